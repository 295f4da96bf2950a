"""Generates tests/golden/reference_layernorm_sm100.npz: the reference's own layer-norm -> affine -> column-quantisation
chain (cu_layernorm_forward, cu_arith_ln_mul / cu_arith_ln_mul_add, cu_gemm_calc_scale_transpose,
cu_gemm_round_transpose; compiled unmodified for sm_100 into oracle/_ref by `make -C oracle ref`) on seeded inputs.

    python tests/golden/make_golden_layernorm.py          (on a machine with an sm_100 GPU)

Inputs are stored next to the outputs; fp16 arrays are stored as uint16 bit patterns.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle.ref_cuda import ReferenceKernels  # noqa: E402
from util import randn_fp16  # noqa: E402

# name -> (shape (batch, n, m), eps, rd_mean, bias)
CASES = {
    "mean_bias": ((2, 96, 64), 1e-5, True, True),
    "rms": ((2, 96, 64), 1e-6, False, False),
    "ragged": ((1, 1100, 10), 1e-5, True, False),        # n > 1024 and not a multiple of 32; m not a multiple of 8
    "hidden4096": ((1, 4096, 8), 1e-6, False, False),
    "ragged_rms_bias": ((3, 70, 24), 1e-5, False, True),
}


def u16(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def inputs(name):
    shape, eps, rd_mean, bias = CASES[name]
    seed = sum(ord(c) for c in name)
    x = (randn_fp16(shape, seed, 1.5).float() + 0.3).half()
    alpha = (randn_fp16((shape[1],), seed + 1, 0.1).float() + 1.0).half()
    beta = randn_fp16((shape[1],), seed + 2, 0.1) if bias else None
    return x, alpha, beta, eps, rd_mean


def main():
    out_path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "reference_layernorm_sm100.npz")
    ref = ReferenceKernels()
    out = {}
    for name in CASES:
        x, alpha, beta, eps, rd_mean = inputs(name)
        xd, ad = x.cuda(), alpha.cuda()
        ln = ref.layernorm_forward(xd, eps, rd_mean)
        aff = ref.arith_ln_mul_add(ln, ad, beta.cuda()) if beta is not None else ref.arith_ln_mul(ln, ad)
        scale = ref.gemm_calc_scale_transpose(aff)
        codes = ref.gemm_round_transpose(aff, scale)
        torch.cuda.synchronize()
        out[name + "_x"] = u16(x)
        out[name + "_alpha"] = u16(alpha)
        if beta is not None:
            out[name + "_beta"] = u16(beta)
        out[name + "_ln"] = u16(ln)
        out[name + "_affine"] = u16(aff)
        out[name + "_scale"] = u16(scale)
        out[name + "_codes"] = codes.cpu().numpy()
    np.savez_compressed(out_path, **out)
    print("wrote", out_path, len(out), "arrays")


if __name__ == "__main__":
    main()
