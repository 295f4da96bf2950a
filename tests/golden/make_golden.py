"""Generates tests/golden/reference_sm100.npz: outputs of the reference's own device code.

Run on a machine with an sm_100 GPU after `make -C oracle ref` has compiled the reference's unmodified
cuda/gemm.cu and cuda/gemv.cu into oracle/_ref/ (that step needs the reference checkout; this one does not):

    python tests/golden/make_golden.py --out tests/golden/reference_sm100.npz

Inputs are seeded (CPU generator) and stored next to the outputs, so the fixture is self-contained.
Every array is what the reference's kernel wrote, byte for byte; fp16 arrays are stored as uint16.
"""
import argparse
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle.ref_cuda import ReferenceKernels, ReferenceCublasLt  # noqa: E402
from util import randn_fp16, edge_case_matrix  # noqa: E402


def u16(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.join(ROOT, "tests", "golden", "reference_sm100.npz"))
    args = ap.parse_args()
    ref = ReferenceKernels()
    out = {}

    cases = {
        "a": ((2, 48, 96), 1.0, 101),        # activations-like
        "w": ((1, 40, 160), 0.02, 102),      # weights-like
        "s": ((3, 12, 12), 1.0, 103),        # the reference's smallest odd test shape (tests/test_gemm.py:47)
        "e": (None, None, None),             # edge cases
    }
    for key, (shape, std, seed) in cases.items():
        x = edge_case_matrix() if key == "e" else randn_fp16(shape, seed, std)
        xd = x.cuda()
        sr = ref.gemm_calc_scale(xd)
        sc = ref.gemm_calc_scale_transpose(xd)
        qr = ref.gemm_round(xd, sr)
        qc = ref.gemm_round_transpose(xd, sc)
        out[key + "_x"] = u16(x)
        out[key + "_scale_rows"] = u16(sr)
        out[key + "_scale_cols"] = u16(sc)
        out[key + "_codes_rows"] = qr.cpu().numpy()
        out[key + "_codes_cols"] = qc.cpu().numpy()

    # out-of-range quotients: what (int8_t)nearbyintf(x / s) yields beyond [-128, 127], for inf and for NaN
    cx = np.array([0.0, -0.0, 1.0, -1.0, 0.5, 1.5, 2.5, 127.0, 128.0, 129.0, 200.0, 255.0, 256.0, 300.0, 1000.0, -1000.0, 32768.0,
                   40000.0, 65504.0, -65504.0, 3.0, 7.0, 100.0, -100.0, 1e-3, 6e-8, -6e-8, np.inf, -np.inf, np.nan, 12345.0, -12345.0],
                  dtype=np.float16)
    cs = np.array([1.0, 0.5, 0.25, 2.0 ** -8, 2.0 ** -10, 2.0 ** -14, 2.0 ** -16, 2.0 ** -20, 2.0 ** -24, 0.0, np.inf, np.nan, 3.0, 1e-3,
                   65504.0, 7e-5], dtype=np.float16)
    cxm = torch.from_numpy(np.tile(cx[None, None, :], (1, len(cs), 1)).copy())
    csm = torch.from_numpy(cs[None, :].copy())
    out["c_x"], out["c_s"] = u16(cxm), u16(csm)
    out["c_codes"] = ref.gemm_round(cxm.cuda(), csm.cuda()).cpu().numpy()

    # dequantisation, both broadcast settings (cuda/gemm.cu:37-57)
    g = torch.Generator(device="cpu").manual_seed(104)
    acc = torch.randint(-2_000_000, 2_000_000, (2, 24, 40), generator=g, dtype=torch.int32)
    sx = randn_fp16((2, 24), 105, 0.01).abs()
    sy = randn_fp16((2, 40), 106, 0.001).abs()
    out["d_acc"], out["d_sx"], out["d_sy"] = acc.numpy(), u16(sx), u16(sy)
    out["d_out_ff"] = u16(ref.gemm_scale(acc.cuda(), sx.cuda(), sy.cuda(), False, False))
    out["d_out_tf"] = u16(ref.gemm_scale(acc.cuda(), sx[:1].contiguous().cuda(), sy.cuda(), True, False))
    out["d_out_ft"] = u16(ref.gemm_scale(acc.cuda(), sx.cuda(), sy[:1].contiguous().cuda(), False, True))
    big = torch.tensor([[[2_000_000_000, -2_000_000_000, 16_777_217, 123_456_789]]], dtype=torch.int32)
    bsx = torch.tensor([[1.0]], dtype=torch.float16)
    bsy = torch.tensor([[1.0, 0.5, 2.0 ** -10, 2.0 ** -14]], dtype=torch.float16)
    out["d_big_acc"], out["d_big_sx"], out["d_big_sy"] = big.numpy(), u16(bsx), u16(bsy)
    out["d_big_out"] = u16(ref.gemm_scale(big.cuda(), bsx.cuda(), bsy.cuda(), False, False))

    # backward helpers (cuda/gemm.cu:103-172)
    gr = randn_fp16((2, 20, 32), 107, 0.5)
    bsy2 = randn_fp16((2, 32), 108, 0.01).abs() + 1e-3
    bsx2 = randn_fp16((1, 20), 109, 0.01).abs() + 1e-3
    q1, s1 = ref.gemm_backward_round_scale(gr.cuda(), bsy2.cuda(), False)
    q2, s2 = ref.gemm_backward_scale_round(gr.cuda(), bsx2.cuda(), True)
    out["b_grad"], out["b_sy"], out["b_sx"] = u16(gr), u16(bsy2), u16(bsx2)
    out["b_q_rows"], out["b_s_rows"] = q1.cpu().numpy(), u16(s1)
    out["b_q_cols"], out["b_s_cols"] = q2.cpu().numpy(), u16(s2)

    # GEMV: the reference's own kernels (cuda/gemv.cu:57-164); pinned only within its test tolerances
    mat = randn_fp16((2, 24, 64), 110, 0.1)
    vec = randn_fp16((2, 64), 111, 1.0)
    out["v_mat"], out["v_vec"] = u16(mat), u16(vec)
    out["v_out_rows"] = u16(ref.gemv_fp16_light(mat.cuda(), vec.cuda()))
    mt = mat.transpose(1, 2).contiguous()
    out["v_out_transpose"] = u16(ref.gemv_fp16_transpose_light(mt.cuda(), vec.cuda()))
    out["v_out_shared"] = u16(ref.gemv_broadcast_mat_fp16_light(mat[0].contiguous().cuda(), vec.cuda()))
    qm = torch.randint(-127, 128, (24, 64), generator=g, dtype=torch.int8)
    qv = torch.randint(-127, 128, (2, 64), generator=g, dtype=torch.int8)
    sm = randn_fp16((24,), 112, 0.01).abs()
    sv = randn_fp16((2,), 113, 0.01).abs()
    out["v_qm"], out["v_qv"], out["v_sm"], out["v_sv"] = qm.numpy(), qv.numpy(), u16(sm), u16(sv)
    out["v_out_int8"] = u16(ref.gemv_broadcast_mat_int8(sm.cuda(), qm.cuda(), sv.cuda(), qv.cuda()))

    # the cublasLt int8 GEMM with the reference's layouts, where the library accepts them on this device
    m, k, n = 16, 32, 8
    for aT in (False, True):
        for bT in (False, True):
            A = torch.randint(-127, 128, (2, m, k) if aT else (2, k, m), generator=g, dtype=torch.int8)
            B = torch.randint(-127, 128, (1, k, n) if bT else (1, n, k), generator=g, dtype=torch.int8)
            tag = "g_%d%d" % (aT, bT)
            out[tag + "_A"], out[tag + "_B"] = A.numpy(), B.numpy()
            try:
                lt = ReferenceCublasLt()
                res = torch.empty((2, n, m), dtype=torch.int32, device="cuda")
                lt.gemm_int8(m, k, n, 2, 1, aT, bT, A.cuda(), B.cuda(), res)
                torch.cuda.synchronize()
                out[tag + "_out"] = res.cpu().numpy()
            except RuntimeError as e:
                print("cublasLt int8 aT=%s bT=%s: %s" % (aT, bT, e))
    torch.cuda.synchronize()
    os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
    np.savez_compressed(args.out, **out)
    print("wrote %s (%d arrays, %d bytes)" % (args.out, len(out), os.path.getsize(args.out)))


if __name__ == "__main__":
    main()
