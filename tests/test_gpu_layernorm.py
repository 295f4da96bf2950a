"""GPU parity of the fused layer norm -> affine -> column quantisation with the reference's own four-kernel chain:
bit for bit against its recorded outputs (tests/golden/reference_layernorm_sm100.npz) and, where the reference's device
code was built (oracle/_ref), against that chain run live at the sizes of a CPM layer."""
import os

import numpy as np
import pytest
import torch

import cpm_kernels_b200.torch as ct
from oracle import ref_cuda
from util import randn_fp16, np16

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_layernorm_sm100.npz"))
# name -> (eps, rd_mean), as tests/golden/make_golden_layernorm.py generated them
CASES = {"mean_bias": (1e-5, True), "rms": (1e-6, False), "hidden4096": (1e-6, False), "ragged_rms_bias": (1e-5, False)}


@pytest.fixture(scope="module")
def G():
    import gpu_util
    return gpu_util


def t16(name):
    return torch.from_numpy(GOLD[name].view(np.float16).copy())


@pytest.mark.parametrize("name", sorted(CASES))
def test_recorded_reference_outputs(G, name):
    eps, rd_mean = CASES[name]
    x = t16(name + "_x").cuda()
    alpha = t16(name + "_alpha").cuda()
    beta = t16(name + "_beta").cuda() if name + "_beta" in GOLD else None
    scale, codes = ct.layernorm_quantize(x, eps, alpha, beta, rd_mean)
    assert (G.host(scale).view(np.uint16) == GOLD[name + "_scale"]).all()
    assert (G.host(codes) == GOLD[name + "_codes"]).all()
    G.assert_no_device_error()


@pytest.fixture(scope="module")
def ref():
    if not (ref_cuda.available() and os.path.exists(os.path.join(ref_cuda.REF_DIR, "layernorm.fatbin"))
            and os.path.exists(os.path.join(ref_cuda.REF_DIR, "arith.fatbin"))):
        pytest.skip("the reference's layer-norm device code was not built (oracle/_ref)")
    return ref_cuda.ReferenceKernels()


@pytest.mark.parametrize("shape,eps,rd_mean,bias", [((8, 4096, 512), 1e-6, False, False), ((2, 1100, 72), 1e-5, True, True),
                                                    ((1, 2560, 1024), 1e-5, True, False), ((3, 40, 8), 1e-5, False, True),
                                                    ((1, 5000, 200), 1e-6, True, True)])
def test_against_the_reference_chain(G, ref, shape, eps, rd_mean, bias):
    x = (randn_fp16(shape, shape[1] + shape[2], 1.5).float() + 0.3).half().cuda()
    alpha = (randn_fp16((shape[1],), 5, 0.1).float() + 1.0).half().cuda()
    beta = randn_fp16((shape[1],), 6, 0.1).cuda() if bias else None
    ln = ref.layernorm_forward(x, eps, rd_mean)
    aff = ref.arith_ln_mul_add(ln, alpha, beta) if bias else ref.arith_ln_mul(ln, alpha)
    want_scale = ref.gemm_calc_scale_transpose(aff)
    want_codes = ref.gemm_round_transpose(aff, want_scale)
    scale, codes = ct.layernorm_quantize(x, eps, alpha, beta, rd_mean)
    assert torch.equal(scale.view(torch.int16), want_scale.view(torch.int16))
    assert torch.equal(codes, want_codes)
    G.assert_no_device_error()


def test_feeds_the_int8_linear(G, ref):
    """bmm(W, False, affine(layernorm(x)), False, int8=True) == bmm_quantized_b(W, False, *layernorm_quantize(x), False)."""
    x = randn_fp16((2, 512, 256), 1, 1.0).cuda()          # (batch, hidden, seq)
    alpha = (randn_fp16((512,), 2, 0.1).float() + 1.0).half().cuda()
    w = randn_fp16((1, 384, 512), 3, 0.05).cuda()          # (1, N, K = hidden)
    aff = ref.arith_ln_mul(ref.layernorm_forward(x, 1e-6, False), alpha)
    want = ct.bmm(w, False, aff, False, int8=True)
    scale, codes = ct.layernorm_quantize(x, 1e-6, alpha, None, False)
    got = ct.bmm_quantized_b(w, False, scale, codes, False)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
