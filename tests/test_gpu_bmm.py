"""GPU parity of the torch-level entry point ``bmm(A, aT, B, bT, int8=True)`` (cpm_kernels/torch/gemm.py:233)
against the oracle's restatement of GEMMInt8.forward, for every storage order and broadcast."""
import numpy as np
import pytest
import torch

import cpm_kernels_b200.torch as ct
from cpm_kernels_b200.library import cpmk
from oracle import quant_linear as ql
from oracle import test_formula
from util import randn_fp16, np16

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def G():
    import gpu_util
    return gpu_util


def make(batch, m, k, n, tp, aT, bT, seed):
    """As generate_matrix in tests/test_gemm.py:62-85, seeded: values randn / k**0.25, optional broadcast, optional transposed storage."""
    skk = float(k) ** 0.25
    bA, bB = (batch, batch) if tp == 0 else ((1, batch) if tp == 1 else (batch, 1))
    a = randn_fp16((bA, m, k), seed, 1.0 / skk)
    b = randn_fp16((bB, k, n), seed + 1, 1.0 / skk)
    if aT:
        a = a.transpose(-1, -2).contiguous()
    if bT:
        b = b.transpose(-1, -2).contiguous()
    return a, b


# tests/test_gemm.py:43-60 (batch, m, k, n); the three largest are covered at full size by the checksum test below
CASES = [(1, 4, 4, 4), (2, 4, 4, 4), (1, 8, 8, 8), (3, 12, 12, 12), (1, 16, 16, 16), (1, 32, 32, 32), (1, 64, 64, 64),
         (1, 128, 128, 128), (4, 128, 128, 128), (8, 128, 128, 128), (8, 112, 224, 112), (2, 512, 1024, 256), (2, 500, 512, 796)]


@pytest.mark.parametrize("batch,m,k,n", CASES)
@pytest.mark.parametrize("aT,bT", [(False, False), (True, False), (False, True), (True, True)])
@pytest.mark.parametrize("tp", [0, 1, 2])
def test_bmm_int8_forward(G, batch, m, k, n, aT, bT, tp):
    a, b = make(batch, m, k, n, tp, aT, bT, seed=batch + m + k + n)
    want = ql.bmm_int8(np16(a), aT, np16(b), bT)
    out = ct.bmm(a.cuda(), aT, b.cuda(), bT, int8=True)
    assert out.shape == want["out"].shape
    assert G.same_bits(out, want["out"])                                    # bit-exact, hence within rtol 1e-3 / atol 1e-2
    # and the reference's own acceptance test (tests/test_gemm.py:96-98)
    ans = test_formula.real_bmm(a, aT, b, bT, True)
    assert torch.isclose(out.cpu().float(), ans.float(), rtol=5e-1, atol=5e-1).all()
    G.assert_no_device_error()


def test_linear_layer_uses_tensor_core_kernel(G):
    """nn.Linear convention: x (1, M, K) row-major, W (1, N, K) row-major -> bmm(x, False, W, True)."""
    x = randn_fp16((1, 512, 2560), 0)
    w = randn_fp16((1, 10240, 2560), 1, 0.02)
    out = ct.bmm(x.cuda(), False, w.cuda(), True, int8=True)            # configuration 1
    assert cpmk.last_gemm_path() == 1
    want = ql.bmm_int8(np16(x), False, np16(w), True)
    assert G.same_bits(out, want["out"])
    # the saved tensors of the autograd function are the separate passes' results
    from cpm_kernels_b200.torch.gemm import quantize
    s, q = quantize(x.cuda(), False)
    assert G.same_bits(s, want["scale_A"]) and (G.host(q) == want["quant_A"]).all()
    s, q = quantize(w.cuda(), False)
    assert G.same_bits(s, want["scale_B"]) and (G.host(q) == want["quant_B"]).all()


def test_attention_scores_shape(G):
    """Configuration 4 at reduced batch: Q (b, 512, 128) x K (b, 512, 128)^T -> (b, 512, 512)."""
    q = randn_fp16((6, 512, 128), 2)
    kk = randn_fp16((6, 512, 128), 3)
    out = ct.bmm(q.cuda(), False, kk.cuda(), True, int8=True)
    assert cpmk.last_gemm_path() == 1
    assert G.same_bits(out, ql.bmm_int8(np16(q), False, np16(kk), True)["out"])


def test_attention_scores_full_batch(G):
    """Configuration 4 at its full size: batch 256 (8 sequences x 32 heads), Q and K (256, 512, 128) -> (256, 512, 512):
    1024 pair tiles, the batch coordinate of the tensor maps at size."""
    q = randn_fp16((256, 512, 128), 2)
    kk = randn_fp16((256, 512, 128), 3)
    out = ct.bmm(q.cuda(), False, kk.cuda(), True, int8=True)
    assert cpmk.last_gemm_path() == 1
    want = ql.bmm_int8(np16(q), False, np16(kk), True)
    assert G.same_bits(out, want["out"])
    G.assert_no_device_error()


def test_linear_at_16384_tokens(G):
    """The token count of configuration 5 on the attention-out shape: x (1, 16384, 4096), W (1, 4096, 4096)."""
    x = randn_fp16((1, 16384, 4096), 4)
    w = randn_fp16((1, 4096, 4096), 5, 0.02)
    out = ct.bmm(x.cuda(), False, w.cuda(), True, int8=True)
    assert cpmk.last_gemm_path() == 1
    assert G.same_bits(out, ql.bmm_int8(np16(x), False, np16(w), True)["out"])
    G.assert_no_device_error()


def test_backward_matches_composition_of_oracle_steps(G):
    """GEMMInt8.backward (torch/gemm.py:116-179) restated with the oracle's step functions."""
    for (aT, bT, bA, bB) in [(False, False, 2, 2), (True, False, 2, 1), (False, True, 1, 2), (True, True, 2, 2)]:
        M, K, N = 24, 40, 16
        a = randn_fp16((bA, K, M) if aT else (bA, M, K), 5, 0.5)
        b = randn_fp16((bB, N, K) if bT else (bB, K, N), 6, 0.5)
        batch = max(bA, bB)
        grad = randn_fp16((batch, M, N), 7, 0.3)
        ad, bd = a.cuda().requires_grad_(), b.cuda().requires_grad_()
        out = ct.bmm(ad, aT, bd, bT, int8=True)
        out.backward(gradient=grad.cuda())
        fw = ql.bmm_int8(np16(a), aT, np16(b), bT)
        g = np16(grad)

        def gemm_and_scale(qA, sA, qB, sB, aT_, bT_):
            M_ = qA.shape[2] if aT_ else qA.shape[1]
            K_ = qA.shape[1] if aT_ else qA.shape[2]
            N_ = qB.shape[1] if bT_ else qB.shape[2]
            acc = ql.gemm_int8(N_, K_, M_, bT_, aT_, qB, qA)
            if sA is not None:
                return ql.gemm_scale_x(acc, sA)
            return ql.gemm_scale_y(acc, sB)

        qGa, sGa = ql.gemm_backward_round_scale(g, fw["scale_B"], bB == 1)
        gA = gemm_and_scale(fw["quant_B"], None, qGa, sGa, bT, True) if aT else gemm_and_scale(qGa, sGa, fw["quant_B"], None, False, not bT)
        qGb, sGb = ql.gemm_backward_scale_round(g, fw["scale_A"], bA == 1)
        gB = gemm_and_scale(qGb, sGb, fw["quant_A"], None, True, aT) if bT else gemm_and_scale(fw["quant_A"], None, qGb, sGb, not aT, False)
        if bA == 1 and gA.shape[0] > 1:
            gA = torch.from_numpy(gA).cuda().sum(dim=0, keepdim=True).cpu().numpy()
        if bB == 1 and gB.shape[0] > 1:
            gB = torch.from_numpy(gB).cuda().sum(dim=0, keepdim=True).cpu().numpy()
        assert np.isclose(G.host(ad.grad).astype(np.float32), gA.astype(np.float32), rtol=1e-3, atol=1e-2).all(), (aT, bT)
        assert np.isclose(G.host(bd.grad).astype(np.float32), gB.astype(np.float32), rtol=1e-3, atol=1e-2).all(), (aT, bT)


def test_float_branch_is_a_plain_matmul(G):
    a, b = make(2, 32, 64, 48, 0, False, True, 9)
    out = ct.bmm(a.cuda(), False, b.cuda(), True, int8=False)
    ans = torch.matmul(a.double(), b.double().transpose(-1, -2)).half()       # the exact product, rounded once
    assert torch.isclose(out.cpu().float(), ans.float(), rtol=1e-3, atol=1e-2).all()


@pytest.mark.skipif(not __import__("oracle.ref_cuda", fromlist=["x"]).available(), reason="oracle/_ref fatbins not built")
@pytest.mark.parametrize("batch,m,k,n,tp,aT,bT", [
    (8, 512, 4096, 2048, 0, False, False), (8, 500, 4096, 7996, 2, True, False), (8, 512, 10240, 4096, 1, False, True),
    (8, 1024, 512, 4096, 0, True, True), (1, 4096, 4096, 12288, 0, False, True), (1, 4096, 10240, 4096, 0, False, False)])
def test_full_size_bmm_equals_the_references_own_pipeline(G, batch, m, k, n, tp, aT, bT):
    """The largest shapes of the reference's test list (tests/test_gemm.py:54-59) and two CPM-Bee-10B linears: the result
    of bmm(int8=True) must equal, bit for bit, what the reference's own kernels (compiled from its sources) and its
    cublasLt call sequence produce for the same tensors on the same GPU: calc_scale, round, gemm_int8, gemm_scale
    (cpm_kernels/torch/gemm.py:98-104)."""
    from oracle import ref_cuda
    g = torch.Generator(device="cuda").manual_seed(batch + m + n)
    bA, bB = (batch, batch) if tp == 0 else ((1, batch) if tp == 1 else (batch, 1))
    skk = float(k) ** 0.25
    a = (torch.randn((bA, k, m) if aT else (bA, m, k), generator=g, device="cuda") / skk).half()
    b = (torch.randn((bB, n, k) if bT else (bB, k, n), generator=g, device="cuda") / skk).half()
    out = ct.bmm(a, aT, b, bT, int8=True)
    ref = ref_cuda.ReferenceKernels()
    lt = ref_cuda.ReferenceCublasLt()
    sa = ref.gemm_calc_scale_transpose(a) if aT else ref.gemm_calc_scale(a)
    sb = ref.gemm_calc_scale(b) if bT else ref.gemm_calc_scale_transpose(b)
    qa = ref.gemm_round_transpose(a, sa) if aT else ref.gemm_round(a, sa)
    qb = ref.gemm_round(b, sb) if bT else ref.gemm_round_transpose(b, sb)
    acc = torch.empty((max(bA, bB), m, n), dtype=torch.int32, device="cuda")
    lt.gemm_int8(n, k, m, bB, bA, bT, aT, qb, qa, acc)                      # operands swapped as torch/gemm.py:45-52
    want = ref.gemm_scale(acc, sa, sb, bA == 1, bB == 1)
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), want.view(torch.int16))
    G.assert_no_device_error()
