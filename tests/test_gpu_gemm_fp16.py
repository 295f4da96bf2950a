"""GPU parity of the fp16 GEMM (the int8=False branch of bmm) against the exact float64 products rounded once to
fp16, at rtol 1e-3 / atol 1e-2 (the reference's own test allows 0.5 / 0.5, tests/test_gemm.py:98)."""
import os

import numpy as np
import pytest
import torch

import cpm_kernels_b200.kernels as ck
import cpm_kernels_b200.torch as ct
from cpm_kernels_b200.library import cpmk
from oracle import quant_linear as ql
from util import randn_fp16, np16

pytestmark = pytest.mark.gpu
RTOL, ATOL = 1e-3, 1e-2


@pytest.fixture(scope="module")
def G():
    import gpu_util
    return gpu_util


def close(got_fp16, want_f64):
    want16 = want_f64.astype(np.float16).astype(np.float64)
    return np.isclose(got_fp16.astype(np.float64), want16, rtol=RTOL, atol=ATOL)


def run_kernel(G, m, k, n, bA, bB, aT, bT, seed=0):
    ssk = float(k) ** 0.25
    A = randn_fp16((bA, m, k) if aT else (bA, k, m), seed + 1, 1.0 / ssk)
    B = randn_fp16((bB, k, n) if bT else (bB, n, k), seed + 2, 1.0 / ssk)
    Ad, Bd = A.cuda(), B.cuda()
    out = torch.full((max(bA, bB), n, m), 77.0, dtype=torch.half, device="cuda")
    ck.gemm_fp16(m, k, n, bA, bB, aT, bT, Ad.data_ptr(), Bd.data_ptr(), out.data_ptr(), G.stream())
    want = ql.gemm_fp16(m, k, n, aT, bT, np16(A), np16(B))
    got = G.host(out)
    G.assert_no_device_error()
    return got, want


# (m, k, n, batchA, batchB): extents that are multiples of 8 take the tcgen05 kernel
TC_SHAPES = [
    (256, 64, 256, 1, 1), (256, 128, 512, 1, 1), (512, 256, 256, 2, 2),
    (264, 200, 520, 1, 1),          # ragged tiles in both directions, k tail inside a stage
    (128, 8, 64, 3, 1),             # k shorter than one stage; fewer rows than a tile; broadcast B
    (1000, 72, 200, 1, 4),          # row blocks that end inside the second 64-row box of an MN-major tile
    (4096, 512, 768, 1, 1),
]


@pytest.mark.parametrize("aT,bT", [(True, False), (False, False), (True, True), (False, True)])
@pytest.mark.parametrize("shape", TC_SHAPES)
def test_tensor_core_kernel(G, shape, aT, bT):
    m, k, n, bA, bB = shape
    got, want = run_kernel(G, m, k, n, bA, bB, aT, bT, seed=m + n)
    assert cpmk.last_gemm_path() == 1
    ok = close(got, want)
    assert ok.all(), "mismatches: %d of %d" % ((~ok).sum(), ok.size)


@pytest.mark.parametrize("aT,bT", [(True, False), (False, True)])
@pytest.mark.parametrize("shape", [(4, 4, 4, 1, 1), (12, 6, 10, 3, 3), (130, 50, 66, 2, 1), (64, 64, 64, 1, 2)])
def test_generic_kernel(G, shape, aT, bT, monkeypatch):
    m, k, n, bA, bB = shape
    if m % 8 == 0:
        monkeypatch.setenv("CPMK_GEMM_VARIANT", "generic")
    got, want = run_kernel(G, m, k, n, bA, bB, aT, bT, seed=7)
    assert cpmk.last_gemm_path() == 2
    assert close(got, want).all()


def test_linear_shape_full_k(G):
    """One CPM-Bee-sized case (attention-out: N = K = 4096) at M = 1024 tokens, through bmm."""
    x = randn_fp16((1, 1024, 4096), 1, 1.0 / 8.0)
    w = randn_fp16((1, 4096, 4096), 2, 1.0 / 8.0)
    y = ct.bmm(x.cuda(), False, w.cuda(), True, int8=False)
    want = np.matmul(np16(x).astype(np.float64), np.swapaxes(np16(w).astype(np.float64), 1, 2))
    assert cpmk.last_gemm_path() == 1
    assert close(G.host(y), want).all()


@pytest.mark.parametrize("aT,bT", [(False, False), (True, False), (False, True), (True, True)])
def test_bmm_fp16_forward_backward_matches_torch(G, aT, bT):
    b, M, K, N = 2, 64, 96, 128
    a = randn_fp16((b, K, M) if aT else (b, M, K), 3, 0.3).cuda()
    w = randn_fp16((1, N, K) if bT else (1, K, N), 4, 0.3).cuda()
    a1, w1 = a.clone().requires_grad_(), w.clone().requires_grad_()
    a2, w2 = a.clone().float().requires_grad_(), w.clone().float().requires_grad_()
    out = ct.bmm(a1, aT, w1, bT, int8=False)
    ref = torch.matmul(a2.transpose(1, 2) if aT else a2, w2.transpose(1, 2) if bT else w2)
    g = randn_fp16(tuple(out.shape), 5, 0.5).cuda()
    out.backward(g)
    ref.backward(g.float())
    assert torch.allclose(out.float(), ref, rtol=2e-3, atol=2e-2)
    assert torch.allclose(a1.grad.float(), a2.grad, rtol=2e-3, atol=2e-2)
    assert torch.allclose(w1.grad.float(), w2.grad, rtol=2e-3, atol=5e-2)
    G.assert_no_device_error()


def test_empty_and_zero_k(G):
    ck.gemm_fp16(0, 8, 8, 1, 1, True, False, 0, 0, 0, G.stream())
    out = torch.full((1, 8, 8), 3.0, dtype=torch.half, device="cuda")
    ck.gemm_fp16(8, 0, 8, 1, 1, True, False, 0, 0, out.data_ptr(), G.stream())
    assert (G.host(out) == 0).all()
    with pytest.raises(AssertionError):
        ck.gemm_fp16(3, 8, 8, 1, 1, True, False, 0, 0, out.data_ptr(), G.stream())
