"""GPU parity of GELU -- standalone and chained after the int8 GEMM -- against the reference's own kernel,
whose complete behaviour (all 65536 fp16 inputs) is recorded in tests/golden/reference_gelu_sm100.npz.  Bit-exact."""
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
TABLE = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_gelu_sm100.npz"))["gelu_of_every_fp16"]


@pytest.fixture(scope="module")
def G():
    import gpu_util
    return gpu_util


def lookup(x_fp16: np.ndarray) -> np.ndarray:
    return TABLE[x_fp16.view(np.uint16)]


def test_every_fp16_value(G):
    x = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.float16).reshape(4, 16384).cuda()
    out = torch.empty_like(x)
    ck.gelu_forward(4, 16384, x.data_ptr(), out.data_ptr(), G.stream())
    assert (G.host(out).view(np.uint16).reshape(-1) == TABLE).all()
    assert (ql.gelu_forward(G.host(x)).view(np.uint16).reshape(-1) == TABLE).all()


@pytest.mark.parametrize("batch,n", [(1, 5), (3, 1000), (2, (1 << 20) + 8), (3, (1 << 20) + 3), (1, 4096 * 10240)])
def test_sizes_and_in_place(G, batch, n):
    """Small inputs evaluate the expression; from 2^21 elements on the table kernel runs (with a ragged tail when the
    count is not a multiple of 8)."""
    x = randn_fp16((batch, n), 5, 1.5)
    want = lookup(np16(x))
    xd = x.cuda()
    out = torch.empty_like(xd)
    ck.gelu_forward(batch, n, xd.data_ptr(), out.data_ptr(), G.stream())
    assert (G.host(out).view(np.uint16) == want).all()
    ck.gelu_inplace_forward(batch, n, xd.data_ptr(), G.stream())
    assert (G.host(xd).view(np.uint16) == want).all()
    assert (G.host(ct.gelu(x.cuda())).view(np.uint16) == want).all()
    G.assert_no_device_error()


@pytest.mark.parametrize("m,k,n,aT,bT,generic", [(512, 256, 512, True, False, False), (272, 128, 528, False, True, False),
                                                 (12, 8, 20, True, False, True), (256, 128, 256, True, False, True)])
def test_gemm_gelu_equals_two_calls(G, m, k, n, aT, bT, generic, monkeypatch):
    if generic and m % 16 == 0:
        monkeypatch.setenv("CPMK_GEMM_VARIANT", "generic")
    rng = np.random.default_rng(m + n)
    A = torch.from_numpy(rng.integers(-127, 128, size=(1, m, k) if aT else (1, k, m), dtype=np.int8)).cuda()
    B = torch.from_numpy(rng.integers(-127, 128, size=(1, k, n) if bT else (1, n, k), dtype=np.int8)).cuda()
    sx = (randn_fp16((1, n), 1, 0.004).abs() + 1e-3).cuda()
    sy = (randn_fp16((1, m), 2, 0.004).abs() + 1e-3).cuda()
    plain = torch.empty((1, n, m), dtype=torch.half, device="cuda")
    fused = torch.empty_like(plain)
    ck.gemm_int8_scale(m, k, n, 1, 1, aT, bT, A.data_ptr(), B.data_ptr(), sx.data_ptr(), sy.data_ptr(), False, False, plain.data_ptr(), G.stream())
    ck.gemm_int8_scale_gelu(m, k, n, 1, 1, aT, bT, A.data_ptr(), B.data_ptr(), sx.data_ptr(), sy.data_ptr(), False, False, fused.data_ptr(), G.stream())
    assert cpmk.last_gemm_path() == (2 if generic else 1)          # GELU runs after either GEMM kernel
    got = G.host(fused).view(np.uint16)
    assert (got == lookup(G.host(plain))).all()
    if k >= 128:
        assert np.abs(G.host(plain).astype(np.float32)).max() > 1.0      # the activation is exercised beyond its linear range
    G.assert_no_device_error()


def test_bmm_gelu(G):
    x = randn_fp16((2, 256, 512), 1, 1.0).cuda()
    w = randn_fp16((1, 384, 512), 2, 0.05).cuda()
    y = ct.bmm(x, False, w, True, int8=True)
    z = ct.bmm_gelu(x, False, w, True)
    assert (G.host(z).view(np.uint16) == lookup(G.host(y))).all()
    y2 = y.clone()
    ct.gelu_inplace(y2)
    assert torch.equal(y2.view(torch.int16), z.view(torch.int16))


def test_backward_matches_the_references_own_kernel_on_every_input(G):
    """gelu_backward for every fp16 x, against cu_gelu_backward compiled from the reference's source and run on the same
    GPU (bit for bit), and against the binary64 restatement of its formula (to a tolerance: the device's coshf / tanhf
    are not correctly rounded)."""
    from oracle import ref_cuda
    x = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.float16).reshape(4, 16384).cuda()
    for scale in (1.0, -0.37, 24.0):
        g = (randn_fp16((4, 16384), 17) * scale).half().cuda()
        grad = torch.empty_like(x)
        ck.gelu_backward(4, 16384, g.data_ptr(), x.data_ptr(), grad.data_ptr(), G.stream())
        got = G.host(grad)
        if ref_cuda.available():
            want = ref_cuda.ReferenceKernels().gelu_backward(g, x)
            assert (got.view(np.uint16) == G.host(want).view(np.uint16)).all()
        exact = ql.gelu_backward(G.host(g), G.host(x))
        finite = np.isfinite(exact) & (np.abs(exact) < 6e4)
        assert np.isclose(got.astype(np.float64)[finite], exact[finite], rtol=2e-3, atol=1e-3).all()
    G.assert_no_device_error()


@pytest.mark.parametrize("batch,n", [(1, 5), (3, 1001), (2, 70000)])
def test_autograd_backward_runs_on_the_kernel(G, batch, n):
    """torch.gelu's backward (cpm_kernels/torch/gelu.py:17-32): odd sizes (scalar tail), unaligned views are refused."""
    x = randn_fp16((batch, n), 6, 2.0)
    g = randn_fp16((batch, n), 7, 0.5)
    xd = x.cuda().requires_grad_()
    y = ct.gelu(xd)
    y.backward(gradient=g.cuda())
    exact = ql.gelu_backward(np16(g), np16(x))
    assert np.isclose(G.host(xd.grad).astype(np.float64), exact, rtol=2e-3, atol=1e-3).all()
    if batch > 1:
        with pytest.raises(AssertionError):
            y2 = ct.gelu(x.cuda().requires_grad_())
            y2.backward(gradient=g.cuda().t().contiguous().t())       # not contiguous
