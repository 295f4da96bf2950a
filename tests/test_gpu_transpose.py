"""GPU parity of the batched fp16 transpose (cpm_kernels/kernels/transpose.py, torch/transpose.py) against the CPU
oracle, bit for bit: through the C ABI, through the torch-level autograd function, and through the loadable module
under the reference's own launch shape; the reference's device code, where built, is held to the same oracle."""
import os

import numpy as np
import pytest
import torch

import cpm_kernels_b200.kernels as ck
import cpm_kernels_b200.torch as ct
from cpm_kernels_b200 import build
from cpm_kernels_b200.library import cpmk
from oracle import quant_linear as ql
from oracle import ref_cuda
from util import randn_fp16, np16

pytestmark = pytest.mark.gpu

# the shapes of the reference's tests/test_transpose.py:9-19, then: odd sizes, sizes that are multiples of 8 but
# not of 64 (ragged tiles of the 16-byte path), one element, a batch beyond 65535, the activation of the bench
REFERENCE_SHAPES = [(1, 2, 32), (4, 128, 128), (16, 128, 32), (4, 16, 128), (123, 512, 321), (123, 768, 321), (233, 1024, 321),
                    (4, 123, 16), (4, 321, 16)]
MORE_SHAPES = [(1, 1, 1), (3, 7, 5), (2, 8, 8), (2, 72, 136), (1, 200, 8), (1, 8, 200), (70000, 2, 3), (66000, 8, 8), (5, 33, 66),
               (1, 4096, 4096), (2, 10240, 512)]


@pytest.fixture(scope="module")
def G():
    import gpu_util
    return gpu_util


def rows_tagged(shape, seed):
    """Random fp16 values; every bit pattern is data here, so NaN payloads and infinities are included."""
    rng = np.random.default_rng(seed)
    return torch.from_numpy(rng.integers(0, 65536, size=shape, dtype=np.uint16).view(np.int16).copy()).view(torch.float16)


@pytest.mark.parametrize("shape", REFERENCE_SHAPES + MORE_SHAPES)
def test_c_abi_against_oracle(G, shape):
    x = rows_tagged(shape, sum(shape))
    want = ql.transpose(np16(x)).view(np.uint16)
    xd = x.cuda()
    out = torch.full((shape[0], shape[2], shape[1]), -1.0, dtype=torch.half, device="cuda")
    ck.transpose(shape[0], shape[1], shape[2], xd.data_ptr(), out.data_ptr(), G.stream())
    assert (G.host(out).view(np.uint16) == want).all()
    G.assert_no_device_error()


def test_unaligned_pointers_take_the_element_path(G):
    """A view that starts 2 bytes into an allocation cannot use 16-byte accesses; the result is the same."""
    b, n, m = 2, 64, 128
    buf = rows_tagged((b * n * m + 1,), 3).cuda()
    outbuf = torch.zeros(b * n * m + 1, dtype=torch.half, device="cuda")
    ck.transpose(b, n, m, buf.data_ptr() + 2, outbuf.data_ptr() + 2, G.stream())
    want = ql.transpose(G.host(buf)[1:].reshape(b, n, m)).view(np.uint16)
    assert (G.host(outbuf)[1:].view(np.uint16).reshape(b, m, n) == want).all()


def test_twice_is_identity_full_size(G):
    """Size-independent property at the bench's activation size: transposing twice returns the input."""
    x = randn_fp16((4, 4096, 10240), 9, 1.0).cuda()
    y = ct.transpose(ct.transpose(x))
    assert torch.equal(y.view(torch.int16), x.view(torch.int16))
    assert torch.equal(ct.transpose(x).view(torch.int16), ct.transposeTH(x).contiguous().view(torch.int16))


@pytest.mark.parametrize("shape", [(4, 128, 128), (123, 512, 321), (4, 123, 16)])
def test_autograd_like_the_reference_test(G, shape):
    """tests/test_transpose.py:20-36: forward and gradient equal to x.transpose(1, 2)."""
    x = randn_fp16(shape, 1, 1.0).cuda()
    x1 = x.clone().requires_grad_()
    x2 = x.clone().requires_grad_()
    y1 = ct.transposeTH(x1)
    y2 = ct.transpose(x2)
    assert torch.equal(y1, y2)
    rd = randn_fp16((shape[0], shape[2], shape[1]), 2, 1.0).cuda()
    y1.backward(gradient=rd)
    y2.backward(gradient=rd)
    assert torch.equal(x1.grad, x2.grad)


def test_rejects_in_place_and_negative_sizes(G):
    x = torch.zeros(64, dtype=torch.half, device="cuda")
    with pytest.raises(RuntimeError):
        ck.transpose(1, 8, 8, x.data_ptr(), x.data_ptr(), G.stream())
    with pytest.raises(RuntimeError):
        ck.transpose(1, -8, 8, x.data_ptr(), x.data_ptr() + 0, G.stream())
    assert "transpose" in cpmk.last_error() or "negative" in cpmk.last_error()
    ck.transpose(0, 8, 8, x.data_ptr(), x.data_ptr(), G.stream())          # nothing to do: accepted


@pytest.mark.parametrize("shape", REFERENCE_SHAPES + [(3, 7, 5), (2, 72, 136), (1, 4096, 4096)])
def test_module_under_the_reference_launch(G, shape):
    """lib/transpose.fatbin loaded and launched exactly as kernels/transpose.py:11-27 does."""
    assert os.path.exists(build.module_path("transpose")), "kernel module not built"
    mod = ref_cuda.ReferenceKernels(fatbin_dir=build.LIB_DIR)
    x = rows_tagged(shape, 5 + sum(shape))
    want = ql.transpose(np16(x)).view(np.uint16)
    assert (G.host(mod.transpose(x.cuda())).view(np.uint16) == want).all()
    if ref_cuda.available() and os.path.exists(os.path.join(ref_cuda.REF_DIR, "transpose.fatbin")):
        ref = ref_cuda.ReferenceKernels()
        assert (G.host(ref.transpose(x.cuda())).view(np.uint16) == want).all()
