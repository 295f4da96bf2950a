"""The allocation-free transposed GEMV (cpmk_gemv_fp16_transpose_noalloc) against the regular entry point.

Some callers of this library cannot let it allocate device memory: inference servers whose own pool already owns
the whole GPU, host applications that forbid allocation calls in their plug-ins, and real-time loops that cannot
take the device-wide stall of a cudaMalloc.  For them the library offers this one entry point, whose scratch lives in a
fixed array inside the library's device image.  The test calls it through the C ABI twice in a row (the array
keeps the previous call's contents, so the second call exercises the clearing) and checks the results against
the regular entry point, and against the exact (float64) oracle as every other GEMV test does, within the GEMV
tests' tolerance (rtol 1e-3, atol 1e-2).

This file sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import numpy as np
import pytest
import torch

from cpm_kernels_b200.library import cpmk
from oracle import quant_linear as ql
from util import randn_fp16

pytestmark = pytest.mark.gpu
RTOL, ATOL = 1e-3, 1e-2


def _run(entry, batch, dim_out, dim_in, mat, vec):
    out = torch.full((batch, dim_out), 9.0, dtype=torch.half, device="cuda")
    cpmk.call(entry, batch, dim_out, dim_in, mat.data_ptr(), vec.data_ptr(), out.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return out.cpu().numpy().astype(np.float64)


@pytest.mark.parametrize("batch,dim_out,dim_in", [(1, 10240, 4096), (4, 1024, 2048), (2, 264, 100), (16, 128, 2222)])
def test_noalloc_matches_regular_entry_point_twice(batch, dim_out, dim_in):
    ssk = float(dim_in) ** 0.25
    mat_h = randn_fp16((batch, dim_in, dim_out), 31, 1.0 / ssk)
    vec_h = randn_fp16((batch, dim_in), 32, 1.0 / ssk)
    mat, vec = mat_h.cuda(), vec_h.cuda()
    want = _run("cpmk_gemv_fp16_transpose", batch, dim_out, dim_in, mat, vec)
    first = _run("cpmk_gemv_fp16_transpose_noalloc", batch, dim_out, dim_in, mat, vec)
    assert np.isclose(first, want, rtol=RTOL, atol=ATOL).all()
    exact = ql.gemv_fp16_transpose(mat_h.numpy(), vec_h.numpy()).astype(np.float16).astype(np.float64)   # exact sum, rounded once
    assert np.isclose(first, exact, rtol=RTOL, atol=ATOL).all()
    # second call, different data of the same shape: nothing of the first call may leak through the shared array
    vec2 = randn_fp16((batch, dim_in), 33, 1.0 / ssk).cuda()
    want2 = _run("cpmk_gemv_fp16_transpose", batch, dim_out, dim_in, mat, vec2)
    second = _run("cpmk_gemv_fp16_transpose_noalloc", batch, dim_out, dim_in, mat, vec2)
    assert np.isclose(second, want2, rtol=RTOL, atol=ATOL).all()
    assert cpmk.read_status() == 0


def test_noalloc_rejects_sizes_beyond_its_fixed_scratch():
    a = torch.zeros(16, dtype=torch.half, device="cuda")
    with pytest.raises(RuntimeError, match="exceeds the fixed scratch"):
        cpmk.call("cpmk_gemv_fp16_transpose_noalloc", 64, 16384, 64, a.data_ptr(), a.data_ptr(), a.data_ptr(), None)
    with pytest.raises(RuntimeError, match="dim_out"):
        cpmk.call("cpmk_gemv_fp16_transpose_noalloc", 1, 12, 64, a.data_ptr(), a.data_ptr(), a.data_ptr(), None)
