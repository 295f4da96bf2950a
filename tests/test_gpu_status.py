"""The give-up path of the library's device-side waits, exercised without faulting or hanging anything: a one-block
kernel waits, with a 1 ms limit, on a barrier on which nothing arrives.  The wait must end by itself, the failure must
reach the host as CPMK_EDEVICE exactly once, and the library must work normally afterwards (status word and ticket
counters cleared).  Also: the workspace table (one workspace per stream, released on request)."""
import numpy as np
import pytest
import torch

import cpm_kernels_b200.torch as ct
from cpm_kernels_b200.library import cpmk
from oracle import quant_linear as ql
from util import randn_fp16, np16

pytestmark = pytest.mark.gpu


def test_bounded_wait_runs_out_and_the_library_recovers():
    s = torch.cuda.current_stream().cuda_stream
    assert cpmk.read_status() == 0
    # the wait gives up after ~1 ms; the call returns CPMK_OK because giving up is what the self-test expects
    cpmk.call("cpmk_selftest_bounded_wait", 1000, s)
    # the failure code the kernel left is reported once, as CPMK_EDEVICE, and cleared
    with pytest.raises(RuntimeError, match=r"status 4.*0x901"):
        cpmk.check_stream(s)
    cpmk.check_stream(s)                                  # second read: clean
    assert cpmk.read_status() == 0
    # the context is intact: a tensor-core GEMM and a ticketed kernel on the same stream are bit-exact afterwards
    x = randn_fp16((1, 300, 512), 11)
    w = randn_fp16((1, 520, 512), 12, 0.02)
    out = ct.bmm(x.cuda(), False, w.cuda(), True, int8=True)
    assert cpmk.last_gemm_path() == 1
    want = ql.bmm_int8(np16(x), False, np16(w), True)["out"]
    assert (out.cpu().numpy().view(np.uint16) == want.view(np.uint16)).all()
    from cpm_kernels_b200.torch.gemm import quantize
    a = randn_fp16((2, 700, 264), 13)
    sc, q = quantize(a.cuda(), True)                      # column quantisation: scratch + workspace
    assert (sc.cpu().numpy().view(np.uint16) == ql.gemm_calc_scale_transpose(np16(a)).view(np.uint16)).all()
    cpmk.check_stream(s)


def test_read_status_reports_the_code_too():
    s = torch.cuda.current_stream().cuda_stream
    cpmk.call("cpmk_selftest_bounded_wait", 500, s)
    assert cpmk.read_status() == 0x901
    assert cpmk.read_status() == 0


def test_selftest_rejects_limits_out_of_range():
    with pytest.raises(RuntimeError, match="limit_us"):
        cpmk.call("cpmk_selftest_bounded_wait", 0, None)
    with pytest.raises(RuntimeError, match="limit_us"):
        cpmk.call("cpmk_selftest_bounded_wait", 10_000_000, None)


def test_one_workspace_per_stream_released_on_request():
    """More streams than the old process-wide cap of 64 each get a workspace; releasing gives the slot back."""
    import cpm_kernels_b200.kernels as ck
    a = randn_fp16((1, 64, 128), 14).cuda()
    want = None
    streams = [torch.cuda.Stream() for _ in range(70)]
    for st in streams:
        sc = torch.empty((1, 128), dtype=torch.half, device="cuda")
        q = torch.empty((1, 64, 128), dtype=torch.int8, device="cuda")
        with torch.cuda.stream(st):
            ck.gemm_quantize_cols(1, 64, 128, a.data_ptr(), sc.data_ptr(), q.data_ptr(), st.cuda_stream)
        st.synchronize()
        if want is None:
            want = (sc.clone(), q.clone())
        assert torch.equal(sc, want[0]) and torch.equal(q, want[1])
    for st in streams:
        cpmk.release_workspace(st.cuda_stream)
    cpmk.release_workspace(streams[0].cuda_stream)       # releasing twice is harmless
    assert cpmk.read_status() == 0


def test_tensor_map_cache_holds_a_model_worth_of_buffers():
    """240 distinct weight buffers in turn (more than the 32 encodings the cache once held), twice over: every product
    exact both times."""
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randint(-127, 128, (1, 256, 256), generator=g, device="cuda", dtype=torch.int8)
    ws = [torch.randint(-127, 128, (1, 256, 256), generator=g, device="cuda", dtype=torch.int8) for _ in range(240)]
    import gpu_util as G
    for _ in range(2):
        for i in (0, 1, 100, 239):
            out = G.gemm_int8(256, 256, 256, True, False, ws[i], x)
            want = torch.matmul(x[0].double(), ws[i][0].double().t()).to(torch.int32)
            assert torch.equal(out[0], want)
        for w in ws:
            G.gemm_int8(256, 256, 256, True, False, w, x)
    G.assert_no_device_error()
