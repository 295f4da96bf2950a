"""GPU parity of the fp16 decode GEMVs against the exact (float64) oracle, within rtol 1e-3 / atol 1e-2
(the reference pins its cublasLt GEMV to 1e-3 and its own kernels to 5e-2: tests/test_gemv.py:81,103)."""
import numpy as np
import pytest
import torch

import cpm_kernels_b200.kernels as ck
from oracle import quant_linear as ql
from util import randn_fp16, np16

pytestmark = pytest.mark.gpu
RTOL, ATOL = 1e-3, 1e-2


@pytest.fixture(scope="module")
def G():
    import gpu_util
    return gpu_util


def close(got_fp16, want_f64):
    got = got_fp16.astype(np.float64)
    want16 = want_f64.astype(np.float16).astype(np.float64)      # the exact sum, rounded once to fp16
    return np.isclose(got, want16, rtol=RTOL, atol=ATOL).all()


ROWS = [(16, 2222, 128), (1, 10240, 4096), (4, 1024, 4096), (3, 37, 24), (2, 9, 4100), (1, 5, 30), (2, 8, 7),
        (3, 1000, 1032), (2, 2371, 6400),
        (1, 2371, 1032), (1, 5000, 2056), (1, 2400, 4088), (1, 3000, 3072),   # one matrix, rows <= 4096: the vector lives in registers
        (4, 10240, 4096), (16, 10240, 4096)]                       # configuration 3 with per-batch matrices at full size                          # streaming kernel: ragged row groups, longest rows it takes


@pytest.mark.parametrize("batch,dim_out,dim_in", ROWS)
def test_gemv_fp16(G, batch, dim_out, dim_in):
    ssk = float(dim_in) ** 0.25
    mat = randn_fp16((batch, dim_out, dim_in), 1, 1.0 / ssk)
    vec = randn_fp16((batch, dim_in), 2, 1.0 / ssk)
    out = torch.full((batch, dim_out), 9.0, dtype=torch.half, device="cuda")
    md, vd = mat.cuda(), vec.cuda()
    ck.gemv_fp16(batch, dim_out, dim_in, md.data_ptr(), vd.data_ptr(), out.data_ptr(), G.stream())
    want = ql.gemv_fp16(np16(mat), np16(vec))
    assert close(G.host(out), want)
    if dim_in % 2 == 0:
        out2 = torch.empty_like(out)
        ck.gemv_fp16_light(batch, dim_out, dim_in, md.data_ptr(), vd.data_ptr(), out2.data_ptr(), G.stream())
        assert torch.equal(out, out2)


COLS = [(16, 128, 2222), (1, 10240, 4096), (1, 4096, 10240), (4, 1024, 4096), (3, 40, 24), (2, 12, 9), (2, 264, 100),
        (4, 4096, 2048), (8, 2056, 1000), (16, 10240, 1024),
        (4, 10240, 4096), (16, 10240, 4096), (4, 4096, 10240),
        (2, 4096, 8192), (1, 3000, 5000),                         # many row ranges per strip (batches; ragged strip, empty ranges)
        (1, 10008, 3000), (1, 9472, 1024), (1, 18944, 1100), (1, 9480, 16384)]   # one matrix, whole columns per block: ragged last strip and last box, fewer boxes than ring slots, the widest strip, the longest vector


@pytest.mark.parametrize("batch,dim_out,dim_in", COLS)
def test_gemv_fp16_transpose(G, batch, dim_out, dim_in):
    ssk = float(dim_in) ** 0.25
    mat = randn_fp16((batch, dim_in, dim_out), 3, 1.0 / ssk)
    vec = randn_fp16((batch, dim_in), 4, 1.0 / ssk)
    want = ql.gemv_fp16_transpose(np16(mat), np16(vec))
    md, vd = mat.cuda(), vec.cuda()
    outs = []
    for _ in range(3):                              # repeated calls: tickets and scratch are left clean
        out = torch.full((batch, dim_out), 9.0, dtype=torch.half, device="cuda")
        ck.gemv_fp16_transpose(batch, dim_out, dim_in, md.data_ptr(), vd.data_ptr(), out.data_ptr(), G.stream())
        outs.append(out)
    assert close(G.host(outs[0]), want)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])      # deterministic
    G.assert_no_device_error()


@pytest.mark.parametrize("batch,dim_out,dim_in", [(16, 22222, 4444), (1, 10240, 4096), (4, 10240, 4096), (16, 10240, 4096), (5, 33, 64), (3, 7, 10),
                                                  (1, 2999, 2056)])
def test_gemv_broadcast_mat_fp16(G, batch, dim_out, dim_in):
    ssk = float(dim_in) ** 0.25
    mat = randn_fp16((dim_out, dim_in), 5, 1.0 / ssk)
    vec = randn_fp16((batch, dim_in), 6, 1.0 / ssk)
    out = torch.full((batch, dim_out), 9.0, dtype=torch.half, device="cuda")
    md, vd = mat.cuda(), vec.cuda()
    ck.gemv_broadcast_mat_fp16(batch, dim_out, dim_in, md.data_ptr(), vd.data_ptr(), out.data_ptr(), G.stream())
    assert close(G.host(out), ql.gemv_broadcast_mat_fp16(np16(mat), np16(vec)))


def test_int8_gemv_chain(G):
    """tests/test_gemv.py:8-59: quantise matrix rows and vectors, int8 dot products, dequantise -- bit-exact here."""
    batch, n, m = 16, 4444, 8888
    mat = randn_fp16((n, m), 7)
    vec = randn_fp16((batch, m), 8)
    md, vd = mat.cuda(), vec.cuda()
    ms = torch.empty(n, dtype=torch.half, device="cuda")
    mq = torch.empty((n, m), dtype=torch.int8, device="cuda")
    ck.gemm_calc_scale(1, n, m, md.data_ptr(), ms.data_ptr(), G.stream())
    ck.gemm_round(1, n, m, md.data_ptr(), ms.data_ptr(), mq.data_ptr(), G.stream())
    vs = torch.empty(batch, dtype=torch.half, device="cuda")
    vq = torch.empty((batch, m), dtype=torch.int8, device="cuda")
    ck.gemv_calc_scale(batch, m, vd.data_ptr(), vs.data_ptr(), G.stream())
    ck.gemv_round(batch, m, vd.data_ptr(), vs.data_ptr(), vq.data_ptr(), G.stream())
    out = torch.empty((batch, n), dtype=torch.half, device="cuda")
    ck.gemv_broadcast_mat_int8(batch, n, m, ms.data_ptr(), mq.data_ptr(), vs.data_ptr(), vq.data_ptr(), out.data_ptr(), G.stream())
    wms = ql.gemm_calc_scale(np16(mat)[None])[0]
    wmq = ql.gemm_round(np16(mat)[None], wms[None])[0]
    wvs = ql.gemm_calc_scale(np16(vec)[None])[0]
    wvq = ql.gemm_round(np16(vec)[None], wvs[None])[0]
    assert G.same_bits(ms, wms) and (G.host(mq) == wmq).all() and G.same_bits(vs, wvs) and (G.host(vq) == wvq).all()
    assert G.same_bits(out, ql.gemv_broadcast_mat_int8(wms, wmq, wvs, wvq))
