"""The multi-destination forms on one GPU (every destination is local memory): the row quantiser that writes its scales
and codes to several destinations, and the one-call column-parallel linear, against the oracle bit for bit.  The same
entry points run across GPUs in tests/test_gpu_multi.py."""
import numpy as np
import pytest
import torch

import cpm_kernels_b200.kernels as ck
from cpm_kernels_b200.library import cpmk
from cpm_kernels_b200.sharded import FusedColumnParallelInt8Linear
from oracle import quant_linear as ql
from util import randn_fp16, np16

pytestmark = pytest.mark.gpu


def _s():
    return torch.cuda.current_stream().cuda_stream


@pytest.mark.parametrize("rows,m,n_dst,n1", [(512, 4096, 3, 256), (100, 264, 2, 0), (37, 10240, 8, 19), (64, 64, 1, 64), (1000, 1032, 4, 3)])
def test_quantize_rows_pair_scatter(rows, m, n_dst, n1):
    """Operand 0: rows [lo, lo+rows) of a larger activation; every destination holds the full (total, m) code buffer and the
    rows land at their offset.  Operand 1 (the weight rows) is quantised by the same launch."""
    total, lo = rows * 2 + 5, rows + 3                    # m % 8 == 0, so the code destination lo * m is 8-byte aligned
    x = randn_fp16((1, rows, m), 21)
    w = randn_fp16((1, max(n1, 1), m), 22, 0.02)
    xd, wd = x.cuda(), w.cuda()
    codes = [torch.full((total, m), 99, dtype=torch.int8, device="cuda") for _ in range(n_dst)]
    scales = [torch.full((total,), 7.0, dtype=torch.half, device="cuda") for _ in range(n_dst)]
    sw = torch.full((1, max(n1, 1)), 7.0, dtype=torch.half, device="cuda")
    qw = torch.full((1, max(n1, 1), m), 99, dtype=torch.int8, device="cuda")
    ck.gemm_quantize_rows_pair_scatter(rows, xd.data_ptr(), [t.data_ptr() + 2 * lo for t in scales], [t.data_ptr() + lo * m for t in codes],
                                       n1, wd.data_ptr(), sw.data_ptr(), qw.data_ptr(), m, _s())
    want_s = ql.gemm_calc_scale(np16(x))
    want_q = ql.gemm_round(np16(x), want_s)
    for c, s in zip(codes, scales):
        assert (c[lo:lo + rows].cpu().numpy() == want_q[0]).all()
        assert (s[lo:lo + rows].cpu().numpy().view(np.uint16) == want_s[0].view(np.uint16)).all()
        assert (c[:lo] == 99).all() and (c[lo + rows:] == 99).all()            # nothing outside the rows is touched
        assert (s[:lo] == 7.0).all() and (s[lo + rows:] == 7.0).all()
    if n1:
        ws = ql.gemm_calc_scale(np16(w))
        assert (sw.cpu().numpy().view(np.uint16) == ws.view(np.uint16)).all()
        assert (qw.cpu().numpy() == ql.gemm_round(np16(w), ws)).all()
    else:
        assert (qw == 99).all()
    torch.cuda.synchronize()
    assert cpmk.read_status() == 0


def test_scatter_quantiser_refuses_what_it_cannot_do():
    a = torch.zeros(64, dtype=torch.half, device="cuda")
    with pytest.raises(RuntimeError, match="multiple of 8"):
        ck.gemm_quantize_rows_pair_scatter(2, a.data_ptr(), [a.data_ptr()], [a.data_ptr()], 0, 0, 0, 0, 12, None)
    with pytest.raises(AssertionError):
        ck.gemm_quantize_rows_pair_scatter(2, a.data_ptr(), [a.data_ptr()] * 9, [a.data_ptr()] * 9, 0, 0, 0, 0, 16, None)


@pytest.mark.parametrize("tokens,k,n", [(512, 512, 1024), (1000, 1024, 768), (300, 2560, 520)])
def test_one_call_linear_single_rank(tokens, k, n):
    """The layer object on one GPU (one rank: plain device memory, no barrier): both forms of its forward pass."""
    x = randn_fp16((1, tokens, k), 23)
    w = randn_fp16((1, n, k), 24, 0.02)
    want = ql.bmm_int8(np16(x), False, np16(w), True)
    layer = FusedColumnParallelInt8Linear(w.cuda())
    for slot in (0, 1, 0):
        y = layer.forward(x.cuda(), slot=slot)
        torch.cuda.synchronize()
        assert (y.cpu().numpy().view(np.uint16) == want["out"].view(np.uint16)).all()
    buf = layer._buffers_for(tokens)
    assert (buf.qx[0].cpu().numpy() == want["quant_A"]).all() and (layer.q_w.cpu().numpy() == want["quant_B"]).all()
    y = layer.forward_sharded(x.cuda(), slot=1)             # one rank: its row shard is the whole tensor
    torch.cuda.synchronize()
    assert (y.cpu().numpy().view(np.uint16) == want["out"].view(np.uint16)).all()
    assert cpmk.read_status() == 0


def test_linear_scatter_to_two_local_destinations():
    """n_dst = 2 with both destinations in local memory, pitched: what two ranks' buffers would receive."""
    tokens, k, n_local, n_total = 512, 1024, 512, 1280
    x = randn_fp16((1, tokens, k), 25)
    w = randn_fp16((1, n_local, k), 26, 0.02)
    xd, wd = x.cuda(), w.cuda()
    ys = [torch.full((tokens, n_total), 5.0, dtype=torch.half, device="cuda") for _ in range(2)]
    sx = torch.empty((tokens,), dtype=torch.half, device="cuda")
    qx = torch.empty((tokens, k), dtype=torch.int8, device="cuda")
    sw = torch.empty((n_local,), dtype=torch.half, device="cuda")
    qw = torch.empty((n_local, k), dtype=torch.int8, device="cuda")
    col0 = 256
    ck.linear_int8_scatter(tokens, k, n_local, xd.data_ptr(), wd.data_ptr(), sx.data_ptr(), qx.data_ptr(), sw.data_ptr(), qw.data_ptr(),
                           [y.data_ptr() + 2 * col0 for y in ys], n_total, _s())
    torch.cuda.synchronize()
    want = ql.bmm_int8(np16(x), False, np16(w), True)["out"][0]
    for y in ys:
        got = y.cpu().numpy()
        assert (got[:, col0:col0 + n_local].view(np.uint16) == want.view(np.uint16)).all()
        assert (got[:, :col0] == 5.0).all() and (got[:, col0 + n_local:] == 5.0).all()
    assert cpmk.read_status() == 0


@pytest.mark.parametrize("tokens,k,n_local,n_dst", [(4096, 1024, 1536, 4), (1000, 512, 520, 3), (256, 4096, 256, 8), (2048, 10240, 512, 2)])
def test_forwarding_ctas_equal_direct_stores(tokens, k, n_local, n_dst):
    """With more than one destination a few CTAs of the GEMM's grid forward finished tiles from destination 0 to the
    others.  Every destination must receive exactly what the direct form (every computing CTA stores everywhere) and the
    oracle give, for many tiles per forwarding CTA, ragged edges, and fewer tiles than forwarding CTAs."""
    x = randn_fp16((1, tokens, k), 27)
    w = randn_fp16((1, n_local, k), 28, 0.02)
    xd, wd = x.cuda(), w.cuda()
    n_total = n_local * n_dst
    sx = torch.empty((tokens,), dtype=torch.half, device="cuda")
    qx = torch.empty((tokens, k), dtype=torch.int8, device="cuda")
    sw = torch.empty((n_local,), dtype=torch.half, device="cuda")
    qw = torch.empty((n_local, k), dtype=torch.int8, device="cuda")
    want = ql.bmm_int8(np16(x), False, np16(w), True)["out"][0].view(np.uint16)
    try:
        for forward_sms in (0, 16, 6):
            cpmk.set_gemm_forward_sms(forward_sms)
            for rep in range(2):                                                  # twice: the tile counters start from zero each call
                ys = [torch.full((tokens, n_total), 5.0, dtype=torch.half, device="cuda") for _ in range(n_dst)]
                ck.linear_int8_scatter(tokens, k, n_local, xd.data_ptr(), wd.data_ptr(), sx.data_ptr(), qx.data_ptr(), sw.data_ptr(), qw.data_ptr(),
                                       [y.data_ptr() + 2 * n_local * d for d, y in enumerate(ys)], n_total, _s())
                torch.cuda.synchronize()
                for d, y in enumerate(ys):
                    got = y.cpu().numpy()
                    assert (got[:, n_local * d:n_local * (d + 1)].view(np.uint16) == want).all(), (forward_sms, rep, d)
                    got[:, n_local * d:n_local * (d + 1)] = 5.0
                    assert (got == 5.0).all()                                      # nothing else is touched
            assert cpmk.read_status() == 0
    finally:
        cpmk.set_gemm_forward_sms(-1)
