"""GPU parity of the quantisation passes (scale, round, fused forms, dequant) against the CPU oracle,
bit for bit, through the C ABI; and against the reference's own device code where its fatbins are present."""
import numpy as np
import pytest
import torch

from oracle import quant_linear as ql
from oracle import ref_cuda
from util import randn_fp16, np16, edge_case_matrix

pytestmark = pytest.mark.gpu

ROW_SHAPES = [
    (1, 4, 4), (2, 4, 8), (3, 12, 12),            # the reference's smallest cases (tests/test_gemm.py:43-47): generic path
    (1, 7, 500), (2, 5, 7996),                   # m % 8 != 0
    (1, 33, 64), (4, 100, 128), (2, 40, 512), (1, 130, 1024),
    (1, 512, 2560),                               # configuration 1 activations
    (1, 96, 4096), (1, 24, 10240), (1, 5, 12288), (1, 3, 16384),
    (1, 2, 20000),                                # longer than the register-resident limit
    (1, 70000, 8),                                # more rows than the reference's grid.y allows
    (8, 512, 128),                                # attention-score operands (batch x heads folded)
]


@pytest.fixture(scope="module")
def G():
    import gpu_util
    return gpu_util


@pytest.mark.parametrize("shape", ROW_SHAPES)
def test_row_quantisation_matches_oracle(G, shape):
    std = 0.02 if shape[2] in (2560, 4096) else 1.0
    x = randn_fp16(shape, seed=shape[1] * 31 + shape[2], std=std)
    xh = np16(x)
    want_s = ql.gemm_calc_scale(xh)
    want_q = ql.gemm_round(xh, want_s)
    xd = x.cuda()
    s = G.calc_scale(xd)
    assert G.same_bits(s, want_s)
    assert (G.host(G.round_i8(xd, s)) == want_q).all()
    s2, q2 = G.quantize(xd)
    assert G.same_bits(s2, want_s)
    assert (G.host(q2) == want_q).all()
    G.assert_no_device_error()


COL_SHAPES = [
    (1, 4, 4), (3, 12, 12), (2, 33, 40),           # generic path
    (1, 7, 8), (2, 31, 64), (1, 32, 72), (1, 1000, 200),
    (1, 1024, 1536), (8, 512, 256), (1, 4096, 512), (2, 65, 4096),
    (1, 16000, 2056), (3, 7000, 1600), (2, 16411, 1024),  # streaming kernels: ragged strips, ragged row ranges, batches
]


@pytest.mark.parametrize("shape", COL_SHAPES)
def test_column_quantisation_matches_oracle(G, shape):
    x = randn_fp16(shape, seed=shape[1] * 17 + shape[2], std=1.0)
    xh = np16(x)
    want_s = ql.gemm_calc_scale_transpose(xh)
    want_q = ql.gemm_round_transpose(xh, want_s)
    xd = x.cuda()
    s = G.calc_scale(xd, transpose=True)
    assert G.same_bits(s, want_s)
    assert (G.host(G.round_i8(xd, s, transpose=True)) == want_q).all()
    s2, q2 = G.quantize(xd, transpose=True)
    assert G.same_bits(s2, want_s)
    assert (G.host(q2) == want_q).all()
    # twice in a row on the same stream: the scratch the fused form uses carries nothing over
    s3, q3 = G.quantize(xd, transpose=True)
    assert G.same_bits(s3, want_s) and (G.host(q3) == want_q).all()
    G.assert_no_device_error()


# the resident-strip kernel (operand read once; clusters of 1 to 8 CTAs hold a 64-column strip in shared memory)
RESIDENT_SHAPES = [
    (1, 4096, 10240),      # cluster of 8, 512 rows per CTA: the operand of the benchmark
    (1, 6144, 1024),       # the tallest it takes: 8 x 768 rows
    (1, 6145, 1024),       # one row too many: the two-pass kernels
    (1, 10240, 4096),      # taller still: the two-pass streaming kernels
    (2, 700, 2056),        # one CTA per strip; m % 64 = 8: a ragged last strip; rows not a multiple of the 128-row boxes
    (1, 1500, 1416),       # cluster of 2, ragged rows and columns
    (1, 3001, 1000),       # cluster of 4; the last CTA holds 697 of its 768 rows
    (8, 4096, 512),        # batched: (batch, hidden, seq) activations
]


@pytest.mark.parametrize("shape", RESIDENT_SHAPES)
def test_column_quantisation_resident_strips(G, shape):
    x = randn_fp16(shape, seed=shape[1] * 13 + shape[2], std=1.0)
    xh = np16(x)
    want_s = ql.gemm_calc_scale_transpose(xh)
    want_q = ql.gemm_round_transpose(xh, want_s)
    xd = x.cuda()
    for _ in range(2):
        s, q = G.quantize(xd, transpose=True)
        assert G.same_bits(s, want_s)
        assert (G.host(q) == want_q).all()
    G.assert_no_device_error()


def test_column_quantisation_resident_strips_edge_columns(G):
    """Columns that leave the division-free rule's domain, inside an operand large enough for the resident-strip
    kernel: all zero (scale 0: 0/0), subnormal scale, NaN, +-inf, the largest finite value, exact .5 ties."""
    x = randn_fp16((1, 2048, 1024), 77).numpy().copy()
    x[0, :, 0] = 0
    x[0, :, 1] = np.float16(6e-8) * (np.arange(2048) % 5)
    x[0, :, 2] = np.float16(2e-5) * ((np.arange(2048) % 7) - 3)
    x[0, 100, 3] = np.float16(np.nan)
    x[0, 200, 4] = np.float16(np.inf)
    x[0, 300, 4] = -np.float16(np.inf)
    x[0, 5, 5] = np.float16(65504.0)
    x[0, :, 6] = 0
    x[0, 0, 6] = np.float16(127.0)                                   # scale exactly 1: k + 0.5 are exact ties
    x[0, 1:200, 6] = (np.arange(199) % 100 - 50).astype(np.float16) + np.float16(0.5)
    x[0, :, 7] = np.float16(-0.0)
    x[0, :, 1023] = x[0, :, 6]
    want_s = ql.gemm_calc_scale_transpose(x)
    want_q = ql.gemm_round_transpose(x, want_s)
    s, q = G.quantize(torch.from_numpy(x).cuda(), transpose=True)
    assert G.same_bits(s, want_s)
    assert (G.host(q) == want_q).all()
    if ref_cuda.available():
        ref = ref_cuda.ReferenceKernels()
        xd = torch.from_numpy(x).cuda()
        rs = ref.gemm_calc_scale_transpose(xd)
        assert G.same_bits(s, rs)
        assert (G.host(q) == G.host(ref.gemm_round_transpose(xd, rs))).all()
    G.assert_no_device_error()


def test_round_with_foreign_scales(G):
    """gemm_round / gemm_round_transpose take any scale, not only the absmax one: values far outside
    [-127, 127], zero, subnormal, inf and NaN scales must give what the reference expression gives."""
    x = randn_fp16((1, 16, 64), 21)
    xh = np16(x)
    rows = np.array([[1.0, 0.001, 100.0, 0.0, 6e-8, 2e-5, np.inf, np.nan, 0.5, 0.25, 3e-3, 65504.0, 1e-4, 7e-5, 0.0313, 2.0]],
                    dtype=np.float16)
    q = G.host(G.round_i8(x.cuda(), G.dev(rows)))
    assert (q == ql.gemm_round(xh, rows)).all()
    cols = np.tile(rows[:, :16], (1, 4))
    q = G.host(G.round_i8(x.cuda(), G.dev(cols), transpose=True))
    assert (q == ql.gemm_round_transpose(xh, cols)).all()


def test_edge_cases_match_oracle_and_reference_device_code(G):
    x = edge_case_matrix()
    xh = np16(x)
    xd = x.cuda()
    s, q = G.quantize(xd)
    sc, qc = G.quantize(xd, transpose=True)
    assert G.same_bits(s, ql.gemm_calc_scale(xh))
    assert (G.host(q) == ql.gemm_round(xh, ql.gemm_calc_scale(xh))).all()
    assert G.same_bits(sc, ql.gemm_calc_scale_transpose(xh))
    assert (G.host(qc) == ql.gemm_round_transpose(xh, ql.gemm_calc_scale_transpose(xh))).all()
    if ref_cuda.available():
        ref = ref_cuda.ReferenceKernels()
        rs = ref.gemm_calc_scale(xd)
        assert G.same_bits(s, rs)
        assert (G.host(q) == G.host(ref.gemm_round(xd, rs))).all()
        rsc = ref.gemm_calc_scale_transpose(xd)
        assert G.same_bits(sc, rsc)
        assert (G.host(qc) == G.host(ref.gemm_round_transpose(xd, rsc))).all()


@pytest.mark.skipif(not ref_cuda.available(), reason="oracle/_ref fatbins not built")
@pytest.mark.parametrize("shape,std", [((1, 4096, 4096), 1.0), ((1, 10240, 2560), 0.02), ((8, 512, 4096), 1.0), ((1, 4096, 12288), 0.02)])
def test_full_size_operands_match_reference_device_code(G, shape, std):
    """Configuration-2 sized operands: codes and scales byte-identical to the reference's kernels run on the same GPU."""
    g = torch.Generator(device="cuda").manual_seed(5)
    x = (torch.randn(shape, generator=g, device="cuda") * std).half()
    ref = ref_cuda.ReferenceKernels()
    rs = ref.gemm_calc_scale(x)
    rq = ref.gemm_round(x, rs)
    s, q = G.quantize(x)
    assert torch.equal(s.view(torch.int16), rs.view(torch.int16))
    assert torch.equal(q, rq)
    rsc = ref.gemm_calc_scale_transpose(x)
    rqc = ref.gemm_round_transpose(x, rsc)
    sc, qc = G.quantize(x, transpose=True)
    assert torch.equal(sc.view(torch.int16), rsc.view(torch.int16))
    assert torch.equal(qc, rqc)
    # size-independent property: no code exceeds 127 in magnitude and every row / column reaches it
    assert int(q.abs().max()) == 127 and int(q.to(torch.int16).abs().amax(dim=2).min()) == 127
    assert int(qc.to(torch.int16).abs().amax(dim=1).min()) == 127
    G.assert_no_device_error()


@pytest.mark.parametrize("shape", [(1, 4, 4), (2, 24, 40), (3, 12, 12), (1, 100, 500), (2, 64, 4096), (1, 512, 10240)])
@pytest.mark.parametrize("bx,by", [(False, False), (True, False), (False, True), (True, True)])
def test_dequant_matches_oracle(G, shape, bx, by):
    b, n, m = shape
    g = torch.Generator(device="cpu").manual_seed(n * m)
    acc = torch.randint(-30_000_000, 30_000_000, shape, generator=g, dtype=torch.int32)
    sx = randn_fp16((1 if bx else b, n), 1, 0.01).abs()
    sy = randn_fp16((1 if by else b, m), 2, 0.001).abs()
    want = ql.gemm_scale(acc.numpy(), np16(sx), np16(sy), bx, by)
    got = G.gemm_scale(acc.cuda(), sx.cuda(), sy.cuda(), bx, by)
    assert G.same_bits(got, want)


def test_dequant_single_scale_forms(G):
    import cpm_kernels_b200.kernels as ck
    g = torch.Generator(device="cpu").manual_seed(3)
    acc = torch.randint(-3_000_000, 3_000_000, (2, 20, 48), generator=g, dtype=torch.int32)
    sx = randn_fp16((2, 20), 4, 0.01).abs()
    sy = randn_fp16((2, 48), 5, 0.01).abs()
    accd, out = acc.cuda(), torch.empty((2, 20, 48), dtype=torch.half, device="cuda")
    sxd, syd = sx.cuda(), sy.cuda()
    ck.gemm_scale_x(2, 20, 48, accd.data_ptr(), sxd.data_ptr(), out.data_ptr(), G.stream())
    assert G.same_bits(out, ql.gemm_scale_x(acc.numpy(), np16(sx)))
    ck.gemm_scale_y(2, 20, 48, accd.data_ptr(), syd.data_ptr(), out.data_ptr(), G.stream())
    assert G.same_bits(out, ql.gemm_scale_y(acc.numpy(), np16(sy)))


def test_backward_helpers_match_oracle(G):
    import cpm_kernels_b200.kernels as ck
    gr = randn_fp16((2, 20, 32), 107, 0.5)
    sy = randn_fp16((2, 32), 108, 0.01).abs() + 1e-3
    sx = randn_fp16((1, 20), 109, 0.01).abs() + 1e-3
    q = torch.empty((2, 20, 32), dtype=torch.int8, device="cuda")
    s = torch.empty((2, 20), dtype=torch.half, device="cuda")
    grd, syd, sxd = gr.cuda(), sy.cuda(), sx.cuda()
    ck.gemm_backward_round_scale(2, 20, 32, grd.data_ptr(), syd.data_ptr(), q.data_ptr(), s.data_ptr(), False, G.stream())
    wq, ws = ql.gemm_backward_round_scale(np16(gr), np16(sy), False)
    assert (G.host(q) == wq).all() and G.same_bits(s, ws)
    s2 = torch.empty((2, 32), dtype=torch.half, device="cuda")
    ck.gemm_backward_scale_round(2, 20, 32, grd.data_ptr(), sxd.data_ptr(), q.data_ptr(), s2.data_ptr(), True, G.stream())
    wq, ws = ql.gemm_backward_scale_round(np16(gr), np16(sx), True)
    assert (G.host(q) == wq).all() and G.same_bits(s2, ws)


def test_empty_inputs(G):
    import cpm_kernels_b200.kernels as ck
    ck.gemm_calc_scale(0, 4, 8, 0, 0, G.stream())
    ck.gemm_round(1, 0, 8, 0, 0, 0, G.stream())
    ck.gemm_quantize_cols(0, 4, 8, 0, 0, 0, G.stream())
    ck.gemm_scale(1, 0, 8, 0, 0, 0, 0, False, False, G.stream())
    torch.cuda.synchronize()


def test_non_default_stream_and_second_device_state(G):
    x = randn_fp16((1, 256, 512), 33)
    xh = np16(x)
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        xd = x.cuda()
        s, q = G.quantize(xd, transpose=True)
    st.synchronize()
    want_s = ql.gemm_calc_scale_transpose(xh)
    assert G.same_bits(s, want_s) and (G.host(q) == ql.gemm_round_transpose(xh, want_s)).all()


@pytest.mark.parametrize("rows0,rows1,m", [((1, 64), (1, 96), 4096), ((2, 33), (1, 7), 512), ((1, 5), (3, 4), 20), ((1, 4096), (1, 1000), 10240),
                                           ((1, 16), (1, 8), 128), ((1, 0), (1, 8), 64)])
def test_two_operands_in_one_launch(G, rows0, rows1, m):
    """cpmk_quantize_rows_pair gives what two cpmk_quantize_rows calls give (and so the oracle's bits)."""
    import cpm_kernels_b200.kernels as ck
    x0 = randn_fp16((rows0[0], rows0[1], m), 1, 1.0)
    x1 = randn_fp16((rows1[0], rows1[1], m), 2, 0.02)
    outs = []
    for x in (x0, x1):
        xd = x.cuda()
        outs.append((xd, torch.full(x.shape[:2], 9.0, dtype=torch.half, device="cuda"), torch.full(x.shape, 9, dtype=torch.int8, device="cuda")))
    (a, sa, qa), (b, sb, qb) = outs
    ck.gemm_quantize_rows_pair(rows0[0], rows0[1], a.data_ptr(), sa.data_ptr(), qa.data_ptr(),
                               rows1[0], rows1[1], b.data_ptr(), sb.data_ptr(), qb.data_ptr(), m, G.stream())
    for x, s, q in ((x0, sa, qa), (x1, sb, qb)):
        if x.numel() == 0:
            continue
        want_s = ql.gemm_calc_scale(np16(x))
        assert G.same_bits(s, want_s)
        assert (G.host(q) == ql.gemm_round(np16(x), want_s)).all()
    G.assert_no_device_error()
