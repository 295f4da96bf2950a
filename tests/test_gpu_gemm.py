"""GPU parity of the int8 GEMM (tcgen05 kernel and generic kernel) and of its fused dequantising epilogue:
int32 accumulators exact, fp16 outputs bit-identical to the oracle's gemm_scale of those accumulators."""
import numpy as np
import pytest
import torch

from oracle import quant_linear as ql
from oracle import ref_cuda
from cpm_kernels_b200.library import cpmk
from util import randn_fp16, np16

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def G():
    import gpu_util
    return gpu_util


def rand_i8(shape, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randint(-127, 128, shape, generator=g, dtype=torch.int8)


def operands(m, k, n, bA, bB, aT, bT, seed):
    A = rand_i8((bA, m, k) if aT else (bA, k, m), seed)
    B = rand_i8((bB, k, n) if bT else (bB, n, k), seed + 1)
    return A, B


# (m, k, n): sizes from the reference's test list (tests/test_gemm.py:43-60, kernel-level m = N, n = M) plus ragged ones
SMALL = [(4, 4, 4), (8, 8, 8), (12, 12, 12), (16, 16, 16), (32, 32, 32), (64, 64, 64), (128, 128, 128), (112, 224, 112),
         (36, 20, 68), (260, 48, 132)]


@pytest.mark.parametrize("m,k,n", SMALL)
@pytest.mark.parametrize("aT,bT", [(True, False), (False, False), (True, True), (False, True)])
@pytest.mark.parametrize("bA,bB", [(1, 1), (3, 3), (1, 3), (3, 1)])
def test_all_layouts_and_broadcasts(G, m, k, n, aT, bT, bA, bB):
    A, B = operands(m, k, n, bA, bB, aT, bT, seed=m + k + n + bA)
    want = ql.gemm_int8(m, k, n, aT, bT, A.numpy(), B.numpy())
    got = G.gemm_int8(m, k, n, aT, bT, A.cuda(), B.cuda())
    assert (G.host(got) == want).all()
    # the tensor-core kernels need the contiguous extent of each operand to be a multiple of 16 bytes
    expect_tc = (k % 16 == 0 if aT else m % 16 == 0) and (n % 16 == 0 if bT else k % 16 == 0)
    assert cpmk.last_gemm_path() == (1 if expect_tc else 2)
    G.assert_no_device_error()


# shapes that exercise the tensor-core kernel's pipeline: several k blocks, several tiles per CTA, ragged edges in
# every dimension, k not a multiple of the 128-byte stage, more tiles than SMs, batches
TC_SHAPES = [
    (256, 128, 128, 1, 1), (256, 1024, 128, 1, 1), (512, 4096, 256, 1, 1), (768, 640, 384, 1, 1),
    (260, 144, 132, 1, 1), (1000, 2064, 500, 1, 1), (7996, 4096, 500, 1, 1),
    (4096, 512, 2048, 1, 1), (512, 128, 512, 16, 16), (512, 128, 512, 1, 6), (384, 256, 200, 5, 1),
    (10240, 2560, 512, 1, 1),                      # configuration 1
]


@pytest.fixture
def variant(request, monkeypatch):
    """Forces one form of the tensor-core kernel (one-CTA tiles / CTA-pair tiles) for the duration of a test."""
    monkeypatch.setenv("CPMK_GEMM_VARIANT", request.param)
    return {"1cta": 1, "2cta": 2}[request.param]


@pytest.mark.parametrize("variant", ["1cta", "2cta"], indirect=True)
@pytest.mark.parametrize("m,k,n,bA,bB", TC_SHAPES)
def test_tensor_core_kernel_exact(G, variant, m, k, n, bA, bB):
    A, B = operands(m, k, n, bA, bB, True, False, seed=m + n)
    want = ql.gemm_int8(m, k, n, True, False, A.numpy(), B.numpy())
    Ad, Bd = A.cuda(), B.cuda()
    got = G.gemm_int8(m, k, n, True, False, Ad, Bd)
    assert cpmk.last_gemm_path() == 1 and cpmk.last_gemm_variant() == variant
    assert (G.host(got) == want).all()
    # extreme codes: every product +-127*127 (or 128*128), accumulators at their largest magnitude
    Ae = torch.full_like(A, -128).cuda()
    Be = torch.full_like(B, -128).cuda()
    got = G.gemm_int8(m, k, n, True, False, Ae, Be)
    assert int(got.min()) == int(got.max()) == 128 * 128 * k
    G.assert_no_device_error()


@pytest.mark.parametrize("m,k,n,bA,bB", [(256, 128, 128, 1, 1), (260, 144, 132, 2, 2), (1000, 2064, 500, 1, 1), (516, 256, 200, 3, 1),
                                         (512, 128, 512, 1, 4), (2560, 4096, 384, 1, 1), (5120, 1024, 1024, 1, 1)])
@pytest.mark.parametrize("path", ["tc", "tc2", "generic"])
def test_fused_dequant_epilogue(G, m, k, n, bA, bB, path, monkeypatch):
    monkeypatch.setenv("CPMK_GEMM_VARIANT", {"tc": "1cta", "tc2": "2cta", "generic": "generic"}[path])
    aT, bT = (True, False) if path != "generic" else (False, True)
    A, B = operands(m, k, n, bA, bB, aT, bT, seed=m * 3 + n)
    batch = max(bA, bB)
    bx, by = bB == 1, bA == 1                       # scale_x pairs with the n axis (operand B), scale_y with m (operand A)
    sx = randn_fp16((1 if bx else batch, n), 7, 0.01).abs()
    sy = randn_fp16((1 if by else batch, m), 8, 0.001).abs()
    acc = ql.gemm_int8(m, k, n, aT, bT, A.numpy(), B.numpy())
    want = ql.gemm_scale(acc, np16(sx), np16(sy), bx, by)
    got = G.gemm_int8_scale(m, k, n, aT, bT, A.cuda(), B.cuda(), sx.cuda(), sy.cuda(), bx, by)
    assert cpmk.last_gemm_path() == (2 if path == "generic" else 1)
    assert cpmk.last_gemm_variant() == {"tc": 1, "tc2": 2, "generic": 0}[path]
    assert G.same_bits(got, want)
    G.assert_no_device_error()


@pytest.mark.parametrize("m,k,n,bA,bB", [(512, 384, 256, 1, 1), (1024, 4096, 512, 1, 1), (272, 144, 400, 2, 2), (2048, 1000, 304, 1, 3),
                                         (4096, 2560, 768, 1, 1)])
@pytest.mark.parametrize("aT,bT", [(False, False), (True, True), (False, True)])
def test_tensor_core_kernel_other_storage_orders(G, m, k, n, bA, bB, aT, bT):
    """The reference's three other storage orders (an operand whose k axis is the slow one: the transposed-weight and
    (hidden, seq) activation layouts) on the tensor-core kernel, exact, plus the fused dequantising epilogue."""
    if (not aT and m % 16) or (bT and n % 16) or ((aT or not bT) and k % 16):
        pytest.skip("extent not a multiple of 16 bytes: generic kernel")
    A, B = operands(m, k, n, bA, bB, aT, bT, seed=m + 7 * n)
    want = ql.gemm_int8(m, k, n, aT, bT, A.numpy(), B.numpy())
    Ad, Bd = A.cuda(), B.cuda()
    got = G.gemm_int8(m, k, n, aT, bT, Ad, Bd)
    assert cpmk.last_gemm_path() == 1 and cpmk.last_gemm_variant() == 2
    assert (G.host(got) == want).all()
    batch = max(bA, bB)
    bx, by = bB == 1, bA == 1
    sx = randn_fp16((1 if bx else batch, n), 7, 0.01).abs()
    sy = randn_fp16((1 if by else batch, m), 8, 0.001).abs()
    fused = G.gemm_int8_scale(m, k, n, aT, bT, Ad, Bd, sx.cuda(), sy.cuda(), bx, by)
    assert G.same_bits(fused, ql.gemm_scale(want, np16(sx), np16(sy), bx, by))
    G.assert_no_device_error()


FULL = [(12288, 4096, 4096), (4096, 4096, 4096), (10240, 4096, 4096), (4096, 10240, 4096)]   # (m = N, k = K, n = M tokens)


@pytest.mark.parametrize("m,k,n", FULL)
def test_full_size_shapes_by_checksum_and_library(G, m, k, n):
    """CPM-Bee-10B linears at M = 4096 tokens.  The oracle does not finish these in seconds, so the result is held to
    (1) a checksum of checksums: sum_i out[j, i] == sum_l B[j, l] * (sum_i A[i, l]), in int64;
    (2) sampled rows recomputed in int64;  (3) the vendor library's int8 GEMM, entry by entry."""
    g = torch.Generator(device="cuda").manual_seed(m + k)
    A = torch.randint(-127, 128, (1, m, k), generator=g, device="cuda", dtype=torch.int8)
    B = torch.randint(-127, 128, (1, n, k), generator=g, device="cuda", dtype=torch.int8)
    out = G.gemm_int8(m, k, n, True, False, A, B)
    assert cpmk.last_gemm_path() == 1 and cpmk.last_gemm_variant() == 2
    colsum_A = A[0].to(torch.int64).sum(dim=0)                                      # (k,)
    want_rowsum = (B[0].to(torch.float64) @ colsum_A.to(torch.float64)).to(torch.int64)   # exact: < 2**53
    assert torch.equal(out[0].to(torch.int64).sum(dim=1), want_rowsum)
    rows = torch.tensor([0, 1, 127, 128, n // 2 + 3, n - 1], device="cuda")
    want_rows = (B[0][rows].to(torch.float64) @ A[0].to(torch.float64).T).to(torch.int64)
    assert torch.equal(out[0][rows].to(torch.int64), want_rows)
    lib = torch._int_mm(B[0], A[0].T)                                               # cublasLt, (n, m) int32
    assert torch.equal(out[0], lib)
    G.assert_no_device_error()


@pytest.mark.skipif(not ref_cuda.available(), reason="oracle/_ref fatbins not built")
def test_against_reference_cublaslt_call_sequence(G):
    """The reference's own GEMM path (its cublasLt call sequence) on the same GPU, for the layouts the library accepts."""
    m, k, n = 512, 256, 384
    try:
        lt = ref_cuda.ReferenceCublasLt()
    except RuntimeError as e:
        pytest.skip(str(e))
    for aT, bT in [(True, False), (False, False), (True, True), (False, True)]:
        A, B = operands(m, k, n, 2, 1, aT, bT, seed=11)
        Ad, Bd = A.cuda(), B.cuda()
        mine = G.gemm_int8(m, k, n, aT, bT, Ad, Bd)
        theirs = torch.empty_like(mine)
        try:
            lt.gemm_int8(m, k, n, 2, 1, aT, bT, Ad, Bd, theirs)
        except RuntimeError:
            continue                                   # cublasLt rejects this plain-layout combination on this device
        torch.cuda.synchronize()
        assert torch.equal(mine, theirs), (aT, bT)


def test_argument_errors(G):
    import cpm_kernels_b200.kernels as ck
    with pytest.raises(AssertionError):
        ck.gemm_int8(6, 8, 8, 1, 1, True, False, 0, 0, 0, G.stream())
    A = torch.zeros(64, dtype=torch.int8, device="cuda")
    with pytest.raises(RuntimeError, match="status 1"):
        cpmk.call("cpmk_gemm_int8", 8, 8, 8, 2, 3, 1, 0, A.data_ptr(), A.data_ptr(), A.data_ptr(), None)
    with pytest.raises(RuntimeError, match="null"):
        cpmk.call("cpmk_gemm_int8", 8, 8, 8, 1, 1, 1, 0, None, A.data_ptr(), A.data_ptr(), None)
    # k == 0: the sum is empty, the output is zero
    out = torch.full((1, 4, 4), 5, dtype=torch.int32, device="cuda")
    ck.gemm_int8(4, 0, 4, 1, 1, True, False, A.data_ptr(), A.data_ptr(), out.data_ptr(), G.stream())
    assert int(out.abs().max()) == 0


@pytest.mark.parametrize("m,k,n,batch", [(512, 256, 384, 1), (1536, 1024, 1000, 1), (256, 128, 300, 3)])
def test_scattered_output_to_pitched_destinations(G, m, k, n, batch):
    """cpmk_gemm_int8_dequant_scatter on one GPU: two destinations, each a column slice of a wider buffer (the layout a
    column-parallel rank writes into every rank's full-width output).  Slices equal the plain call; nothing else is touched."""
    import cpm_kernels_b200.kernels as ck
    A, B = operands(m, k, n, batch, batch, True, False, seed=m + n)
    sx = randn_fp16((batch, n), 7, 0.01).abs()
    sy = randn_fp16((batch, m), 8, 0.001).abs()
    Ad, Bd, sxd, syd = A.cuda(), B.cuda(), sx.cuda(), sy.cuda()
    plain = G.gemm_int8_scale(m, k, n, True, False, Ad, Bd, sxd, syd, False, False)
    pitch = 3 * m
    bufs = [torch.full((batch, n, pitch), -7.0, dtype=torch.half, device="cuda") for _ in range(2)]
    offs = [0, 2 * m]
    dst = [b.data_ptr() + 2 * o for b, o in zip(bufs, offs)]
    ck.gemm_int8_scale_scatter(m, k, n, batch, batch, True, False, Ad.data_ptr(), Bd.data_ptr(), sxd.data_ptr(), syd.data_ptr(), False, False,
                               dst, pitch, G.stream())
    torch.cuda.synchronize()
    for b, o in zip(bufs, offs):
        assert torch.equal(b[:, :, o:o + m].view(torch.int16), plain.view(torch.int16))
        rest = torch.cat([b[:, :, :o], b[:, :, o + m:]], dim=2)
        assert bool((rest == -7.0).all())
    G.assert_no_device_error()
    with pytest.raises(RuntimeError, match="pitch"):
        ck.gemm_int8_scale_scatter(m, k, n, batch, batch, True, False, Ad.data_ptr(), Bd.data_ptr(), sxd.data_ptr(), syd.data_ptr(), False, False,
                                   dst, m - 8, G.stream())
