"""The loadable kernel modules (lib/gemm.fatbin, lib/gemv.fatbin) run through the reference's own loading and
launch convention: cuModuleLoadData, cuModuleGetFunction by the reference's symbol names, cuLaunchKernel with the
grids, blocks and ctypes parameters its Python launchers compute (oracle/ref_cuda.py mirrors them, citing each).
Results are held to the CPU oracle bit for bit, and to the reference's own device code where it was built."""
import ctypes
import os

import numpy as np
import pytest
import torch

from cpm_kernels_b200 import build
from oracle import quant_linear as ql
from oracle import ref_cuda
from util import randn_fp16, np16, bits, edge_case_matrix

pytestmark = pytest.mark.gpu
RTOL, ATOL = 1e-3, 1e-2


@pytest.fixture(scope="module")
def mod():
    assert os.path.exists(build.module_path("gemm")) and os.path.exists(build.module_path("gemv")), "kernel modules not built"
    return ref_cuda.ReferenceKernels(fatbin_dir=build.LIB_DIR)


@pytest.fixture(scope="module")
def ref():
    if not ref_cuda.available():
        pytest.skip("the reference's device code was not built (oracle/_ref)")
    return ref_cuda.ReferenceKernels()


def host(t):
    torch.cuda.synchronize()
    return t.cpu().numpy()


# m = 20 and 4 give blocks that are not a multiple of 32 threads; 7996 is not a multiple of 8 (scalar path);
# 4100 > 1024 threads' worth of 2-byte elements
SHAPES = [(1, 4, 4), (3, 12, 12), (2, 5, 20), (1, 7, 500), (2, 5, 7996), (1, 33, 64), (4, 100, 128), (1, 130, 1024),
          (1, 512, 2560), (1, 96, 4096), (1, 24, 10240), (2, 9, 4100), (8, 64, 128)]


@pytest.mark.parametrize("shape", SHAPES)
def test_row_kernels(mod, shape):
    x = randn_fp16(shape, seed=shape[1] * 31 + shape[2], std=0.02 if shape[2] in (2560, 4096) else 1.0)
    xh, xd = np16(x), x.cuda()
    want_s = ql.gemm_calc_scale(xh)
    s = mod.gemm_calc_scale(xd)
    assert (bits(host(s)) == bits(want_s)).all()
    assert (host(mod.gemm_round(xd, s)) == ql.gemm_round(xh, want_s)).all()


@pytest.mark.parametrize("shape", SHAPES)
def test_column_kernels(mod, shape):
    x = randn_fp16(shape, seed=shape[1] * 17 + shape[2], std=1.0)
    xh, xd = np16(x), x.cuda()
    want_s = ql.gemm_calc_scale_transpose(xh)
    s = mod.gemm_calc_scale_transpose(xd)
    assert (bits(host(s)) == bits(want_s)).all()
    assert (host(mod.gemm_round_transpose(xd, s)) == ql.gemm_round_transpose(xh, want_s)).all()


def test_edge_cases_match_the_reference_device_code(mod, ref):
    """Zero rows, subnormal scales, NaN, inf, exact ties: the casts the C standard leaves undefined must come out as
    the reference's build produces them."""
    x = edge_case_matrix().cuda()
    for transpose in (False, True):
        calc = "gemm_calc_scale_transpose" if transpose else "gemm_calc_scale"
        rnd = "gemm_round_transpose" if transpose else "gemm_round"
        s_ref = getattr(ref, calc)(x)
        s_mod = getattr(mod, calc)(x)
        assert (bits(host(s_mod)) == bits(host(s_ref))).all()
        assert (host(getattr(mod, rnd)(x, s_ref)) == host(getattr(ref, rnd)(x, s_ref))).all()


@pytest.mark.parametrize("shape,bx,by", [((2, 12, 40), False, False), ((3, 33, 64), True, False), ((2, 128, 512), False, True),
                                         ((4, 7, 20), True, True), ((1, 512, 10240), False, False)])
def test_dequant_kernels(mod, shape, bx, by):
    b, n, m = shape
    rng = np.random.default_rng(b * 100 + n)
    acc = rng.integers(-(2 ** 27), 2 ** 27, size=shape, dtype=np.int32)
    sx = np16(randn_fp16((1 if bx else b, n), 5, 0.01)).copy()
    sy = np16(randn_fp16((1 if by else b, m), 6, 0.01)).copy()
    accd, sxd, syd = torch.from_numpy(acc).cuda(), torch.from_numpy(sx).cuda(), torch.from_numpy(sy).cuda()
    got = host(mod.gemm_scale(accd, sxd, syd, bx, by))
    assert (bits(got) == bits(ql.gemm_scale(acc, sx, sy, bx, by))).all()
    if not bx and not by:
        assert (bits(host(mod.gemm_scale_x(accd, sxd))) == bits(ql.gemm_scale_x(acc, sx))).all()
        assert (bits(host(mod.gemm_scale_y(accd, syd))) == bits(ql.gemm_scale_y(acc, sy))).all()


@pytest.mark.parametrize("shape,bcast", [((2, 12, 40), False), ((3, 33, 64), True), ((2, 100, 520), False), ((1, 64, 2048), True)])
def test_backward_kernels(mod, shape, bcast):
    b, n, m = shape
    x = randn_fp16(shape, 11, 1.0)
    sy = randn_fp16((1 if bcast else b, m), 12, 0.05).abs() + 1e-3
    sx = randn_fp16((1 if bcast else b, n), 13, 0.05).abs() + 1e-3
    q, s = mod.gemm_backward_round_scale(x.cuda(), sy.cuda(), bcast)
    want_q, want_s = ql.gemm_backward_round_scale(np16(x), np16(sy), bcast)
    assert (host(q) == want_q).all() and (bits(host(s)) == bits(want_s)).all()
    q, s = mod.gemm_backward_scale_round(x.cuda(), sx.cuda(), bcast)
    want_q, want_s = ql.gemm_backward_scale_round(np16(x), np16(sx), bcast)
    assert (host(q) == want_q).all() and (bits(host(s)) == bits(want_s)).all()


def close(got_fp16, want_f64):
    want16 = want_f64.astype(np.float16).astype(np.float64)
    return np.isclose(got_fp16.astype(np.float64), want16, rtol=RTOL, atol=ATOL).all()


@pytest.mark.parametrize("batch,dim_out,dim_in", [(1, 10240, 4096), (4, 256, 4096), (3, 37, 24), (2, 9, 4100), (2, 40, 30)])
def test_gemv_kernels(mod, batch, dim_out, dim_in):
    ssk = float(dim_in) ** 0.25
    mat = randn_fp16((batch, dim_out, dim_in), 1, 1.0 / ssk)
    vec = randn_fp16((batch, dim_in), 2, 1.0 / ssk)
    md, vd = mat.cuda(), vec.cuda()
    assert close(host(mod.gemv_fp16_light(md, vd)), ql.gemv_fp16(np16(mat), np16(vec)))
    shared = md[0].contiguous()
    assert close(host(mod.gemv_broadcast_mat_fp16_light(shared, vd)), ql.gemv_broadcast_mat_fp16(np16(mat)[0], np16(vec)))
    matT = md.transpose(1, 2).contiguous()                       # (batch, dim_in, dim_out)
    assert close(host(mod.gemv_fp16_transpose_light(matT, vd)), ql.gemv_fp16_transpose(np16(matT.cpu()), np16(vec)))


@pytest.mark.parametrize("batch,dim_out,dim_in", [(1, 1024, 4096), (4, 100, 256), (3, 37, 24), (2, 9, 4100)])
def test_gemv_int8_kernels(mod, batch, dim_out, dim_in):
    vec = randn_fp16((batch, dim_in), 21, 1.0)
    mat = randn_fp16((1, dim_out, dim_in), 22, 0.02)
    vh = np16(vec)
    want_sv = ql.gemm_calc_scale(vh[None])[0]
    want_qv = ql.gemm_round(vh[None], want_sv[None])[0]
    vd = vec.cuda()
    sv = mod.gemv_calc_scale(vd)
    assert (bits(host(sv)) == bits(want_sv)).all()
    qv = mod.gemv_round(vd, sv)
    assert (host(qv) == want_qv).all()
    sm = ql.gemm_calc_scale(np16(mat))[0]
    qm = ql.gemm_round(np16(mat), sm[None])[0]
    got = host(mod.gemv_broadcast_mat_int8(torch.from_numpy(sm).cuda(), torch.from_numpy(qm).cuda(), sv, qv))
    assert (bits(got) == bits(ql.gemv_broadcast_mat_int8(sm, qm, want_sv, want_qv))).all()


def test_other_launch_shapes(mod):
    """The kernels read their work split from gridDim / blockDim: a clamped grid and odd blocks give the same bits."""
    shape = (2, 70, 520)
    x = randn_fp16(shape, 3, 1.0)
    xh, xd = np16(x), x.cuda()
    b, n, m = shape
    i32, ptr, stream = ctypes.c_int32, (lambda t: ctypes.c_void_p(t.data_ptr())), torch.cuda.current_stream().cuda_stream
    for grid, block in (((1, 7, 1), (96, 1, 1)), ((2, 3, 1), (20, 3, 1)), ((b, n, 1), (1000, 1, 1))):
        s = torch.empty((b, n), dtype=torch.half, device="cuda")
        q = torch.empty(shape, dtype=torch.int8, device="cuda")
        mod.drv.launch(mod._fn("gemm", "cu_gemm_calc_scale"), grid, block, stream, [i32(b), i32(n), i32(m), ptr(xd), ptr(s)])
        mod.drv.launch(mod._fn("gemm", "cu_gemm_round"), grid, block, stream, [i32(b), i32(n), i32(m), ptr(xd), ptr(s), ptr(q)])
        want_s = ql.gemm_calc_scale(xh)
        assert (bits(host(s)) == bits(want_s)).all() and (host(q) == ql.gemm_round(xh, want_s)).all()
        st = torch.empty((b, m), dtype=torch.half, device="cuda")
        qt = torch.empty(shape, dtype=torch.int8, device="cuda")
        mod.drv.launch(mod._fn("gemm", "cu_gemm_calc_scale_transpose"), grid, block, stream, [i32(b), i32(n), i32(m), ptr(xd), ptr(st)])
        mod.drv.launch(mod._fn("gemm", "cu_gemm_round_transpose"), grid, block, stream, [i32(b), i32(n), i32(m), ptr(xd), ptr(st), ptr(qt)])
        want_st = ql.gemm_calc_scale_transpose(xh)
        assert (bits(host(st)) == bits(want_st)).all() and (host(qt) == ql.gemm_round_transpose(xh, want_st)).all()
