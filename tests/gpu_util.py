"""Helpers of the GPU parity tests: every call goes through cpm_kernels_b200.kernels, i.e. ctypes -> C ABI."""
import numpy as np
import torch

import cpm_kernels_b200.kernels as ck
from cpm_kernels_b200.library import cpmk


def stream():
    return torch.cuda.current_stream().cuda_stream


def dev(a):
    if isinstance(a, np.ndarray):
        a = torch.from_numpy(np.ascontiguousarray(a))
    return a.contiguous().cuda()


def host(t):
    return t.detach().cpu().contiguous().numpy()


def calc_scale(x, transpose=False):
    b, n, m = x.shape
    out = torch.full((b, m if transpose else n), 7.0, dtype=torch.half, device="cuda")
    (ck.gemm_calc_scale_transpose if transpose else ck.gemm_calc_scale)(b, n, m, x.data_ptr(), out.data_ptr(), stream())
    return out


def round_i8(x, scale, transpose=False):
    b, n, m = x.shape
    out = torch.full((b, n, m), 99, dtype=torch.int8, device="cuda")
    (ck.gemm_round_transpose if transpose else ck.gemm_round)(b, n, m, x.data_ptr(), scale.data_ptr(), out.data_ptr(), stream())
    return out


def quantize(x, transpose=False):
    b, n, m = x.shape
    scale = torch.full((b, m if transpose else n), 7.0, dtype=torch.half, device="cuda")
    out = torch.full((b, n, m), 99, dtype=torch.int8, device="cuda")
    (ck.gemm_quantize_cols if transpose else ck.gemm_quantize_rows)(b, n, m, x.data_ptr(), scale.data_ptr(), out.data_ptr(), stream())
    return scale, out


def gemm_int8(m, k, n, aT, bT, A, B):
    bA, bB = A.shape[0], B.shape[0]
    out = torch.full((max(bA, bB), n, m), -12345, dtype=torch.int32, device="cuda")
    ck.gemm_int8(m, k, n, bA, bB, aT, bT, A.data_ptr(), B.data_ptr(), out.data_ptr(), stream())
    return out


def gemm_int8_scale(m, k, n, aT, bT, A, B, sx, sy, bx, by):
    bA, bB = A.shape[0], B.shape[0]
    out = torch.full((max(bA, bB), n, m), 777.0, dtype=torch.half, device="cuda")
    ck.gemm_int8_scale(m, k, n, bA, bB, aT, bT, A.data_ptr(), B.data_ptr(), sx.data_ptr(), sy.data_ptr(), bx, by, out.data_ptr(), stream())
    return out


def gemm_scale(acc, sx, sy, bx, by):
    b, n, m = acc.shape
    out = torch.full((b, n, m), 777.0, dtype=torch.half, device="cuda")
    ck.gemm_scale(b, n, m, acc.data_ptr(), sx.data_ptr(), sy.data_ptr(), out.data_ptr(), bx, by, stream())
    return out


def assert_no_device_error():
    torch.cuda.synchronize()
    assert cpmk.read_status() == 0


def same_bits(a, b):
    """fp16 tensors / arrays equal as bit patterns."""
    a = host(a) if isinstance(a, torch.Tensor) else a
    b = host(b) if isinstance(b, torch.Tensor) else b
    return (np.ascontiguousarray(a).view(np.uint16) == np.ascontiguousarray(b).view(np.uint16)).all()
