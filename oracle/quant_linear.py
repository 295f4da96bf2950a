"""TEST INFRASTRUCTURE ONLY -- numpy restatement of the cpm_kernels quantised-linear hot path.

This module is the checker the CUDA kernels are compared against.  The shipped package never
imports it; only ``tests/``, the smoke check and the CPU-baseline leg of the benchmark do.

Two restatements live side by side and are tested against each other:

* the functions below (vectorised numpy, usable at the benchmark's full sizes), and
* ``oracle/quant_linear.c`` (scalar C that follows the reference's device code operation by
  operation; reached through :class:`COracle`).

Parity pin: the reference holds no golden vectors for this path.  The pin is the reference's
own device code (``cuda/gemm.cu``, ``cuda/gemv.cu``), compiled unmodified for sm_100 by
``oracle/Makefile`` (target ``ref``) and run on a B200 by ``tests/golden/make_golden.py``; its
outputs on seeded inputs are committed under ``tests/golden/`` and ``tests/test_oracle_golden.py``
holds both restatements to them bit for bit.

All fp16 tensors are ``np.float16`` arrays; int8 codes ``np.int8``; accumulators ``np.int32``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))


# --------------------------------------------------------------------------------------------
# numpy restatement
# --------------------------------------------------------------------------------------------
def _scale_from_amax(amax_f32: np.ndarray) -> np.ndarray:
    """``__float2half(local_max / 127.0)``: double division, narrowed to float, then to half
    (cuda/gemm.cu:74, :96)."""
    return (amax_f32.astype(np.float64) / 127.0).astype(np.float32).astype(np.float16)


def _absmax(x_f32: np.ndarray, axis: int) -> np.ndarray:
    """``fmaxf(fabsf(x), running)`` starting from 0: NaN elements are dropped (fmaxf returns the
    non-NaN operand), as in cuda/gemm.cu:67-69."""
    a = np.abs(x_f32)
    a = np.where(np.isnan(a), np.float32(0), a)
    return a.max(axis=axis, initial=np.float32(0)).astype(np.float32)


def cast_i8(v_f32: np.ndarray) -> np.ndarray:
    """float -> int8 as the reference's sm_100 build performs it (observed; tests/golden/reference_sm100.npz,
    arrays c_*): saturating round-toward-zero conversion to a 32-bit integer (NaN -> 0), low byte kept.  Equal to
    the C cast wherever that is defined (|v| <= 127)."""
    v = np.asarray(v_f32, dtype=np.float32).astype(np.float64)
    t = np.trunc(np.where(np.isnan(v), 0.0, v))
    w = np.clip(t, -2147483648.0, 2147483647.0).astype(np.int64)
    return (w & 0xFF).astype(np.uint8).view(np.int8)


def gemm_calc_scale(mat: np.ndarray) -> np.ndarray:
    """cuda/gemm.cu:60-76.  mat (batch, n, m) fp16 -> (batch, n) fp16."""
    assert mat.dtype == np.float16 and mat.ndim == 3
    return _scale_from_amax(_absmax(mat.astype(np.float32), axis=2))


def gemm_calc_scale_transpose(mat: np.ndarray) -> np.ndarray:
    """cuda/gemm.cu:79-98.  mat (batch, n, m) fp16 -> (batch, m) fp16 (reduction over n)."""
    assert mat.dtype == np.float16 and mat.ndim == 3
    return _scale_from_amax(_absmax(mat.astype(np.float32), axis=1))


def _round_div(x_f32: np.ndarray, s_f32: np.ndarray) -> np.ndarray:
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        q = x_f32 / s_f32                      # IEEE binary32 division, round to nearest even
        return cast_i8(np.rint(q))             # nearbyintf: round half to even


def gemm_round(mat: np.ndarray, scale: np.ndarray) -> np.ndarray:
    """cuda/gemm.cu:6-18.  mat (batch, n, m), scale (batch, n) -> int8 (batch, n, m)."""
    assert mat.dtype == np.float16 and scale.dtype == np.float16
    return _round_div(mat.astype(np.float32), scale.astype(np.float32)[:, :, None])


def gemm_round_transpose(mat: np.ndarray, scale: np.ndarray) -> np.ndarray:
    """cuda/gemm.cu:22-33.  mat (batch, n, m), scale (batch, m) -> int8 (batch, n, m)."""
    assert mat.dtype == np.float16 and scale.dtype == np.float16
    return _round_div(mat.astype(np.float32), scale.astype(np.float32)[:, None, :])


def gemm_int8(m: int, k: int, n: int, aT: bool, bT: bool, A: np.ndarray, B: np.ndarray) -> np.ndarray:
    """cpm_kernels/kernels/gemm.py:127-186.  A (bA, k, m) or (bA, m, k) if aT; B (bB, n, k) or
    (bB, k, n) if bT; returns int32 (max(bA, bB), n, m) with out[b,j,i] = sum_l Aop[b,l,i]*Bop[b,j,l].
    Computed in float64 (exact: |sum| <= 128*128*k < 2**53)."""
    assert A.dtype == np.int8 and B.dtype == np.int8
    a_km = A.transpose(0, 2, 1) if aT else A                  # (bA, k, m)
    b_nk = B.transpose(0, 2, 1) if bT else B                  # (bB, n, k)
    assert a_km.shape[1:] == (k, m) and b_nk.shape[1:] == (n, k)
    assert A.shape[0] == B.shape[0] or A.shape[0] == 1 or B.shape[0] == 1
    out = np.matmul(b_nk.astype(np.float64), a_km.astype(np.float64))
    return np.rint(out).astype(np.int32)


def gemm_fp16(m: int, k: int, n: int, aT: bool, bT: bool, A: np.ndarray, B: np.ndarray) -> np.ndarray:
    """cpm_kernels/kernels/gemm.py:188-256 gemm_fp16, same storage conventions as gemm_int8: A (bA, k, m) or
    (bA, m, k) if aT; B (bB, n, k) or (bB, k, n) if bT.  Returns the exact products in float64 (b, n, m); the
    reference's cublasLt call accumulates in fp16 and is pinned by its tests to 0.5 / 0.5 only
    (tests/test_gemm.py:98)."""
    a = A.astype(np.float64)
    b = B.astype(np.float64)
    a_km = np.swapaxes(a, 1, 2) if aT else a          # (bA, k, m)
    b_nk = np.swapaxes(b, 1, 2) if bT else b          # (bB, n, k)
    assert a_km.shape[1:] == (k, m) and b_nk.shape[1:] == (n, k)
    return np.matmul(b_nk, a_km)


def gemm_scale(mat: np.ndarray, scale_x: np.ndarray, scale_y: np.ndarray,
               broad_cast_x: bool, broad_cast_y: bool) -> np.ndarray:
    """cuda/gemm.cu:37-57.  mat int32 (batch, n, m); scale_x (batch or 1, n); scale_y (batch or 1, m).
    out = half(((float)mat * sx) * sy), the two multiplies in binary32, left to right."""
    assert mat.dtype == np.int32
    sx = scale_x.astype(np.float32).reshape(-1, mat.shape[1])
    sy = scale_y.astype(np.float32).reshape(-1, mat.shape[2])
    sx = sx[0:1] if broad_cast_x else sx
    sy = sy[0:1] if broad_cast_y else sy
    with np.errstate(over="ignore", invalid="ignore"):
        v = mat.astype(np.float32) * sx[:, :, None]
        v = v * sy[:, None, :]
        return v.astype(np.float16)


def gemm_scale_x(mat: np.ndarray, scale_x: np.ndarray) -> np.ndarray:
    """cuda/gemm.cu:176-189."""
    with np.errstate(over="ignore"):
        return (scale_x.astype(np.float32)[:, :, None] * mat.astype(np.float32)).astype(np.float16)


def gemm_scale_y(mat: np.ndarray, scale_y: np.ndarray) -> np.ndarray:
    """cuda/gemm.cu:192-205."""
    with np.errstate(over="ignore"):
        return (mat.astype(np.float32) * scale_y.astype(np.float32)[:, None, :]).astype(np.float16)


def gemm_backward_round_scale(mat: np.ndarray, scale_y: np.ndarray, broad_cast_y: bool):
    """cuda/gemm.cu:103-134.  Returns (codes int8 (b,n,m), scale_x fp16 (b,n)).  The divisor of the
    rounding step is the float scale *before* it is narrowed to fp16."""
    sy = scale_y.astype(np.float32).reshape(-1, mat.shape[2])
    sy = sy[0:1] if broad_cast_y else sy
    v = mat.astype(np.float32) * sy[:, None, :]
    s = (_absmax(v, axis=2).astype(np.float64) / 127.0).astype(np.float32)
    return _round_div(v, s[:, :, None]), s.astype(np.float16)


def gemm_backward_scale_round(mat: np.ndarray, scale_x: np.ndarray, broad_cast_x: bool):
    """cuda/gemm.cu:137-172.  Returns (codes int8 (b,n,m), scale_y fp16 (b,m))."""
    sx = scale_x.astype(np.float32).reshape(-1, mat.shape[1])
    sx = sx[0:1] if broad_cast_x else sx
    v = mat.astype(np.float32) * sx[:, :, None]
    s = (_absmax(v, axis=1).astype(np.float64) / 127.0).astype(np.float32)
    return _round_div(v, s[:, None, :]), s.astype(np.float16)


def gemv_fp16(mat: np.ndarray, vec: np.ndarray) -> np.ndarray:
    """cuda/gemv.cu:79-106 / kernels/gemv.py:82-127.  mat (batch, dim_out, dim_in), vec (batch, dim_in);
    returns the exact sums in float64 (batch, dim_out).  The reference's own two implementations differ
    in accumulation order and precision; its tests pin them to 1e-3 (tests/test_gemv.py:81)."""
    return np.einsum("boi,bi->bo", mat.astype(np.float64), vec.astype(np.float64))


def gemv_fp16_transpose(mat: np.ndarray, vec: np.ndarray) -> np.ndarray:
    """cuda/gemv.cu:109-135.  mat (batch, dim_in, dim_out), vec (batch, dim_in) -> float64 (batch, dim_out)."""
    return np.einsum("bio,bi->bo", mat.astype(np.float64), vec.astype(np.float64))


def gemv_broadcast_mat_fp16(mat: np.ndarray, vec: np.ndarray) -> np.ndarray:
    """cuda/gemv.cu:138-164.  mat (dim_out, dim_in) shared, vec (batch, dim_in) -> float64 (batch, dim_out)."""
    return vec.astype(np.float64) @ mat.astype(np.float64).T


def gemv_broadcast_mat_int8(scale_mat, mat, scale_vec, vec) -> np.ndarray:
    """cuda/gemv.cu:57-76.  out[b,o] = half(((float)dot * scale_vec[b]) * scale_mat[o])."""
    acc = np.rint(vec.astype(np.float64) @ mat.astype(np.float64).T).astype(np.int32)
    with np.errstate(over="ignore"):
        v = acc.astype(np.float32) * scale_vec.astype(np.float32)[:, None]
        v = v * scale_mat.astype(np.float32)[None, :]
        return v.astype(np.float16)


def gelu_forward(x: np.ndarray) -> np.ndarray:
    """cuda/gelu.cu:6-17 cu_gelu_forward on an fp16 array of any shape:
        x = (float)h;  x = 0.5 * x * (1.0 + tanhf(0.7978845608028654 * x * (1.0 + 0.044715 * x * x)));  out = half(x)
    The literals are doubles, so every product and sum is carried out in binary64; the argument of tanhf is narrowed
    to binary32 first and its result widened again; the final product is narrowed to binary32, then to fp16.  tanhf is
    taken as correctly rounded here; against the reference's own device code this agrees on all 65536 fp16 inputs
    (tests/golden/reference_gelu_sm100.npz).  NaN results carry the bit pattern 0x7fff that __float2half writes."""
    assert x.dtype == np.float16
    with np.errstate(all="ignore"):
        xd = x.astype(np.float32).astype(np.float64)
        inner = (0.7978845608028654 * xd * (1.0 + 0.044715 * xd * xd)).astype(np.float32)
        th = np.tanh(inner.astype(np.float64)).astype(np.float32)
        y = (0.5 * xd * (1.0 + th.astype(np.float64))).astype(np.float32).astype(np.float16)
    bits = y.view(np.uint16).copy()
    bits[np.isnan(y)] = 0x7FFF
    return bits.view(np.float16)


def gelu_backward(grad_out: np.ndarray, mat: np.ndarray) -> np.ndarray:
    """cuda/gelu.cu:20-44 cu_gelu_backward in binary64: grad = gelu'(mat) * grad_out with
        gelu'(x) = 0.5 + (0.398942 x + 0.0535161 x^3) sech^2(u) + 0.5 tanh(u),  u = 0.797885 x + 0.0356774 x^3   for -5 < x < 5,
        gelu'(x) = 0 (x < 0) or 1 otherwise.
    The device evaluates coshf / tanhf in binary32 with its own (not correctly rounded) routines, so this restatement
    pins the kernel to a tolerance (rtol 2e-3, atol 1e-3 on the fp16 result), not bit for bit; bit parity of the
    backward kernel is checked against the reference's own device code where it is available."""
    assert grad_out.dtype == np.float16 and mat.dtype == np.float16
    with np.errstate(all="ignore"):
        x = mat.astype(np.float64)
        u = 0.797885 * x + 0.0356774 * x ** 3
        g = 0.5 + (0.398942 * x + 0.0535161 * x ** 3) / np.cosh(u) ** 2 + 0.5 * np.tanh(u)
        g = np.where((x > -5) & (x < 5), g, np.where(x < 0, 0.0, 1.0))
        return g * grad_out.astype(np.float64)


def transpose(x: np.ndarray) -> np.ndarray:
    """cuda/transpose.cu:6-22 cu_transpose: out[b, c, r] = in[b, r, c] for a (batch, n, m) array; no arithmetic."""
    assert x.ndim == 3
    return np.ascontiguousarray(np.swapaxes(x, 1, 2))


def _shuffle_down_sum32(v: np.ndarray) -> np.ndarray:
    """Lane 0 of the reference's warpReduceSum (cuda/includes/reduce.cuh:6-10) over the last axis (length 32), in
    binary32: x += shfl_down(x, 16), then 8, 4, 2, 1."""
    a = v[..., :16] + v[..., 16:32]
    b = a[..., :8] + a[..., 8:16]
    c = b[..., :4] + b[..., 4:8]
    d = c[..., :2] + c[..., 2:4]
    return d[..., 0] + d[..., 1]


def _layernorm_column_sum(v: np.ndarray) -> np.ndarray:
    """The reference's nested summation of one quantity over the rows (cuda/layernorm.cu:19-45): v is (batch, n, m)
    binary32; rows are taken in chunks of 1024, each chunk as 32 blocks of 32 rows; a block's 32 rows and a chunk's 32
    block sums are each combined by the shuffle tree above (missing rows / blocks count as zero), and the chunk sums are
    accumulated in order."""
    b, n, m = v.shape
    n_pad = (n + 1023) // 1024 * 1024
    vp = np.zeros((b, n_pad, m), np.float32)
    vp[:, :n, :] = v
    blocks = vp.reshape(b, n_pad // 1024, 32, 32, m)                  # (batch, chunk, block, row lane, column)
    block_sums = _shuffle_down_sum32(np.moveaxis(blocks, 3, -1))       # (batch, chunk, block, column)
    chunk_sums = _shuffle_down_sum32(np.moveaxis(block_sums, 2, -1))   # (batch, chunk, column)
    total = np.zeros((b, m), np.float32)
    for c in range(chunk_sums.shape[1]):
        total = total + chunk_sums[:, c, :]
    return total


def layernorm_forward(x: np.ndarray, eps: float, rd_mean: bool) -> np.ndarray:
    """cuda/layernorm.cu:6-71 cu_layernorm_forward: x (batch, n, m) fp16, normalised over the MIDDLE axis n per
    (batch, column).  mean = S1 / n, var = S2 / n - mean * mean (one fused multiply-add, as nvcc contracts it),
    rstd = rsqrtf(var + eps), out = half(((float)x - mean) * rstd)  [rd_mean]  or  half((float)x * rstd).
    rsqrtf is taken as correctly rounded here; the device's approximation differs from that in the last place for
    some arguments, which moves a few outputs by one fp16 step (tests/test_oracle_golden.py states how many)."""
    assert x.dtype == np.float16 and x.ndim == 3
    n = x.shape[1]
    xf = x.astype(np.float32)
    with np.errstate(all="ignore"):
        s2 = _layernorm_column_sum(xf * xf) / np.float32(n)
        if rd_mean:
            mean = _layernorm_column_sum(xf) / np.float32(n)
            var = (s2.astype(np.float64) - mean.astype(np.float64) * mean.astype(np.float64)).astype(np.float32)   # fma
        else:
            mean = np.zeros_like(s2)
            var = s2
        rstd = (1.0 / np.sqrt((var + np.float32(eps)).astype(np.float64))).astype(np.float32)
        if rd_mean:
            y = (xf - mean[:, None, :]) * rstd[:, None, :]
        else:
            y = xf * rstd[:, None, :]
        return y.astype(np.float16)


def arith_ln_mul(x: np.ndarray, alpha: np.ndarray) -> np.ndarray:
    """cuda/arith.cu:115-127: out = __hmul2(x, alpha[row]) -- one rounding to fp16."""
    return (x.astype(np.float32) * alpha.astype(np.float32)[None, :, None]).astype(np.float16)


def arith_ln_mul_add(x: np.ndarray, alpha: np.ndarray, beta: np.ndarray) -> np.ndarray:
    """cuda/arith.cu:97-112: out = __hfma2(x, alpha[row], beta[row]) -- fused, one rounding to fp16."""
    prod = x.astype(np.float64) * alpha.astype(np.float64)[None, :, None]
    return (prod + beta.astype(np.float64)[None, :, None]).astype(np.float16)


def layernorm_quantize_cols(x: np.ndarray, eps: float, rd_mean: bool, alpha: np.ndarray, beta=None):
    """The chain layer norm -> affine -> column quantisation that feeds a CPM-layout linear
    (torch/layernorm.py:8-30, torch/gemm.py:98-102): returns (scale (batch, m) fp16, codes (batch, n, m) int8)."""
    y = layernorm_forward(x, eps, rd_mean)
    y = arith_ln_mul_add(y, alpha, beta) if beta is not None else arith_ln_mul(y, alpha)
    scale = gemm_calc_scale_transpose(y)
    return scale, gemm_round_transpose(y, scale)


def bmm_int8(A: np.ndarray, aT: bool, B: np.ndarray, bT: bool):
    """cpm_kernels/torch/gemm.py:86-113 GEMMInt8.forward, restated with the functions above.
    A (bA, M, K) [or (bA, K, M) if aT], B (bB, K, N) [or (bB, N, K) if bT], fp16.
    Returns dict with scale_A, quant_A, scale_B, quant_B, acc (int32), out (fp16 (b, M, N))."""
    scale_A = gemm_calc_scale_transpose(A) if aT else gemm_calc_scale(A)
    scale_B = gemm_calc_scale(B) if bT else gemm_calc_scale_transpose(B)
    qA = gemm_round_transpose(A, scale_A) if aT else gemm_round(A, scale_A)
    qB = gemm_round(B, scale_B) if bT else gemm_round_transpose(B, scale_B)
    M = A.shape[2] if aT else A.shape[1]
    K = A.shape[1] if aT else A.shape[2]
    N = B.shape[1] if bT else B.shape[2]
    # torch/gemm.py:45-52: operands swapped so that the (n, m) = (M, N) result is row-major C
    acc = gemm_int8(N, K, M, bT, aT, qB, qA)
    out = gemm_scale(acc, scale_A, scale_B, A.shape[0] == 1, B.shape[0] == 1)
    return dict(scale_A=scale_A, quant_A=qA, scale_B=scale_B, quant_B=qB, acc=acc, out=out)


# --------------------------------------------------------------------------------------------
# C restatement (oracle/quant_linear.c) through ctypes
# --------------------------------------------------------------------------------------------
def build_c_oracle() -> str:
    """Compile oracle/quant_linear.c (and, where a reference checkout is present, the reference's
    own device code into oracle/_ref/) with oracle/Makefile; return the path of the C library."""
    subprocess.run(["make", "-s", "-C", _HERE, "all", "REFERENCE_DIR=" + reference_dir()], check=True, stdout=subprocess.DEVNULL)
    return os.path.join(_HERE, "_build", "libquant_linear_oracle.so")


def reference_dir() -> str:
    """Where a cpm_kernels checkout is looked for: $CPM_KERNELS_REFERENCE_DIR, else a directory named ``reference``
    beside this repository.  Empty when there is none (the prebuilt oracle/_ref files are then used as they are)."""
    cand = os.environ.get("CPM_KERNELS_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    return cand if os.path.exists(os.path.join(cand, "cuda", "gemm.cu")) else ""


def _c_oracle_path() -> str:
    """The C library, rebuilt by make when quant_linear.c is newer (the reference's device code is left alone)."""
    subprocess.run(["make", "-s", "-C", _HERE, "oracle"], check=True, stdout=subprocess.DEVNULL)
    return os.path.join(_HERE, "_build", "libquant_linear_oracle.so")


class COracle:
    """ctypes view of oracle/quant_linear.c.  Arrays are numpy, C-contiguous."""

    def __init__(self, path: str | None = None):
        path = path or _c_oracle_path()
        self.lib = ctypes.CDLL(path)

    @staticmethod
    def _p(a: np.ndarray):
        assert a.flags["C_CONTIGUOUS"]
        return a.ctypes.data_as(ctypes.c_void_p)

    def gemm_calc_scale(self, mat):
        b, n, m = mat.shape
        out = np.empty((b, n), np.float16)
        self.lib.orc_gemm_calc_scale(b, n, m, self._p(mat), self._p(out))
        return out

    def gelu_forward(self, x):
        out = np.empty(x.shape, np.float16)
        self.lib.orc_gelu_forward(ctypes.c_int64(x.size), self._p(x), self._p(out))
        return out

    def gemm_calc_scale_transpose(self, mat):
        b, n, m = mat.shape
        out = np.empty((b, m), np.float16)
        self.lib.orc_gemm_calc_scale_transpose(b, n, m, self._p(mat), self._p(out))
        return out

    def gemm_round(self, mat, scale):
        b, n, m = mat.shape
        out = np.empty((b, n, m), np.int8)
        self.lib.orc_gemm_round(b, n, m, self._p(mat), self._p(scale), self._p(out))
        return out

    def gemm_round_transpose(self, mat, scale):
        b, n, m = mat.shape
        out = np.empty((b, n, m), np.int8)
        self.lib.orc_gemm_round_transpose(b, n, m, self._p(mat), self._p(scale), self._p(out))
        return out

    def gemm_int8(self, m, k, n, aT, bT, A, B, threads: int | None = None):
        bA, bB = A.shape[0], B.shape[0]
        out = np.empty((max(bA, bB), n, m), np.int32)
        threads = threads or min(os.cpu_count() or 1, max(1, n))
        bounds = np.linspace(0, n, threads + 1).astype(int)

        def run(t):
            self.lib.orc_gemm_int8_rows(m, k, n, bA, bB, int(aT), int(bT), self._p(A), self._p(B),
                                        self._p(out), int(bounds[t]), int(bounds[t + 1]))
        with ThreadPoolExecutor(threads) as ex:
            list(ex.map(run, range(threads)))
        return out

    def gemm_scale(self, mat, scale_x, scale_y, bx, by):
        b, n, m = mat.shape
        out = np.empty((b, n, m), np.float16)
        self.lib.orc_gemm_scale(b, n, m, self._p(mat), self._p(scale_x), self._p(scale_y), self._p(out), int(bx), int(by))
        return out

    def gemm_scale_x(self, mat, scale_x):
        b, n, m = mat.shape
        out = np.empty((b, n, m), np.float16)
        self.lib.orc_gemm_scale_x(b, n, m, self._p(mat), self._p(scale_x), self._p(out))
        return out

    def gemm_scale_y(self, mat, scale_y):
        b, n, m = mat.shape
        out = np.empty((b, n, m), np.float16)
        self.lib.orc_gemm_scale_y(b, n, m, self._p(mat), self._p(scale_y), self._p(out))
        return out

    def gemm_backward_round_scale(self, mat, scale_y, by):
        b, n, m = mat.shape
        out = np.empty((b, n, m), np.int8)
        sx = np.empty((b, n), np.float16)
        self.lib.orc_gemm_backward_round_scale(b, n, m, self._p(mat), self._p(scale_y), self._p(out), self._p(sx), int(by))
        return out, sx

    def gemm_backward_scale_round(self, mat, scale_x, bx):
        b, n, m = mat.shape
        out = np.empty((b, n, m), np.int8)
        sy = np.empty((b, m), np.float16)
        self.lib.orc_gemm_backward_scale_round(b, n, m, self._p(mat), self._p(scale_x), self._p(out), self._p(sy), int(bx))
        return out, sy

    def gemv_fp16(self, mat, vec):
        b, o, i = mat.shape
        out = np.empty((b, o), np.float64)
        self.lib.orc_gemv_fp16(b, o, i, self._p(mat), self._p(vec), self._p(out))
        return out

    def gemv_fp16_transpose(self, mat, vec):
        b, i, o = mat.shape
        out = np.empty((b, o), np.float64)
        self.lib.orc_gemv_fp16_transpose(b, o, i, self._p(mat), self._p(vec), self._p(out))
        return out

    def gemv_broadcast_mat_fp16(self, mat, vec):
        o, i = mat.shape
        b = vec.shape[0]
        out = np.empty((b, o), np.float64)
        self.lib.orc_gemv_broadcast_mat_fp16(b, o, i, self._p(mat), self._p(vec), self._p(out))
        return out

    def gemv_broadcast_mat_int8(self, scale_mat, mat, scale_vec, vec):
        o, i = mat.shape
        b = vec.shape[0]
        out = np.empty((b, o), np.float16)
        self.lib.orc_gemv_broadcast_mat_int8(b, o, i, self._p(scale_mat), self._p(mat), self._p(scale_vec), self._p(vec), self._p(out))
        return out

    def round_one(self, x_bits: int, s_bits: int) -> int:
        self.lib.orc_round_one.restype = ctypes.c_int8
        return int(self.lib.orc_round_one(ctypes.c_uint16(x_bits), ctypes.c_uint16(s_bits)))
