"""Launchers of the quantisation passes and the int8 GEMM, with the signatures of
cpm_kernels/kernels/gemm.py (positional order, meaning and preconditions unchanged).

All pointers are raw device addresses (``DevicePointer = int``), sizes are Python ints and ``stream``
is a ``cudaStream_t`` value.  Work is enqueued on ``stream``; nothing synchronises.  Shape
preconditions raise ``AssertionError`` as in the reference; CUDA failures raise ``RuntimeError``.
"""
from ..library import cpmk
from .base import DevicePointer, CUDAStream, stream_arg


def gemm_round(batch: int, n: int, m: int,
               mat: DevicePointer,      # (b, n, m) fp16
               scale: DevicePointer,    # (b, n)    fp16
               out: DevicePointer,      # (b, n, m) int8
               stream: CUDAStream):
    """kernels/gemm.py:21-41.  out = (int8) nearbyintf(mat / scale[b, row])."""
    cpmk.call("cpmk_gemm_round", batch, n, m, mat, scale, out, stream_arg(stream))


def gemm_round_transpose(batch: int, n: int, m: int,
                         mat: DevicePointer,    # (b, n, m) fp16
                         scale: DevicePointer,  # (b, m)    fp16
                         out: DevicePointer,    # (b, n, m) int8
                         stream: CUDAStream):
    """kernels/gemm.py:43-63.  out = (int8) nearbyintf(mat / scale[b, column])."""
    cpmk.call("cpmk_gemm_round_transpose", batch, n, m, mat, scale, out, stream_arg(stream))


def gemm_scale(batch: int, n: int, m: int,
               mat: DevicePointer,        # (b, n, m) int32
               scale_x: DevicePointer,    # (b, n)    fp16
               scale_y: DevicePointer,    # (b, m)    fp16
               out: DevicePointer,        # (b, n, m) fp16
               broad_cast_x: bool, broad_cast_y: bool,
               stream: CUDAStream):
    """kernels/gemm.py:65-89.  out = half(((float)mat * scale_x) * scale_y)."""
    cpmk.call("cpmk_gemm_scale", batch, n, m, mat, scale_x, scale_y, out, int(bool(broad_cast_x)), int(bool(broad_cast_y)),
              stream_arg(stream))


def gemm_calc_scale(batch: int, n: int, m: int,
                    mat: DevicePointer,    # (b, n, m) fp16
                    out: DevicePointer,    # (b, n)    fp16
                    stream: CUDAStream):
    """kernels/gemm.py:91-107.  out = half(max_i |mat[b, r, i]| / 127)."""
    cpmk.call("cpmk_gemm_calc_scale", batch, n, m, mat, out, stream_arg(stream))


def gemm_calc_scale_transpose(batch: int, n: int, m: int,
                              inp: DevicePointer,    # (b, n, m) fp16
                              out: DevicePointer,    # (b, m)    fp16
                              stream: CUDAStream):
    """kernels/gemm.py:109-125.  out = half(max_r |inp[b, r, c]| / 127)."""
    cpmk.call("cpmk_gemm_calc_scale_transpose", batch, n, m, inp, out, stream_arg(stream))


def gemm_int8(m: int, k: int, n: int,
              batchA: int, batchB: int,
              aT: bool, bT: bool,
              A: DevicePointer,    # (bA, k, m), or (bA, m, k) if aT     int8
              B: DevicePointer,    # (bB, n, k), or (bB, k, n) if bT     int8
              out: DevicePointer,  # (max(bA, bB), n, m)                 int32
              stream: CUDAStream):
    """kernels/gemm.py:127-186.  out[b, j, i] = sum_l Aop[b, l, i] * Bop[b, j, l] in int32."""
    assert m % 4 == 0 and n % 4 == 0 and k % 4 == 0
    assert batchA == batchB or batchA == 1 or batchB == 1
    cpmk.call("cpmk_gemm_int8", m, k, n, batchA, batchB, int(bool(aT)), int(bool(bT)), A, B, out, stream_arg(stream))


def gemm_fp16(m: int, k: int, n: int,
              batchA: int, batchB: int,
              aT: bool, bT: bool,
              A: DevicePointer,    # (bA, k, m), or (bA, m, k) if aT     fp16
              B: DevicePointer,    # (bB, n, k), or (bB, k, n) if bT     fp16
              out: DevicePointer,  # (max(bA, bB), n, m)                 fp16
              stream: CUDAStream):
    """kernels/gemm.py:188-256.  out[b, j, i] = sum_l Aop[b, l, i] * Bop[b, j, l], fp32 accumulation, fp16 result."""
    assert m % 2 == 0 and n % 2 == 0 and k % 2 == 0
    assert batchA == batchB or batchA == 1 or batchB == 1
    cpmk.call("cpmk_gemm_fp16", m, k, n, batchA, batchB, int(bool(aT)), int(bool(bT)), A, B, out, stream_arg(stream))


def gemm_backward_round_scale(batch: int, n: int, m: int,
                              mat: DevicePointer,        # (batch, n, m) fp16
                              scale_y: DevicePointer,    # (batch, m)    fp16
                              out: DevicePointer,        # (batch, n, m) int8
                              scale_x: DevicePointer,    # (batch, n)    fp16
                              broad_cast_y: bool,
                              stream: CUDAStream):
    """kernels/gemm.py:261-283."""
    cpmk.call("cpmk_gemm_backward_round_scale", batch, n, m, mat, scale_y, out, scale_x, int(bool(broad_cast_y)), stream_arg(stream))


def gemm_backward_scale_round(batch: int, n: int, m: int,
                              mat: DevicePointer,        # (batch, n, m) fp16
                              scale_x: DevicePointer,    # (batch, n)    fp16
                              out: DevicePointer,        # (batch, n, m) int8
                              scale_y: DevicePointer,    # (batch, m)    fp16
                              broad_cast_x: bool,
                              stream: CUDAStream):
    """kernels/gemm.py:285-307."""
    cpmk.call("cpmk_gemm_backward_scale_round", batch, n, m, mat, scale_x, out, scale_y, int(bool(broad_cast_x)), stream_arg(stream))


def gemm_scale_x(batch: int, n: int, m: int,
                 mat: DevicePointer,        # (batch, n, m) int32
                 scale_x: DevicePointer,    # (batch, n)    fp16
                 out: DevicePointer,        # (batch, n, m) fp16
                 stream: CUDAStream):
    """kernels/gemm.py:309-327."""
    cpmk.call("cpmk_gemm_scale_x", batch, n, m, mat, scale_x, out, stream_arg(stream))


def gemm_scale_y(batch: int, n: int, m: int,
                 mat: DevicePointer,        # (batch, n, m) int32
                 scale_y: DevicePointer,    # (batch, m)    fp16
                 out: DevicePointer,        # (batch, n, m) fp16
                 stream: CUDAStream):
    """kernels/gemm.py:329-347."""
    cpmk.call("cpmk_gemm_scale_y", batch, n, m, mat, scale_y, out, stream_arg(stream))


# ---- fused forms (no counterpart function in the reference; each equals two of the calls above) ----

def gemm_quantize_rows(batch: int, n: int, m: int,
                       mat: DevicePointer,      # (b, n, m) fp16
                       scale: DevicePointer,    # (b, n)    fp16, written
                       out: DevicePointer,      # (b, n, m) int8, written
                       stream: CUDAStream):
    """gemm_calc_scale followed by gemm_round on the same tensor (torch/gemm.py:98-102), in one pass."""
    cpmk.call("cpmk_quantize_rows", batch, n, m, mat, scale, out, stream_arg(stream))


def gemm_quantize_cols(batch: int, n: int, m: int,
                       mat: DevicePointer,      # (b, n, m) fp16
                       scale: DevicePointer,    # (b, m)    fp16, written
                       out: DevicePointer,      # (b, n, m) int8, written
                       stream: CUDAStream):
    """gemm_calc_scale_transpose followed by gemm_round_transpose on the same tensor."""
    cpmk.call("cpmk_quantize_cols", batch, n, m, mat, scale, out, stream_arg(stream))


def gemm_quantize_rows_pair(batch0: int, n0: int, mat0: DevicePointer, scale0: DevicePointer, out0: DevicePointer,
                            batch1: int, n1: int, mat1: DevicePointer, scale1: DevicePointer, out1: DevicePointer,
                            m: int, stream: CUDAStream):
    """gemm_quantize_rows on two operands with rows of the same length m, (batch0, n0, m) and (batch1, n1, m), in one
    launch: the activations and the weight of a linear layer (torch/gemm.py:98-102 quantises them back to back)."""
    cpmk.call("cpmk_quantize_rows_pair", batch0, n0, mat0, scale0, out0, batch1, n1, mat1, scale1, out1, m, stream_arg(stream))


def gemm_int8_scale(m: int, k: int, n: int,
                    batchA: int, batchB: int,
                    aT: bool, bT: bool,
                    A: DevicePointer, B: DevicePointer,
                    scale_x: DevicePointer,    # (broad_cast_x ? 1 : batch, n) fp16
                    scale_y: DevicePointer,    # (broad_cast_y ? 1 : batch, m) fp16
                    broad_cast_x: bool, broad_cast_y: bool,
                    out: DevicePointer,        # (max(bA, bB), n, m) fp16
                    stream: CUDAStream):
    """gemm_int8 followed by gemm_scale (torch/gemm.py:45-64) without the int32 tensor in between."""
    assert m % 4 == 0 and n % 4 == 0 and k % 4 == 0
    assert batchA == batchB or batchA == 1 or batchB == 1
    cpmk.call("cpmk_gemm_int8_dequant", m, k, n, batchA, batchB, int(bool(aT)), int(bool(bT)), A, B, scale_x, scale_y,
              int(bool(broad_cast_x)), int(bool(broad_cast_y)), out, stream_arg(stream))


def gemm_int8_scale_gelu(m: int, k: int, n: int,
                         batchA: int, batchB: int,
                         aT: bool, bT: bool,
                         A: DevicePointer, B: DevicePointer,
                         scale_x: DevicePointer, scale_y: DevicePointer,
                         broad_cast_x: bool, broad_cast_y: bool,
                         out: DevicePointer,        # (max(bA, bB), n, m) fp16
                         stream: CUDAStream):
    """gemm_int8_scale followed by gelu_forward on its result in place (kernels/gelu.py:33-50), one call."""
    assert m % 4 == 0 and n % 4 == 0 and k % 4 == 0
    assert batchA == batchB or batchA == 1 or batchB == 1
    cpmk.call("cpmk_gemm_int8_dequant_gelu", m, k, n, batchA, batchB, int(bool(aT)), int(bool(bT)), A, B, scale_x, scale_y,
              int(bool(broad_cast_x)), int(bool(broad_cast_y)), out, stream_arg(stream))


def gemm_int8_scale_scatter(m: int, k: int, n: int,
                            batchA: int, batchB: int,
                            aT: bool, bT: bool,
                            A: DevicePointer, B: DevicePointer,
                            scale_x: DevicePointer, scale_y: DevicePointer,
                            broad_cast_x: bool, broad_cast_y: bool,
                            dst: list,               # device addresses of element (0, 0, 0) of each destination
                            dst_row_pitch: int,      # elements between rows of a destination (>= m)
                            stream: CUDAStream):
    """gemm_int8_scale whose result goes to several pitched destinations (this GPU's and its peers' output buffers):
    the output all-gather of a column-parallel linear, done by the GEMM's epilogue.  No counterpart in the reference."""
    import ctypes
    assert m % 4 == 0 and n % 4 == 0 and k % 4 == 0
    assert batchA == batchB or batchA == 1 or batchB == 1
    arr = dst if not isinstance(dst, (list, tuple)) else (ctypes.c_void_p * len(dst))(*dst)
    cpmk.call("cpmk_gemm_int8_dequant_scatter", m, k, n, batchA, batchB, int(bool(aT)), int(bool(bT)), A, B, scale_x, scale_y,
              int(bool(broad_cast_x)), int(bool(broad_cast_y)), len(dst), arr, dst_row_pitch, stream_arg(stream))


def gemm_quantize_rows_pair_scatter(n0: int, mat0: DevicePointer,
                                    scale_dst0: list,       # where the scales (n0) of these rows go in each destination
                                    q_dst0: list,           # where the codes (n0, m) of these rows go in each destination
                                    n1: int, mat1: DevicePointer, scale1: DevicePointer, out1: DevicePointer,
                                    m: int, stream: CUDAStream):
    """gemm_quantize_rows_pair whose first operand is written to several destinations (this GPU's code buffer and its
    peers'): the all-gather of row-sharded int8 activations, done by the stores of the quantisation pass.  ``n1`` may
    be 0 (no second operand).  No counterpart in the reference."""
    import ctypes
    assert len(scale_dst0) == len(q_dst0) and 1 <= len(q_dst0) <= 8
    sarr = (ctypes.c_void_p * len(scale_dst0))(*scale_dst0)
    qarr = (ctypes.c_void_p * len(q_dst0))(*q_dst0)
    cpmk.call("cpmk_quantize_rows_pair_scatter", n0, mat0, len(q_dst0), sarr, qarr, n1, mat1, scale1, out1, m, stream_arg(stream))


def linear_int8_scatter(tokens: int, k: int, n_local: int,
                        x: DevicePointer,          # (tokens, k)    fp16
                        w: DevicePointer,          # (n_local, k)   fp16: this rank's rows of the weight
                        scale_x: DevicePointer, q_x: DevicePointer, scale_w: DevicePointer, q_w: DevicePointer,   # written
                        dst,                       # ctypes array of device addresses, or a list of them
                        dst_row_pitch: int, stream: CUDAStream, multicast: bool = False):
    """One column-parallel int8 linear in one call: quantise x and w (one launch), GEMM + dequantisation stored to every
    destination (one launch).  Every buffer is the caller's.  torch/gemm.py:86-113 for the sharded layout."""
    import ctypes
    if isinstance(dst, (list, tuple)):
        dst = (ctypes.c_void_p * len(dst))(*dst)
    cpmk.call("cpmk_linear_int8_scatter", tokens, k, n_local, x, w, scale_x, q_x, scale_w, q_w, len(dst), dst, dst_row_pitch,
              int(bool(multicast)), stream_arg(stream))


def gemm_int8_scale_multicast(m: int, k: int, n: int, batchA: int, batchB: int, aT: bool, bT: bool,
                              A: DevicePointer, B: DevicePointer, scale_x: DevicePointer, scale_y: DevicePointer,
                              broad_cast_x: bool, broad_cast_y: bool,
                              dst_local: DevicePointer,        # this GPU's copy of the result slice
                              dst_multicast: DevicePointer,    # the same slice at the buffer's multicast address
                              dst_row_pitch: int, stream: CUDAStream):
    """gemm_int8_scale whose result goes to this GPU's buffer and, through one multimem store per 16 bytes that the NVLink
    switch replicates, to every GPU's copy of a multicast-mapped buffer.  No counterpart in the reference."""
    assert m % 4 == 0 and n % 4 == 0 and k % 4 == 0
    assert batchA == batchB or batchA == 1 or batchB == 1
    cpmk.call("cpmk_gemm_int8_dequant_multicast", m, k, n, batchA, batchB, int(bool(aT)), int(bool(bT)), A, B, scale_x, scale_y,
              int(bool(broad_cast_x)), int(bool(broad_cast_y)), dst_local, dst_multicast, dst_row_pitch, stream_arg(stream))
