"""Launchers of the decode GEMV family, with the signatures of cpm_kernels/kernels/gemv.py.

The reference has two implementations of each fp16 GEMV: a cublasLt n=1 GEMM (``gemv_fp16``) and its own
kernel (``gemv_fp16_light``).  Here both names reach the same kernel, which accumulates in fp32."""
from ..library import cpmk
from .base import DevicePointer, CUDAStream, stream_arg


def gemv_calc_scale(batch: int, n: int,
                    vec: DevicePointer,    # (batch, n) fp16
                    out: DevicePointer,    # (batch,)   fp16
                    stream: CUDAStream):
    """kernels/gemv.py:18-33."""
    cpmk.call("cpmk_gemv_calc_scale", batch, n, vec, out, stream_arg(stream))


def gemv_round(batch: int, n: int,
               vec: DevicePointer,      # (batch, n) fp16
               scale: DevicePointer,    # (batch,)   fp16
               out: DevicePointer,      # (batch, n) int8
               stream: CUDAStream):
    """kernels/gemv.py:35-53."""
    cpmk.call("cpmk_gemv_round", batch, n, vec, scale, out, stream_arg(stream))


def gemv_broadcast_mat_int8(batch: int, dim_out: int, dim_in: int,
                            scale_mat: DevicePointer,    # (dim_out,)        fp16
                            mat: DevicePointer,          # (dim_out, dim_in) int8
                            scale_vec: DevicePointer,    # (batch,)          fp16
                            vec: DevicePointer,          # (batch, dim_in)   int8
                            out: DevicePointer,          # (batch, dim_out)  fp16
                            stream: CUDAStream):
    """kernels/gemv.py:56-79."""
    assert dim_in % 4 == 0
    cpmk.call("cpmk_gemv_broadcast_mat_int8", batch, dim_out, dim_in, scale_mat, mat, scale_vec, vec, out, stream_arg(stream))


def gemv_fp16(batch: int, dim_out: int, dim_in: int,
              mat: DevicePointer,    # (batch, dim_out, dim_in) fp16
              vec: DevicePointer,    # (batch, dim_in)          fp16
              out: DevicePointer,    # (batch, dim_out)         fp16
              stream: CUDAStream):
    """kernels/gemv.py:82-127.  out[b, o] = sum_i mat[b, o, i] * vec[b, i]."""
    cpmk.call("cpmk_gemv_fp16", batch, dim_out, dim_in, mat, vec, out, stream_arg(stream))


def gemv_fp16_light(batch: int, dim_out: int, dim_in: int, mat: DevicePointer, vec: DevicePointer, out: DevicePointer,
                    stream: CUDAStream):
    """kernels/gemv.py:129-148."""
    assert dim_in % 2 == 0
    gemv_fp16(batch, dim_out, dim_in, mat, vec, out, stream)


def gemv_fp16_transpose(batch: int, dim_out: int, dim_in: int,
                        mat: DevicePointer,    # (batch, dim_in, dim_out) fp16
                        vec: DevicePointer,    # (batch, dim_in)          fp16
                        out: DevicePointer,    # (batch, dim_out)         fp16
                        stream: CUDAStream):
    """kernels/gemv.py:151-196.  out[b, o] = sum_i mat[b, i, o] * vec[b, i]."""
    cpmk.call("cpmk_gemv_fp16_transpose", batch, dim_out, dim_in, mat, vec, out, stream_arg(stream))


def gemv_fp16_transpose_light(batch: int, dim_out: int, dim_in: int, mat: DevicePointer, vec: DevicePointer, out: DevicePointer,
                              stream: CUDAStream):
    """kernels/gemv.py:198-216."""
    gemv_fp16_transpose(batch, dim_out, dim_in, mat, vec, out, stream)


def gemv_broadcast_mat_fp16(batch: int, dim_out: int, dim_in: int,
                            mat: DevicePointer,    # (dim_out, dim_in) fp16, shared by the batch
                            vec: DevicePointer,    # (batch, dim_in)
                            out: DevicePointer,    # (batch, dim_out)
                            stream: CUDAStream):
    """kernels/gemv.py:218-262."""
    cpmk.call("cpmk_gemv_broadcast_mat_fp16", batch, dim_out, dim_in, mat, vec, out, stream_arg(stream))


def gemv_broadcast_mat_fp16_light(batch: int, dim_out: int, dim_in: int, mat: DevicePointer, vec: DevicePointer, out: DevicePointer,
                                  stream: CUDAStream):
    """kernels/gemv.py:264-283."""
    assert dim_in % 2 == 0
    gemv_broadcast_mat_fp16(batch, dim_out, dim_in, mat, vec, out, stream)
