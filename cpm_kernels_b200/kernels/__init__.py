"""Flat namespace of launchers, as cpm_kernels/kernels/__init__.py:3-5 re-exports them."""
from .base import DevicePointer, CUDAStream, round_up
from .gemm import (gemm_calc_scale, gemm_calc_scale_transpose, gemm_round, gemm_round_transpose, gemm_scale,
                   gemm_int8, gemm_fp16, gemm_backward_round_scale, gemm_backward_scale_round, gemm_scale_x, gemm_scale_y,
                   gemm_quantize_rows, gemm_quantize_rows_pair, gemm_quantize_cols, gemm_int8_scale, gemm_int8_scale_gelu, gemm_int8_scale_scatter,
                   gemm_quantize_rows_pair_scatter, linear_int8_scatter, gemm_int8_scale_multicast)
from .gelu import gelu_forward, gelu_inplace_forward, gelu_backward
from .layernorm import layernorm_quantize_cols
from .transpose import transpose
from .gemv import (gemv_fp16, gemv_fp16_light, gemv_fp16_transpose, gemv_fp16_transpose_light,
                   gemv_broadcast_mat_fp16, gemv_broadcast_mat_fp16_light, gemv_calc_scale, gemv_round,
                   gemv_broadcast_mat_int8)
