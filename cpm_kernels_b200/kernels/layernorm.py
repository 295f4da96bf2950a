"""Launcher of the fused layer norm -> affine -> column quantisation (no single counterpart in the reference, which
runs kernels/layernorm.py:18-38, kernels/arith.py:134-215 and kernels/gemm.py:43-63, 109-125 one after another)."""
from .base import DevicePointer, CUDAStream, stream_arg
from ..library import cpmk


def layernorm_quantize_cols(batch: int, n: int, m: int,
                            mat: DevicePointer,        # (batch, n, m) fp16
                            eps: float, rd_mean: bool,
                            alpha: DevicePointer,      # (n) fp16
                            beta: DevicePointer,       # (n) fp16, or 0 for the multiply-only form
                            scale_out: DevicePointer,  # (batch, m) fp16
                            q_out: DevicePointer,      # (batch, n, m) int8
                            stream: CUDAStream):
    """q, scale = quantise_cols(affine(layernorm(mat))) with the layer norm over the middle axis n."""
    assert m % 8 == 0
    cpmk.call("cpmk_layernorm_quantize_cols", batch, n, m, mat, float(eps), int(bool(rd_mean)), alpha, beta or None, scale_out, q_out,
              stream_arg(stream))
