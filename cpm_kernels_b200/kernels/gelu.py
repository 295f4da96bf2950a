"""Launchers with the signatures of cpm_kernels/kernels/gelu.py: the activation that follows the feed-forward block's
first int8 linear, and its backward pass."""
from .base import DevicePointer, CUDAStream, stream_arg
from ..library import cpmk


def gelu_forward(batch: int, n: int,
                 mat: DevicePointer,    # (batch, n) fp16
                 out: DevicePointer,    # (batch, n) fp16
                 stream: CUDAStream):
    """kernels/gelu.py:14-31."""
    cpmk.call("cpmk_gelu_forward", batch, n, mat, out, stream_arg(stream))


def gelu_inplace_forward(batch: int, n: int,
                         mat: DevicePointer,    # (batch, n) fp16, overwritten
                         stream: CUDAStream):
    """kernels/gelu.py:33-50."""
    cpmk.call("cpmk_gelu_forward", batch, n, mat, mat, stream_arg(stream))


def gelu_backward(batch: int, n: int,
                  grad_out: DevicePointer,   # (batch, n) fp16
                  mat: DevicePointer,        # (batch, n) fp16: the forward pass's input
                  grad: DevicePointer,       # (batch, n) fp16, written
                  stream: CUDAStream):
    """kernels/gelu.py:50-69.  grad = gelu'(mat) * grad_out."""
    cpmk.call("cpmk_gelu_backward", batch, n, grad_out, mat, grad, stream_arg(stream))
