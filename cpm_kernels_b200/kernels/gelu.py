"""Launchers with the signatures of cpm_kernels/kernels/gelu.py (forward only: the activation that follows the
feed-forward block's first int8 linear)."""
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
