"""Launcher with the signature of cpm_kernels/kernels/transpose.py."""
from .base import DevicePointer, CUDAStream, stream_arg
from ..library import cpmk


def transpose(batch: int, n: int, m: int,
              inp: DevicePointer,    # (batch, n, m) fp16
              out: DevicePointer,    # (batch, m, n) fp16
              stream: CUDAStream):
    """kernels/transpose.py:11-27."""
    cpmk.call("cpmk_transpose", batch, n, m, inp, out, stream_arg(stream))
