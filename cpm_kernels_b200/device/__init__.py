"""Current-device query.  Stands in for cpm_kernels/device/__init__.py:106-157 on this path: the
reference keeps one cublasLt handle per device and gates fp16 accumulation on ``architecture < 62``;
this package keeps its per-device state inside the C library and gates on ``architecture >= 100``."""
from ..library import cpmk


class Device:
    def __init__(self, architecture: int):
        self._architecture = architecture

    @property
    def architecture(self) -> int:
        """major * 10 + minor, as Device.architecture in the reference (device/__init__.py:143-145)."""
        return self._architecture


def current_device() -> Device:
    """The CUDA device current on this thread.  Raises RuntimeError unless it is compute capability 10.x."""
    return Device(cpmk.check_device())
