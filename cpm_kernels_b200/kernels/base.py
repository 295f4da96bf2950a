"""Types shared by the launchers (cpm_kernels/kernels/base.py:7-13)."""
import ctypes

DevicePointer = int            # raw device address, e.g. torch.Tensor.data_ptr()
CUDAStream = ctypes.c_void_p   # cudaStream_t value, e.g. torch.cuda.current_stream().cuda_stream


def round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


def stream_arg(stream) -> ctypes.c_void_p:
    """Accept an int, None or a ctypes pointer for the stream, as the reference's callers pass them."""
    if isinstance(stream, ctypes.c_void_p):
        return stream
    return ctypes.c_void_p(stream or 0)
