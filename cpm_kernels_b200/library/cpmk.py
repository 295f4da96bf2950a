"""ctypes binding of ``libcpmk_b200.so`` (declared in ``include/cpmk_b200.h``).

Takes the place of cpm_kernels/library/cublaslt.py (the GEMM the reference delegates to cublasLt)
and of the fatbin loader cpm_kernels/kernels/base.py:15-71 (the reference launches its own kernels
with cuModuleLoadData + cuLaunchKernel; here the library launches them itself).  A non-zero status
becomes ``RuntimeError`` with the library's own message, as the reference does for CUDA and cuBLAS
statuses (library/cublaslt.py:96-100).
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_int32, c_uint32, c_void_p, POINTER

from .base import Lib

ABI_VERSION = 1

OK, EINVAL, EARCH, ECUDA, EDEVICE, ENOMEM = 0, 1, 2, 3, 4, 5

lib = Lib()

_i = c_int32
_p = c_void_p

# name -> argument types (every function returns int32 status unless noted)
SIGNATURES = {
    "cpmk_check_device": [POINTER(c_int32)],
    "cpmk_read_status": [POINTER(c_uint32)],
    "cpmk_check_stream": [_p],
    "cpmk_release_workspace": [_p],
    "cpmk_selftest_bounded_wait": [c_uint32, _p],
    "cpmk_quantize_rows_pair_scatter": [_i, _p, _i, POINTER(c_void_p), POINTER(c_void_p), _i, _p, _p, _p, _i, _p],
    "cpmk_linear_int8_scatter": [_i, _i, _i, _p, _p, _p, _p, _p, _p, _i, POINTER(c_void_p), ctypes.c_int64, _i, _p],
    "cpmk_gemm_int8_dequant_multicast": [_i, _i, _i, _i, _i, _i, _i, _p, _p, _p, _p, _i, _i, _p, _p, ctypes.c_int64, _p],
    "cpmk_gemm_calc_scale": [_i, _i, _i, _p, _p, _p],
    "cpmk_gemm_calc_scale_transpose": [_i, _i, _i, _p, _p, _p],
    "cpmk_gemm_round": [_i, _i, _i, _p, _p, _p, _p],
    "cpmk_gemm_round_transpose": [_i, _i, _i, _p, _p, _p, _p],
    "cpmk_quantize_rows": [_i, _i, _i, _p, _p, _p, _p],
    "cpmk_quantize_cols": [_i, _i, _i, _p, _p, _p, _p],
    "cpmk_gemm_scale": [_i, _i, _i, _p, _p, _p, _p, _i, _i, _p],
    "cpmk_gemm_scale_x": [_i, _i, _i, _p, _p, _p, _p],
    "cpmk_gemm_scale_y": [_i, _i, _i, _p, _p, _p, _p],
    "cpmk_gemm_backward_round_scale": [_i, _i, _i, _p, _p, _p, _p, _i, _p],
    "cpmk_gemm_backward_scale_round": [_i, _i, _i, _p, _p, _p, _p, _i, _p],
    "cpmk_gemm_int8": [_i, _i, _i, _i, _i, _i, _i, _p, _p, _p, _p],
    "cpmk_gemm_int8_dequant": [_i, _i, _i, _i, _i, _i, _i, _p, _p, _p, _p, _i, _i, _p, _p],
    "cpmk_gemm_int8_dequant_scatter": [_i, _i, _i, _i, _i, _i, _i, _p, _p, _p, _p, _i, _i, _i, POINTER(c_void_p), ctypes.c_int64, _p],
    "cpmk_quantize_rows_pair": [_i, _i, _p, _p, _p, _i, _i, _p, _p, _p, _i, _p],
    "cpmk_layernorm_quantize_cols": [_i, _i, _i, _p, ctypes.c_float, _i, _p, _p, _p, _p, _p],
    "cpmk_set_gemm_sm_margin": [_i],
    "cpmk_set_gemm_forward_sms": [_i],
    "cpmk_gelu_forward": [_i, _i, _p, _p, _p],
    "cpmk_gelu_backward": [_i, _i, _p, _p, _p, _p],
    "cpmk_transpose": [_i, _i, _i, _p, _p, _p],
    "cpmk_gemm_int8_dequant_gelu": [_i, _i, _i, _i, _i, _i, _i, _p, _p, _p, _p, _i, _i, _p, _p],
    "cpmk_gemm_fp16": [_i, _i, _i, _i, _i, _i, _i, _p, _p, _p, _p],
    "cpmk_gemv_fp16": [_i, _i, _i, _p, _p, _p, _p],
    "cpmk_gemv_fp16_transpose": [_i, _i, _i, _p, _p, _p, _p],
    "cpmk_gemv_fp16_transpose_noalloc": [_i, _i, _i, _p, _p, _p, _p],
    "cpmk_probe_read": [_i, _i, _i, _p, _p, _p],
    "cpmk_gemv_broadcast_mat_fp16": [_i, _i, _i, _p, _p, _p, _p],
    "cpmk_gemv_calc_scale": [_i, _i, _p, _p, _p],
    "cpmk_gemv_round": [_i, _i, _p, _p, _p, _p],
    "cpmk_gemv_broadcast_mat_int8": [_i, _i, _i, _p, _p, _p, _p, _p, _p],
}

for _name, _args in SIGNATURES.items():
    lib.bind(_name, _args, c_int32)
lib.bind("cpmk_abi_version", [], c_int32)
lib.bind("cpmk_last_error", [], c_char_p)
lib.bind("cpmk_last_gemm_path", [], c_int32)
lib.bind("cpmk_last_gemm_variant", [], c_int32)

if lib.cpmk_abi_version() != ABI_VERSION:
    raise RuntimeError("%s has ABI version %d, this package expects %d" % (lib.path, lib.cpmk_abi_version(), ABI_VERSION))


def last_error() -> str:
    msg = lib.cpmk_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def check_status(status: int, what: str) -> None:
    if status != OK:
        raise RuntimeError("%s failed (status %d): %s" % (what, status, last_error()))


def call(name: str, *args) -> None:
    """Call a status-returning entry point; raise RuntimeError on failure."""
    check_status(getattr(lib, name)(*args), name)


def check_device() -> int:
    """Compute capability (major*10+minor) of the current device; raises unless it is 10.x."""
    arch = c_int32(0)
    check_status(lib.cpmk_check_device(ctypes.byref(arch)), "cpmk_check_device")
    return arch.value


def read_status() -> int:
    """The bounded-wait status word of the current device (0 = no kernel gave up a wait); clears it.
    Synchronises the device."""
    word = c_uint32(0)
    check_status(lib.cpmk_read_status(ctypes.byref(word)), "cpmk_read_status")
    return word.value


def check_stream(stream) -> None:
    """Wait for ``stream``; raise RuntimeError (status CPMK_EDEVICE) if a kernel on it gave up a bounded wait."""
    call("cpmk_check_stream", stream)


def release_workspace(stream) -> None:
    """Free the library's workspace of (current device, ``stream``); call before destroying the stream."""
    call("cpmk_release_workspace", stream)


def set_gemm_sm_margin(sms: int) -> None:
    """Keep the persistent GEMM grid off ``sms`` SMs (0: use all; negative: follow CPMK_GEMM_SM_MARGIN)."""
    call("cpmk_set_gemm_sm_margin", int(sms))


def set_gemm_forward_sms(sms: int) -> None:
    """How many SMs of a scattering GEMM forward finished tiles to the other destinations (0: none; negative: default)."""
    call("cpmk_set_gemm_forward_sms", int(sms))


def last_gemm_variant() -> int:
    """1 = one-CTA tiles, 2 = CTA-pair tiles (cta_group::2), 0 = the generic kernel, for the last int8 GEMM of this thread."""
    return lib.cpmk_last_gemm_variant()


def last_gemm_path() -> int:
    """1 = tcgen05 kernel, 2 = generic kernel, for the last int8 GEMM issued by this thread."""
    return lib.cpmk_last_gemm_path()
