"""The C-ABI library loads without a GPU and exports exactly what include/cpmk_b200.h declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "cpmk_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cpmk_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_path():
    syms = declared_symbols()
    for must in ("cpmk_gemm_calc_scale", "cpmk_gemm_calc_scale_transpose", "cpmk_gemm_round", "cpmk_gemm_round_transpose",
                 "cpmk_gemm_int8", "cpmk_gemm_scale", "cpmk_gemv_fp16", "cpmk_gemv_fp16_transpose",
                 "cpmk_quantize_rows", "cpmk_quantize_cols", "cpmk_gemm_int8_dequant"):
        assert must in syms


def test_library_exports_every_declared_symbol(built_library):
    lib = ctypes.CDLL(built_library)
    missing = [s for s in declared_symbols() if not hasattr(lib, s)]
    assert not missing, missing
    lib.cpmk_abi_version.restype = ctypes.c_int32
    assert lib.cpmk_abi_version() == 1


def test_python_binding_covers_every_declared_symbol(built_library):
    from cpm_kernels_b200.library import cpmk
    bound = set(cpmk.SIGNATURES) | {"cpmk_abi_version", "cpmk_last_error", "cpmk_last_gemm_path", "cpmk_last_gemm_variant"}
    assert sorted(bound) == declared_symbols()


def test_argument_counts_match_the_header(built_library):
    from cpm_kernels_b200.library import cpmk
    text = open(os.path.join(ROOT, "include", "cpmk_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    for name, args in cpmk.SIGNATURES.items():
        m = re.search(r"\b%s\s*\((.*?)\)\s*;" % name, text, flags=re.S)
        assert m, name
        params = [p for p in m.group(1).split(",") if p.strip() and p.strip() != "void"]
        assert len(params) == len(args), (name, len(params), len(args))


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from cpm_kernels_b200.library import base
    monkeypatch.setenv(base.ENV_LIB, str(tmp_path / "nope.so"))
    try:
        base.find_library()
    except RuntimeError as e:
        assert "no CPU fallback" in str(e)
    else:
        raise AssertionError("expected RuntimeError")


def test_calls_without_a_gpu_report_an_error_instead_of_computing(built_library):
    import torch
    if torch.cuda.is_available():
        return
    from cpm_kernels_b200.library import cpmk
    try:
        cpmk.check_device()
    except RuntimeError as e:
        assert "cpmk_check_device" in str(e)
    else:
        raise AssertionError("expected RuntimeError without a CUDA device")


def test_kernel_level_preconditions_are_the_references(built_library):
    # kernels/gemm.py:139-140: m, n, k multiples of 4; batches equal or 1 -- AssertionError before any CUDA call
    import pytest
    import cpm_kernels_b200.kernels as ck
    with pytest.raises(AssertionError):
        ck.gemm_int8(6, 8, 8, 1, 1, True, False, 0, 0, 0, 0)
    with pytest.raises(AssertionError):
        ck.gemm_int8(8, 8, 8, 2, 3, True, False, 0, 0, 0, 0)
    with pytest.raises(AssertionError):
        ck.gemv_broadcast_mat_int8(1, 8, 6, 0, 0, 0, 0, 0, 0)


def test_kernel_modules_are_built_and_export_the_reference_symbols():
    """lib/gemm.fatbin, lib/gemv.fatbin and lib/transpose.fatbin exist after a build, and their sources define every kernel name the
    reference's loader looks up (cpm_kernels/kernels/gemm.py:6-19, kernels/gemv.py:6-16, kernels/transpose.py:4-9)."""
    import os
    import re
    from cpm_kernels_b200 import build
    build.build_library()
    names = {
        "gemm": ["cu_gemm_round", "cu_gemm_round_transpose", "cu_gemm_scale", "cu_gemm_calc_scale", "cu_gemm_calc_scale_transpose",
                 "cu_gemm_backward_round_scale", "cu_gemm_backward_scale_round", "cu_gemm_scale_x", "cu_gemm_scale_y"],
        "gemv": ["cu_gemv_calc_scale", "cu_gemv_round", "cu_gemv_broadcast_mat_int8", "cu_gemv_fp16", "cu_gemv_fp16_transpose",
                 "cu_gemv_broadcast_mat_fp16"],
        "transpose": ["cu_transpose"],
    }
    for mod, kernels in names.items():
        assert os.path.getsize(build.module_path(mod)) > 0
        src = open(os.path.join(build.CSRC, "modules", build.MODULES[mod])).read()
        for k in kernels:
            assert re.search(r'extern "C" __global__ void %s\(' % k, src), k
