"""TEST INFRASTRUCTURE ONLY -- runs the *reference's own* device code on the GPU.

``oracle/Makefile`` (target ``ref``) compiles the reference's unmodified ``cuda/gemm.cu`` and
``cuda/gemv.cu`` for sm_100 into ``oracle/_ref/*.fatbin``.  This module loads those fatbins with the
driver API and launches their kernels with the launch shapes the reference's Python launchers use
(cited per function), and reproduces the reference's cublasLt call sequence for the int8 GEMM.  It is
what pins the CPU restatements: ``tests/golden/make_golden.py`` records its outputs on seeded inputs,
and the GPU tests compare this package's kernels with it directly.

It is never imported by the shipped package.
"""
from __future__ import annotations

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(_HERE, "_ref")


def available() -> bool:
    return os.path.exists(os.path.join(REF_DIR, "gemm.fatbin")) and os.path.exists(os.path.join(REF_DIR, "gemv.fatbin"))


def _round_up(x, m):
    return (x + m - 1) // m * m


class _Driver:
    def __init__(self):
        self.lib = ctypes.CDLL("libcuda.so.1")
        self.lib.cuModuleLoadData.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p]
        self.lib.cuModuleGetFunction.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p, ctypes.c_char_p]
        self.lib.cuLaunchKernel.argtypes = [ctypes.c_void_p] + [ctypes.c_uint] * 6 + [ctypes.c_uint, ctypes.c_void_p,
                                                                                      ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p]

    def check(self, status, what):
        if status != 0:
            raise RuntimeError("%s failed with CUresult %d" % (what, status))

    def load(self, image: bytes):
        mod = ctypes.c_void_p()
        buf = ctypes.create_string_buffer(image, len(image))
        self.check(self.lib.cuModuleLoadData(ctypes.byref(mod), buf), "cuModuleLoadData")
        return mod

    def function(self, mod, name: str):
        fn = ctypes.c_void_p()
        self.check(self.lib.cuModuleGetFunction(ctypes.byref(fn), mod, name.encode()), "cuModuleGetFunction(%s)" % name)
        return fn

    def launch(self, fn, grid, block, stream, params):
        # cpm_kernels/library/cuda.py:249-267: params is an array of pointers to the argument values
        arr = (ctypes.c_void_p * len(params))(*[ctypes.addressof(p) for p in params])
        self.check(self.lib.cuLaunchKernel(fn, grid[0], grid[1], grid[2], block[0], block[1], block[2], 0,
                                           ctypes.c_void_p(stream), arr, None), "cuLaunchKernel")


class ReferenceKernels:
    """The reference's quantisation / GEMV kernels, compiled from its sources, on the current device."""

    def __init__(self, fatbin_dir: str = None):
        """``fatbin_dir``: where ``gemm.fatbin`` / ``gemv.fatbin`` are read from.  Default: the reference's own
        device code in ``oracle/_ref``.  Tests also point it at this package's kernel modules, which export the
        same symbols, to run them under the reference's launch shapes."""
        if fatbin_dir is None:
            if not available():
                raise RuntimeError("oracle/_ref/*.fatbin not built (run `make -C oracle ref` where the reference checkout is)")
            fatbin_dir = REF_DIR
        torch.cuda.init()
        torch.zeros(1, device="cuda")       # make the primary context current
        self.drv = _Driver()
        self._fns = {}
        for name in ("gemm", "gemv", "gelu", "layernorm", "arith", "transpose"):
            path = os.path.join(fatbin_dir, name + ".fatbin")
            if name not in ("gemm", "gemv") and not os.path.exists(path):
                continue                                  # only needed by the functions of that file
            with open(path, "rb") as f:
                setattr(self, "_mod_" + name, self.drv.load(f.read()))

    def _fn(self, mod, name):
        if name not in self._fns:
            self._fns[name] = self.drv.function(getattr(self, "_mod_" + mod), name)
        return self._fns[name]

    @staticmethod
    def _stream():
        return torch.cuda.current_stream().cuda_stream

    @staticmethod
    def _i(v):
        return ctypes.c_int32(v)

    @staticmethod
    def _p(t: torch.Tensor):
        return ctypes.c_void_p(t.data_ptr())

    # ---- cpm_kernels/kernels/gemm.py -------------------------------------------------------------
    def gemm_calc_scale(self, mat: torch.Tensor) -> torch.Tensor:
        """kernels/gemm.py:91-107: grid (batch, n), block min(round_up(m, 32), 1024)."""
        b, n, m = mat.shape
        out = torch.empty((b, n), dtype=torch.half, device=mat.device)
        self.drv.launch(self._fn("gemm", "cu_gemm_calc_scale"), (b, n, 1), (min(_round_up(m, 32), 1024), 1, 1), self._stream(),
                        [self._i(b), self._i(n), self._i(m), self._p(mat), self._p(out)])
        return out

    def gemm_calc_scale_transpose(self, mat: torch.Tensor) -> torch.Tensor:
        """kernels/gemm.py:109-125: grid (batch, round_up(m, 32) / 32), block (32, 32)."""
        b, n, m = mat.shape
        out = torch.empty((b, m), dtype=torch.half, device=mat.device)
        self.drv.launch(self._fn("gemm", "cu_gemm_calc_scale_transpose"), (b, _round_up(m, 32) // 32, 1), (32, 32, 1), self._stream(),
                        [self._i(b), self._i(n), self._i(m), self._p(mat), self._p(out)])
        return out

    def gemm_round(self, mat: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
        """kernels/gemm.py:21-41: grid (batch, n), block min(m, 1024)."""
        b, n, m = mat.shape
        out = torch.empty((b, n, m), dtype=torch.int8, device=mat.device)
        self.drv.launch(self._fn("gemm", "cu_gemm_round"), (b, n, 1), (min(m, 1024), 1, 1), self._stream(),
                        [self._i(b), self._i(n), self._i(m), self._p(mat), self._p(scale), self._p(out)])
        return out

    def gemm_round_transpose(self, mat: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
        """kernels/gemm.py:43-63: grid (batch, n), block min(m, 1024)."""
        b, n, m = mat.shape
        out = torch.empty((b, n, m), dtype=torch.int8, device=mat.device)
        self.drv.launch(self._fn("gemm", "cu_gemm_round_transpose"), (b, n, 1), (min(m, 1024), 1, 1), self._stream(),
                        [self._i(b), self._i(n), self._i(m), self._p(mat), self._p(scale), self._p(out)])
        return out

    def gemm_scale(self, mat: torch.Tensor, scale_x: torch.Tensor, scale_y: torch.Tensor, bx: bool, by: bool) -> torch.Tensor:
        """kernels/gemm.py:65-89: grid (batch, n), block min(m, 1024)."""
        b, n, m = mat.shape
        out = torch.empty((b, n, m), dtype=torch.half, device=mat.device)
        self.drv.launch(self._fn("gemm", "cu_gemm_scale"), (b, n, 1), (min(m, 1024), 1, 1), self._stream(),
                        [self._i(b), self._i(n), self._i(m), self._p(mat), self._p(scale_x), self._p(scale_y), self._p(out),
                         ctypes.c_bool(bx), ctypes.c_bool(by)])
        return out

    def gemm_backward_round_scale(self, mat, scale_y, by: bool):
        """kernels/gemm.py:261-283: grid (batch, n), block min(round_up(m, 32), 1024)."""
        b, n, m = mat.shape
        out = torch.empty((b, n, m), dtype=torch.int8, device=mat.device)
        scale_x = torch.empty((b, n), dtype=torch.half, device=mat.device)
        self.drv.launch(self._fn("gemm", "cu_gemm_backward_round_scale"), (b, n, 1), (min(_round_up(m, 32), 1024), 1, 1), self._stream(),
                        [self._i(b), self._i(n), self._i(m), self._p(mat), self._p(scale_y), self._p(out), self._p(scale_x), ctypes.c_bool(by)])
        return out, scale_x

    def gemm_backward_scale_round(self, mat, scale_x, bx: bool):
        """kernels/gemm.py:285-307: grid (batch, round_up(m, 32) / 32), block (32, 32)."""
        b, n, m = mat.shape
        out = torch.empty((b, n, m), dtype=torch.int8, device=mat.device)
        scale_y = torch.empty((b, m), dtype=torch.half, device=mat.device)
        self.drv.launch(self._fn("gemm", "cu_gemm_backward_scale_round"), (b, _round_up(m, 32) // 32, 1), (32, 32, 1), self._stream(),
                        [self._i(b), self._i(n), self._i(m), self._p(mat), self._p(scale_x), self._p(out), self._p(scale_y), ctypes.c_bool(bx)])
        return out, scale_y

    def gemm_scale_x(self, mat: torch.Tensor, scale_x: torch.Tensor) -> torch.Tensor:
        """kernels/gemm.py:309-326: grid (batch, n), block min(m, 1024)."""
        b, n, m = mat.shape
        out = torch.empty((b, n, m), dtype=torch.half, device=mat.device)
        self.drv.launch(self._fn("gemm", "cu_gemm_scale_x"), (b, n, 1), (min(m, 1024), 1, 1), self._stream(),
                        [self._i(b), self._i(n), self._i(m), self._p(mat), self._p(scale_x), self._p(out)])
        return out

    def gemm_scale_y(self, mat: torch.Tensor, scale_y: torch.Tensor) -> torch.Tensor:
        """kernels/gemm.py:329-347: grid (batch, n), block min(m, 1024)."""
        b, n, m = mat.shape
        out = torch.empty((b, n, m), dtype=torch.half, device=mat.device)
        self.drv.launch(self._fn("gemm", "cu_gemm_scale_y"), (b, n, 1), (min(m, 1024), 1, 1), self._stream(),
                        [self._i(b), self._i(n), self._i(m), self._p(mat), self._p(scale_y), self._p(out)])
        return out

    # ---- cpm_kernels/kernels/gelu.py -------------------------------------------------------------
    def gelu_forward(self, mat: torch.Tensor) -> torch.Tensor:
        """kernels/gelu.py:14-31: threads = min(round_up(n, 32), 1024); grid (batch, round_up(n, threads) / threads)."""
        b, n = mat.shape
        out = torch.empty_like(mat)
        threads = min(_round_up(n, 32), 1024)
        self.drv.launch(self._fn("gelu", "cu_gelu_forward"), (b, _round_up(n, threads) // threads, 1), (threads, 1, 1), self._stream(),
                        [self._i(b), self._i(n), self._p(mat), self._p(out)])
        return out

    def gelu_backward(self, grad_out: torch.Tensor, mat: torch.Tensor) -> torch.Tensor:
        """kernels/gelu.py:50-69: the launch shape of gelu_forward."""
        b, n = mat.shape
        grad = torch.empty_like(mat)
        threads = min(_round_up(n, 32), 1024)
        self.drv.launch(self._fn("gelu", "cu_gelu_backward"), (b, _round_up(n, threads) // threads, 1), (threads, 1, 1), self._stream(),
                        [self._i(b), self._i(n), self._p(grad_out), self._p(mat), self._p(grad)])
        return grad

    # ---- cpm_kernels/kernels/transpose.py --------------------------------------------------------
    def transpose(self, mat: torch.Tensor) -> torch.Tensor:
        """kernels/transpose.py:11-27: grid (batch, round_up(n, 32) / 32, round_up(m, 32) / 32), block (32, 32)."""
        b, n, m = mat.shape
        out = torch.empty((b, m, n), dtype=torch.half, device=mat.device)
        self.drv.launch(self._fn("transpose", "cu_transpose"), (b, _round_up(n, 32) // 32, _round_up(m, 32) // 32), (32, 32, 1), self._stream(),
                        [self._i(b), self._i(n), self._i(m), self._p(mat), self._p(out)])
        return out

    # ---- cpm_kernels/kernels/layernorm.py, arith.py ----------------------------------------------
    def layernorm_forward(self, mat: torch.Tensor, eps: float, rd_mean: bool) -> torch.Tensor:
        """kernels/layernorm.py:18-38: grid (batch, round_up(m, 32) / 32), block (32, 32)."""
        b, n, m = mat.shape
        out = torch.empty_like(mat)
        self.drv.launch(self._fn("layernorm", "cu_layernorm_forward"), (b, _round_up(m, 32) // 32, 1), (32, 32, 1), self._stream(),
                        [self._i(b), self._i(n), self._i(m), self._p(mat), self._p(out), ctypes.c_float(eps), ctypes.c_bool(rd_mean)])
        return out

    def arith_ln_mul(self, x: torch.Tensor, alpha: torch.Tensor) -> torch.Tensor:
        """kernels/arith.py:188-215: m halved (half2 elements); threads = min(round_up(m, 32), 1024); grid (batch, n, round_up(m, threads) / threads)."""
        b, n, m = x.shape
        assert m % 2 == 0
        out = torch.empty_like(x)
        m2 = m // 2
        threads = min(_round_up(m2, 32), 1024)
        self.drv.launch(self._fn("arith", "cu_arith_ln_mul"), (b, n, _round_up(m2, threads) // threads), (threads, 1, 1), self._stream(),
                        [ctypes.c_int64(b), ctypes.c_int64(n), ctypes.c_int64(m2), self._p(x), self._p(alpha), self._p(out)])
        return out

    def arith_ln_mul_add(self, x: torch.Tensor, alpha: torch.Tensor, beta: torch.Tensor) -> torch.Tensor:
        """kernels/arith.py:134-161: as arith_ln_mul with a per-row addend."""
        b, n, m = x.shape
        assert m % 2 == 0
        out = torch.empty_like(x)
        m2 = m // 2
        threads = min(_round_up(m2, 32), 1024)
        self.drv.launch(self._fn("arith", "cu_arith_ln_mul_add"), (b, n, _round_up(m2, threads) // threads), (threads, 1, 1), self._stream(),
                        [ctypes.c_int64(b), ctypes.c_int64(n), ctypes.c_int64(m2), self._p(x), self._p(alpha), self._p(beta), self._p(out)])
        return out

    # ---- cpm_kernels/kernels/gemv.py -------------------------------------------------------------
    def gemv_calc_scale(self, vec: torch.Tensor) -> torch.Tensor:
        """kernels/gemv.py:18-35: grid (batch,), block min(1024, round_up(n, 32))."""
        b, n = vec.shape
        out = torch.empty((b,), dtype=torch.half, device=vec.device)
        self.drv.launch(self._fn("gemv", "cu_gemv_calc_scale"), (b, 1, 1), (min(1024, _round_up(n, 32)), 1, 1), self._stream(),
                        [self._i(b), self._i(n), self._p(vec), self._p(out)])
        return out

    def gemv_round(self, vec: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
        """kernels/gemv.py:37-54: threads = min(1024, round_up(n, 32)); grid (batch, round_up(n, threads) / threads)."""
        b, n = vec.shape
        out = torch.empty((b, n), dtype=torch.int8, device=vec.device)
        threads = min(1024, _round_up(n, 32))
        self.drv.launch(self._fn("gemv", "cu_gemv_round"), (b, _round_up(n, threads) // threads, 1), (threads, 1, 1), self._stream(),
                        [self._i(b), self._i(n), self._p(vec), self._p(scale), self._p(out)])
        return out

    def gemv_fp16_light(self, mat: torch.Tensor, vec: torch.Tensor) -> torch.Tensor:
        """kernels/gemv.py:129-148: grid (batch, dim_out), block min(1024, round_up(dim_in / 2, 32))."""
        b, o, i = mat.shape
        out = torch.empty((b, o), dtype=torch.half, device=mat.device)
        self.drv.launch(self._fn("gemv", "cu_gemv_fp16"), (b, o, 1), (min(1024, _round_up(i // 2, 32)), 1, 1), self._stream(),
                        [self._i(b), self._i(o), self._i(i), self._p(mat), self._p(vec), self._p(out)])
        return out

    def gemv_fp16_transpose_light(self, mat: torch.Tensor, vec: torch.Tensor) -> torch.Tensor:
        """kernels/gemv.py:198-216: grid (batch, round_up(dim_out, 32) / 32), block (32, 32)."""
        b, i, o = mat.shape
        out = torch.empty((b, o), dtype=torch.half, device=mat.device)
        self.drv.launch(self._fn("gemv", "cu_gemv_fp16_transpose"), (b, _round_up(o, 32) // 32, 1), (32, 32, 1), self._stream(),
                        [self._i(b), self._i(o), self._i(i), self._p(mat), self._p(vec), self._p(out)])
        return out

    def gemv_broadcast_mat_fp16_light(self, mat: torch.Tensor, vec: torch.Tensor) -> torch.Tensor:
        """kernels/gemv.py:264-283: grid (batch, dim_out), block min(1024, round_up(dim_in / 2, 32))."""
        o, i = mat.shape
        b = vec.shape[0]
        out = torch.empty((b, o), dtype=torch.half, device=mat.device)
        self.drv.launch(self._fn("gemv", "cu_gemv_broadcast_mat_fp16"), (b, o, 1), (min(1024, _round_up(i // 2, 32)), 1, 1), self._stream(),
                        [self._i(b), self._i(o), self._i(i), self._p(mat), self._p(vec), self._p(out)])
        return out

    def gemv_broadcast_mat_int8(self, scale_mat, mat, scale_vec, vec) -> torch.Tensor:
        """kernels/gemv.py:56-79: grid (batch, dim_out), block min(1024, round_up(dim_in / 4, 32))."""
        o, i = mat.shape
        b = vec.shape[0]
        out = torch.empty((b, o), dtype=torch.half, device=mat.device)
        self.drv.launch(self._fn("gemv", "cu_gemv_broadcast_mat_int8"), (b, o, 1), (min(1024, _round_up(i // 4, 32)), 1, 1), self._stream(),
                        [self._i(b), self._i(o), self._i(i), self._p(scale_mat), self._p(mat), self._p(scale_vec), self._p(vec), self._p(out)])
        return out


class ReferenceCublasLt:
    """The reference's int8 GEMM: the cublasLt call sequence of cpm_kernels/kernels/gemm.py:127-186 with the
    bindings of cpm_kernels/library/cublaslt.py (plain column-major layouts, CUBLAS_COMPUTE_32I, no workspace,
    heuristic algorithm).  Descriptors are created and destroyed per call, as the reference does."""

    CUDA_R_8I, CUDA_R_32I = 3, 10                     # library/cublaslt.py:7-19
    COMPUTE_32I = 72                                  # library/cublaslt.py:21-33 (CUBLAS_COMPUTE_32I)
    ATTR_BATCH_COUNT, ATTR_BATCH_OFFSET = 5, 6        # CUBLASLT_MATRIX_LAYOUT_BATCH_COUNT / STRIDED_BATCH_OFFSET
    DESC_TRANSA, DESC_TRANSB = 3, 4                   # CUBLASLT_MATMUL_DESC_TRANSA / TRANSB
    OP_T = 1

    def __init__(self):
        path = None
        for cand in ("/usr/local/cuda/lib64/libcublasLt.so", "libcublasLt.so.12", "libcublasLt.so"):
            try:
                self.lib = ctypes.CDLL(cand)
                path = cand
                break
            except OSError:
                continue
        if path is None:
            raise RuntimeError("libcublasLt not found")
        self.handle = ctypes.c_void_p()
        self._check(self.lib.cublasLtCreate(ctypes.byref(self.handle)), "cublasLtCreate")

    @staticmethod
    def _check(status, what):
        if status != 0:
            raise RuntimeError("%s failed with cublasStatus %d" % (what, status))

    def _layout(self, dtype, rows, cols, ld, batch, stride):
        lay = ctypes.c_void_p()
        self._check(self.lib.cublasLtMatrixLayoutCreate(ctypes.byref(lay), ctypes.c_int(dtype), ctypes.c_uint64(rows),
                                                         ctypes.c_uint64(cols), ctypes.c_int64(ld)), "cublasLtMatrixLayoutCreate")
        bc = ctypes.c_int32(batch)
        st = ctypes.c_int64(stride)
        self._check(self.lib.cublasLtMatrixLayoutSetAttribute(lay, self.ATTR_BATCH_COUNT, ctypes.byref(bc), ctypes.c_size_t(4)), "set batch count")
        self._check(self.lib.cublasLtMatrixLayoutSetAttribute(lay, self.ATTR_BATCH_OFFSET, ctypes.byref(st), ctypes.c_size_t(8)), "set batch stride")
        return lay

    def gemm_int8(self, m, k, n, batchA, batchB, aT, bT, A: torch.Tensor, B: torch.Tensor, out: torch.Tensor):
        """Arguments as kernels/gemm.py:127-135; A, B int8, out int32 (max(bA, bB), n, m)."""
        batchC = max(batchA, batchB)
        layA = self._layout(self.CUDA_R_8I, k if aT else m, m if aT else k, k if aT else m, batchC, 0 if batchA == 1 else m * k)
        layB = self._layout(self.CUDA_R_8I, n if bT else k, k if bT else n, n if bT else k, batchC, 0 if batchB == 1 else n * k)
        layC = self._layout(self.CUDA_R_32I, m, n, m, batchC, m * n)
        desc = ctypes.c_void_p()
        self._check(self.lib.cublasLtMatmulDescCreate(ctypes.byref(desc), ctypes.c_int(self.COMPUTE_32I), ctypes.c_int(self.CUDA_R_32I)),
                    "cublasLtMatmulDescCreate")
        op_t = ctypes.c_int32(self.OP_T)
        try:
            if aT:
                self._check(self.lib.cublasLtMatmulDescSetAttribute(desc, self.DESC_TRANSA, ctypes.byref(op_t), ctypes.c_size_t(4)), "set transa")
            if bT:
                self._check(self.lib.cublasLtMatmulDescSetAttribute(desc, self.DESC_TRANSB, ctypes.byref(op_t), ctypes.c_size_t(4)), "set transb")
            alpha, beta = ctypes.c_int32(1), ctypes.c_int32(0)
            # library/cublaslt.py:126-150: algo NULL, workspace NULL / 0
            self._check(self.lib.cublasLtMatmul(self.handle, desc, ctypes.byref(alpha), ctypes.c_void_p(A.data_ptr()), layA,
                                                ctypes.c_void_p(B.data_ptr()), layB, ctypes.byref(beta), ctypes.c_void_p(out.data_ptr()), layC,
                                                ctypes.c_void_p(out.data_ptr()), layC, None, None, ctypes.c_size_t(0),
                                                ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "cublasLtMatmul")
        finally:
            self.lib.cublasLtMatmulDescDestroy(desc)
            self.lib.cublasLtMatrixLayoutDestroy(layA)
            self.lib.cublasLtMatrixLayoutDestroy(layB)
            self.lib.cublasLtMatrixLayoutDestroy(layC)
        return out
