"""``bmm`` and its autograd functions, as cpm_kernels/torch/gemm.py.

PyTorch is used for what the reference uses it for: allocating the outputs, ``data_ptr()``, the current
stream and autograd bookkeeping.  All arithmetic of the int8 path runs in this package's CUDA kernels.

The forward pass issues three kernels where the reference issues six (torch/gemm.py:98-104): each operand
is quantised by one fused scale+round pass, and the int8 GEMM writes dequantised fp16 directly, so neither
the fp16 operands are read twice nor does an int32 tensor travel through HBM.  The tensors saved for
backward and every value returned are bit-identical to what the six separate passes produce.
"""
from typing import Optional

import torch

from ..kernels import (gemm_calc_scale, gemm_calc_scale_transpose, gemm_round, gemm_round_transpose, gemm_scale, gemm_int8, gemm_fp16,
                       gemm_backward_round_scale, gemm_backward_scale_round, gemm_scale_x, gemm_scale_y,
                       gemm_quantize_rows, gemm_quantize_rows_pair, gemm_quantize_cols, gemm_int8_scale, gemm_int8_scale_gelu)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def calc_scale(mat: torch.Tensor, transpose: bool) -> torch.Tensor:
    """torch/gemm.py:5-19.  (b, n, m) -> (b, m) if transpose else (b, n)."""
    assert mat.is_contiguous() and mat.is_cuda
    with torch.cuda.device(mat.device):
        if transpose:
            out = torch.empty((mat.size(0), mat.size(2)), dtype=torch.half, device=mat.device)
            gemm_calc_scale_transpose(mat.size(0), mat.size(1), mat.size(2), mat.data_ptr(), out.data_ptr(), _stream())
        else:
            out = torch.empty((mat.size(0), mat.size(1)), dtype=torch.half, device=mat.device)
            gemm_calc_scale(mat.size(0), mat.size(1), mat.size(2), mat.data_ptr(), out.data_ptr(), _stream())
    return out


def round_i8(mat: torch.Tensor, scale: torch.Tensor, transpose: bool) -> torch.Tensor:
    """torch/gemm.py:21-38."""
    assert mat.is_contiguous() and mat.is_cuda
    assert scale.is_contiguous() and scale.is_cuda
    out = torch.empty(mat.size(), dtype=torch.int8, device=mat.device)
    with torch.cuda.device(mat.device):
        if transpose:
            gemm_round_transpose(mat.size(0), mat.size(1), mat.size(2), mat.data_ptr(), scale.data_ptr(), out.data_ptr(), _stream())
        else:
            gemm_round(mat.size(0), mat.size(1), mat.size(2), mat.data_ptr(), scale.data_ptr(), out.data_ptr(), _stream())
    return out


def quantize(mat: torch.Tensor, transpose: bool):
    """calc_scale + round_i8 in one pass over ``mat``.  Returns (scale fp16, codes int8)."""
    assert mat.is_contiguous() and mat.is_cuda and mat.dtype == torch.half and mat.ndim == 3
    b, n, m = mat.shape
    codes = torch.empty(mat.size(), dtype=torch.int8, device=mat.device)
    with torch.cuda.device(mat.device):
        if transpose:
            scale = torch.empty((b, m), dtype=torch.half, device=mat.device)
            gemm_quantize_cols(b, n, m, mat.data_ptr(), scale.data_ptr(), codes.data_ptr(), _stream())
        else:
            scale = torch.empty((b, n), dtype=torch.half, device=mat.device)
            gemm_quantize_rows(b, n, m, mat.data_ptr(), scale.data_ptr(), codes.data_ptr(), _stream())
    return scale, codes


def gemm_and_scale(quantA: torch.Tensor, scaleA: Optional[torch.Tensor], quantB: torch.Tensor, scaleB: Optional[torch.Tensor],
                   aT: bool, bT: bool) -> torch.Tensor:
    """torch/gemm.py:40-82.  quantA (bA, M, K) [(bA, K, M) if aT], quantB (bB, K, N) [(bB, N, K) if bT] -> fp16 (b, M, N).
    The operands are passed swapped (torch/gemm.py:45-52) so that the kernel-level (n, m) = (M, N) output is row-major C."""
    M = quantA.size(2) if aT else quantA.size(1)
    K = quantA.size(1) if aT else quantA.size(2)
    N = quantB.size(1) if bT else quantB.size(2)
    batch = max(quantA.size(0), quantB.size(0))
    result_fp = torch.empty((batch, M, N), dtype=torch.float16, device=quantA.device)
    with torch.cuda.device(quantA.device):
        if scaleA is not None and scaleB is not None:
            gemm_int8_scale(N, K, M, quantB.size(0), quantA.size(0), bT, aT, quantB.data_ptr(), quantA.data_ptr(),
                            scaleA.data_ptr(), scaleB.data_ptr(), quantA.size(0) == 1, quantB.size(0) == 1,
                            result_fp.data_ptr(), _stream())
            return result_fp
        result_i32 = torch.empty((batch, M, N), dtype=torch.int32, device=quantA.device)
        gemm_int8(N, K, M, quantB.size(0), quantA.size(0), bT, aT, quantB.data_ptr(), quantA.data_ptr(), result_i32.data_ptr(), _stream())
        if scaleA is not None:
            gemm_scale_x(batch, M, N, result_i32.data_ptr(), scaleA.data_ptr(), result_fp.data_ptr(), _stream())
        else:
            assert scaleB is not None
            gemm_scale_y(batch, M, N, result_i32.data_ptr(), scaleB.data_ptr(), result_fp.data_ptr(), _stream())
    return result_fp


def _int8_forward(A: torch.Tensor, aT: bool, B: torch.Tensor, bT: bool, gelu: bool = False):
    """The three launches of the forward pass with one device guard and one stream lookup.
    Returns (result, scale_A, quantized_A, scale_B, quantized_B).  ``gelu``: GELU is applied to the result in place."""
    dev = A.device
    bA, bB = A.size(0), B.size(0)
    M = A.size(2) if aT else A.size(1)
    K = A.size(1) if aT else A.size(2)
    N = B.size(1) if bT else B.size(2)
    scale_A = torch.empty((bA, M), dtype=torch.half, device=dev)
    scale_B = torch.empty((bB, N), dtype=torch.half, device=dev)
    quantized_A = torch.empty(A.shape, dtype=torch.int8, device=dev)
    quantized_B = torch.empty(B.shape, dtype=torch.int8, device=dev)
    result = torch.empty((max(bA, bB), M, N), dtype=torch.float16, device=dev)
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream().cuda_stream
        if not aT and bT:
            # both operands are stored with K contiguous (activations (M, K), nn.Linear weights (N, K)): one launch for both
            gemm_quantize_rows_pair(bA, A.size(1), A.data_ptr(), scale_A.data_ptr(), quantized_A.data_ptr(),
                                    bB, B.size(1), B.data_ptr(), scale_B.data_ptr(), quantized_B.data_ptr(), K, stream)
        else:
            # A is quantised along K per row of the (M, K) operand: by columns of its storage when it is stored (K, M)
            (gemm_quantize_cols if aT else gemm_quantize_rows)(bA, A.size(1), A.size(2), A.data_ptr(), scale_A.data_ptr(),
                                                              quantized_A.data_ptr(), stream)
            (gemm_quantize_rows if bT else gemm_quantize_cols)(bB, B.size(1), B.size(2), B.data_ptr(), scale_B.data_ptr(),
                                                              quantized_B.data_ptr(), stream)
        # operands swapped (torch/gemm.py:45-52) so that the kernel-level (n, m) = (M, N) output is row-major C
        (gemm_int8_scale_gelu if gelu else gemm_int8_scale)(N, K, M, bB, bA, bT, aT, quantized_B.data_ptr(), quantized_A.data_ptr(),
                                                            scale_A.data_ptr(), scale_B.data_ptr(), bA == 1, bB == 1, result.data_ptr(), stream)
    return result, scale_A, quantized_A, scale_B, quantized_B


class GEMMInt8(torch.autograd.Function):
    """torch/gemm.py:84-179."""

    @staticmethod
    def forward(ctx, A: torch.Tensor, aT: bool, B: torch.Tensor, bT: bool):
        """A (batchA, M, K) [(batchA, K, M) if aT], B (batchB, K, N) [(batchB, N, K) if bT] -> (batch, M, N)."""
        assert A.is_cuda and B.is_cuda and A.device == B.device
        assert A.is_contiguous() and B.is_contiguous()
        assert A.dtype == torch.half and B.dtype == torch.half

        result, scale_A, quantized_A, scale_B, quantized_B = _int8_forward(A, aT, B, bT)

        ctx.save_for_backward(scale_A, quantized_A, scale_B, quantized_B)
        ctx.aT = aT
        ctx.bT = bT
        return result

    @staticmethod
    def backward(ctx, grad_f: torch.Tensor):
        assert grad_f.is_contiguous() and grad_f.is_cuda and grad_f.dtype == torch.float16
        scale_A, quantized_A, scale_B, quantized_B = ctx.saved_tensors
        aT, bT = ctx.aT, ctx.bT
        batch, m, n = grad_f.size()

        with torch.cuda.device(grad_f.device):
            scale_G_a = torch.empty((batch, m), dtype=torch.half, device=grad_f.device)
            quant_G_a = torch.empty((batch, m, n), dtype=torch.int8, device=grad_f.device)
            gemm_backward_round_scale(batch, m, n, grad_f.data_ptr(), scale_B.data_ptr(), quant_G_a.data_ptr(), scale_G_a.data_ptr(),
                                      scale_B.size(0) == 1, _stream())
        if aT:
            grad_A = gemm_and_scale(quantized_B, None, quant_G_a, scale_G_a, bT, True)
        else:
            grad_A = gemm_and_scale(quant_G_a, scale_G_a, quantized_B, None, False, not bT)
        del scale_G_a, quant_G_a

        with torch.cuda.device(grad_f.device):
            scale_G_b = torch.empty((batch, n), dtype=torch.half, device=grad_f.device)
            quant_G_b = torch.empty((batch, m, n), dtype=torch.int8, device=grad_f.device)
            gemm_backward_scale_round(batch, m, n, grad_f.data_ptr(), scale_A.data_ptr(), quant_G_b.data_ptr(), scale_G_b.data_ptr(),
                                      scale_A.size(0) == 1, _stream())
        if bT:
            grad_B = gemm_and_scale(quant_G_b, scale_G_b, quantized_A, None, True, aT)
        else:
            grad_B = gemm_and_scale(quantized_A, None, quant_G_b, scale_G_b, not aT, False)

        if scale_A.size(0) == 1 and grad_A.size(0) > 1:
            grad_A = grad_A.sum(dim=0, keepdim=True)
        if scale_B.size(0) == 1 and grad_B.size(0) > 1:
            grad_B = grad_B.sum(dim=0, keepdim=True)
        return grad_A, None, grad_B, None


def gemm_pth_fp16(A: torch.Tensor, aT: bool, B: torch.Tensor, bT: bool) -> torch.Tensor:
    """torch/gemm.py:182-195: the fp16 GEMM with the operands swapped so that the result is row-major (b, M, N)."""
    M = A.size(2) if aT else A.size(1)
    K = A.size(1) if aT else A.size(2)
    N = B.size(1) if bT else B.size(2)
    out = torch.empty((max(A.size(0), B.size(0)), M, N), dtype=torch.float16, device=A.device)
    gemm_fp16(N, K, M, B.size(0), A.size(0), bT, aT, B.data_ptr(), A.data_ptr(), out.data_ptr(),
                 torch.cuda.current_stream().cuda_stream)
    return out


class GEMMFloat(torch.autograd.Function):
    """torch/gemm.py:197-231: the ``int8=False`` branch of ``bmm``.  The reference hands this fp16 GEMM to
    cublasLt (kernels/gemm.py:188-256); here it runs on the library's own tcgen05 ``kind::f16`` kernel
    (``cpmk_gemm_fp16``: fp32 accumulation, one rounding to fp16)."""

    @staticmethod
    def forward(ctx, A: torch.Tensor, aT, B: torch.Tensor, bT):
        assert A.is_cuda and A.is_contiguous() and A.dtype == torch.half
        assert B.is_cuda and B.is_contiguous() and B.dtype == torch.half
        assert A.device == B.device
        ctx.save_for_backward(A, B)
        ctx.aT = aT
        ctx.bT = bT
        return gemm_pth_fp16(A, aT, B, bT)

    @staticmethod
    def backward(ctx, grad_f):
        assert grad_f.is_cuda and grad_f.is_contiguous() and grad_f.dtype == torch.float16
        aT, bT = ctx.aT, ctx.bT
        A, B = ctx.saved_tensors
        grad_A = gemm_pth_fp16(B, bT, grad_f, True) if aT else gemm_pth_fp16(grad_f, False, B, not bT)
        grad_B = gemm_pth_fp16(grad_f, True, A, aT) if bT else gemm_pth_fp16(A, not aT, grad_f, False)
        if A.size(0) == 1 and grad_A.size(0) > 1:
            grad_A = grad_A.sum(dim=0, keepdim=True)
        if B.size(0) == 1 and grad_B.size(0) > 1:
            grad_B = grad_B.sum(dim=0, keepdim=True)
        return grad_A, None, grad_B, None


def bmm(A: torch.Tensor, aT: bool, B: torch.Tensor, bT: bool, int8: bool = False) -> torch.Tensor:
    """torch/gemm.py:233-239."""
    assert A.ndim == 3
    assert B.ndim == 3
    if int8:
        if torch.is_grad_enabled() and (A.requires_grad or B.requires_grad):
            return GEMMInt8.apply(A, aT, B, bT)
        # nothing to differentiate: the same forward without the autograd bookkeeping
        assert A.is_cuda and B.is_cuda and A.device == B.device
        assert A.is_contiguous() and B.is_contiguous()
        assert A.dtype == torch.half and B.dtype == torch.half
        return _int8_forward(A, aT, B, bT)[0]
    return GEMMFloat.apply(A, aT, B, bT)


def bmm_gelu(A: torch.Tensor, aT: bool, B: torch.Tensor, bT: bool) -> torch.Tensor:
    """``gelu(bmm(A, aT, B, bT, int8=True))`` (cpm_kernels.torch.gelu after cpm_kernels.torch.bmm, as the feed-forward
    block chains them) without a second tensor: the activation runs in place on the GEMM's result while it is still
    in L2.  Forward only; same bits as the two calls."""
    assert A.ndim == 3 and B.ndim == 3
    assert A.is_cuda and B.is_cuda and A.device == B.device
    assert A.is_contiguous() and B.is_contiguous()
    assert A.dtype == torch.half and B.dtype == torch.half
    return _int8_forward(A, aT, B, bT, gelu=True)[0]


def layernorm_quantize(x: torch.Tensor, eps: float, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, rd_mean: bool = True):
    """Layer norm of ``x`` (batch, hidden, seq) over the hidden axis, times ``weight`` (plus ``bias``), quantised per
    (batch, seq) column: ``(scale (batch, seq) fp16, codes (batch, hidden, seq) int8)``, the operand B that
    ``bmm(W, False, layernorm(x), False, int8=True)`` would quantise, without the fp16 tensors in between
    (cpm_kernels/torch/layernorm.py:8-30 and torch/gemm.py:98-102 in one call; same bits).  Forward only."""
    from ..kernels import layernorm_quantize_cols
    assert x.is_cuda and x.is_contiguous() and x.ndim == 3 and x.dtype == torch.half
    assert weight.is_cuda and weight.is_contiguous() and weight.ndim == 1 and weight.dtype == torch.half and weight.numel() == x.size(1)
    if bias is not None:
        assert bias.is_cuda and bias.is_contiguous() and bias.dtype == torch.half and bias.numel() == x.size(1)
    scale = torch.empty((x.size(0), x.size(2)), dtype=torch.half, device=x.device)
    codes = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    with torch.cuda.device(x.device):
        layernorm_quantize_cols(x.size(0), x.size(1), x.size(2), x.data_ptr(), eps, rd_mean, weight.data_ptr(),
                                bias.data_ptr() if bias is not None else 0, scale.data_ptr(), codes.data_ptr(),
                                torch.cuda.current_stream().cuda_stream)
    return scale, codes


def bmm_quantized_b(A: torch.Tensor, aT: bool, scale_B: torch.Tensor, quantized_B: torch.Tensor, bT: bool) -> torch.Tensor:
    """``bmm(A, aT, B, bT, int8=True)`` for an operand B that is already quantised along K (``layernorm_quantize``
    gives it for bT = False): A is quantised here, then the GEMM with its dequantising epilogue.  Forward only."""
    assert A.ndim == 3 and quantized_B.ndim == 3
    assert A.is_cuda and A.is_contiguous() and A.dtype == torch.half
    assert quantized_B.is_cuda and quantized_B.is_contiguous() and quantized_B.dtype == torch.int8
    scale_A, quantized_A = quantize(A, aT)
    return gemm_and_scale(quantized_A, scale_A, quantized_B, scale_B, aT, bT)
