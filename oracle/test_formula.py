"""TEST INFRASTRUCTURE ONLY -- the reference's *test* formulas, on CPU with torch.

These are the expressions the reference's unit tests hold its kernels to (tests/test_gemm.py:8-41,
tests/test_gemv.py:80,125).  They are looser than the kernels' own arithmetic -- the scale stays in
fp32 instead of being rounded to fp16, so about half a percent of the int8 codes differ by one --
and are therefore used for two things only: the timed CPU baseline of the benchmark, and a coarse
(rtol 0.5 / atol 0.5, tests/test_gemm.py:98) sanity check of the end-to-end result.
"""
import torch


def calc_scale(x: torch.Tensor) -> torch.Tensor:
    """tests/test_gemm.py:8-9."""
    return x.abs().max(dim=-1, keepdim=True)[0] / 127


def scale_round(x: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """tests/test_gemm.py:12-13."""
    return torch.round(x / scale) * scale


def real_bmm(a: torch.Tensor, aT: bool, b: torch.Tensor, bT: bool, int8: bool) -> torch.Tensor:
    """tests/test_gemm.py:25-41 (forward only): fake-quantise both operands along K in fp32, fp32 matmul."""
    if a.ndim == 2:
        a = a.unsqueeze(0)
    if b.ndim == 2:
        b = b.unsqueeze(0)
    if aT:
        a = a.transpose(-1, -2)
    if bT:
        b = b.transpose(-1, -2)
    if int8:
        old_type = a.dtype
        a = a.to(torch.float32)
        b = b.to(torch.float32)
        a = scale_round(a, calc_scale(a))
        # tests/test_gemm.py:36-37 quantises `b` (k, n) along its last axis as well; the kernels
        # quantise B along K.  The linear-layer configurations are timed with the kernels' axis.
        bt = b.transpose(-1, -2)
        bt = scale_round(bt, calc_scale(bt))
        return torch.matmul(a, bt.transpose(-1, -2)).to(old_type)
    return torch.matmul(a, b)


def gemv(mat: torch.Tensor, vec: torch.Tensor) -> torch.Tensor:
    """tests/test_gemv.py:80: the GEMV is checked against a plain matmul.  mat (b, out, in), vec (b, in)."""
    return torch.matmul(mat.float(), vec.float().unsqueeze(-1)).squeeze(-1).to(mat.dtype)
