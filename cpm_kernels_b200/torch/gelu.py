"""``gelu`` / ``gelu_inplace`` with the interface of cpm_kernels/torch/gelu.py: the activation that follows the
feed-forward block's first linear.  Forward and backward both run on the library's kernels, which evaluate the
reference's expressions (cuda/gelu.cu:6-44) as the reference compiles them: same bits as its kernels."""
import torch

from ..kernels import gelu_forward, gelu_inplace_forward, gelu_backward


class OpGeLU(torch.autograd.Function):
    """torch/gelu.py:4-44."""

    @staticmethod
    def forward(ctx, x: torch.Tensor):
        assert x.is_contiguous() and x.is_cuda and x.dtype == torch.half
        ctx.save_for_backward(x)
        ret = torch.empty_like(x)
        with torch.cuda.device(x.device):
            gelu_forward(x.size(0), x.stride(0), x.data_ptr(), ret.data_ptr(), torch.cuda.current_stream().cuda_stream)
        return ret

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        """torch/gelu.py:17-32."""
        assert grad_output.is_contiguous() and grad_output.is_cuda and grad_output.dtype == torch.half
        x = ctx.saved_tensors[0]
        grad = torch.empty_like(x)
        with torch.cuda.device(x.device):
            gelu_backward(x.size(0), x.stride(0), grad_output.data_ptr(), x.data_ptr(), grad.data_ptr(), torch.cuda.current_stream().cuda_stream)
        return grad


def gelu(x: torch.Tensor) -> torch.Tensor:
    """torch/gelu.py:46-47."""
    if torch.is_grad_enabled() and x.requires_grad:
        return OpGeLU.apply(x)
    return OpGeLU.forward(_NoCtx(), x)


class _NoCtx:
    def save_for_backward(self, *a):
        pass


def gelu_inplace(x: torch.Tensor) -> None:
    """torch/gelu.py:60-68."""
    assert x.is_contiguous() and x.is_cuda and x.dtype == torch.half
    with torch.cuda.device(x.device):
        gelu_inplace_forward(x.size(0), x.stride(0), x.data_ptr(), torch.cuda.current_stream().cuda_stream)
