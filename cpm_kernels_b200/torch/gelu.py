"""``gelu`` / ``gelu_inplace`` with the interface of cpm_kernels/torch/gelu.py: the activation that follows the
feed-forward block's first linear.  Forward on the library's kernel (same bits as the reference's); the backward of
the autograd function evaluates the reference's derivative formula (cuda/gelu.cu:20-44) with torch operations."""
import torch

from ..kernels import gelu_forward, gelu_inplace_forward


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
        x = ctx.saved_tensors[0].float()
        x3 = x * x * x
        inner = 0.797885 * x + 0.0356774 * x3
        sech2 = (1.0 / torch.cosh(inner)) ** 2
        g = 0.5 + (0.398942 * x + 0.0535161 * x3) * sech2 + 0.5 * torch.tanh(inner)
        g = torch.where((x > -5) & (x < 5), g, (x >= 0).float())
        return (g * grad_output.float()).half()


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
