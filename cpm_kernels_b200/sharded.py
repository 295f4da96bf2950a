"""Column-parallel (N-sharded) int8 linear over ``torch.distributed``.

The reference has no multi-GPU code; its linear layer shards naturally along the output features: rank r holds
rows [r*N/g, (r+1)*N/g) of the weight W (N, K), the activations x (M, K) are replicated, and because both
quantisations are per row (x rows along K, W rows along K) every rank's slice of y = x W^T is bit-identical to
the same slice of the unsharded result.  The only exchange is an all-gather of the fp16 output slices.

One process per GPU; the process group is the caller's (NCCL on GPUs; gloo works for the host logic).
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def shard_bounds(n: int, world: int, rank: int) -> Tuple[int, int]:
    """Rows [lo, hi) of an N-row weight that rank ``rank`` of ``world`` holds.  N must divide evenly: the all-gather
    moves equal slices."""
    if n % world != 0:
        raise ValueError("output features (%d) must be a multiple of the number of ranks (%d)" % (n, world))
    per = n // world
    return rank * per, (rank + 1) * per


def _default_compute(x: torch.Tensor, w_shard: torch.Tensor) -> torch.Tensor:
    from .torch import bmm            # imported here so that the host logic can be exercised without the CUDA library
    return bmm(x, False, w_shard, True, int8=True)


class ColumnParallelInt8Linear:
    """y = int8_linear(x, W) with W sharded along N.

    ``weight_shard``: this rank's rows of W, fp16 (1, N/g, K), contiguous.
    ``compute``: the local linear; defaults to this package's CUDA ``bmm(x, False, w, True, int8=True)``.  Tests of the
    host logic pass a CPU function here; the default never falls back to one.
    """

    def __init__(self, weight_shard: torch.Tensor, group: Optional[dist.ProcessGroup] = None,
                 compute: Optional[Callable[[torch.Tensor, torch.Tensor], torch.Tensor]] = None):
        assert weight_shard.ndim == 3 and weight_shard.size(0) == 1 and weight_shard.is_contiguous()
        self.weight = weight_shard
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.compute = compute or _default_compute

    def local(self, x: torch.Tensor) -> torch.Tensor:
        """This rank's output slice (1, M, N/g)."""
        return self.compute(x, self.weight)

    def gather(self, y_local: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """All-gather the slices into (g, M, N/g) (rank-major, what the collective produces without a copy)."""
        _, m, n_local = y_local.shape
        if out is None:
            out = torch.empty((self.world, m, n_local), dtype=y_local.dtype, device=y_local.device)
        if self.world == 1:
            out.copy_(y_local)
        else:
            dist.all_gather_into_tensor(out, y_local.contiguous(), group=self.group)
        return out

    @staticmethod
    def to_token_major(gathered: torch.Tensor) -> torch.Tensor:
        """(g, M, N/g) -> (1, M, N): the layout of the unsharded result (one re-layout pass)."""
        g, m, n_local = gathered.shape
        return gathered.permute(1, 0, 2).reshape(1, m, g * n_local)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.to_token_major(self.gather(self.local(x)))

    __call__ = forward


class FusedColumnParallelInt8Linear:
    """The same layer with the all-gather done by the GEMM: every rank's epilogue stores its N/g output columns straight
    into columns [r*N/g, (r+1)*N/g) of every rank's full-width, token-major y (TMA stores over NVLink into peer-mapped
    symmetric memory), so there is no gather kernel, no second read of the slice and no re-layout pass.

    ``y`` lives in symmetric memory owned by the layer (one buffer per token count, reused call after call): the caller
    must be done reading the previous result on every rank before calling again, or pass ``sync_before=True``.
    CUDA only (there is no host form of peer-mapped stores); NCCL process group for the rendezvous.
    """

    def __init__(self, weight_shard: torch.Tensor, group: Optional[dist.ProcessGroup] = None):
        assert weight_shard.ndim == 3 and weight_shard.size(0) == 1 and weight_shard.is_contiguous() and weight_shard.is_cuda
        self.weight = weight_shard
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self._buffers = {}

    def _buffer(self, m_tokens: int):
        import torch.distributed._symmetric_memory as symm_mem
        if m_tokens not in self._buffers:
            n_total = self.weight.size(1) * self.world
            y = symm_mem.empty((1, m_tokens, n_total), dtype=torch.half, device=self.weight.device)
            handle = symm_mem.rendezvous(y, self.group)
            self._buffers[m_tokens] = (y, handle)
        return self._buffers[m_tokens]

    def forward(self, x: torch.Tensor, sync_before: bool = False) -> torch.Tensor:
        from .kernels import gemm_int8_scale_scatter, gemm_quantize_rows_pair
        assert x.ndim == 3 and x.size(0) == 1 and x.is_contiguous() and x.is_cuda
        m_tokens, k = x.size(1), x.size(2)
        n_local = self.weight.size(1)
        n_total = n_local * self.world
        y, handle = self._buffer(m_tokens)
        # activations and this rank's weight rows in one launch (both are stored with K contiguous)
        dev = x.device
        scale_x = torch.empty((1, m_tokens), dtype=torch.half, device=dev)
        q_x = torch.empty(x.shape, dtype=torch.int8, device=dev)
        scale_w = torch.empty((1, n_local), dtype=torch.half, device=dev)
        q_w = torch.empty(self.weight.shape, dtype=torch.int8, device=dev)
        with torch.cuda.device(dev):
            gemm_quantize_rows_pair(1, m_tokens, x.data_ptr(), scale_x.data_ptr(), q_x.data_ptr(), 1, n_local, self.weight.data_ptr(),
                                    scale_w.data_ptr(), q_w.data_ptr(), k, torch.cuda.current_stream().cuda_stream)
        if sync_before:
            handle.barrier(channel=0)
        dst = [int(handle.buffer_ptrs[p]) + 2 * self.rank * n_local for p in range(self.world)]
        with torch.cuda.device(x.device):
            # kernel-level (m, k, n) = (N_local, K, M): A = weights, B = activations, out rows = tokens
            gemm_int8_scale_scatter(n_local, k, m_tokens, 1, 1, True, False, q_w.data_ptr(), q_x.data_ptr(), scale_x.data_ptr(),
                                    scale_w.data_ptr(), True, True, dst, n_total, torch.cuda.current_stream().cuda_stream)
        handle.barrier(channel=1)          # every rank's stores have landed before anyone reads y
        return y

    __call__ = forward
