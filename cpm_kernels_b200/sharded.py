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
