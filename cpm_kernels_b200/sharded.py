"""Column-parallel (N-sharded) int8 linear over ``torch.distributed``.

The reference has no multi-GPU code; its linear layer shards naturally along the output features: rank r holds
rows [r*N/g, (r+1)*N/g) of the weight W (N, K), and because both quantisations are per row (x rows along K, W rows
along K) every rank's slice of y = x W^T is bit-identical to the same slice of the unsharded result.  Two exchanges
exist, both done by the stores of this package's own kernels into peer-mapped (symmetric) memory:

* the all-gather of the fp16 outputs: the GEMM's epilogue stores its N/g columns into every rank's full-width y;
* (optional) the all-gather of the int8 activations: a rank that holds only rows [r*M/g, (r+1)*M/g) of x quantises
  them once and the quantising kernel stores codes and scales into every rank's full code buffer -- 1 byte per element
  over NVLink instead of every rank loading (or uploading) the whole fp16 tensor.

One process per GPU; the process group is the caller's (NCCL on GPUs; gloo works for the host logic of the
NCCL-gather layer).
"""
from __future__ import annotations

import ctypes
import math
from typing import Callable, List, Optional, Tuple

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
    """y = int8_linear(x, W) with W sharded along N and an NCCL all-gather of the output slices.

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


# ------------------------------------------------------------------------------------------------
# peer-mapped buffers
# ------------------------------------------------------------------------------------------------
def _align(x: int, a: int = 256) -> int:
    return (x + a - 1) // a * a


class SymmetricArena:
    """One symmetric-memory allocation per rank (same size on every rank), carved into buffers that sit at the same
    offset on every rank, so that a peer's copy of a buffer is ``base[peer] + offset``.  One rendezvous for everything
    instead of one per tensor.  With a single rank (or no process group) it is ordinary device memory and the barrier
    does nothing, so the same layer code runs on one GPU."""

    def __init__(self, nbytes: int, device: torch.device, group: Optional[dist.ProcessGroup] = None):
        self.distributed = dist.is_available() and dist.is_initialized()
        self.group = (group if group is not None else dist.group.WORLD) if self.distributed else None
        self.world = dist.get_world_size(self.group) if self.distributed else 1
        self.rank = dist.get_rank(self.group) if self.distributed else 0
        self.nbytes = _align(max(int(nbytes), 256))
        self.used = 0
        if self.world > 1:
            import torch.distributed._symmetric_memory as symm_mem
            self.buf = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
            self.handle = symm_mem.rendezvous(self.buf, self.group)
            self.base = [int(self.handle.buffer_ptrs[p]) for p in range(self.world)]
            # the same allocation mapped through an NVLink multicast object (0 when the system has none): one store to
            # multicast_base + offset lands in every rank's copy
            self.multicast_base = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        else:
            self.buf = torch.empty(self.nbytes, dtype=torch.uint8, device=device)
            self.handle = None
            self.base = [self.buf.data_ptr()]
            self.multicast_base = 0

    def carve(self, shape, dtype: torch.dtype) -> Tuple[torch.Tensor, int]:
        """A (local tensor, offset) pair; the peers' copies are at ``peer_ptr(p, offset)``."""
        n = math.prod(shape) * torch.empty((), dtype=dtype).element_size()
        off = self.used
        if off + n > self.nbytes:
            raise RuntimeError("symmetric arena of %d bytes is full (%d used, %d asked)" % (self.nbytes, off, n))
        self.used = _align(off + n)
        return self.buf[off:off + n].view(dtype).view(shape), off

    def peer_ptr(self, peer: int, offset: int) -> int:
        return self.base[peer] + offset

    def barrier(self, channel: int = 0) -> None:
        """Every rank's work enqueued so far on its current stream (stores into peers included) has completed when the
        stream passes this point on any rank."""
        if self.handle is not None:
            self.handle.barrier(channel=channel)


class ExchangeBuffers:
    """The peer-mapped buffers of one linear shape (tokens, K) -> (tokens, N): per slot the full-width fp16 output
    y (1, tokens, N), the gathered int8 activations qx (1, tokens, K) and their scales sx (1, tokens).  Two slots let
    step s+1 be written while step s is still being read."""

    def __init__(self, arena: SymmetricArena, tokens: int, k: int, n_total: int, slots: int = 2):
        self.arena, self.tokens, self.k, self.n_total, self.slots = arena, tokens, k, n_total, slots
        self.y, self.qx, self.sx = [], [], []
        self.y_off, self.qx_off, self.sx_off = [], [], []
        for _ in range(slots):
            t, off = arena.carve((1, tokens, n_total), torch.half)
            self.y.append(t)
            self.y_off.append(off)
            t, off = arena.carve((1, tokens, k), torch.int8)
            self.qx.append(t)
            self.qx_off.append(off)
            t, off = arena.carve((1, tokens), torch.half)
            self.sx.append(t)
            self.sx_off.append(off)

    @staticmethod
    def nbytes(tokens: int, k: int, n_total: int, slots: int = 2) -> int:
        return slots * (_align(2 * tokens * n_total) + _align(tokens * k) + _align(2 * tokens))


def recommended_forward_sms(world: int) -> int:
    """How many SMs of a scattering GEMM to give to forwarding CTAs (``cpmk.set_gemm_forward_sms``) for ``world`` ranks.
    With two ranks a GPU sends its output once whether its computing CTAs or forwarding CTAs store it, and the computing
    CTAs' own stores measured faster; from four ranks on every output tile crosses the link three or more times, and
    taking those stores off the computing CTAs measured faster (4 ranks: 0.350 against 0.379 ms per benchmark step)."""
    return 24 if world >= 4 else 0


def _peer_order(rank: int, world: int) -> List[int]:
    """Destinations in the order rank, rank+1, rank+2, ...: the rank's own buffer first (the scattering GEMM computes into
    destination 0 and forwards from there), then the peers starting with its neighbour, so that at any moment the ranks
    store to different peers instead of all converging on rank 0."""
    return [(rank + i) % world for i in range(world)]


class FusedColumnParallelInt8Linear:
    """The column-parallel layer with the all-gather done by the GEMM: every rank's epilogue stores its N/g output
    columns straight into columns [r*N/g, (r+1)*N/g) of every rank's full-width, token-major y (TMA stores over NVLink
    into peer-mapped memory), so there is no gather kernel, no second read of the slice and no re-layout pass.

    ``weight_shard``: this rank's rows of W, fp16 (1, N/g, K).  ``buffers``: the peer-mapped buffers of this shape
    (shared by all layers of the shape); without them the layer allocates its own on first use -- a collective call.
    ``weight_scratch``: (codes int8 (1, N/g, K), scales fp16 (1, N/g)) for the quantised weight; layers of one shape may
    share it, because the weight is re-quantised on every call as the reference's ``bmm`` does.

    Two forms of the forward pass:
      * ``forward(x)``: x (1, tokens, K) is present in full on every rank; one library call quantises x and the weight
        rows and runs the scattering GEMM; one barrier afterwards.
      * ``quantize_shard(x_rows)`` + barrier + ``gemm()`` + barrier (``forward_sharded``): each rank holds only its
        tokens/g rows of x; the quantising kernel distributes codes and scales to every rank.
    ``y`` lives in the buffers' slot: the caller must be done reading a slot on every rank before it is written again
    (alternate slots, or pass ``sync_before=True``).  CUDA only.
    """

    def __init__(self, weight_shard: torch.Tensor, group: Optional[dist.ProcessGroup] = None,
                 buffers: Optional[ExchangeBuffers] = None, weight_scratch: Optional[Tuple[torch.Tensor, torch.Tensor]] = None):
        assert weight_shard.ndim == 3 and weight_shard.size(0) == 1 and weight_shard.is_contiguous() and weight_shard.is_cuda
        assert weight_shard.dtype == torch.half
        self.weight = weight_shard
        self.distributed = dist.is_available() and dist.is_initialized()
        self.group = (group if group is not None else dist.group.WORLD) if self.distributed else None
        self.world = dist.get_world_size(self.group) if self.distributed else 1
        self.rank = dist.get_rank(self.group) if self.distributed else 0
        self.n_local, self.k = weight_shard.size(1), weight_shard.size(2)
        self.n_total = self.n_local * self.world
        self.buffers = buffers
        if weight_scratch is None:
            weight_scratch = (torch.empty(weight_shard.shape, dtype=torch.int8, device=weight_shard.device),
                              torch.empty((1, self.n_local), dtype=torch.half, device=weight_shard.device))
        self.q_w, self.scale_w = weight_scratch
        assert self.q_w.shape == weight_shard.shape and self.q_w.dtype == torch.int8
        self._own = {}
        self._dst_cache = {}

    # ---- buffers and destination lists ----
    def _buffers_for(self, tokens: int) -> ExchangeBuffers:
        if self.buffers is not None:
            assert self.buffers.tokens == tokens and self.buffers.k == self.k and self.buffers.n_total == self.n_total
            return self.buffers
        if tokens not in self._own:
            arena = SymmetricArena(ExchangeBuffers.nbytes(tokens, self.k, self.n_total), self.weight.device, self.group)
            self._own[tokens] = ExchangeBuffers(arena, tokens, self.k, self.n_total)
        return self._own[tokens]

    def _dsts(self, buf: ExchangeBuffers, slot: int, only_local: bool = False, multicast: bool = False):
        """(y destinations, code destinations, scale destinations) of this rank's contribution, as ctypes arrays.
        multicast: the y destinations are this rank's copy and the buffer's multicast address."""
        key = (id(buf), slot, only_local, multicast)
        if key not in self._dst_cache:
            arena = buf.arena
            peers = [self.rank] if only_local else _peer_order(self.rank, self.world)
            rows = buf.tokens // self.world
            y = [arena.peer_ptr(p, buf.y_off[slot]) + 2 * self.rank * self.n_local for p in peers]
            if multicast and not only_local:
                assert arena.multicast_base, "the symmetric arena has no multicast mapping on this system"
                y = [y[0], arena.multicast_base + buf.y_off[slot] + 2 * self.rank * self.n_local]
            qx = [arena.peer_ptr(p, buf.qx_off[slot]) + self.rank * rows * self.k for p in peers]
            sx = [arena.peer_ptr(p, buf.sx_off[slot]) + 2 * self.rank * rows for p in peers]
            self._dst_cache[key] = tuple((ctypes.c_void_p * len(v))(*v) for v in (y, qx, sx))
        return self._dst_cache[key]

    @staticmethod
    def _stream() -> int:
        return torch.cuda.current_stream().cuda_stream

    # ---- x present in full on every rank ----
    def launch(self, x: torch.Tensor, slot: int = 0, only_local: bool = False, multicast: bool = False) -> torch.Tensor:
        """Quantise x and the weight rows, run the scattering GEMM (two launches, one library call); no barrier.
        ``only_local``: store this rank's columns into its own y only (the compute phase without the exchange).
        ``multicast``: reach the other ranks through the buffers' NVLink multicast mapping (one multimem store per 16
        bytes, replicated by the switch) instead of one store per peer."""
        from .kernels import linear_int8_scatter
        assert x.ndim == 3 and x.size(0) == 1 and x.is_contiguous() and x.is_cuda and x.dtype == torch.half and x.size(2) == self.k
        tokens = x.size(1)
        buf = self._buffers_for(tokens)
        multicast = multicast and not only_local and self.world > 1
        y_dst, _, _ = self._dsts(buf, slot, only_local, multicast)
        with torch.cuda.device(x.device):
            linear_int8_scatter(tokens, self.k, self.n_local, x.data_ptr(), self.weight.data_ptr(), buf.sx[slot].data_ptr(),
                                buf.qx[slot].data_ptr(), self.scale_w.data_ptr(), self.q_w.data_ptr(), y_dst, self.n_total, self._stream(),
                                multicast=multicast)
        return buf.y[slot]

    def forward(self, x: torch.Tensor, sync_before: bool = False, slot: int = 0, multicast: bool = False) -> torch.Tensor:
        buf = self._buffers_for(x.size(1))
        if sync_before:
            buf.arena.barrier(0)           # every rank is done reading the slot's previous contents
        y = self.launch(x, slot, multicast=multicast)
        buf.arena.barrier(1)               # every rank's stores have landed before anyone reads y
        return y

    __call__ = forward

    # ---- x sharded by rows ----
    def quantize_shard(self, x_rows: torch.Tensor, slot: int = 0, tokens: Optional[int] = None) -> None:
        """x_rows (1, tokens/g, K): this rank's rows [r*tokens/g, (r+1)*tokens/g) of the activations.  One launch
        quantises them into every rank's code buffer (at that row offset) and this rank's weight rows into its scratch.
        A barrier must follow before ``gemm`` reads the gathered codes."""
        from .kernels import gemm_quantize_rows_pair_scatter
        assert x_rows.ndim == 3 and x_rows.size(0) == 1 and x_rows.is_contiguous() and x_rows.is_cuda and x_rows.dtype == torch.half
        rows = x_rows.size(1)
        tokens = rows * self.world if tokens is None else tokens
        assert rows * self.world == tokens and x_rows.size(2) == self.k
        buf = self._buffers_for(tokens)
        _, q_dst, s_dst = self._dsts(buf, slot)
        with torch.cuda.device(x_rows.device):
            gemm_quantize_rows_pair_scatter(rows, x_rows.data_ptr(), s_dst, q_dst, self.n_local, self.weight.data_ptr(),
                                            self.scale_w.data_ptr(), self.q_w.data_ptr(), self.k, self._stream())

    def gemm(self, tokens: int, slot: int = 0, only_local: bool = False) -> torch.Tensor:
        """The scattering GEMM on the slot's gathered codes and this rank's quantised weight rows."""
        from .kernels import gemm_int8_scale_scatter
        buf = self._buffers_for(tokens)
        y_dst, _, _ = self._dsts(buf, slot, only_local)
        with torch.cuda.device(self.weight.device):
            # kernel-level (m, k, n) = (N_local, K, tokens): A = weight codes, B = activation codes, output rows = tokens
            gemm_int8_scale_scatter(self.n_local, self.k, tokens, 1, 1, True, False, self.q_w.data_ptr(), buf.qx[slot].data_ptr(),
                                    buf.sx[slot].data_ptr(), self.scale_w.data_ptr(), True, True, y_dst, self.n_total, self._stream())
        return buf.y[slot]

    def forward_sharded(self, x_rows: torch.Tensor, slot: int = 0) -> torch.Tensor:
        tokens = x_rows.size(1) * self.world
        buf = self._buffers_for(tokens)
        self.quantize_shard(x_rows, slot, tokens)
        buf.arena.barrier(0)               # every rank's codes and scales have landed
        y = self.gemm(tokens, slot)
        buf.arena.barrier(1)               # every rank's output columns have landed
        return y
