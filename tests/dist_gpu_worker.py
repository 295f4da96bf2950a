"""Worker of the multi-GPU test (tests/test_gpu_multi.py), one process per GPU: the column-parallel layers against the
unsharded oracle, bit for bit -- the NCCL-gather layer, and both forms of the layer whose kernels do the exchanges
(activations present in full: one call, GEMM epilogue scatters; activations sharded by rows: the quantising kernel
scatters the int8 codes, then the GEMM scatters its columns), on shared and on layer-owned buffers, alternating slots."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from cpm_kernels_b200.library import cpmk  # noqa: E402
from cpm_kernels_b200.sharded import (ColumnParallelInt8Linear, ExchangeBuffers, FusedColumnParallelInt8Linear, SymmetricArena,  # noqa: E402
                                      shard_bounds)
from oracle import quant_linear as ql  # noqa: E402
from util import randn_fp16  # noqa: E402


def same(t, want) -> bool:
    return bool((t.cpu().numpy().view(np.uint16) == want.view(np.uint16)).all())


def main():
    rank = int(os.environ["RANK"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    world = dist.get_world_size()
    shapes = [(512, 512, 1024), (1000 // world * world, 1024, 2048 * world // 2)]
    arena = SymmetricArena(sum(ExchangeBuffers.nbytes(m, k, n) for m, k, n in shapes) + 4096, torch.device("cuda", local))
    for (m, k, n) in shapes:
        x = randn_fp16((1, m, k), 1)
        w = randn_fp16((1, n, k), 2, 0.02)
        lo, hi = shard_bounds(n, world, rank)
        w_shard = w[:, lo:hi, :].contiguous().cuda()
        want = ql.bmm_int8(x.numpy(), False, w.numpy(), True)
        base = ColumnParallelInt8Linear(w_shard)(x.cuda())
        torch.cuda.synchronize()
        assert same(base, want["out"]), "NCCL-gather layer differs from the oracle"
        # layer-owned buffers, activations in full
        fused = FusedColumnParallelInt8Linear(w_shard)
        for _ in range(2):
            y = fused(x.cuda(), sync_before=True)
            torch.cuda.synchronize()
            assert same(y, want["out"]), "fused scatter layer differs from the oracle"
        # shared buffers in one arena, both slots, both forms
        layer = FusedColumnParallelInt8Linear(w_shard, buffers=ExchangeBuffers(arena, m, k, n))
        rows = m // world
        x_rows = x[:, rank * rows:(rank + 1) * rows, :].contiguous().cuda()
        for slot in (0, 1, 0):
            y = layer.forward(x.cuda(), sync_before=True, slot=slot)
            torch.cuda.synchronize()
            assert same(y, want["out"]), "one-call scatter layer differs from the oracle (slot %d)" % slot
            dist.barrier()
            layer.buffers.y[slot].fill_(3.0)
            layer.buffers.qx[slot].fill_(55)
            torch.cuda.synchronize()
            dist.barrier()
            y = layer.forward_sharded(x_rows, slot=slot)
            torch.cuda.synchronize()
            assert same(y, want["out"]), "row-sharded activations: result differs from the oracle (slot %d)" % slot
            assert (layer.buffers.qx[slot].cpu().numpy() == want["quant_A"]).all(), "gathered int8 codes differ from the unsharded codes"
            assert same(layer.buffers.sx[slot], want["scale_A"]), "gathered scales differ from the unsharded scales"
            dist.barrier()
            # forwarding CTAs: the computing CTAs store to this rank's result only, a few CTAs of the grid copy finished
            # tiles to the peers -- with plain stores, and (where the buffers have a multicast mapping) with multimem stores
            for multicast in ((False, True) if arena.multicast_base else (False,)):
                layer.buffers.y[slot].fill_(3.0)
                torch.cuda.synchronize()
                dist.barrier()
                cpmk.set_gemm_forward_sms(16)
                y = layer.forward(x.cuda(), sync_before=True, slot=slot, multicast=multicast)
                torch.cuda.synchronize()
                cpmk.set_gemm_forward_sms(-1)
                assert same(y, want["out"]), "forwarding CTAs (multicast=%s): result differs from the oracle (slot %d)" % (multicast, slot)
                dist.barrier()
    assert cpmk.read_status() == 0
    dist.barrier()
    dist.destroy_process_group()
    print("rank %d ok" % rank)


if __name__ == "__main__":
    main()
