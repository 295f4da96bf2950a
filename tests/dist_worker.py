"""Worker of the world_size-2 gloo test (tests/test_sharded_host.py): column-parallel linear with the oracle as the
local compute, checked against the unsharded oracle."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from cpm_kernels_b200.sharded import ColumnParallelInt8Linear, shard_bounds  # noqa: E402
from oracle import quant_linear as ql  # noqa: E402
from util import randn_fp16  # noqa: E402


def oracle_compute(x, w):
    return torch.from_numpy(ql.bmm_int8(x.numpy(), False, w.numpy(), True)["out"])


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    m, k, n = 24, 64, 48
    x = randn_fp16((1, m, k), 1)
    w = randn_fp16((1, n, k), 2, 0.02)
    lo, hi = shard_bounds(n, world, rank)
    layer = ColumnParallelInt8Linear(w[:, lo:hi, :].contiguous(), compute=oracle_compute)
    y = layer(x)
    want = ql.bmm_int8(x.numpy(), False, w.numpy(), True)["out"]
    assert y.shape == (1, m, n)
    assert (y.numpy().view(np.uint16) == want.view(np.uint16)).all(), "sharded result differs from the unsharded one"
    # the raw gather is rank-major
    g = layer.gather(layer.local(x))
    assert g.shape == (world, m, n // world)
    assert (g[rank].numpy().view(np.uint16) == want[0, :, lo:hi].view(np.uint16)).all()
    try:
        shard_bounds(50, 4, 0)
    except ValueError:
        pass
    else:
        raise AssertionError("uneven sharding must be refused")
    dist.barrier()
    dist.destroy_process_group()
    print("rank %d ok" % rank)


if __name__ == "__main__":
    main()
