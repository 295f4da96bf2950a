"""Worker of the multi-GPU test (tests/test_gpu_multi.py): fused scatter-GEMM against the NCCL-gather layer and the oracle."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from cpm_kernels_b200.sharded import ColumnParallelInt8Linear, FusedColumnParallelInt8Linear, shard_bounds  # noqa: E402
from oracle import quant_linear as ql  # noqa: E402
from util import randn_fp16  # noqa: E402


def main():
    rank = int(os.environ["RANK"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    world = dist.get_world_size()
    for (m, k, n) in [(512, 512, 1024), (1000, 1024, 2048 * world // 2)]:
        x = randn_fp16((1, m, k), 1)
        w = randn_fp16((1, n, k), 2, 0.02)
        lo, hi = shard_bounds(n, world, rank)
        w_shard = w[:, lo:hi, :].contiguous().cuda()
        want = ql.bmm_int8(x.numpy(), False, w.numpy(), True)["out"]
        base = ColumnParallelInt8Linear(w_shard)(x.cuda())
        torch.cuda.synchronize()
        assert (base.cpu().numpy().view(np.uint16) == want.view(np.uint16)).all(), "NCCL-gather layer differs from the oracle"
        fused = FusedColumnParallelInt8Linear(w_shard)
        for _ in range(2):
            y = fused(x.cuda(), sync_before=True)
            torch.cuda.synchronize()
            assert (y.cpu().numpy().view(np.uint16) == want.view(np.uint16)).all(), "fused scatter layer differs from the oracle"
    dist.barrier()
    dist.destroy_process_group()
    print("rank %d ok" % rank)


if __name__ == "__main__":
    main()
