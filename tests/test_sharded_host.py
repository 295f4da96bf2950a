"""Host logic of the N-sharded path on CPU: two gloo ranks, the oracle as the local compute."""
import os
import socket
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _torchrun(args, nproc=2, timeout=240):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc), "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port())] + args
    env = dict(os.environ, OMP_NUM_THREADS="2")
    return subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)


def test_column_parallel_linear_two_ranks_gloo():
    r = _torchrun([os.path.join(ROOT, "tests", "dist_worker.py")])
    assert r.returncode == 0, r.stdout + r.stderr
    assert "rank 0 ok" in r.stdout and "rank 1 ok" in r.stdout


def test_shard_bounds():
    from cpm_kernels_b200.sharded import shard_bounds
    assert [shard_bounds(12288, 8, r) for r in (0, 7)] == [(0, 1536), (10752, 12288)]
    assert shard_bounds(4096, 1, 0) == (0, 4096)


def test_peer_order_spreads_the_first_destination():
    """Rank r stores to r, r+1, r+2, ...: its own buffer first, and at every position the ranks address different peers."""
    from cpm_kernels_b200.sharded import _peer_order
    for world in (1, 2, 4, 8):
        orders = [_peer_order(r, world) for r in range(world)]
        for r, o in enumerate(orders):
            assert sorted(o) == list(range(world)) and o[0] == r
        for step in range(world):
            assert len({o[step] for o in orders}) == world


def test_arena_carves_aligned_buffers_at_rank_independent_offsets():
    """One rank, host memory: the carving arithmetic (what makes `base[peer] + offset` valid on every rank)."""
    import torch
    from cpm_kernels_b200.sharded import ExchangeBuffers, SymmetricArena
    need = ExchangeBuffers.nbytes(48, 64, 96)
    arena = SymmetricArena(need, torch.device("cpu"))
    assert arena.world == 1 and arena.rank == 0
    buf = ExchangeBuffers(arena, 48, 64, 96)
    assert arena.used <= arena.nbytes == need
    offs = buf.y_off + buf.qx_off + buf.sx_off
    assert all(o % 256 == 0 for o in offs) and len(set(offs)) == 6
    assert buf.y[1].shape == (1, 48, 96) and buf.y[1].dtype == torch.half and buf.qx[0].dtype == torch.int8
    assert buf.y[1].data_ptr() == arena.peer_ptr(0, buf.y_off[1])
    arena.barrier(0)                                           # one rank: nothing to wait for
    try:
        arena.carve((1 << 20,), torch.half)
    except RuntimeError as e:
        assert "full" in str(e)
    else:
        raise AssertionError("an over-full arena must refuse")


def test_reference_arm_under_torchrun_prints_one_line():
    """bench.py --impl reference with two ranks: rank 0 alone runs and prints; the other exits 0 without work."""
    import json
    r = _torchrun([os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "1", "--tokens", "64"])
    assert r.returncode == 0, r.stdout + r.stderr
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["n_gpus"] == 2 and d["cpu_baseline"]["kind"] == "port"
