"""Multi-GPU parity (needs at least two GPUs; skipped otherwise): the column-parallel layer with an NCCL all-gather and the
layer whose kernels do the exchanges themselves (GEMM epilogue scatters the output columns; the quantiser scatters the
int8 codes of row-sharded activations), all against the unsharded oracle, bit for bit.  tests/dist_gpu_worker.py is the
per-rank program.  (bench.py --gpus N repeats the comparison on its own tensors after its timed region.)"""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _run_workers(nproc):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc), "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(ROOT, "tests", "dist_gpu_worker.py")]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    for rank in range(nproc):
        assert "rank %d ok" % rank in r.stdout


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_layers_on_two_gpus():
    _run_workers(2)


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 4, reason="needs four GPUs")
def test_sharded_layers_on_all_gpus():
    _run_workers(8 if torch.cuda.device_count() >= 8 else 4)
