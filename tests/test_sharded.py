"""The table-wise-sharded path: layout arithmetic, the exchange on CPU ranks (gloo, world size 2),
and -- on a box with at least two GPUs -- the fused peer-store exchange against NCCL's all-to-all."""
import os
import socket
import subprocess
import sys

import pytest
import torch

from torchlib_xpu_b200 import sharded

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run_workers(backend, world, timeout=600):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(ROOT, "tests", "sharded_worker.py"), backend]
    env = dict(os.environ, OMP_NUM_THREADS="2")
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "sharded worker ok" in proc.stdout


def test_layout_arithmetic():
    assert sharded.local_tables(1, 4, 10) == [1, 5, 9]
    assert [sharded.owner_of_table(t, 4) for t in range(6)] == [0, 1, 2, 3, 0, 1]
    assert sharded.layout_batch_rows(2, 4, 64) == (32, 48)
    assert sharded.layout_pooled_columns(3, 256) == (768, 1024)
    with pytest.raises(ValueError):
        sharded.layout_batch_rows(0, 3, 64)


def test_exchange_layout_on_two_cpu_ranks():
    _run_workers("gloo", 2)


@pytest.mark.gpu
def test_fused_exchange_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _run_workers("nccl", 2)
