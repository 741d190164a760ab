"""GPU tier, needs two or more GPUs (skipped on a single-GPU box): the row-sharded decode
stream with its all-gather done by peer stores, one process per GPU."""
from __future__ import annotations

import pathlib
import socket
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = pathlib.Path(__file__).resolve().parents[1]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_sharded_stream_two_gpus(rt):
    n_gpus = rt._lib.fm_device_count()
    if n_gpus < 2:
        pytest.skip("needs at least two GPUs")
    world = 2
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                        "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
                        str(ROOT / "tests" / "multi_gpu_worker.py")], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert r.stdout.count("ok") == world
