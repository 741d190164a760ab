"""CPU tier, two gloo ranks: the host side of the row-sharded path — each rank generates
only its own rows, the shards tile the global layer exactly, per-shard oracle outputs
gathered over the process group equal the single-process result bit for bit, and the
max-over-ranks reduction the benchmark uses for its timing works."""
from __future__ import annotations

import os
import pathlib
import socket
import subprocess
import sys

import numpy as np
import pytest

ROOT = pathlib.Path(__file__).resolve().parents[1]

WORKER = r'''
import os, sys
import numpy as np
import torch, torch.distributed as dist
sys.path[:0] = [r"%(pkg)s", r"%(oracle)s"]
import w4_oracle as O
from k100lc_kernels import shard, synth

dist.init_process_group(backend="gloo")
rank, world = dist.get_rank(), dist.get_world_size()
n, k, layers = 64, 1024, 3
r0, r1 = shard.row_range(n, rank, world)
assert shard.stream_blocks(rank, world) == list(range(rank * 8 // world, (rank + 1) * 8 // world))
ys = []
for l in range(layers):
    full = shard.stream_layer_shard(l, 0, 1, n, k)                 # what one GPU would hold
    mine = shard.stream_layer_shard(l, rank, world, n, k)
    assert np.array_equal(mine["wq"], full["wq"][r0:r1]) and np.array_equal(mine["ws"], full["ws"][r0:r1])
    x = synth.stream_layer_x(l, k)[None, :]
    q = O.quant_act(x)
    y_loc = O.gemv_w4(mine["wq"].view(np.uint32), mine["ws"], q["q"], q["scale"], 128)["y"][0]
    parts = [torch.zeros(r1 - r0) for _ in range(world)]
    dist.all_gather(parts, torch.from_numpy(y_loc.copy()))
    y = torch.cat(parts).numpy()
    y_one = O.gemv_w4(full["wq"].view(np.uint32), full["ws"], q["q"], q["scale"], 128)["y"][0]
    assert np.array_equal(y, y_one), "sharded result differs from the single-GPU result"
    ys.append(y)
t = torch.tensor([1.0 + rank], dtype=torch.float64)
dist.all_reduce(t, op=dist.ReduceOp.MAX)
assert float(t) == float(world)
box = [b"id-from-rank-0" if rank == 0 else None]
dist.broadcast_object_list(box, src=0)
assert box[0] == b"id-from-rank-0"
dist.barrier()
dist.destroy_process_group()
print("rank", rank, "ok")
'''


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2])
def test_row_sharding_two_ranks(tmp_path, world):
    script = tmp_path / "worker.py"
    script.write_text(WORKER % {"pkg": ROOT / "k100lc-kernels_b200", "oracle": ROOT / "oracle"})
    env = dict(os.environ, OMP_NUM_THREADS="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                        "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), str(script)],
                       capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert r.stdout.count("ok") == world


def test_shard_arithmetic():
    import sys as _s
    from k100lc_kernels import shard
    assert shard.row_range(17408, 3, 8) == (6528, 8704)
    assert shard.stream_blocks(1, 4) == [2, 3]
    with pytest.raises(ValueError):
        shard.row_range(10, 0, 3)
    with pytest.raises(ValueError):
        shard.row_range(8, 2, 2)
    with pytest.raises(ValueError):
        shard.stream_blocks(0, 3)
