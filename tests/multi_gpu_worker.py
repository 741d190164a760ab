"""Worker of tests/test_gpu_multi.py: one process per GPU (torch.distributed.run), a small
row-sharded decode stream with the all-gather done by peer stores, checked against the
oracle on every rank, and the NCCL all-gather entry checked beside it."""
from __future__ import annotations

import os
import pathlib
import sys

import numpy as np
import torch.distributed as dist

ROOT = pathlib.Path(__file__).resolve().parents[1]
sys.path[:0] = [str(ROOT / "k100lc-kernels_b200"), str(ROOT / "oracle")]
import w4_oracle as O  # noqa: E402
from k100lc_kernels import Runtime, shard, synth  # noqa: E402


def main() -> int:
    dist.init_process_group(backend="gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    os.environ["FM_DEVICE"] = os.environ.get("LOCAL_RANK", "0")
    rt = Runtime()
    n, k, layers = 1024, 5120, 4
    r0, r1 = shard.row_range(n, rank, world)
    rows = r1 - r0
    full = [dict(wq=np.concatenate([synth.stream_layer_block(l, b, n, k)["wq"] for b in range(8)]),
                 ws=np.concatenate([synth.stream_layer_block(l, b, n, k)["ws"] for b in range(8)]),
                 x=synth.stream_layer_x(l, k)) for l in range(layers)]
    x_all = rt.alloc(layers * k * 4)
    rt.upload(x_all, np.stack([L["x"] for L in full]))
    y = rt.alloc(layers * n * 4 + layers * 4)          # the gathered outputs, then one completion counter per layer
    rt.memset(y, 0xFF, layers * n * 4)
    flags = y + layers * n * 4
    rt.memset(flags, 0, layers * 4)
    ptrs = []
    for l, L in enumerate(full):
        pwq, pws = rt.alloc(rows * k // 2), rt.alloc(rows * (k // 128) * 2)
        rt.upload(pwq, L["wq"][r0:r1])
        rt.upload(pws, L["ws"][r0:r1])
        ptrs.append((pwq, pws, x_all + l * k * 4, y + l * n * 4))
    table = rt.stream_table(ptrs, rows, k, r0)
    peers = shard.exchange_ipc(rt, dist, y)
    deltas = rt.stream_peers([peers[r] for r in range(world) if r != rank], y, layers * n * 4 + layers * 4)
    ae, ao = rt.alloc(layers * k // 2), rt.alloc(layers * k // 2)
    asc, asu = rt.alloc(layers * (k // 128) * 4), rt.alloc(layers * (k // 128) * 4)
    status = rt.alloc(4)
    rt.memset(status, 0, 4)
    rt.sync()
    dist.barrier()                     # every rank has initialised its y before anyone stores into it
    rt.launch2d("quant_act", k // 128, layers, 32, 1, [x_all, ae, ao, asc, asu, layers, k])
    rt.launch("w4a8_decode_stream", 1, 1, [table, layers, rows, k, r0, world - 1, deltas, status, ae, ao, asc, asu, flags])
    # acquire side of the completion counters: every CTA of every rank adds one per layer on every receiver, so this
    # GPU's counters reach world x CTAs once all rows of a layer have arrived here — no host barrier in between
    ctas = min(rt.device_attr("sm_count"), rows)
    wstat = rt.alloc(4)
    rt.memset(wstat, 0, 4)
    rt.launch("stream_flag_wait", 1, 128, [flags, layers, world * ctas, wstat, 1000000])
    got = rt.download(y, layers * n, np.float32).reshape(layers, n)      # ordered behind the wait kernel on the stream
    assert int(rt.download(wstat, 1, np.int32)[0]) == 0, "a completion counter did not reach its target in time"
    assert (rt.download(flags, layers, np.uint32) == world * ctas).all()
    assert int(rt.download(status, 1, np.int32)[0]) == 0
    dist.barrier()
    for l, L in enumerate(full):
        q = O.quant_act(L["x"][None, :])
        ref = O.gemv_w4(L["wq"].view(np.uint32), L["ws"], q["q"], q["scale"], 128)["y"][0]
        assert O.rel_err(got[l], ref) < 1e-5, f"rank {rank} layer {l}"

    # NCCL all-gather entry: gather each rank's slice of layer 0 and compare with the peer-store result
    uid = [rt.comm_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(uid, src=0)
    rt.comm_init(uid[0], world, rank)
    recv = rt.alloc(n * 4)
    rt.allgather(recv, y + r0 * 4, rows * 4)
    rt.sync()
    assert np.array_equal(rt.download(recv, n, np.float32), got[0])
    # a peer window that is not an imported allocation is refused
    try:
        rt.stream_peers([y], y, layers * n * 4)
        raise AssertionError("a local address was accepted as a peer window")
    except RuntimeError:
        pass
    rt.comm_destroy()
    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank} ok")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
