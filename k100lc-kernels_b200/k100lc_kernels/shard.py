"""Row sharding of a linear layer over the GPUs of one node (one process per GPU).

Output rows are independent, so rank ``r`` of ``g`` holds rows ``[r*N/g, (r+1)*N/g)`` of the
packed weights and of the scales of every layer, the activations are replicated, and the
only exchange is the all-gather of ``y``.  Summation order inside a row does not depend on
the sharding, so results are bit-identical to a single GPU.  The reference is single-device
(runtime/hsa_rt.cpp:383-396); this module is an addition."""
from __future__ import annotations

import numpy as np

from . import synth


def row_range(n: int, rank: int, world: int) -> tuple[int, int]:
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if n % world:
        raise ValueError(f"N={n} does not split evenly over {world} GPUs")
    rows = n // world
    return rank * rows, (rank + 1) * rows


def stream_blocks(rank: int, world: int) -> list[int]:
    """Generator row blocks (``synth.STREAM_ROW_BLOCKS`` per layer) that rank ``rank`` holds."""
    nb = synth.STREAM_ROW_BLOCKS
    if nb % world:
        raise ValueError(f"{world} GPUs do not divide the {nb} row blocks of a stream layer")
    per = nb // world
    return list(range(rank * per, (rank + 1) * per))


def stream_layer_shard(layer: int, rank: int, world: int, n=synth.N_DEFAULT, k=synth.K_DEFAULT, seed=4) -> dict:
    """This rank's rows of one layer of the decode stream (packed weights, f16 scales)."""
    blks = [synth.stream_layer_block(layer, b, n, k, seed) for b in stream_blocks(rank, world)]
    return dict(wq=np.concatenate([b["wq"] for b in blks]), ws=np.concatenate([b["ws"] for b in blks]))


def exchange_ipc(rt, dist, ptr: int):
    """All ranks export the allocation behind ``ptr`` and open everybody else's; returns
    ``{rank: device address of that rank's ptr in this process}`` (own rank included)."""
    handle, off, size = rt.ipc_export(ptr)
    box = [None] * dist.get_world_size()
    dist.all_gather_object(box, (handle, off, size))
    me = dist.get_rank()
    out = {}
    for r, (h, o, sz) in enumerate(box):
        out[r] = ptr if r == me else rt.ipc_import(h, sz) + o
    return out
