#!/usr/bin/env python3
"""Benchmark of the weight-streaming quantized linear-layer path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (one "step" = one decoded token): 400 independent 17408 x 5120 W4A8 layers at
M = 1 — per layer `quant_act` (fp32 activations -> int8 per 128-group) then
`gemv_w4a8<1,false,1>` over that layer's own int4 weights and f16 group scales
(18.4 GB of weights in total, far larger than L2, so every step streams from HBM).
With G > 1 GPUs rank r holds rows [r*17408/G, (r+1)*17408/G) of every layer and an
all-gather of y follows each layer (strong scaling: the job is fixed).

One JSON line is printed by rank 0; see the keys at the bottom of `run_ours`.
`--impl reference` times the reference project's CPU implementation of the same path —
its NumPy arithmetic as restated in oracle/w4_oracle.py — on the host cores, on a
bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import json
import os
import pathlib
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT / "k100lc-kernels_b200"))

N, K, GROUP = 17408, 5120, 128
NG = K // GROUP
W_BYTES = N * K // 2                       # packed int4 weights of one layer
S_BYTES = N * NG * 2                       # f16 group scales of one layer
LAYER_BYTES = W_BYTES + S_BYTES            # algorithmic bytes of one W4 layer: 45 957 120
NVFP4_LAYER_BYTES = W_BYTES + N * (K // 16)   # E2M1 codes + E4M3 block scales: 50 135 040
METRIC = "decode weight-stream bandwidth, 400 x (17408x5120) W4A8 layers, M=1 (us/layer and ms/token alongside)"
WORKLOAD = "400-layer W4A8 M=1 decode weight stream, N=17408 K=5120 group=128, seed 4"


def log(msg: str) -> None:
    """Progress on stderr (rank-tagged), so that a stall can be located from the log."""
    print(f"[bench {time.strftime('%H:%M:%S')} rank {os.environ.get('RANK', '0')}] {msg}", file=sys.stderr, flush=True)


def watchdog(seconds: int) -> None:
    """End the process if the whole run takes longer than `seconds` (a hung collective must not
    hold the GPUs until someone else's limit expires)."""
    import signal

    def _fire(signum, frame):
        log(f"watchdog: no result after {seconds} s, giving up")
        os._exit(3)
    signal.signal(signal.SIGALRM, _fire)
    signal.alarm(seconds)


def peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "source": "measured (MEASURED_PEAKS.json)"}
    return {"hbm_gbs": 6650.0, "source": "fallback (6.65 TB/s, no MEASURED_PEAKS.json beside bench.py)"}


class ClockSampler:
    """SM clock, power and throttle-reason samples taken while the timed region runs.

    A thread polls NVML (read-only queries) every 2 ms, so that even a 50 ms timed region gets
    tens of samples; `window(t0, t1)` keeps the samples whose host time lies inside the region.
    Without NVML the summary says so instead of inventing numbers."""

    REASONS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20),
               ("sw_power_cap", 0x4))

    def __init__(self, device: int):
        self.samples, self.t0, self.t1 = [], None, None
        self._stop, self._thread, self._h, self._nv = threading.Event(), None, None, None
        vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
        ids = [v for v in vis.split(",") if v.strip().isdigit()]
        self.index = int(ids[device]) if device < len(ids) else device

    def __enter__(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            self._nv, self._h = nv, nv.nvmlDeviceGetHandleByIndex(self.index)
            self.smax = nv.nvmlDeviceGetMaxClockInfo(self._h, nv.NVML_CLOCK_SM)
        except Exception as e:                        # no NVML on this host
            self._why = f"NVML unavailable: {type(e).__name__}"
            return self
        self._thread = threading.Thread(target=self._poll, daemon=True)
        self._thread.start()
        return self

    def _poll(self):
        nv, h = self._nv, self._h
        reasons_of = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
        while not self._stop.is_set():
            try:
                self.samples.append((time.perf_counter(), nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM),
                                     int(reasons_of(h)), nv.nvmlDeviceGetPowerUsage(h) / 1000.0))
            except Exception:
                pass
            time.sleep(0.002)

    def window(self, t0: float, t1: float) -> None:
        self.t0, self.t1 = t0, t1

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
            try:
                self._nv.nvmlShutdown()
            except Exception:
                pass

    def summary(self) -> dict:
        rows = [r for r in self.samples if self.t0 is None or self.t0 <= r[0] <= self.t1]
        note = None
        if not rows and self.samples:
            # a region of a few milliseconds can fall between two polls (each poll is three NVML calls):
            # take the sample closest to it and say how far away it was
            near = min(self.samples, key=lambda r: min(abs(r[0] - self.t0), abs(r[0] - self.t1)))
            rows = [near]
            note = f"closest sample, {1e3 * min(abs(near[0] - self.t0), abs(near[0] - self.t1)):.1f} ms outside the timed region"
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [getattr(self, "_why", "no NVML sample")],
                    "samples": 0}
        bits = 0
        for r in rows:
            bits |= r[2]
        return {"sm_mhz": int(statistics.median(r[1] for r in rows)), "sm_min_mhz": min(r[1] for r in rows),
                "sm_max_mhz": int(self.smax), "power_w": round(statistics.median(r[3] for r in rows), 1),
                "reasons": [name for name, bit in self.REASONS if bits & bit], "samples": len(rows),
                "how": "NVML polled every 2 ms by a host thread during the timed region" + (f" ({note})" if note else "")}


# --------------------------------------------------------------------------- ours
class Stream:
    """The sharded 400-layer weight stream of one rank, resident in HBM."""

    def __init__(self, rt, layers: int, rank: int, world: int, dist=None):
        from k100lc_kernels import synth
        self.rt, self.layers, self.rank, self.world, self.dist = rt, layers, rank, world, dist
        self.rows = N // world
        blocks = synth.STREAM_ROW_BLOCKS // world
        self.wq = rt.alloc(layers * self.rows * (K // 2))
        self.ws = rt.alloc(layers * self.rows * NG * 2)
        self.x = rt.alloc(layers * K * 4)
        self.ysz = layers * N * 4
        self.y = rt.alloc(2 * self.ysz)                           # gathered outputs [layers][N], two buffers
        self.yloc = rt.alloc(layers * self.rows * 4) if world > 1 else self.y
        self.ae, self.ao = rt.alloc(K // 2), rt.alloc(K // 2)
        self.asc, self.asu = rt.alloc(NG * 4), rt.alloc(NG * 4)
        brow = N // synth.STREAM_ROW_BLOCKS
        jobs = [(l, rank * blocks + b) for l in range(layers) for b in range(blocks)]
        with cf.ThreadPoolExecutor(max_workers=min(16, os.cpu_count() or 8)) as ex:
            for (l, b), blk in zip(jobs, ex.map(lambda j: synth.stream_layer_block(j[0], j[1]), jobs)):
                lb = b - rank * blocks
                rt.upload(self.wq + (l * self.rows + lb * brow) * (K // 2), blk["wq"])
                rt.upload(self.ws + (l * self.rows + lb * brow) * NG * 2, blk["ws"])
        self.x_host = rt.pinned((layers, K), np.float32)
        for l in range(layers):
            self.x_host[l] = synth.stream_layer_x(l)
        self.y_host = rt.pinned((layers, N), np.float32)
        rt.upload(self.x, self.x_host)

    def wq_l(self, l): return self.wq + l * self.rows * (K // 2)
    def ws_l(self, l): return self.ws + l * self.rows * NG * 2

    def enqueue_token(self, quant=True, gemv=True, gather=True):
        """One decoded token: per layer quant_act -> gemv_w4a8 (-> all-gather of y)."""
        rt, rows = self.rt, self.rows
        for l in range(self.layers):
            if quant:
                rt.launch("quant_act", NG, 32, [self.x + l * K * 4, self.ae, self.ao, self.asc, self.asu, 1, K])
            if gemv:
                dst = (self.yloc + l * rows * 4) if self.world > 1 else (self.y + l * N * 4)
                rt.launch("gemv_w4a8<1,false,1>", rows // 4, 256,
                          [self.wq_l(l), self.ws_l(l), self.ae, self.ao, self.asc, self.asu, dst, rows, K])
            if gather and self.world > 1:
                rt.allgather(self.y + l * N * 4, self.yloc + l * rows * 4, rows * 4)

    def capture(self, **kw) -> int:
        self.rt.graph_begin()
        self.enqueue_token(**kw)
        return self.rt.graph_end()

    def capture_fused(self, host_mirror: bool = False, x: int | None = None, ybuf: int = 0) -> int:
        """One decoded token as TWO launches: quant_act over the x of all layers (grid y =
        layer), then the multi-layer stream kernel (bulk-copy ring over all layers' weights).
        With several GPUs the kernel's epilogue stores every y row into the y buffer of every
        peer as well (the all-gather, over NVLink peer mappings), so no collective follows.
        With `host_mirror` the pinned host array y_host is one more receiver of this rank's
        rows: the result reaches the host while the kernel runs, with no copy afterwards."""
        rt, nl = self.rt, self.layers
        if not hasattr(self, "tables"):
            base = self.rank * self.rows
            self.tables = [rt.stream_table([(self.wq_l(l), self.ws_l(l), self.x + l * K * 4, self.y + b * self.ysz + l * N * 4)
                                            for l in range(nl)], self.rows, K, base) for b in range(2)]
            self.table = self.tables[0]
            self.status = rt.alloc(4)
            rt.memset(self.status, 0, 4)
            self.ae_all, self.ao_all = rt.alloc(nl * K // 2), rt.alloc(nl * K // 2)
            self.asc_all, self.asu_all = rt.alloc(nl * NG * 4), rt.alloc(nl * NG * 4)
            self.npeers, self.deltas = 0, 0
            if self.world > 1:
                from k100lc_kernels.shard import exchange_ipc
                peers = exchange_ipc(rt, self.dist, self.y)
                bases = [peers[r] for r in range(self.world) if r != self.rank]
                self.deltas = rt.stream_peers(bases, self.y, 2 * self.ysz)
                self.npeers = len(bases)
            self.bases = bases if self.world > 1 else []
        npeers, deltas = self.npeers, self.deltas
        if host_mirror:
            if ybuf != 0:
                raise ValueError("the host receiver mirrors the first y buffer")
            if not hasattr(self, "deltas_host"):
                self.deltas_host = rt.stream_peers(self.bases + [self.y_host.ctypes.data], self.y, self.ysz)
            npeers, deltas = self.npeers + 1, self.deltas_host
        rt.graph_begin()
        rt.launch2d("quant_act", NG, nl, 32, 1, [self.x if x is None else x, self.ae_all, self.ao_all, self.asc_all, self.asu_all, nl, K])
        rt.launch("w4a8_decode_stream", 1, 1, [self.tables[ybuf], nl, self.rows, K, self.rank * self.rows, npeers,
                                               deltas, self.status,
                                               self.ae_all, self.ao_all, self.asc_all, self.asu_all, 0])
        return rt.graph_end()

    def y_digest(self) -> str:
        """SHA-1 of the gathered outputs of all layers on this rank."""
        import hashlib
        self.rt.sync()
        return hashlib.sha1(self.rt.download(self.y, self.layers * N, np.float32).tobytes()).hexdigest()


def time_graph(rt, graph, steps, warmup, barrier, counter=None, clocks=None) -> float:
    """ms per launch of `graph`, CUDA events on the engine stream, barrier + sync both sides.
    `counter`, if given, receives the number of kernels launched inside the timed region;
    `clocks` (a ClockSampler) is told the host-time window of the region."""
    for _ in range(warmup):
        rt.graph_launch(graph)
    rt.sync()
    barrier()
    e0, e1 = rt.event(), rt.event()
    n0 = rt.launch_count()
    t0 = time.perf_counter()
    rt.record(e0)
    for _ in range(steps):
        rt.graph_launch(graph)
    rt.record(e1)
    rt.sync()
    if clocks is not None:
        clocks.window(t0, time.perf_counter())
    barrier()
    if counter is not None:
        counter.append(rt.launch_count() - n0)
    return rt.elapsed_ms(e0, e1) / steps


def path_timings(rt, st: Stream, reps: int) -> dict:
    """us/layer and GB/s of quantiser + GEMV for W4A8, W4A4 and NVFP4 at M=1, each over a
    rotation of distinct layers (> L2) so that the weights come from HBM."""
    from k100lc_kernels import synth
    out = {}
    nl = min(st.layers, 64)
    rows = st.rows
    aq, asc4 = rt.alloc(K // 2), rt.alloc((K // 32) * 4)
    qa, qb, sc16 = rt.alloc(K // 2), rt.alloc(K // 2), rt.alloc((K // 16) * 4)
    nv_layers = min(nl, 64)
    nvs = rt.alloc(nv_layers * rows * (K // 16))
    rng = np.random.default_rng(2)
    from k100lc_kernels.quant import f32_to_e4m3_bits
    sb = f32_to_e4m3_bits(np.exp2(rng.uniform(-4.0, 2.0, size=(rows, K // 16))).astype(np.float32))
    for l in range(nv_layers):
        rt.upload(nvs + l * rows * (K // 16), np.roll(sb, l, axis=0))

    def graph_of(fn, count):
        rt.graph_begin()
        for l in range(count):
            fn(l)
        return rt.graph_end()

    def w4a8(l):
        rt.launch("quant_act", NG, 32, [st.x + l * K * 4, st.ae, st.ao, st.asc, st.asu, 1, K])
        rt.launch("gemv_w4a8<1,false,1>", rows // 4, 256,
                  [st.wq_l(l), st.ws_l(l), st.ae, st.ao, st.asc, st.asu, st.y + l * N * 4, rows, K])

    def w4a4(l):
        rt.launch("quant_act4", K // 32, 32, [st.x + l * K * 4, aq, asc4, 1, K])
        rt.launch("gemv_w4a4<1>", rows // 4, 256, [st.wq_l(l), st.ws_l(l), aq, asc4, st.y + l * N * 4, rows, K])

    def nvfp4(l):
        rt.launch("nvfp4_quant_act", K // 16, 64, [st.x + l * K * 4, qa, qb, sc16, 1, K])
        rt.launch("nvfp4_gemv<1,1>", rows // 4, 256,
                  [st.wq_l(l), nvs + (l % nv_layers) * rows * (K // 16), qa, qb, sc16, st.y + l * N * 4, rows, K, 0.05])

    def w4a8_only(l):
        rt.launch("gemv_w4a8<1,false,1>", rows // 4, 256,
                  [st.wq_l(l), st.ws_l(l), st.ae, st.ao, st.asc, st.asu, st.y + l * N * 4, rows, K])

    def w4a8_one(l):                                    # the quantiser inside the GEMV: one launch per layer
        rt.launch("quant_gemv_w4a8", rows // 4, 256, [st.wq_l(l), st.ws_l(l), st.x + l * K * 4, st.y + l * N * 4, rows, K])

    def w4a4_one(l):
        rt.launch("quant_gemv_w4a4", rows // 4, 256, [st.wq_l(l), st.ws_l(l), st.x + l * K * 4, st.y + l * N * 4, rows, K])

    frac = rows / N
    paths = [("w4a8_m1", w4a8, LAYER_BYTES), ("w4a4_m1", w4a4, LAYER_BYTES), ("nvfp4_m1", nvfp4, NVFP4_LAYER_BYTES),
             ("w4a8_m1_gemv_only", w4a8_only, LAYER_BYTES)]
    if rt.has("quant_gemv_w4a8"):
        paths += [("w4a8_m1_one_launch", w4a8_one, LAYER_BYTES), ("w4a4_m1_one_launch", w4a4_one, LAYER_BYTES)]
    for name, fn, nbytes in paths:
        g = graph_of(fn, nl)
        ms = time_graph(rt, g, reps, 3, lambda: None)
        rt.graph_free(g)
        us = ms * 1e3 / nl
        out[name] = {"us_per_layer": round(us, 3), "gb_per_s": round(nbytes * frac / us / 1e3, 1)}
    # four tokens per layer (the reference's launch sequence: one quantiser launch per token, one GEMV)
    from k100lc_kernels import W4Runner
    runner = W4Runner(rt)
    m4 = lambda kind: (lambda l: runner.gemv_device(kind, st.wq_l(l), st.ws_l(l), None, rows, K, x_dev=st.x + min(l, st.layers - 4) * K * 4,
                                                    y_dev=st.y + min(l, st.layers - 4) * N * 4, m=4, sync=False))
    for name, kind in (("w4a8_m4", "w4a8"), ("w4a4_m4", "w4a4")):
        if st.layers < 4:
            break
        fn = m4(kind)
        fn(0)                                           # the runner's scratch buffers exist before the capture
        rt.sync()
        g = graph_of(fn, nl)
        us = time_graph(rt, g, reps, 3, lambda: None) * 1e3 / nl
        rt.graph_free(g)
        out[name] = {"us_per_layer": round(us, 3), "gb_per_s": round(LAYER_BYTES * frac / us / 1e3, 1)}
    runner.close()
    if st.layers >= 4:                                  # NVFP4, four tokens (one 2-D quantiser launch, grid y = token)
        qa4, qb4, sc4n = rt.alloc(4 * K // 2), rt.alloc(4 * K // 2), rt.alloc(4 * (K // 16) * 4)

        def nvfp4_m4(l):
            lx = min(l, st.layers - 4)
            rt.launch2d("nvfp4_quant_act", K // 16, 4, 64, 1, [st.x + lx * K * 4, qa4, qb4, sc4n, 4, K])
            rt.launch("nvfp4_gemv<4,1>", rows // 4, 256,
                      [st.wq_l(l), nvs + (l % nv_layers) * rows * (K // 16), qa4, qb4, sc4n, st.y + lx * N * 4, rows, K, 0.05])
        g = graph_of(nvfp4_m4, nl)
        us = time_graph(rt, g, reps, 3, lambda: None) * 1e3 / nl
        rt.graph_free(g)
        out["nvfp4_m4"] = {"us_per_layer": round(us, 3), "gb_per_s": round(NVFP4_LAYER_BYTES * frac / us / 1e3, 1)}
        for ptr in (qa4, qb4, sc4n):
            rt.free(ptr)
    # W4A16: compressed-tensors bytes (offset-binary nibbles, bf16 group scales), fp32 activations
    from k100lc_kernels import DotLinear, Workspace
    nd = min(nl, 16)
    bf16_bits = lambda a: (a.astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    with Workspace(rt) as dws:
        dots = [DotLinear(rt, rows, K, "int4", rng.integers(0, 256, size=(rows, K // 2), dtype=np.uint8),
                          (bf16_bits(np.abs(rng.standard_normal((rows, NG))) * 0.01 + 1e-3),), ws=dws, tag=f"bench_dot{i}")
                for i in range(nd)]
        dot_fn = lambda l: dots[l % nd].forward_device(st.x + l * K * 4, 1)
        for l in range(nl):
            dot_fn(l)                                   # output buffers and layer tables exist before the capture
        rt.sync()
        g = graph_of(dot_fn, nl)
        us = time_graph(rt, g, reps, 3, lambda: None) * 1e3 / nl
        rt.graph_free(g)
        out["w4a16_m1"] = {"us_per_layer": round(us, 3), "gb_per_s": round(LAYER_BYTES * frac / us / 1e3, 1),
                           "what": "DotLinear.forward_device: activation split + bulk-copy ring, two launches per layer"}
        # the reference's launch sequence (int4_dot_k + reduce_blocks_k per token) on the same buffers
        for d in dots:
            d.ring = False
        for l in range(nl):
            dot_fn(l)
        rt.sync()
        g = graph_of(dot_fn, nl)
        us = time_graph(rt, g, reps, 3, lambda: None) * 1e3 / nl
        rt.graph_free(g)
        out["w4a16_m1_dot_reduce"] = {"us_per_layer": round(us, 3), "gb_per_s": round(LAYER_BYTES * frac / us / 1e3, 1)}
        # the same layers through the W4A16 stream kernel (activation split + stream, two launches)
        tab16 = rt.stream_table([(d.w, d.tables[0], st.x + i * K * 4, st.y + i * N * 4) for i, d in enumerate(dots)], rows, K, 0)
        st16 = rt.alloc(4)
        rt.memset(st16, 0, 4)
        rt.graph_begin()
        rt.launch("w4a16_decode_stream", 1, 1, [tab16, nd, rows, K, 0, 0, 0, st16, 0])
        g = rt.graph_end()
        us = time_graph(rt, g, reps, 3, lambda: None) * 1e3 / nd
        rt.graph_free(g)
        if int(rt.download(st16, 1, np.int32)[0]) != 0:
            raise RuntimeError("a bounded wait ran out in the W4A16 stream kernel")
        out["w4a16_m1_stream"] = {"us_per_layer": round(us, 3), "gb_per_s": round(LAYER_BYTES * frac / us / 1e3, 1),
                                  "note": f"{nd} layers per launch"}
        rt.free(tab16)
        rt.free(st16)
    # the same layers through the multi-layer stream kernels (two launches for all nl layers)
    table = rt.stream_table([(st.wq_l(l), st.ws_l(l), st.x + l * K * 4, st.y + l * N * 4) for l in range(nl)], rows, K, 0)
    status = rt.alloc(4)
    rt.memset(status, 0, 4)
    ae, ao, sc8, su8 = rt.alloc(nl * K // 2), rt.alloc(nl * K // 2), rt.alloc(nl * NG * 4), rt.alloc(nl * NG * 4)
    aq4, sc4 = rt.alloc(nl * K // 2), rt.alloc(nl * (K // 32) * 4)

    def s8():
        rt.launch2d("quant_act", NG, nl, 32, 1, [st.x, ae, ao, sc8, su8, nl, K])
        rt.launch("w4a8_decode_stream", 1, 1, [table, nl, rows, K, 0, 0, 0, status, ae, ao, sc8, su8, 0])

    def s4():
        rt.launch2d("quant_act4", K // 32, nl, 32, 1, [st.x, aq4, sc4, nl, K])
        rt.launch("w4a4_decode_stream", 1, 1, [table, nl, rows, K, 0, 0, 0, status, aq4, sc4, 0])

    for name, fn in (("w4a8_m1_stream", s8), ("w4a4_m1_stream", s4)):
        rt.graph_begin()
        fn()
        g = rt.graph_end()
        us = time_graph(rt, g, reps, 3, lambda: None) * 1e3 / nl
        rt.graph_free(g)
        out[name] = {"us_per_layer": round(us, 3), "gb_per_s": round(LAYER_BYTES * frac / us / 1e3, 1)}
    # NVFP4 through its stream kernel (one 2-D nvfp4_quant_act launch over the x of all layers in front)
    nvl = min(nl, nv_layers)
    tab_n = rt.stream_table([(st.wq_l(l), nvs + l * rows * (K // 16), st.x + l * K * 4, st.y + l * N * 4) for l in range(nvl)], rows, K, 0)
    qan, qbn, scn = rt.alloc(nvl * K // 2), rt.alloc(nvl * K // 2), rt.alloc(nvl * (K // 16) * 4)
    for key, cfg, what in (("nvfp4_m1_stream", None, "tcgen05 kind::mxf4 consumer (default)"),
                           ("nvfp4_m1_stream_dp4a", "1", "dp4a consumer ($FM_NVFP4_CFG=1)")):
        if cfg is None:
            os.environ.pop("FM_NVFP4_CFG", None)
        else:
            os.environ["FM_NVFP4_CFG"] = cfg
        rt.graph_begin()
        rt.launch2d("nvfp4_quant_act", K // 16, nvl, 64, 1, [st.x, qan, qbn, scn, nvl, K])
        rt.launch("nvfp4_decode_stream", 1, 1, [tab_n, nvl, rows, K, 0, 0, 0, status, qan, qbn, scn, 0.05, 0])
        g = rt.graph_end()
        us = time_graph(rt, g, reps, 3, lambda: None) * 1e3 / nvl
        rt.graph_free(g)
        out[key] = {"us_per_layer": round(us, 3), "gb_per_s": round(NVFP4_LAYER_BYTES * frac / us / 1e3, 1),
                    "note": f"{nvl} layers per launch; {what}"}
    os.environ.pop("FM_NVFP4_CFG", None)
    for ptr in (tab_n, qan, qbn, scn):
        rt.free(ptr)
    # four tokens per layer through the multi-token stream kernel (tokens = columns of the MMA)
    mt, nlm = 4, min(nl, st.layers // 4)
    if nlm > 0:
        tab_m = rt.stream_table([(st.wq_l(l), st.ws_l(l), st.x + l * mt * K * 4, st.y + l * mt * N * 4) for l in range(nlm)],
                                rows, K, (mt - 1) * N)
        aem, aom = rt.alloc(nlm * mt * K // 2), rt.alloc(nlm * mt * K // 2)
        scm, sum_ = rt.alloc(nlm * mt * NG * 4), rt.alloc(nlm * mt * NG * 4)
        rt.graph_begin()
        rt.launch2d("quant_act", NG, nlm * mt, 32, 1, [st.x, aem, aom, scm, sum_, nlm * mt, K])
        rt.launch("w4a8_decode_stream_m", 1, 1, [tab_m, nlm, rows, K, 0, 0, 0, status, aem, aom, scm, sum_, mt, N, 0])
        g = rt.graph_end()
        us = time_graph(rt, g, reps, 3, lambda: None) * 1e3 / nlm
        rt.graph_free(g)
        out["w4a8_m4_stream"] = {"us_per_layer": round(us, 3), "gb_per_s": round(LAYER_BYTES * frac / us / 1e3, 1)}
        for ptr in (aem, aom, scm, sum_):
            rt.free(ptr)
        if rt.has("w4a4_decode_stream_m"):
            aqm, scm = rt.alloc(nlm * mt * K // 2), rt.alloc(nlm * mt * (K // 32) * 4)
            rt.graph_begin()
            rt.launch2d("quant_act4", K // 32, nlm * mt, 32, 1, [st.x, aqm, scm, nlm * mt, K])
            rt.launch("w4a4_decode_stream_m", 1, 1, [tab_m, nlm, rows, K, 0, 0, 0, status, aqm, scm, mt, N, 0])
            g = rt.graph_end()
            us = time_graph(rt, g, reps, 3, lambda: None) * 1e3 / nlm
            rt.graph_free(g)
            out["w4a4_m4_stream"] = {"us_per_layer": round(us, 3), "gb_per_s": round(LAYER_BYTES * frac / us / 1e3, 1)}
            rt.free(aqm)
            rt.free(scm)
        rt.free(tab_m)
    # the same for NVFP4: four tokens per layer on the tcgen05 consumer (12 columns of B per token)
    nlm = min(nv_layers, st.layers) // mt
    if nlm > 0 and rt.has("nvfp4_decode_stream_m"):
        tab_m = rt.stream_table([(st.wq_l(l), nvs + l * rows * (K // 16), st.x + l * mt * K * 4, st.y + l * mt * N * 4)
                                 for l in range(nlm)], rows, K, (mt - 1) * N)
        qam, qbm, scm = rt.alloc(nlm * mt * K // 2), rt.alloc(nlm * mt * K // 2), rt.alloc(nlm * mt * (K // 16) * 4)
        rt.graph_begin()
        rt.launch2d("nvfp4_quant_act", K // 16, nlm * mt, 64, 1, [st.x, qam, qbm, scm, nlm * mt, K])
        rt.launch("nvfp4_decode_stream_m", 1, 1, [tab_m, nlm, rows, K, 0, 0, 0, status, qam, qbm, scm, 0.05, mt, N, 0])
        g = rt.graph_end()
        us = time_graph(rt, g, reps, 3, lambda: None) * 1e3 / nlm
        rt.graph_free(g)
        out["nvfp4_m4_stream"] = {"us_per_layer": round(us, 3), "gb_per_s": round(NVFP4_LAYER_BYTES * frac / us / 1e3, 1)}
        for ptr in (tab_m, qam, qbm, scm):
            rt.free(ptr)
    if int(rt.download(status, 1, np.int32)[0]) != 0:
        raise RuntimeError("a bounded wait ran out in a stream kernel")
    for p in (aq, asc4, qa, qb, sc16, nvs, table, status, ae, ao, sc8, su8, aq4, sc4):
        rt.free(p)
    return out


def gemm_timings(rt, st: "Stream", reps: int = 5) -> dict:
    """Prefill GEMM at M = 2048 (N = 17408, K = 5120): row quantiser + tcgen05 GEMM, W4A4 and W4A8,
    over a rotation of 8 distinct weight layers of the stream (356 MB, larger than L2)."""
    m, nl = 2048, min(8, st.layers)
    ops = 2.0 * m * N * K
    rng = np.random.default_rng(3)
    x = rt.alloc(m * K * 4)
    rt.upload(x, rng.standard_normal((m, K)).astype(np.float32))
    wsc = rt.alloc(NG * N * 4)
    rt.upload(wsc, (np.abs(rng.standard_normal((NG, N))) * 0.01 + 1e-3).astype(np.float32))
    aq4, aq8, asc, c = rt.alloc(m * K // 2), rt.alloc(m * K), rt.alloc(NG * m * 4), rt.alloc(m * N * 4)
    out = {}

    def timed(fn):
        rt.graph_begin()
        for l in range(nl):
            fn(l)
        g = rt.graph_end()
        ms = time_graph(rt, g, reps, 3, lambda: None) / nl
        rt.graph_free(g)
        return ms

    grid = (N // 64) * (m // 128)
    q4 = lambda l: rt.launch("quant_rows_fast_k", m, 256, [aq4, asc, x, K, 128, m, K, 0, NG])
    g4 = lambda l: rt.launch("gemm_w4a4_flat", grid, 256, [aq4, st.wq_l(l), asc, wsc, c, m, N, K, N // 64, 0])
    q8 = lambda l: rt.launch("quant_rows_a8_k", m, 256, [aq8, 0, asc, 0, x, K, 128, m, K, 0])
    g8 = lambda l: rt.launch("gemm_w4a8", grid, 256, [aq8, st.wq_l(l), asc, wsc, c, m, N, K])
    q4(0), q8(0)
    pk_int8 = 2 * json.loads((ROOT / "MEASURED_PEAKS.json").read_text())["bf16_tflops"] if (ROOT / "MEASURED_PEAKS.json").is_file() else 2 * 1590.0
    for name, qf, gf in (("w4a4", q4, g4), ("w4a8", q8, g8)):
        ms_g = timed(gf)
        ms_all = timed(lambda l: (qf(l), gf(l)))
        out[name] = {"gemm_ms": round(ms_g, 4), "quant_plus_gemm_ms": round(ms_all, 4),
                     "gemm_tmac_per_s": round(ops / 2 / ms_g / 1e9, 1), "quant_plus_gemm_tmac_per_s": round(ops / 2 / ms_all / 1e9, 1),
                     "gemm_tops": round(ops / ms_g / 1e9, 1),
                     "frac_of_int8_peak": round(ops / ms_g / 1e9 / pk_int8, 4)}
    out["int8_peak_tops_assumed"] = pk_int8
    # the tensor cores' own int8 rate, measured here: `mma_i8_peak` issues tcgen05.mma.kind::i8 (M128 N128 K32, the
    # GEMM's shape) back to back from shared memory on every SM; ops / device time of the launch
    iters = 8000
    cyc = rt.alloc(8 * rt.device_attr("sm_count"))
    rt.graph_begin()
    rt.launch("mma_i8_peak", 1, 128, [cyc, iters])
    g = rt.graph_end()
    ms_pk = time_graph(rt, g, 5, 3, lambda: None)
    rt.graph_free(g)
    sms = rt.device_attr("sm_count")
    issue_tops = 2.0 * 128 * 128 * 32 * iters * sms / ms_pk / 1e9
    cycles = rt.download(cyc, sms, np.int64)
    rt.free(cyc)
    out["int8_mma_peak_measured"] = {"tops": round(issue_tops, 1), "clocks_per_mma": round(float(np.median(cycles)) / iters, 2),
                                     "mac_per_clock_per_sm": round(128 * 128 * 32 / (float(np.median(cycles)) / iters), 1),
                                     "how": f"mma_i8_peak: {iters} tcgen05.mma.kind::i8 M128 N128 K32 per SM, operands in shared memory"}
    for name in ("w4a4", "w4a8"):
        out[name]["frac_of_measured_mma_peak"] = round(out[name]["gemm_tops"] / issue_tops, 4)
    out["note"] = ("frac_of_measured_mma_peak divides by the int8 tensor-core rate measured in this run; "
                   "frac_of_int8_peak uses 2 x the dense bf16 figure of MEASURED_PEAKS.json")
    if rt.gemm_status() != 0:
        raise RuntimeError("a bounded wait ran out in the GEMM kernel")
    # NVFP4 prefill (nvfp4_quant_act over all rows + nvfp4_gemm_kernel): per-16-block integers on mma.sync m16n8k16
    from k100lc_kernels.quant import f32_to_e4m3_bits
    nvs = rt.alloc(N * (K // 16))
    rt.upload(nvs, f32_to_e4m3_bits(np.exp2(rng.uniform(-4.0, 2.0, size=(N, K // 16))).astype(np.float32)))
    qa, qb, sc16 = rt.alloc(m * K // 2), rt.alloc(m * K // 2), rt.alloc(m * (K // 16) * 4)
    qn = lambda l: rt.launch2d("nvfp4_quant_act", K // 16, m, 64, 1, [x, qa, qb, sc16, m, K])
    gn = lambda l: rt.launch2d("nvfp4_gemm_kernel", N // 64, m // 64, 256, 1, [st.wq_l(l), nvs, qa, qb, sc16, c, m, N, K, 0.05])
    qn(0)
    ms_g, ms_all = timed(gn), timed(lambda l: (qn(l), gn(l)))
    out["nvfp4"] = {"gemm_ms": round(ms_g, 4), "quant_plus_gemm_ms": round(ms_all, 4), "gemm_tmac_per_s": round(ops / 2 / ms_g / 1e9, 1),
                    "gemm_tops": round(ops / ms_g / 1e9, 1),
                    "what": "nvfp4_gemm_kernel: one int32 per (token, row, 16-block), scaled in fp32 block by block"}
    for ptr in (x, wsc, aq4, aq8, asc, c, nvs, qa, qb, sc16):
        rt.free(ptr)
    return out


CPU_SAMPLE_LAYERS = 4      # layers of the stream that the CPU legs time per step (0.9 s per layer on 16 cores)


# The layer table of the checkpoint the reference measured its INT4 path on (docs/INT4.md:170-181): 400 quantized
# linear layers of 7 shapes, 12.54 GB of codes and scales.  (N, K, layers)
SHAPE_TABLE = ((17408, 5120, 128), (5120, 17408, 64), (10240, 5120, 48), (5120, 6144, 64), (6144, 5120, 48),
               (12288, 5120, 16), (1024, 5120, 32))


def shape_table_timings(rt, reps: int = 5) -> dict:
    """One decoded token over the 400-layer / 7-shape table with synthetic weights, per layer `quant_act` +
    `gemv_w4a8<1,false,1>` (W4A8) or `int4_dot_k` + `reduce_blocks_k` (W4A16, the path the reference timed it on: 91.9 ms
    per token there), each as one CUDA graph of by-name launches.  Every layer has its own weights (12.5 GB resident)."""
    rng = np.random.default_rng(7)
    from k100lc_kernels import DotLinear, Workspace
    total_bytes = sum((n * k // 2 + n * (k // 128) * 2) * c for n, k, c in SHAPE_TABLE)
    kmax, nmax = max(k for _, k, _ in SHAPE_TABLE), max(n for n, _, _ in SHAPE_TABLE)
    blk = rng.integers(0, 256, size=32 << 20, dtype=np.uint8)                      # 32 MiB of random codes, tiled
    x = rt.alloc(kmax * 4)
    rt.upload(x, rng.standard_normal(kmax).astype(np.float32))
    y = rt.alloc(nmax * 4)
    ae, ao, asc, asu = rt.alloc(kmax // 2), rt.alloc(kmax // 2), rt.alloc(kmax // 128 * 4), rt.alloc(kmax // 128 * 4)
    layers = []
    for n, k, c in SHAPE_TABLE:
        sc16 = (np.abs(rng.standard_normal((n, k // 128))) * 0.01 + 1e-3).astype(np.float16)
        for _ in range(c):
            wq, ws = rt.alloc(n * k // 2), rt.alloc(n * (k // 128) * 2)
            for off in range(0, n * k // 2, blk.size):
                rt.upload(wq + off, blk[:min(blk.size, n * k // 2 - off)])
            rt.upload(ws, sc16)
            layers.append((n, k, wq, ws))
    order = rng.permutation(len(layers))                   # shapes interleaved, as in a model
    out = {"layers": len(layers), "bytes": total_bytes}
    rt.graph_begin()
    for i in order:
        n, k, wq, ws = layers[i]
        rt.launch("quant_act", k // 128, 32, [x, ae, ao, asc, asu, 1, k])
        rt.launch("gemv_w4a8<1,false,1>", -(-n // 4), 256, [wq, ws, ae, ao, asc, asu, y, n, k])
    g = rt.graph_end()
    ms = time_graph(rt, g, reps, 3, lambda: None)
    rt.graph_free(g)
    out["w4a8_by_name"] = {"ms_per_token": round(ms, 4), "gb_per_s": round(total_bytes / ms / 1e6, 1)}
    per_shape = {}
    for n, k, c in SHAPE_TABLE:                            # each shape on its own (its layers rotate: > L2 except the smallest)
        mine = [l for l in layers if l[0] == n and l[1] == k]
        rt.graph_begin()
        for _n, _k, wq, ws in mine:
            rt.launch("quant_act", k // 128, 32, [x, ae, ao, asc, asu, 1, k])
            rt.launch("gemv_w4a8<1,false,1>", -(-n // 4), 256, [wq, ws, ae, ao, asc, asu, y, n, k])
        g = rt.graph_end()
        us = time_graph(rt, g, reps, 3, lambda: None) * 1e3 / len(mine)
        rt.graph_free(g)
        per_shape[f"{n}x{k}"] = {"layers": c, "us_per_layer": round(us, 3),
                                 "gb_per_s": round((n * k // 2 + n * (k // 128) * 2) / us / 1e3, 1)}
    out["w4a8_per_shape"] = per_shape
    # The same token as ONE launch of w4a8_layers_stream (plus one 2-D quant_act launch per distinct K): every layer has
    # its own input and its own y; a layer's x is padded with zeros to whole chunks of 5120 k, so that its codes are too.
    if rt.has("w4a8_layers_stream"):
        ks = sorted({k for _, k, _ in SHAPE_TABLE})
        kpad = {k: -(-k // 5120) * 5120 for k in ks}
        idx_of = {k: [i for i in order if layers[i][1] == k] for k in ks}        # layers of one K, in model order
        slot = {i: j for k in ks for j, i in enumerate(idx_of[k])}
        bufs = {}
        for k in ks:
            cnt, kp = len(idx_of[k]), kpad[k]
            xk = rt.alloc(cnt * kp * 4)
            xh = np.zeros((cnt, kp), dtype=np.float32)
            xh[:, :k] = rng.standard_normal((cnt, k)).astype(np.float32)
            rt.upload(xk, xh)
            bufs[k] = (xk, rt.alloc(cnt * kp // 2), rt.alloc(cnt * kp // 2), rt.alloc(cnt * kp // 128 * 4), rt.alloc(cnt * kp // 128 * 4))
        yall = rt.alloc(sum(n * c for n, _, c in SHAPE_TABLE) * 4)
        entries, yo = [], 0
        for i in order:
            n, k, wq, ws = layers[i]
            xk, a0, a1, a2, a3 = bufs[k]
            j, kp = slot[i], kpad[k]
            entries += rt.layer_chunks(wq, ws, yall + yo * 4, a0 + j * kp // 2, a1 + j * kp // 2, a2 + j * kp // 128 * 4,
                                       a3 + j * kp // 128 * 4, n, k)
            yo += n
        table, shp = rt.stream_table_var(entries)
        status = rt.alloc(4)
        rt.memset(status, 0, 4)
        rt.graph_begin()
        for k in ks:
            xk, a0, a1, a2, a3 = bufs[k]
            rt.launch2d("quant_act", kpad[k] // 128, len(idx_of[k]), 32, 1, [xk, a0, a1, a2, a3, len(idx_of[k]), kpad[k]])
        rt.launch("w4a8_layers_stream", 1, 1, [table, shp, len(entries), 0, 0, status, 0])
        g = rt.graph_end()
        ms = time_graph(rt, g, reps, 3, lambda: None)
        rt.graph_free(g)
        if int(rt.download(status, 1, np.int32)[0]) != 0:
            raise RuntimeError("w4a8_layers_stream reported a bounded wait that ran out")
        out["w4a8_layers_stream"] = {"ms_per_token": round(ms, 4), "gb_per_s": round(total_bytes / ms / 1e6, 1),
                                     "table_entries": len(entries),
                                     "what": "all 400 layers in one launch (a layer of the table = 5120 k of a weight matrix; "
                                             "longer rows are consecutive entries that add to y), one quant_act launch per K"}
        rt.free(table)
        rt.free(shp)
        per_shape_s = {}
        for n, k, c in SHAPE_TABLE:                        # each shape on its own through the same kernel
            xk, a0, a1, a2, a3 = bufs[k]
            kp = kpad[k]
            ent = []
            for i in [i for i in order if layers[i][0] == n and layers[i][1] == k]:
                j = slot[i]
                ent += rt.layer_chunks(layers[i][2], layers[i][3], yall, a0 + j * kp // 2, a1 + j * kp // 2,
                                       a2 + j * kp // 128 * 4, a3 + j * kp // 128 * 4, n, k)
            tb, sh = rt.stream_table_var(ent)
            rt.graph_begin()
            rt.launch("w4a8_layers_stream", 1, 1, [tb, sh, len(ent), 0, 0, status, 0])
            g = rt.graph_end()
            us = time_graph(rt, g, reps, 3, lambda: None) * 1e3 / c
            rt.graph_free(g)
            rt.free(tb)
            rt.free(sh)
            per_shape_s[f"{n}x{k}"] = {"us_per_layer": round(us, 3), "gb_per_s": round((n * k // 2 + n * (k // 128) * 2) / us / 1e3, 1)}
        out["w4a8_layers_stream_per_shape"] = per_shape_s
        for ptr in (status, yall):
            rt.free(ptr)
        for k in ks:
            for ptr in bufs[k]:
                rt.free(ptr)
    for _n, _k, wq, ws in layers:
        rt.free(wq)
        rt.free(ws)
    for ptr in (x, y, ae, ao, asc, asu):
        rt.free(ptr)
    return out


def cpu_sample(nl: int):
    """The first `nl` layers of the stream as the oracle takes them, and one pass over them
    (quant_act + W4A8 GEMV per layer in NumPy).  Both CPU legs — `cpu_baseline` inside the GPU arm and
    `--impl reference` — time this same function on this same sample, so they report one number."""
    sys.path.insert(0, str(ROOT / "oracle"))
    import w4_oracle as O
    from k100lc_kernels import synth
    lay = []
    for l in range(nl):
        blks = [synth.stream_layer_block(l, b) for b in range(synth.STREAM_ROW_BLOCKS)]
        lay.append((np.concatenate([b["wq"] for b in blks]).view(np.uint32), np.concatenate([b["ws"] for b in blks]),
                    synth.stream_layer_x(l)[None, :]))

    def step():
        for wq, ws, x in lay:
            q = O.quant_act(x)
            O.gemv_w4(wq, ws, q["q"], q["scale"], 128)
    return step


def time_cpu_sample(nl: int, steps: int, warmup: int) -> tuple[float, str]:
    """seconds per step of `cpu_sample(nl)` and the description of the sample."""
    step = cpu_sample(nl)
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    return dt, (f"first {nl} of the 400 layers per step (quant_act + W4A8 GEMV in NumPy, all host BLAS threads); "
                f"{steps} timed steps, {warmup} warm-up")


def cpu_baseline(sample_layers: int) -> dict:
    """The reference's CPU arithmetic (NumPy restatement in oracle/) on the host cores, on the
    first `sample_layers` layers of the same stream."""
    dt, sample = time_cpu_sample(sample_layers, 3, 1)
    return {"value": round(sample_layers * LAYER_BYTES / dt / 1e9, 4), "unit": "GB/s", "cores": os.cpu_count(),
            "kind": "port", "seconds_per_layer": round(dt / sample_layers, 3), "sample": sample}


def run_ours(args) -> int:
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            print(f"bench.py --gpus {args.gpus} must be started with torch.distributed.run "
                  f"--nproc-per-node {args.gpus}", file=sys.stderr)
            return 2
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group(backend="gloo")
    os.environ.setdefault("FM_DEVICE", str(local))
    from k100lc_kernels import Runtime
    rt = Runtime()                                  # raises when the CUDA library or a B200 is missing

    def barrier():
        if dist is not None:
            dist.barrier()

    watchdog(args.watchdog)
    if world > 1:
        box = [rt.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        rt.comm_init(box[0], world, rank)
        log("NCCL communicator ready")

    t_setup = time.perf_counter()
    st = Stream(rt, args.layers, rank, world, dist)
    setup_s = time.perf_counter() - t_setup
    log(f"stream resident after {setup_s:.1f} s")
    if world > 1:
        # NCCL sets up its connections on the first collective; do that eagerly, not inside a capture
        rt.allgather(st.y, st.yloc, st.rows * 4)
        rt.sync()
        barrier()
        log("eager all-gather done")

    fused = args.mode == "fused"
    graph = st.capture_fused() if fused else st.capture()
    log("graph captured")
    counted = []
    with ClockSampler(rt.device_attr("device")) as clocks:
        ms_step = time_graph(rt, graph, args.steps, args.warmup, barrier, counted, clocks)
    gpu_launches = counted[0]                       # kernels of this library inside the timed region

    log(f"timed region done: {ms_step:.3f} ms/step")
    # end to end through the C ABI with host buffers: x of all layers up, y of all layers back, every step.
    # Inputs and outputs are double-buffered on the device so that the copies of neighbouring steps run on the
    # copy engines beside the kernel of this step: the x of step t + 1 is uploaded on the engine's second queue
    # while step t runs (the upload waits for the last reader of its buffer, step t + 1 waits for the upload), and
    # this rank's rows of the y of step t are downloaded on the third queue while step t + 1 runs (step t + 2, the
    # next writer of that y buffer, waits for the download).  Every step still moves its own inputs and results
    # inside the timed region; fm_sync ends it.  --e2e-mirror: the kernel stores its rows into the pinned host array
    # itself instead (one more receiver of the writer warp, no copy afterwards).
    st.y_host[:] = np.nan
    e2e_h2d = world * args.layers * K * 4
    lo = rank * st.rows
    mirror = bool(args.e2e_mirror)

    def fetch_y(t):                                 # this rank's rows of all layers of y buffer t % 2 -> y_host
        if mirror:
            return
        rt.download_beside(st.y_host, st.y + (t % 2) * st.ysz + lo * 4, width=st.rows * 4, height=args.layers,
                           dpitch=N * 4, hpitch=N * 4, host_offset=lo * 4)

    if fused and world > 1:
        # Several GPUs: the activations are replicated, but uploading all of x on every rank makes the host
        # serve N x 8.2 MB per token.  Instead every rank uploads 1/N of x, the copy engines push that slice into
        # every peer's buffer over NVLink (beside the running kernel, no SM involved), and a step starts behind a
        # bounded acquire on N counters that the pushes bump.  Four buffers: a peer can be up to two steps behind
        # when a slice for the step after next arrives.
        from k100lc_kernels.shard import exchange_ipc
        NB, xb = 4, args.layers * K * 4
        sl = xb // world                                             # bytes of one rank's slice
        total_steps = max(1, args.warmup) + args.steps + 2
        xall = rt.alloc(NB * xb + NB * world * 4)
        rt.memset(xall, 0, NB * xb + NB * world * 4)
        fl0 = NB * xb                                                # offset of the counters: [NB][world] u32
        steps_dev = rt.alloc(4 * (total_steps + 2))
        rt.upload(steps_dev, np.arange(total_steps + 2, dtype=np.uint32))
        wstat = rt.alloc(4)
        rt.memset(wstat, 0, 4)
        rt.sync()
        barrier()
        px = exchange_ipc(rt, dist, xall)
        x_flat = st.x_host.reshape(-1).view(np.uint8)
        graphs = [st.capture_fused(host_mirror=mirror, x=xall + b * xb, ybuf=0 if mirror else b % 2) for b in range(NB)]
        step_no = [0]
        e2e_h2d = args.layers * K * 4

        def distribute(step):                                        # this rank's slice of the inputs of `step`
            b = step % NB
            mine = xall + b * xb + rank * sl
            rt.upload_beside(mine, x_flat[rank * sl:(rank + 1) * sl])
            for q in range(world):
                if q != rank:
                    rt.copy_beside(px[q] + b * xb + rank * sl, mine, sl)
            for q in range(world):                                   # counter of (buffer, this rank) := step + 1, after the data
                rt.copy_beside(px[q] + fl0 + (b * world + rank) * 4, steps_dev + 4 * (step + 1), 4)

        distribute(0)

        def e2e_step():
            t = step_no[0]
            distribute(t + 1)                                        # beside step t
            rt.launch("stream_flag_wait", 1, 128, [xall + fl0 + (t % NB) * world * 4, world, t + 1, wstat, 2000000])
            rt.download_join(1)                                      # y[t % 2] was last read by the download of step t - 2
            rt.graph_launch(graphs[t % NB])
            fetch_y(t)
            step_no[0] = t + 1
    elif fused:
        x2 = rt.alloc(args.layers * K * 4)
        xbuf = (st.x, x2)
        graphs = tuple(st.capture_fused(host_mirror=mirror, x=xbuf[b], ybuf=0 if mirror else b) for b in range(2))
        step_no = [0]
        rt.upload(st.x, st.x_host)                  # the very first step's inputs (outside the timed steps)

        def e2e_step():
            t = step_no[0]
            rt.upload_beside(xbuf[(t + 1) % 2], st.x_host)     # inputs of the next step, beside this one
            rt.download_join(1)
            rt.graph_launch(graphs[t % 2])
            rt.upload_join()
            fetch_y(t)
            step_no[0] = t + 1
    else:
        def e2e_step():
            rt.upload_async(st.x, st.x_host)
            rt.graph_launch(graph)
            rt.download_async(st.y_host, st.y)
    for _ in range(max(1, args.warmup)):
        e2e_step()
    rt.sync()
    barrier()
    e0, e1 = rt.event(), rt.event()
    rt.record(e0)
    for _ in range(args.steps):
        e2e_step()
    rt.record(e1)
    rt.sync()
    barrier()
    ms_e2e = rt.elapsed_ms(e0, e1) / args.steps
    if fused and world > 1:
        if int(rt.download(wstat, 1, np.int32)[0]) != 0:
            raise RuntimeError("an input slice of a peer did not arrive in time (stream_flag_wait gave up)")
        got_x = rt.download(xall + ((step_no[0] - 1) % NB) * xb, args.layers * K, np.float32)
        if not np.array_equal(got_x, st.x_host.reshape(-1)):
            raise RuntimeError("the gathered inputs of the last step differ from the host's x")
    if fused:                                       # what the host received is what the device holds
        last = 0 if mirror else (step_no[0] - 1) % 2
        dev_y = rt.download(st.y + last * st.ysz, args.layers * N, np.float32).reshape(args.layers, N)
        if not np.array_equal(st.y_host[:, lo:lo + st.rows].view(np.uint32), dev_y[:, lo:lo + st.rows].view(np.uint32)):
            raise RuntimeError("the host copy of this rank's rows of y differs from the device copy")

    # read ceiling: the copies of the stream kernel (same producer, ring and stage geometry) with consumers that only
    # release the stages — what the memory system allows this access pattern, measured in the same run
    ms_ceiling = None
    if fused and rt.has("w4a8_stream_read_ceiling"):
        rt.graph_begin()
        rt.launch2d("quant_act", NG, args.layers, 32, 1, [st.x, st.ae_all, st.ao_all, st.asc_all, st.asu_all, args.layers, K])
        rt.launch("w4a8_stream_read_ceiling", 1, 1, [st.tables[0], args.layers, st.rows, K, rank * st.rows, 0, 0, st.status,
                                                     st.ae_all, st.ao_all, st.asc_all, st.asu_all, 0])
        gc = rt.graph_end()
        ms_ceiling = time_graph(rt, gc, args.steps, 3, barrier)
        rt.graph_free(gc)
        log(f"read ceiling: {ms_ceiling:.3f} ms/step")
    # (after the two 20-step regions, which are then measured in the same state of the board)
    # the same graph back to back for at least a second: long enough for the board to settle at its power
    # limit, which a 20-step region (tens of milliseconds) is not
    sustained = None
    if args.sustain_s > 0:
        n_sus = max(args.steps, int(args.sustain_s * 1e3 / ms_step) + 1)
        with ClockSampler(rt.device_attr("device")) as clocks_sus:
            ms_sus = time_graph(rt, graph, n_sus, 3, barrier, None, clocks_sus)
        sustained = (ms_sus, n_sus, clocks_sus.summary())
        log(f"sustained region done: {ms_sus:.3f} ms/step over {n_sus} steps")
    # the dominant kernel alone, for the roofline: the fused stream kernel is the whole step;
    # in per-layer mode it is gemv_w4a8<1,false,1> without the quantiser
    if fused:
        ms_kern = ms_step
        status = int(rt.download(st.status, 1, np.int32)[0])
        if status != 0:
            raise RuntimeError(f"w4a8_decode_stream reported status {status} (a bounded wait ran out)")
        log("e2e done")
        digest = st.y_digest()
        barrier()
        rt.memset(st.y, 0xFF, args.layers * N * 4)
        rt.sync()
        barrier()
        ms_alt = time_graph(rt, st.capture(), max(3, args.steps // 4), 3, barrier)   # per-layer launches, for comparison
        log(f"per-layer launches: {ms_alt:.3f} ms/step")
        same = digest == st.y_digest()              # both schedules must leave identical bits in y
        if dist is not None:
            box = [None] * world
            dist.all_gather_object(box, (digest, same))
            same = all(b[1] for b in box) and len({b[0] for b in box}) == 1
        if not same:
            raise RuntimeError("the stream kernel and the per-layer launches (or two ranks) disagree on y")
    else:
        gk = st.capture(quant=False, gather=False)
        ms_kern = time_graph(rt, gk, max(3, args.steps // 2), 3, barrier)
        ms_alt = None

    log("reducing timings over ranks")
    if dist is not None:
        import torch
        t = torch.tensor([ms_step, ms_e2e, ms_kern, sustained[0] if sustained else 0.0, ms_ceiling or 0.0], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_step, ms_e2e, ms_kern = (float(v) for v in t[:3])
        if sustained:
            sustained = (float(t[3]),) + sustained[1:]
        if ms_ceiling:
            ms_ceiling = float(t[4])

    total_bytes = args.layers * LAYER_BYTES         # whole job, all ranks
    pk = peaks()
    us_kernel = ms_kern * 1e3 / (1 if fused else args.layers)
    bytes_per_launch = (args.layers if fused else 1) * LAYER_BYTES // world
    achieved = bytes_per_launch / us_kernel / 1e3             # GB/s of one GPU's kernel
    line = None
    if rank == 0:
        paths = path_timings(rt, st, 5) if (args.paths and world == 1) else None   # single-GPU diagnostics
        gemm = gemm_timings(rt, st) if (args.paths and world == 1) else None
        cpu = cpu_baseline(args.cpu_layers) if (world == 1 and args.cpu_layers > 0) else None
        shapes = None
        if args.paths and world == 1 and args.layers >= 400:
            # the stream's 18.4 GB go first: 12.5 GB more for the second workload's own weights
            for ptr in (st.wq, st.ws):
                rt.free(ptr)
            shapes = shape_table_timings(rt)
        line = {
            "metric": METRIC, "value": round(total_bytes / ms_step / 1e6, 1), "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 4),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8 x int4 -> int32, f32 scale",
            "data": "synthetic (seeded uniform int4 weights, |N(0,1)|*0.01+1e-3 f16 scales, N(0,1) activations)",
            "config": {"workload": WORKLOAD, "layers": args.layers, "rows_per_gpu": N // world,
                       "sharding": "output rows" + ((", all-gather of y by peer stores from the kernel epilogue (NVLink)"
                                                     if fused else ", all-gather of y per layer (NCCL)") if world > 1 else ""),
                       "y_check": "identical bits in y from the stream kernel and the per-layer launches on every rank"
                                  if fused else None,
                       "launch": ("two launches per token: quant_act over the x of all layers (grid y = layer), then "
                                  "w4a8_decode_stream (gemv_w4a8 of all layers, software-pipelined)") if fused else
                                 "one CUDA graph per token (quant_act + gemv_w4a8 per layer)",
                       "l2": "inputs (18.4 GB of weights) are larger than L2; no flush needed"},
            "ms_per_token": round(ms_step, 4), "us_per_layer": round(ms_step * 1e3 / args.layers, 3),
            "e2e": {"value": round(total_bytes / ms_e2e / 1e6, 1), "unit": "GB/s", "ms_per_step": round(ms_e2e, 4),
                    "h2d_bytes_per_step": e2e_h2d, "d2h_bytes_per_step": args.layers * N * 4,
                    "api": (("per step: fm_upload_beside(this rank's 1/N of the next step's x) + fm_copy_beside of that slice into every "
                             "peer's buffer (copy engines over NVLink) + stream_flag_wait on the N arrival counters + fm_graph_launch; "
                             if world > 1 else
                             "per step: fm_upload_beside(x of all layers for the next step, second device buffer) + fm_graph_launch + "
                             "fm_upload_join; ") +
                            ("the stream kernel stores each rank's rows of y into a pinned host array (fm_host_alloc, registered "
                             "through fm_stream_peers) while it runs; " if mirror else
                             "fm_download_beside of this rank's rows of the step's y into a pinned host array (third queue, beside "
                             "the next step; two y buffers, fm_download_join(1) before the next writer); ") +
                            "fm_sync ends the run") if fused else
                           "fm_upload_async(x) + fm_graph_launch + fm_download_async(y), pinned host buffers"},
            "gpu_launches": int(gpu_launches),
            "per_layer_launches": None if ms_alt is None else {
                "ms_per_token": round(ms_alt, 4), "us_per_layer": round(ms_alt * 1e3 / args.layers, 3),
                "gb_per_s": round(total_bytes / ms_alt / 1e6, 1),
                "what": "the same token as 800 by-name launches (quant_act, gemv_w4a8<1,false,1>) in one CUDA graph"
                        + (", plus an NCCL all-gather of y per layer" if world > 1 else "")},
            "roofline": {"bound": "hbm", "kernel": "w4a8_decode_stream" if fused else "gemv_w4a8<1,false,1>", "achieved": round(achieved, 1),
                         "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4),
                         "frac_of_nominal_8000": round(achieved / 8000.0, 4), "peak_source": pk["source"],
                         "us_per_launch": round(us_kernel, 3), "bytes_per_launch": bytes_per_launch,
                         "sustained": None if (sustained is None or not fused) else {
                             "ms_per_token": round(sustained[0], 4), "steps": sustained[1],
                             "achieved": round(bytes_per_launch / sustained[0] / 1e6, 1),
                             "frac": round(bytes_per_launch / sustained[0] / 1e6 / pk["hbm_gbs"], 4),
                             "frac_of_nominal_8000": round(bytes_per_launch / sustained[0] / 1e6 / 8000.0, 4),
                             "clocks": sustained[2],
                             "what": "the same graph launched back to back for at least --sustain-s seconds"},
                         "read_ceiling": None if not ms_ceiling else {
                             "ms_per_token": round(ms_ceiling, 4), "achieved": round(bytes_per_launch / ms_ceiling / 1e6, 1),
                             "frac_of_ceiling": round(ms_ceiling / ms_kern, 4),
                             "what": "w4a8_stream_read_ceiling: the stream kernel's copies (same ring and stages) with consumers "
                                     "that release every stage unread; frac_of_ceiling = its time / the stream kernel's time"},
                         # DRAM bytes of one launch: an ncu capture of the same kernel on 24 layers read
                         # 1 103 145 000 B and wrote 5 141 000 B; every weight byte is read once, so the traffic
                         # of a launch is that figure scaled by its layer count
                         "traffic": int(round((1103145000 + 5141000) / 24 * bytes_per_launch / LAYER_BYTES)) if fused else None,
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of a 24-layer launch of the "
                                           "same kernel, scaled by the layer count" if fused else None},
            "cpu_baseline": cpu, "clocks": clocks.summary(), "paths_m1": paths, "prefill_gemm_m2048": gemm,
            "shape_table_400_layers": shapes, "setup_seconds": round(setup_s, 1),
        }
    if line is not None:
        print(json.dumps(line), flush=True)
    if world > 1:
        log("result printed; tearing down")
        barrier()
        rt.comm_destroy()          # also releases the captured graphs that hold NCCL collectives
        dist.destroy_process_group()
    return 0


# ---------------------------------------------------------------------- reference arm
def run_reference(args) -> int:
    """The reference's CPU implementation of the path on the host cores: each step is a
    bounded sample (the first `--cpu-layers` layers) of the same stream."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    world = int(os.environ.get("WORLD_SIZE", "1"))
    nl = max(1, min(args.cpu_layers, CPU_SAMPLE_LAYERS))
    steps, warmup = max(1, min(args.steps, 3)), max(1, min(args.warmup, 1))
    dt, sample = time_cpu_sample(nl, steps, warmup)
    val = round(nl * LAYER_BYTES / dt / 1e9, 4)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "GB/s", "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": round(dt * 1e3 * 400 / nl, 1), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8 x int4 -> int32, f32 scale", "data": "synthetic",
        "config": {"workload": WORKLOAD, "layers": 400, "sampled_layers": nl},
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": os.cpu_count(), "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference's device code targets gfx926 and cannot run here; its CPU path is the NumPy "
                "oracle of its self-test, restated in oracle/w4_oracle.py and pinned to it by tests/golden"}), flush=True)
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=400)
    ap.add_argument("--mode", default="fused", choices=["fused", "graph"],
                    help="fused: one multi-layer kernel per token; graph: 2 by-name launches per layer")
    ap.add_argument("--cpu-layers", type=int, default=CPU_SAMPLE_LAYERS, help="layers of the stream timed on the CPU (0 = skip)")
    ap.add_argument("--no-paths", dest="paths", action="store_false", help="skip the per-path M=1 timings")
    ap.add_argument("--watchdog", type=int, default=600, help="give up after this many seconds")
    ap.add_argument("--e2e-mirror", action="store_true",
                    help="end to end: the kernel stores y into the pinned host array itself instead of a download beside the next step")
    ap.add_argument("--sustain-s", type=float, default=1.0,
                    help="also time the step back to back for this many seconds (0 = skip)")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup) if args.impl == "ours" else args.warmup
    return run_reference(args) if args.impl == "reference" else run_ours(args)


if __name__ == "__main__":
    raise SystemExit(main())
