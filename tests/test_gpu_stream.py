"""GPU tier: the multi-layer decode stream (one 2-D quant_act launch over all layers, then
w4a8_decode_stream) against the per-layer kernels and the oracle, and the validation of
its layer table."""
from __future__ import annotations

import numpy as np
import pytest

import w4_oracle as O
from gpu_util import Bufs
from k100lc_kernels import W4Runner, synth

pytestmark = pytest.mark.gpu
REL = 1e-5
K = 5120


class Codes:
    """quant_act outputs of all layers: x [L][K] -> ae, ao [L][K/2], asc, asu [L][K/128]."""

    def __init__(self, rt, b, layers):
        nl = len(layers)
        self.x = b.put(np.stack([L["x"][0] for L in layers]))
        self.ae, self.ao = b.zeros(nl * K // 2, np.int8), b.zeros(nl * K // 2, np.int8)
        self.asc, self.asu = b.zeros(nl * K // 128), b.zeros(nl * K // 128, np.int32)
        self.args = [self.ae, self.ao, self.asc, self.asu]
        self.nl = nl

    def quantise(self, rt):
        rt.launch2d("quant_act", K // 128, self.nl, 32, 1, [self.x, self.ae, self.ao, self.asc, self.asu, self.nl, K])


def _run_stream(rt, b, layers, rows, row_base=0, n_out=None):
    n_out = n_out or rows
    ptrs, ys = [], []
    codes = Codes(rt, b, layers)
    for i, L in enumerate(layers):
        py = b.zeros(n_out, np.float32, np.nan)
        ys.append(py)
        ptrs.append((b.put(L["wq"]), b.put(L["ws"]), codes.x + i * K * 4, py))
    table = rt.stream_table(ptrs, rows, K, row_base)
    status = b.zeros(1, np.int32)
    codes.quantise(rt)
    rt.launch("w4a8_decode_stream", 1, 1, [table, len(layers), rows, K, row_base, 0, 0, status] + codes.args + [0])
    out = [b.get(py, n_out) for py in ys]
    assert int(b.get(status, 1, np.int32)[0]) == 0
    rt.free(table)
    return out, ptrs


@pytest.mark.parametrize("rows,nlayers", [(1000, 5), (148, 3), (100, 2), (17408, 3)])
def test_stream_matches_per_layer_and_oracle(rt, rows, nlayers):
    layers = [synth.rt4_layer(rows, K, 1, seed=700 + i) for i in range(nlayers)]
    runner = W4Runner(rt)
    with Bufs(rt) as b:
        got, ptrs = _run_stream(rt, b, layers, rows)
        for L, y, (pwq, pws, px, _py) in zip(layers, got, ptrs):
            q = O.quant_act(L["x"])
            ref = O.gemv_w4(L["wq"], L["ws"], q["q"], q["scale"], 128)["y"][0]
            assert O.rel_err(y, ref) < REL
            per_layer = runner.gemv("w4a8", pwq, pws, L["x"], rows, K)[0]
            assert O.rel_err(y, per_layer) < REL
    runner.close()


def test_stream_row_base_and_repeat(rt):
    """A rank's shard writes rows [row_base, row_base+rows) of a longer y; a second launch on
    the same table gives the same bits."""
    rows, base, n_out = 520, 1040, 2080
    layers = [synth.rt4_layer(rows, K, 1, seed=800 + i) for i in range(4)]
    with Bufs(rt) as b:
        ptrs, ys = [], []
        codes = Codes(rt, b, layers)
        for i, L in enumerate(layers):
            py = b.zeros(n_out, np.float32, np.nan)
            ys.append(py)
            ptrs.append((b.put(L["wq"]), b.put(L["ws"]), codes.x + i * K * 4, py))
        table = rt.stream_table(ptrs, rows, K, base)
        status = b.zeros(1, np.int32)
        argv = [table, 4, rows, K, base, 0, 0, status] + codes.args + [0]
        codes.quantise(rt)
        rt.launch("w4a8_decode_stream", 1, 1, argv)
        first = [b.get(py, n_out) for py in ys]
        rt.launch("w4a8_decode_stream", 1, 1, argv)
        second = [b.get(py, n_out) for py in ys]
        for L, y1, y2 in zip(layers, first, second):
            q = O.quant_act(L["x"])
            ref = O.gemv_w4(L["wq"], L["ws"], q["q"], q["scale"], 128)["y"][0]
            assert O.rel_err(y1[base:base + rows], ref) < REL
            assert np.isnan(y1[:base]).all() and np.isnan(y1[base + rows:]).all()
            assert np.array_equal(y1[base:base + rows], y2[base:base + rows])
        # the table is only accepted as validated, with the shapes it was validated for
        with pytest.raises(RuntimeError, match="rc=-4"):
            rt.launch("w4a8_decode_stream", 1, 1, [table, 4, rows + 8, K, base, 0, 0, status] + codes.args + [0])
        rt.memset(table, 0, 32)                         # overwriting it un-validates it
        with pytest.raises(RuntimeError, match="rc=-4"):
            rt.launch("w4a8_decode_stream", 1, 1, argv)
        rt.free(table)
        # a table whose y is too short for row_base + rows is refused
        with pytest.raises(RuntimeError, match="fm_stream_table"):
            rt.stream_table([(ptrs[0][0], ptrs[0][1], ptrs[0][2], ys[0])], rows, K, n_out)
        assert int(b.get(status, 1, np.int32)[0]) == 0


def test_w4a4_stream_matches_oracle(rt):
    """The int4-activation variant: one 2-D quant_act4 launch, then w4a4_decode_stream."""
    rows, nl = 1000, 4
    layers = [synth.rt4_layer(rows, K, 1, seed=850 + i) for i in range(nl)]
    with Bufs(rt) as b:
        x = b.put(np.stack([L["x"][0] for L in layers]))
        aq, asc = b.zeros(nl * K // 2, np.uint8), b.zeros(nl * K // 32)
        ptrs, ys = [], []
        for i, L in enumerate(layers):
            py = b.zeros(rows, np.float32, np.nan)
            ys.append(py)
            ptrs.append((b.put(L["wq"]), b.put(L["ws"]), x + i * K * 4, py))
        table = rt.stream_table(ptrs, rows, K, 0)
        status = b.zeros(1, np.int32)
        rt.launch2d("quant_act4", K // 32, nl, 32, 1, [x, aq, asc, nl, K])
        rt.launch("w4a4_decode_stream", 1, 1, [table, nl, rows, K, 0, 0, 0, status, aq, asc, 0])
        got = [b.get(py, rows) for py in ys]
        assert int(b.get(status, 1, np.int32)[0]) == 0
        rt.free(table)
    for L, y in zip(layers, got):
        q = O.quant_act4(L["x"])
        assert O.rel_err(y, O.gemv_w4(L["wq"], L["ws"], q["q"], q["scale"], 32)["y"][0]) < REL


@pytest.mark.parametrize("kernel,cfg", [("w4a8_decode_stream", None), ("w4a4_decode_stream", None), ("w4a8_decode_stream", "6")])
def test_stream_delivers_y_to_pinned_host_memory(rt, monkeypatch, kernel, cfg):
    """A pinned host buffer registered through fm_stream_peers is one more receiver of y: after
    fm_sync it holds the bits of the device copy, rows outside the shard untouched.  ($FM_STREAM_CFG=6: whole stages
    per CTA from a position that moves with the layer, here with CTAs that have no row in a layer.)"""
    if cfg is not None:
        monkeypatch.setenv("FM_STREAM_CFG", cfg)
    rows, base, n_out, nl = 1500, 500, 2500, 5
    a4 = kernel.startswith("w4a4")
    layers = [synth.rt4_layer(rows, K, 1, seed=870 + i) for i in range(nl)]
    host = rt.pinned((nl, n_out), np.float32)
    host[:] = np.nan
    with Bufs(rt) as b:
        x = b.put(np.stack([L["x"][0] for L in layers]))
        y = b.zeros(nl * n_out, np.float32, np.nan)
        ptrs = [(b.put(L["wq"]), b.put(L["ws"]), x + i * K * 4, y + i * n_out * 4) for i, L in enumerate(layers)]
        table = rt.stream_table(ptrs, rows, K, base)
        status = b.zeros(1, np.int32)
        # ordinary (pageable) host memory is not an accepted receiver
        with pytest.raises(RuntimeError, match="fm_stream_peers"):
            rt.stream_peers([np.zeros(nl * n_out, np.float32).ctypes.data], y, nl * n_out * 4)
        deltas = rt.stream_peers([host.ctypes.data], y, nl * n_out * 4)
        if a4:
            aq, asc = b.zeros(nl * K // 2, np.uint8), b.zeros(nl * K // 32)
            rt.launch2d("quant_act4", K // 32, nl, 32, 1, [x, aq, asc, nl, K])
            rt.launch(kernel, 1, 1, [table, nl, rows, K, base, 1, deltas, status, aq, asc, 0])
        else:
            ae, ao = b.zeros(nl * K // 2, np.int8), b.zeros(nl * K // 2, np.int8)
            asc, asu = b.zeros(nl * K // 128), b.zeros(nl * K // 128, np.int32)
            rt.launch2d("quant_act", K // 128, nl, 32, 1, [x, ae, ao, asc, asu, nl, K])
            rt.launch(kernel, 1, 1, [table, nl, rows, K, base, 1, deltas, status, ae, ao, asc, asu, 0])
        dev = b.get(y, nl * n_out).reshape(nl, n_out)          # drains the stream
        assert int(b.get(status, 1, np.int32)[0]) == 0
        rt.free(table)
        rt.free(deltas)
    assert np.array_equal(host.view(np.uint32), dev.view(np.uint32))
    assert np.isnan(host[:, :base]).all() and np.isnan(host[:, base + rows:]).all()
    for i, L in enumerate(layers):
        q = O.quant_act4(L["x"]) if a4 else O.quant_act(L["x"])
        ref = O.gemv_w4(L["wq"], L["ws"], q["q"], q["scale"], 32 if a4 else 128)["y"][0]
        assert O.rel_err(host[i, base:base + rows], ref) < REL


def test_stream_many_rows_per_cta(rt):
    """More rows per CTA than the shared-memory output tile holds (512): y is then stored row by
    row.  The oracle checks the first and last rows, the per-layer kernel all of them."""
    sms = rt.device_attr("sm_count")
    rows = sms * 512 + 64
    rng = np.random.default_rng(890)                       # (synth.rt4_layer is too slow for 75 840 rows)
    L = {"wq": rng.integers(0, 2**32, size=(rows, K // 8), dtype=np.uint32),
         "ws": (np.abs(rng.standard_normal((rows, K // 128))) * 0.01 + 1e-3).astype(np.float16),
         "x": rng.standard_normal((1, K)).astype(np.float32)}
    runner = W4Runner(rt)
    with Bufs(rt) as b:
        got, ptrs = _run_stream(rt, b, [L], rows)
        per_layer = runner.gemv("w4a8", ptrs[0][0], ptrs[0][1], L["x"], rows, K)[0]
        assert np.array_equal(got[0].view(np.uint32), per_layer.view(np.uint32))
    runner.close()
    q = O.quant_act(L["x"])
    for sl in (slice(0, 1024), slice(rows - 1024, rows)):
        ref = O.gemv_w4(L["wq"][sl], L["ws"][sl], q["q"], q["scale"], 128)["y"][0]
        assert O.rel_err(got[0][sl], ref) < REL


@pytest.mark.parametrize("m,rows,row_base", [(2, 1000, 0), (3, 148, 0), (4, 17408, 0), (4, 700, 300)])
def test_stream_several_tokens_matches_oracle(rt, monkeypatch, m, rows, row_base):
    """w4a8_decode_stream_m: M tokens per layer as the columns of the MMA; y of a layer is token-major.  The default
    schedule (two consumer groups) and the one-group schedule ($FM_STREAM_M_CFG=0, whose accumulators the _iacc entry
    dumps) leave identical bits."""
    nl = 3
    ystride = row_base + rows + 24
    layers = [synth.rt4_layer(rows, K, m, seed=900 + 10 * m + i) for i in range(nl)]
    with Bufs(rt) as b:
        x = b.put(np.stack([L["x"] for L in layers]))                       # [nl][m][K]
        ae, ao = b.zeros(nl * m * K // 2, np.int8), b.zeros(nl * m * K // 2, np.int8)
        asc, asu = b.zeros(nl * m * K // 128), b.zeros(nl * m * K // 128, np.int32)
        y = b.zeros(nl * m * ystride, np.float32, np.nan)
        ptrs = [(b.put(L["wq"]), b.put(L["ws"]), x + i * m * K * 4, y + i * m * ystride * 4) for i, L in enumerate(layers)]
        table = rt.stream_table(ptrs, rows, K, row_base + (m - 1) * ystride)   # footprint of all m tokens
        status = b.zeros(1, np.int32)
        rt.launch2d("quant_act", K // 128, nl * m, 32, 1, [x, ae, ao, asc, asu, nl * m, K])
        argv = [table, nl, rows, K, row_base, 0, 0, status, ae, ao, asc, asu, m, ystride, 0]
        rt.launch("w4a8_decode_stream_m", 1, 1, argv)
        got = b.get(y, nl * m * ystride).reshape(nl, m, ystride)
        assert int(b.get(status, 1, np.int32)[0]) == 0
        monkeypatch.setenv("FM_STREAM_M_CFG", "0")
        rt.memset(y, 0xFF, nl * m * ystride * 4)
        rt.launch("w4a8_decode_stream_m", 1, 1, argv)
        one_group = b.get(y, nl * m * ystride).reshape(nl, m, ystride)
        monkeypatch.delenv("FM_STREAM_M_CFG")
        assert np.array_equal(got[:, :, row_base:row_base + rows].view(np.uint32),
                              one_group[:, :, row_base:row_base + rows].view(np.uint32))
        with pytest.raises(RuntimeError, match="rc=-4"):                    # a table validated for one token is refused
            t1 = rt.stream_table(ptrs, rows, K, row_base)
            try:
                rt.launch("w4a8_decode_stream_m", 1, 1, [t1] + argv[1:])
            finally:
                rt.free(t1)
        rt.free(table)
    for i, L in enumerate(layers):
        q = O.quant_act(L["x"])
        ref = O.gemv_w4(L["wq"], L["ws"], q["q"], q["scale"], 128)["y"]          # [m][rows]
        assert O.rel_err(got[i, :, row_base:row_base + rows], ref) < REL
        assert np.isnan(got[i, :, :row_base]).all() and np.isnan(got[i, :, row_base + rows:]).all()


def test_stream_several_tokens_delivers_to_host(rt):
    """The multi-token kernel stores to every additional receiver too (here: pinned host memory)."""
    m, rows, nl = 2, 900, 4
    ystride = rows + 8
    layers = [synth.rt4_layer(rows, K, m, seed=950 + i) for i in range(nl)]
    host = rt.pinned((nl, m, ystride), np.float32)
    host[:] = np.nan
    with Bufs(rt) as b:
        x = b.put(np.stack([L["x"] for L in layers]))
        ae, ao = b.zeros(nl * m * K // 2, np.int8), b.zeros(nl * m * K // 2, np.int8)
        asc, asu = b.zeros(nl * m * K // 128), b.zeros(nl * m * K // 128, np.int32)
        y = b.zeros(nl * m * ystride, np.float32, np.nan)
        ptrs = [(b.put(L["wq"]), b.put(L["ws"]), x + i * m * K * 4, y + i * m * ystride * 4) for i, L in enumerate(layers)]
        table = rt.stream_table(ptrs, rows, K, (m - 1) * ystride)
        deltas = rt.stream_peers([host.ctypes.data], y, nl * m * ystride * 4)
        status = b.zeros(1, np.int32)
        rt.launch2d("quant_act", K // 128, nl * m, 32, 1, [x, ae, ao, asc, asu, nl * m, K])
        rt.launch("w4a8_decode_stream_m", 1, 1, [table, nl, rows, K, 0, 1, deltas, status, ae, ao, asc, asu, m, ystride, 0])
        dev = b.get(y, nl * m * ystride).reshape(nl, m, ystride)
        assert int(b.get(status, 1, np.int32)[0]) == 0
        rt.free(table)
        rt.free(deltas)
    assert np.array_equal(host.view(np.uint32), dev.view(np.uint32))
    for i, L in enumerate(layers):
        q = O.quant_act(L["x"])
        assert O.rel_err(host[i, :, :rows], O.gemv_w4(L["wq"], L["ws"], q["q"], q["scale"], 128)["y"]) < REL


@pytest.mark.parametrize("rows,nlayers", [(1000, 4), (17408, 2)])
def test_nvfp4_stream_matches_per_layer_and_oracle(rt, rows, nlayers):
    """nvfp4_decode_stream: one 2-D nvfp4_quant_act launch over all layers, then the stream kernel; agrees with
    nvfp4_gemv<1,1> layer by layer (another association of the fp32 sums, so 1e-6 and not bits) and with the oracle."""
    layers = [synth.nvfp4_layer(rows, K, 1, seed=970 + i) for i in range(nlayers)]
    gscale = float(layers[0]["gscale"])
    with Bufs(rt) as b:
        x = b.put(np.stack([L["x"][0] for L in layers]))
        qa, qb = b.zeros(nlayers * K // 2, np.int8), b.zeros(nlayers * K // 2, np.int8)
        sc = b.zeros(nlayers * K // 16)
        ys, ptrs = [], []
        for i, L in enumerate(layers):
            py = b.zeros(rows, np.float32, np.nan)
            ys.append(py)
            ptrs.append((b.put(L["wq"]), b.put(L["ws"]), x + i * K * 4, py))
        table = rt.stream_table(ptrs, rows, K, 0)
        status = b.zeros(1, np.int32)
        rt.launch2d("nvfp4_quant_act", K // 16, nlayers, 64, 1, [x, qa, qb, sc, nlayers, K])   # grid y = layer
        rt.launch("nvfp4_decode_stream", 1, 1, [table, nlayers, rows, K, 0, 0, 0, status, qa, qb, sc, gscale, 0])
        got = [b.get(py, rows) for py in ys]
        assert int(b.get(status, 1, np.int32)[0]) == 0
        for i, (L, yv) in enumerate(zip(layers, got)):
            q = O.nvfp4_quant_act(L["x"])
            ref = O.nvfp4_gemv(L["wq"], L["ws"], q["q"], q["scale"], gscale)["y"][0]
            assert O.rel_err(yv, ref) < REL
            py2 = b.zeros(rows, np.float32, np.nan)
            rt.launch("nvfp4_gemv<1,1>", -(-rows // 4), 256, [ptrs[i][0], ptrs[i][1], qa + i * K // 2, qb + i * K // 2,
                                                             sc + i * (K // 16) * 4, py2, rows, K, gscale])
            assert O.rel_err(b.get(py2, rows), yv) < 1e-6
        # a table whose scale buffers are too short for NVFP4 (rows * K/16 bytes) is refused
        short = b.zeros(rows * (K // 128) * 2 // 4 + 4, np.float32)
        t2 = rt.stream_table([(ptrs[0][0], short, ptrs[0][2], ys[0])], rows, K, 0)
        with pytest.raises(RuntimeError, match="rc=-4"):
            rt.launch("nvfp4_decode_stream", 1, 1, [t2, 1, rows, K, 0, 0, 0, status, qa, qb, sc, gscale, 0])
        rt.free(t2)
        rt.free(table)


@pytest.mark.parametrize("rows,nlayers", [(1000, 4), (17408, 2)])
def test_w4a16_stream_matches_oracle(rt, rows, nlayers):
    """w4a16_decode_stream: compressed-tensors INT4 layers with fp32 activations through the ring; the
    activations are read from the table's x entries and split on the device."""
    layers = [synth.w4a16_layer(rows, K, seed=990 + i) for i in range(nlayers)]
    with Bufs(rt) as b:
        ys, ptrs = [], []
        for L in layers:
            py = b.zeros(rows, np.float32, np.nan)
            ys.append(py)
            ptrs.append((b.put(L["packed"]), b.put(L["scale_bf16"]), b.put(L["x"]), py))
        table = rt.stream_table(ptrs, rows, K, 0)
        status = b.zeros(1, np.int32)
        rt.launch("w4a16_decode_stream", 1, 1, [table, nlayers, rows, K, 0, 0, 0, status, 0])
        got = [b.get(py, rows) for py in ys]
        assert int(b.get(status, 1, np.int32)[0]) == 0
        # a table without x entries is refused by this kernel
        t2 = rt.stream_table([(w, s, 0, y) for (w, s, _x, y) in ptrs], rows, K, 0)
        with pytest.raises(RuntimeError, match="rc=-4"):
            rt.launch("w4a16_decode_stream", 1, 1, [t2, nlayers, rows, K, 0, 0, 0, status, 0])
        rt.free(t2)
        rt.free(table)
    for L, yv in zip(layers, got):
        assert O.rel_err(yv, O.w4a16_gemv(L["packed"], L["scale_bf16"], L["x"])[0]) < REL


def test_freed_buffers_unvalidate_tables_peers_and_cached_plans(rt):
    """Freeing an allocation that a validated layer table, a peer-offset array or a cached launch plan
    points into makes the next launch come back with -4 (nothing is launched on the rejected paths);
    unrelated frees leave them valid."""
    from k100lc_kernels import LaunchPlan
    rows, nl = 200, 2
    layers = [synth.rt4_layer(rows, K, 1, seed=990 + i) for i in range(nl)]
    host = rt.pinned((nl, rows), np.float32)
    with Bufs(rt) as b:
        codes = Codes(rt, b, layers)
        y = b.zeros(nl * rows, np.float32, np.nan)
        wq1 = rt.alloc(layers[1]["wq"].nbytes)                 # freed by hand below
        rt.upload(wq1, layers[1]["wq"])
        ptrs = [(b.put(layers[0]["wq"]), b.put(layers[0]["ws"]), codes.x, y),
                (wq1, b.put(layers[1]["ws"]), codes.x + K * 4, y + rows * 4)]
        table = rt.stream_table(ptrs, rows, K, 0)
        status = b.zeros(1, np.int32)
        deltas = rt.stream_peers([host.ctypes.data], y, nl * rows * 4)
        argv = [table, nl, rows, K, 0, 0, 0, status] + codes.args + [0]
        argv_host = [table, nl, rows, K, 0, 1, deltas, status] + codes.args + [0]
        codes.quantise(rt)
        rt.launch("w4a8_decode_stream", 1, 1, argv_host)
        plan = LaunchPlan(rt, [("w4a8_decode_stream", 1, 1, argv)])
        plan.run()
        plan.run()                                             # replayed from the cached graph
        first = b.get(y, nl * rows).copy()
        assert int(b.get(status, 1, np.int32)[0]) == 0
        assert np.array_equal(host.reshape(-1).view(np.uint32), first.view(np.uint32))
        scratch = rt.alloc(4096)
        rt.free(scratch)                                       # an unrelated free: the table stays valid
        rt.launch("w4a8_decode_stream", 1, 1, argv)
        plan.run()
        assert np.array_equal(b.get(y, nl * rows).view(np.uint32), first.view(np.uint32))
        rt.free_pinned(host)                                   # the receiver goes away: its offsets are dropped
        with pytest.raises(RuntimeError, match="rc=-4"):
            rt.launch("w4a8_decode_stream", 1, 1, argv_host)
        rt.launch("w4a8_decode_stream", 1, 1, argv)            # the table itself is still fine
        rt.free(wq1)                                           # a layer's weights go away: the table is dropped
        with pytest.raises(RuntimeError, match="rc=-4"):
            rt.launch("w4a8_decode_stream", 1, 1, argv)
        with pytest.raises(RuntimeError):                      # the cached graph is not replayed either
            plan.run()
        assert int(b.get(status, 1, np.int32)[0]) == 0
        rt.free(table)
        rt.free(deltas)


@pytest.mark.parametrize("rows,nlayers", [(17408, 2), (2176, 3), (300, 2)])
def test_stream_accumulators_w4a8_and_w4a4(rt, rows, nlayers):
    """The integer accumulators of the stream kernels themselves (tensor-core consumer for W4A8 — both the
    schedule for many stages per layer and the one for a single stage per layer, which 2176 rows on 148 CTAs
    select — and the dp4a consumer for W4A4), bit for bit against the oracle."""
    layers = [synth.rt4_layer(rows, K, 1, seed=1200 + i) for i in range(nlayers)]
    with Bufs(rt) as b:
        codes = Codes(rt, b, layers)
        ys, ptrs = [], []
        for i, L in enumerate(layers):
            py = b.zeros(rows, np.float32, np.nan)
            ys.append(py)
            ptrs.append((b.put(L["wq"]), b.put(L["ws"]), codes.x + i * K * 4, py))
        table = rt.stream_table(ptrs, rows, K, 0)
        status = b.zeros(1, np.int32)
        codes.quantise(rt)
        pi = b.zeros(nlayers * rows * (K // 128), np.int32, -7)
        rt.launch("w4a8_decode_stream_iacc", 1, 1, [table, nlayers, rows, K, 0, 0, 0, status] + codes.args + [0, pi])
        acc8 = b.get(pi, nlayers * rows * (K // 128), np.int32).reshape(nlayers, rows, -1)
        y8 = [b.get(py, rows) for py in ys]
        aq, asc4 = b.zeros(nlayers * K // 2, np.uint8), b.zeros(nlayers * K // 32)
        rt.launch2d("quant_act4", K // 32, nlayers, 32, 1, [codes.x, aq, asc4, nlayers, K])
        pi4 = b.zeros(nlayers * rows * (K // 32), np.int32, -7)
        rt.launch("w4a4_decode_stream_iacc", 1, 1, [table, nlayers, rows, K, 0, 0, 0, status, aq, asc4, 0, pi4])
        acc4 = b.get(pi4, nlayers * rows * (K // 32), np.int32).reshape(nlayers, rows, -1)
        y4 = [b.get(py, rows) for py in ys]
        assert int(b.get(status, 1, np.int32)[0]) == 0
        rt.free(table)
    for i, L in enumerate(layers):
        q = O.quant_act(L["x"])
        ref = O.gemv_w4(L["wq"], L["ws"], q["q"], q["scale"], 128)
        assert np.array_equal(acc8[i], ref["acc"][0]), "W4A8 stream accumulators differ"
        assert O.rel_err(y8[i], ref["y"][0]) < REL
        q4 = O.quant_act4(L["x"])
        ref4 = O.gemv_w4(L["wq"], L["ws"], q4["q"], q4["scale"], 32)
        assert np.array_equal(acc4[i], ref4["acc"][0]), "W4A4 stream accumulators differ"
        assert O.rel_err(y4[i], ref4["y"][0]) < REL


@pytest.mark.parametrize("m,rows", [(2, 600), (4, 17408)])
def test_stream_accumulators_several_tokens(rt, m, rows):
    nl = 2
    ystride = rows + 8
    layers = [synth.rt4_layer(rows, K, m, seed=1300 + 10 * m + i) for i in range(nl)]
    with Bufs(rt) as b:
        x = b.put(np.stack([L["x"] for L in layers]))
        ae, ao = b.zeros(nl * m * K // 2, np.int8), b.zeros(nl * m * K // 2, np.int8)
        asc, asu = b.zeros(nl * m * K // 128), b.zeros(nl * m * K // 128, np.int32)
        y = b.zeros(nl * m * ystride, np.float32, np.nan)
        ptrs = [(b.put(L["wq"]), b.put(L["ws"]), x + i * m * K * 4, y + i * m * ystride * 4) for i, L in enumerate(layers)]
        table = rt.stream_table(ptrs, rows, K, (m - 1) * ystride)
        status = b.zeros(1, np.int32)
        rt.launch2d("quant_act", K // 128, nl * m, 32, 1, [x, ae, ao, asc, asu, nl * m, K])
        pi = b.zeros(nl * m * rows * (K // 128), np.int32, -7)
        rt.launch("w4a8_decode_stream_m_iacc", 1, 1, [table, nl, rows, K, 0, 0, 0, status, ae, ao, asc, asu, m, ystride, 0, pi])
        acc = b.get(pi, nl * m * rows * (K // 128), np.int32).reshape(nl, m, rows, -1)
        got = b.get(y, nl * m * ystride).reshape(nl, m, ystride)
        assert int(b.get(status, 1, np.int32)[0]) == 0
        rt.free(table)
    for i, L in enumerate(layers):
        q = O.quant_act(L["x"])
        ref = O.gemv_w4(L["wq"], L["ws"], q["q"], q["scale"], 128)
        assert np.array_equal(acc[i], ref["acc"])
        assert O.rel_err(got[i, :, :rows], ref["y"]) < REL


@pytest.mark.parametrize("m,rows,row_base,nl", [(2, 600, 0, 3), (3, 148, 0, 5), (4, 17408, 0, 2), (4, 700, 300, 6), (3, 1001, 8, 7)])
def test_w4a4_stream_several_tokens(rt, m, rows, row_base, nl):
    """w4a4_decode_stream_m: 2..4 tokens per layer on the W4A4 tensor-core consumer (two tokens share an MMA: the
    second one rides in the accumulator column that a lane owns beside its own).  The int32 of every
    (token, row, 32-group) bit for bit; y against the oracle, also at a pinned host receiver; a one-token table is
    refused."""
    ystride = row_base + rows + 24
    layers = [synth.rt4_layer(rows, K, m, seed=1350 + 10 * m + i) for i in range(nl)]
    host = rt.pinned((nl, m, ystride), np.float32)
    host[:] = np.nan
    with Bufs(rt) as b:
        x = b.put(np.stack([L["x"] for L in layers]))                       # [nl][m][K]
        aq, asc = b.zeros(nl * m * K // 2, np.uint8), b.zeros(nl * m * K // 32)
        y = b.zeros(nl * m * ystride, np.float32, np.nan)
        ptrs = [(b.put(L["wq"]), b.put(L["ws"]), x + i * m * K * 4, y + i * m * ystride * 4) for i, L in enumerate(layers)]
        table = rt.stream_table(ptrs, rows, K, row_base + (m - 1) * ystride)
        deltas = rt.stream_peers([host.ctypes.data], y, nl * m * ystride * 4)
        status = b.zeros(1, np.int32)
        rt.launch2d("quant_act4", K // 32, nl * m, 32, 1, [x, aq, asc, nl * m, K])
        pi = b.zeros(nl * m * rows * (K // 32), np.int32, -7)
        rt.launch("w4a4_decode_stream_m_iacc", 1, 1, [table, nl, rows, K, row_base, 0, 0, status, aq, asc, m, ystride, 0, pi])
        acc = b.get(pi, nl * m * rows * (K // 32), np.int32).reshape(nl, m, rows, -1)
        dumped = b.get(y, nl * m * ystride).reshape(nl, m, ystride)
        rt.memset(y, 0xFF, nl * m * ystride * 4)
        rt.launch("w4a4_decode_stream_m", 1, 1, [table, nl, rows, K, row_base, 1, deltas, status, aq, asc, m, ystride, 0])
        got = b.get(y, nl * m * ystride).reshape(nl, m, ystride)
        assert int(b.get(status, 1, np.int32)[0]) == 0
        with pytest.raises(RuntimeError, match="2..4 tokens"):
            rt.launch("w4a4_decode_stream_m", 1, 1, [table, nl, rows, K, row_base, 0, 0, status, aq, asc, 1, ystride, 0])
        with pytest.raises(RuntimeError, match="rc=-4"):                    # a table validated for one token is refused
            t1 = rt.stream_table(ptrs, rows, K, row_base)
            try:
                rt.launch("w4a4_decode_stream_m", 1, 1, [t1, nl, rows, K, row_base, 0, 0, status, aq, asc, m, ystride, 0])
            finally:
                rt.free(t1)
        rt.free(table)
        rt.free(deltas)
    sl = slice(row_base, row_base + rows)
    assert np.array_equal(got[:, :, sl].view(np.uint32), dumped[:, :, sl].view(np.uint32))
    assert np.array_equal(host[:, :, sl].view(np.uint32), got[:, :, sl].view(np.uint32))
    for i, L in enumerate(layers):
        q = O.quant_act4(L["x"])
        ref = O.gemv_w4(L["wq"], L["ws"], q["q"], q["scale"], 32)
        assert np.array_equal(acc[i], ref["acc"]), "W4A4 multi-token stream accumulators differ"
        assert O.rel_err(got[i, :, sl], ref["y"]) < REL
        assert np.isnan(got[i, :, :row_base]).all() and np.isnan(got[i, :, row_base + rows:]).all()
        assert np.isnan(host[i, :, :row_base]).all() and np.isnan(host[i, :, row_base + rows:]).all()


@pytest.mark.parametrize("cfg", [None, "3", "1", "0", "2"])
@pytest.mark.parametrize("rows,nlayers", [(17408, 2), (520, 3)])
def test_stream_accumulators_nvfp4(rt, monkeypatch, rows, nlayers, cfg):
    """nvfp4_decode_stream: the int32 of every (row, 16-block), bit for bit, from the default consumer (tcgen05
    kind::mxf4: the integer is rebuilt from the exact fp32 block sums of the base-7 digits of the activation codes), the dp4a consumer ($FM_NVFP4_CFG=1) and the mma.sync consumer (0; 2 = two groups, same arithmetic)."""
    if cfg is None:
        monkeypatch.delenv("FM_NVFP4_CFG", raising=False)
    else:
        monkeypatch.setenv("FM_NVFP4_CFG", cfg)
    layers = [synth.nvfp4_layer(rows, K, 1, seed=1400 + i) for i in range(nlayers)]
    gscale = float(layers[0]["gscale"])
    with Bufs(rt) as b:
        x = b.put(np.stack([L["x"][0] for L in layers]))
        qa, qb = b.zeros(nlayers * K // 2, np.int8), b.zeros(nlayers * K // 2, np.int8)
        sc = b.zeros(nlayers * K // 16)
        ys, ptrs = [], []
        for i, L in enumerate(layers):
            py = b.zeros(rows, np.float32, np.nan)
            ys.append(py)
            ptrs.append((b.put(L["wq"]), b.put(L["ws"]), x + i * K * 4, py))
        table = rt.stream_table(ptrs, rows, K, 0)
        status = b.zeros(1, np.int32)
        rt.launch2d("nvfp4_quant_act", K // 16, nlayers, 64, 1, [x, qa, qb, sc, nlayers, K])
        pi = b.zeros(nlayers * rows * (K // 16), np.int32, -7)
        rt.launch("nvfp4_decode_stream_iacc", 1, 1, [table, nlayers, rows, K, 0, 0, 0, status, qa, qb, sc, gscale, 0, pi])
        acc = b.get(pi, nlayers * rows * (K // 16), np.int32).reshape(nlayers, rows, -1)
        got = [b.get(py, rows) for py in ys]
        rt.launch("nvfp4_decode_stream", 1, 1, [table, nlayers, rows, K, 0, 0, 0, status, qa, qb, sc, gscale, 0])
        got2 = [b.get(py, rows) for py in ys]
        assert all(np.array_equal(a_, b_) for a_, b_ in zip(got, got2))
        assert int(b.get(status, 1, np.int32)[0]) == 0
        rt.free(table)
    for i, L in enumerate(layers):
        q = O.nvfp4_quant_act(L["x"])
        ref = O.nvfp4_gemv(L["wq"], L["ws"], q["q"], q["scale"], gscale)
        assert np.array_equal(acc[i], ref["acc"][0])
        assert O.rel_err(got[i], ref["y"][0]) < REL


def test_nvfp4_stream_counters_host_receiver_and_extreme_codes(rt, monkeypatch):
    """The tcgen05 consumer of nvfp4_decode_stream with a pinned host receiver and completion counters: rows that do
    not fill the last 128-row tile, fewer tiles per layer than CTAs, activation codes over the whole int8 range
    (-128 and 127 included, written directly instead of through the quantiser) and every finite E4M3 scale code."""
    monkeypatch.setenv("FM_NVFP4_CFG", "3")            # the tcgen05 consumer or an error, no other consumer in its place
    rows, nl = 333, 7
    sms = rt.device_attr("sm_count")
    layers = [synth.nvfp4_layer(rows, K, 1, seed=1700 + i) for i in range(nl)]
    rng = np.random.default_rng(5)
    finite = np.array([c for c in range(256) if (c & 0x7F) != 0x7F], dtype=np.uint8)
    for i, L in enumerate(layers):
        ws = np.asarray(L["ws"]).reshape(rows, K // 16).copy()
        ws[i % rows, :] = finite[rng.integers(0, len(finite), size=K // 16)]
        ws[(i + 1) % rows, :len(finite)] = finite
        L["ws"] = ws
    q = rng.integers(-128, 128, size=(nl, K)).astype(np.int8)
    q[:, 0:16] = -128
    q[:, 16:32] = 127
    q[:, 32:48:2] = -128
    asc = np.exp2(rng.uniform(-8.0, -2.0, size=(nl, K // 16))).astype(np.float32)
    gscale = float(layers[0]["gscale"])
    with Bufs(rt) as b:
        qa, qb = b.put(np.ascontiguousarray(q[:, 0::2])), b.put(np.ascontiguousarray(q[:, 1::2]))
        sc = b.put(asc)
        ybytes = nl * rows * 4
        buf = b.zeros((ybytes + nl * 4) // 4, np.float32, 0)
        host = rt.pinned(((ybytes + nl * 4) // 4,), np.float32)
        host[:] = 0
        flags = buf + ybytes
        ptrs = [(b.put(L["wq"]), b.put(L["ws"]), 0, buf + i * rows * 4) for i, L in enumerate(layers)]
        table = rt.stream_table(ptrs, rows, K, 0)
        deltas = rt.stream_peers([host.ctypes.data], buf, ybytes + nl * 4)
        status = b.zeros(1, np.int32)
        rt.launch("nvfp4_decode_stream", 1, 1, [table, nl, rows, K, 0, 1, deltas, status, qa, qb, sc, gscale, flags])
        wstat = b.zeros(1, np.int32)
        rt.launch("stream_flag_wait", 1, 128, [flags, nl, sms, wstat, 1000])
        dev = b.get(buf, (ybytes + nl * 4) // 4)
        assert int(b.get(status, 1, np.int32)[0]) == 0 and int(b.get(wstat, 1, np.int32)[0]) == 0
        assert (dev[ybytes // 4:].view(np.uint32) == sms).all() and (host[ybytes // 4:].view(np.uint32) == sms).all()
        assert np.array_equal(host[:ybytes // 4].view(np.uint32), dev[:ybytes // 4].view(np.uint32))
        pi = b.zeros(nl * rows * (K // 16), np.int32, -7)
        rt.launch("nvfp4_decode_stream_iacc", 1, 1, [table, nl, rows, K, 0, 0, 0, status, qa, qb, sc, gscale, 0, pi])
        acc = b.get(pi, nl * rows * (K // 16), np.int32).reshape(nl, rows, -1)
        assert int(b.get(status, 1, np.int32)[0]) == 0
        rt.free(table)
        rt.free(deltas)
    for i, L in enumerate(layers):
        ref = O.nvfp4_gemv(L["wq"], L["ws"], q[i:i + 1].astype(np.int32), asc[i:i + 1], gscale)
        assert np.array_equal(acc[i], ref["acc"][0])
        assert O.rel_err(host[i * rows:(i + 1) * rows], ref["y"][0]) < REL


@pytest.mark.parametrize("rows,nl", [(1, 1), (127, 2), (128, 3), (129, 1), (2176, 5)])
def test_nvfp4_tcgen05_stream_tile_edges(rt, monkeypatch, rows, nl):
    """The tcgen05 consumer on row counts around its 128-row tile (one row; one short of, exactly and one past a tile;
    the 17-tile shard of eight GPUs) with one and several layers: accumulators bit for bit, y within 1e-5, rows
    outside the layer untouched."""
    monkeypatch.setenv("FM_NVFP4_CFG", "3")
    layers = [synth.nvfp4_layer(rows, K, 1, seed=1800 + 7 * rows + i) for i in range(nl)]
    gscale = float(layers[0]["gscale"])
    with Bufs(rt) as b:
        x = b.put(np.stack([L["x"][0] for L in layers]))
        qa, qb = b.zeros(nl * K // 2, np.int8), b.zeros(nl * K // 2, np.int8)
        sc = b.zeros(nl * K // 16)
        y = b.zeros(nl * (rows + 8), np.float32, np.nan)
        ptrs = [(b.put(L["wq"]), b.put(L["ws"]), x + i * K * 4, y + i * (rows + 8) * 4) for i, L in enumerate(layers)]
        table = rt.stream_table(ptrs, rows, K, 3)                    # rows land at y[3 .. 3 + rows)
        status = b.zeros(1, np.int32)
        rt.launch2d("nvfp4_quant_act", K // 16, nl, 64, 1, [x, qa, qb, sc, nl, K])
        pi = b.zeros(nl * rows * (K // 16), np.int32, -7)
        rt.launch("nvfp4_decode_stream_iacc", 1, 1, [table, nl, rows, K, 3, 0, 0, status, qa, qb, sc, gscale, 0, pi])
        acc = b.get(pi, nl * rows * (K // 16), np.int32).reshape(nl, rows, -1)
        got = b.get(y, nl * (rows + 8)).reshape(nl, rows + 8)
        assert int(b.get(status, 1, np.int32)[0]) == 0
        rt.free(table)
    for i, L in enumerate(layers):
        q = O.nvfp4_quant_act(L["x"])
        ref = O.nvfp4_gemv(L["wq"], L["ws"], q["q"], q["scale"], gscale)
        assert np.array_equal(acc[i], ref["acc"][0])
        assert O.rel_err(got[i, 3:3 + rows], ref["y"][0]) < REL
        assert np.isnan(got[i, :3]).all() and np.isnan(got[i, 3 + rows:]).all()


@pytest.mark.parametrize("m,rows,nl,row_base", [(2, 300, 3, 0), (3, 129, 2, 5), (4, 1000, 2, 0), (4, 17408, 2, 0)])
def test_nvfp4_stream_several_tokens(rt, m, rows, nl, row_base):
    """nvfp4_decode_stream_m: 2..4 tokens per layer on the tcgen05 consumer (12 columns of B per token).  The int32 of
    every (token, row, 16-block) bit for bit, y (token-major) within 1e-5, a pinned host receiver with the same bits."""
    ystride = row_base + rows + 8
    layers = [synth.nvfp4_layer(rows, K, m, seed=2100 + 10 * m + i) for i in range(nl)]
    gscale = float(layers[0]["gscale"])
    host = rt.pinned((nl, m, ystride), np.float32)
    host[:] = np.nan
    with Bufs(rt) as b:
        x = b.put(np.stack([L["x"] for L in layers]))                       # [nl][m][K]
        qa, qb = b.zeros(nl * m * K // 2, np.int8), b.zeros(nl * m * K // 2, np.int8)
        sc = b.zeros(nl * m * K // 16)
        y = b.zeros(nl * m * ystride, np.float32, np.nan)
        ptrs = [(b.put(L["wq"]), b.put(L["ws"]), x + i * m * K * 4, y + i * m * ystride * 4) for i, L in enumerate(layers)]
        table = rt.stream_table(ptrs, rows, K, row_base + (m - 1) * ystride)
        deltas = rt.stream_peers([host.ctypes.data], y, nl * m * ystride * 4)
        status = b.zeros(1, np.int32)
        rt.launch2d("nvfp4_quant_act", K // 16, nl * m, 64, 1, [x, qa, qb, sc, nl * m, K])
        pi = b.zeros(nl * m * rows * (K // 16), np.int32, -7)
        rt.launch("nvfp4_decode_stream_m_iacc", 1, 1, [table, nl, rows, K, row_base, 0, 0, status, qa, qb, sc, gscale, m, ystride, 0, pi])
        acc = b.get(pi, nl * m * rows * (K // 16), np.int32).reshape(nl, m, rows, -1)
        rt.memset(y, 0xFF, nl * m * ystride * 4)
        rt.launch("nvfp4_decode_stream_m", 1, 1, [table, nl, rows, K, row_base, 1, deltas, status, qa, qb, sc, gscale, m, ystride, 0])
        dev = b.get(y, nl * m * ystride).reshape(nl, m, ystride)
        assert int(b.get(status, 1, np.int32)[0]) == 0
        with pytest.raises(RuntimeError, match="rc=-4"):                    # one token belongs to nvfp4_decode_stream
            rt.launch("nvfp4_decode_stream_m", 1, 1, [table, nl, rows, K, row_base, 0, 0, status, qa, qb, sc, gscale, 1, ystride, 0])
        rt.free(table)
        rt.free(deltas)
    sl = slice(row_base, row_base + rows)
    assert np.array_equal(host[:, :, sl].view(np.uint32), dev[:, :, sl].view(np.uint32))
    for i, L in enumerate(layers):
        q = O.nvfp4_quant_act(L["x"])
        ref = O.nvfp4_gemv(L["wq"], L["ws"], q["q"], q["scale"], gscale)
        assert np.array_equal(acc[i], ref["acc"])
        assert O.rel_err(dev[i, :, sl], ref["y"]) < REL
    rt.free_pinned(host)


def test_layers_of_different_shapes_in_one_launch(rt):
    """w4a8_layers_stream: weight matrices of different (rows, K) in one launch — K = 5120, 6144 (a full and a 1024-k
    chunk) and 17408 (three full chunks and one of 2048 k), row counts from a few to thousands, a pinned host receiver
    and completion counters.  y within 1e-5 of the oracle over the whole K, and the bits of gemv_w4a8<1,false,1> where
    the row is a single chunk."""
    shapes = [(300, 5120), (200, 6144), (2176, 5120), (150, 17408), (1024, 5120), (37, 6144), (5120, 17408)]
    sms = rt.device_attr("sm_count")
    layers = [synth.rt4_layer(n, k, 1, seed=2000 + i) for i, (n, k) in enumerate(shapes)]
    ytot = sum(n for n, _ in shapes)
    with Bufs(rt) as b:
        entries, outs, acts = [], [], []
        nchunks = sum(-(-k // 5120) for _, k in shapes)
        buf = b.zeros(ytot + nchunks, np.float32, np.nan)            # every y, then one counter per table entry
        host = rt.pinned((ytot + nchunks,), np.float32)
        host[:] = 0
        rt.memset(buf + ytot * 4, 0, nchunks * 4)
        off = 0
        for (n, k), L in zip(shapes, layers):
            kp = -(-k // 5120) * 5120                              # the code arrays are padded with zeros to whole chunks
            x = b.put(L["x"][0])
            ae, ao = b.zeros(kp // 2, np.int8), b.zeros(kp // 2, np.int8)
            asc, asu = b.zeros(kp // 128), b.zeros(kp // 128, np.int32)
            rt.launch("quant_act", k // 128, 32, [x, ae, ao, asc, asu, 1, k])
            wq, ws = b.put(L["wq"]), b.put(L["ws"])
            entries += rt.layer_chunks(wq, ws, buf + off * 4, ae, ao, asc, asu, n, k)
            outs.append(off)
            acts.append((wq, ws, ae, ao, asc, asu))
            off += n
        table, shp = rt.stream_table_var(entries)
        deltas = rt.stream_peers([host.ctypes.data], buf, (ytot + nchunks) * 4)
        status = b.zeros(1, np.int32)
        flags = buf + ytot * 4
        rt.launch("w4a8_layers_stream", 1, 1, [table, shp, len(entries), 1, deltas, status, flags])
        dev = b.get(buf, ytot + nchunks)
        assert int(b.get(status, 1, np.int32)[0]) == 0
        ctas = min(sms, max(n for n, _ in shapes))
        assert (dev[ytot:].view(np.uint32) == ctas).all() and (host[ytot:].view(np.uint32) == ctas).all()
        assert np.array_equal(host[:ytot].view(np.uint32), dev[:ytot].view(np.uint32))
        for (n, k), L, o, (wq, ws, ae, ao, asc, asu) in zip(shapes, layers, outs, acts):
            q = O.quant_act(L["x"])
            ref = O.gemv_w4(L["wq"], L["ws"], q["q"], q["scale"], 128)["y"][0]
            assert O.rel_err(dev[o:o + n], ref) < REL, (n, k)
            if k == 5120:
                y1 = b.zeros(n, np.float32, np.nan)
                rt.launch("gemv_w4a8<1,false,1>", -(-n // 4), 256, [wq, ws, ae, ao, asc, asu, y1, n, k])
                assert np.array_equal(b.get(y1, n).view(np.uint32), dev[o:o + n].view(np.uint32))
        # a shape the kernel does not take, and a table that was not validated, are refused
        bad = list(entries[0])
        bad[11] = 2560 + 16
        with pytest.raises(RuntimeError, match="not a shape this kernel takes"):
            rt.stream_table_var([tuple(bad)])
        with pytest.raises(RuntimeError, match="adds to y"):            # a later chunk without the chunk before it
            rt.stream_table_var([entries[2]])
        with pytest.raises(RuntimeError, match="rc=-4"):
            rt.launch("w4a8_layers_stream", 1, 1, [table, shp + 64, len(entries) - 1, 0, 0, status, 0])
        rt.free(table)
        rt.free(shp)
        rt.free(deltas)
    rt.free_pinned(host)


@pytest.mark.parametrize("cfg", [None, "6"])
def test_read_ceiling_kernel_copies_and_writes_nothing(rt, monkeypatch, cfg):
    """w4a8_stream_read_ceiling takes the arguments of w4a8_decode_stream, walks all stages (status 0) and leaves y as
    it was; a table of another shape is refused.  (6: the whole-stage split of the rows.)"""
    if cfg is not None:
        monkeypatch.setenv("FM_STREAM_CFG", cfg)
    rows, nl = 2176, 6
    layers = [synth.rt4_layer(rows, K, 1, seed=1900 + i) for i in range(nl)]
    with Bufs(rt) as b:
        codes = Codes(rt, b, layers)
        y = b.zeros(nl * rows, np.float32, np.nan)
        ptrs = [(b.put(L["wq"]), b.put(L["ws"]), codes.x + i * K * 4, y + i * rows * 4) for i, L in enumerate(layers)]
        table = rt.stream_table(ptrs, rows, K, 0)
        status = b.zeros(1, np.int32)
        codes.quantise(rt)
        rt.launch("w4a8_stream_read_ceiling", 1, 1, [table, nl, rows, K, 0, 0, 0, status] + codes.args + [0])
        assert int(b.get(status, 1, np.int32)[0]) == 0
        assert np.isnan(b.get(y, nl * rows)).all()
        with pytest.raises(RuntimeError, match="rc=-4"):
            rt.launch("w4a8_stream_read_ceiling", 1, 1, [table, nl, rows + 16, K, 0, 0, 0, status] + codes.args + [0])
        rt.free(table)


def test_stream_schedules_give_identical_bits(rt, monkeypatch):
    """Every schedule of the W4A8 stream kernel ($FM_STREAM_CFG, with and without a suspend hint on the
    barrier waits) leaves the bits of gemv_w4a8<1,false,1> in y, on a shape with many stages per CTA and
    layer, on one with a single (partial) stage, on fewer rows than CTAs and on a row count that is no multiple of
    the stage."""
    runner = W4Runner(rt)
    for rows, nl in ((17408, 2), (2176, 6), (100, 9), (7111, 3)):
        layers = [synth.rt4_layer(rows, K, 1, seed=1500 + i) for i in range(nl)]
        with Bufs(rt) as b:
            want = None
            # (5 / 6: rows / grid per CTA / whole 16-row stages per CTA from a position that moves with the layer —
            #  the default picks between them by the row count; 7111 rows end in a partial stage under both)
            for cfg in (None, 0, 1, 2, 3, 4, 5, 6, 7):
                for hint in ((0, 2000) if cfg is None else (0,)):
                    if cfg is None:
                        monkeypatch.delenv("FM_STREAM_CFG", raising=False)
                    else:
                        monkeypatch.setenv("FM_STREAM_CFG", str(cfg))
                    monkeypatch.setenv("FM_STREAM_HINT_NS", str(hint))
                    got, ptrs = _run_stream(rt, b, layers, rows)
                    if want is None:
                        want = [runner.gemv("w4a8", pwq, pws, L["x"], rows, K)[0] for L, (pwq, pws, _x, _y) in zip(layers, ptrs)]
                    for i in range(nl):
                        assert np.array_equal(got[i].view(np.uint32), want[i].view(np.uint32)), (rows, cfg, hint, i)
        monkeypatch.delenv("FM_STREAM_CFG", raising=False)
        monkeypatch.delenv("FM_STREAM_HINT_NS", raising=False)
    runner.close()


def test_stream_completion_counters_and_bounded_acquire(rt):
    """flags[layer] ends at the number of CTAs on every receiver (local and pinned host); stream_flag_wait
    returns at once when the target is met and, for a target that no producer will reach, gives up after
    its bounded number of polls with status 9 (the context stays usable)."""
    rows, nl = 1200, 5
    sms = rt.device_attr("sm_count")
    layers = [synth.rt4_layer(rows, K, 1, seed=1600 + i) for i in range(nl)]
    with Bufs(rt) as b:
        codes = Codes(rt, b, layers)
        # y of all layers and the counters live in one allocation, mirrored in one pinned host buffer
        ybytes = nl * rows * 4
        buf = b.zeros((ybytes + nl * 4) // 4, np.float32, 0)
        host = rt.pinned(((ybytes + nl * 4) // 4,), np.float32)
        host[:] = 0
        flags = buf + ybytes
        ptrs = [(b.put(L["wq"]), b.put(L["ws"]), codes.x + i * K * 4, buf + i * rows * 4) for i, L in enumerate(layers)]
        table = rt.stream_table(ptrs, rows, K, 0)
        deltas = rt.stream_peers([host.ctypes.data], buf, ybytes + nl * 4)
        status = b.zeros(1, np.int32)
        codes.quantise(rt)
        rt.launch("w4a8_decode_stream", 1, 1, [table, nl, rows, K, 0, 1, deltas, status] + codes.args + [flags])
        wstat = b.zeros(1, np.int32)
        rt.launch("stream_flag_wait", 1, 128, [flags, nl, sms, wstat, 1000])
        dev = b.get(buf, (ybytes + nl * 4) // 4)
        assert int(b.get(status, 1, np.int32)[0]) == 0 and int(b.get(wstat, 1, np.int32)[0]) == 0
        cnt_dev = dev[ybytes // 4:].view(np.uint32)
        cnt_host = host[ybytes // 4:].view(np.uint32)
        assert (cnt_dev == sms).all() and (cnt_host == sms).all()
        assert np.array_equal(host[:ybytes // 4].view(np.uint32), dev[:ybytes // 4].view(np.uint32))
        # a producer that never comes: the target is one more than anyone will add
        rt.launch("stream_flag_wait", 1, 128, [flags, nl, sms + 1, wstat, 200])
        assert int(b.get(wstat, 1, np.int32)[0]) == 9
        # flags outside the validated window are refused
        other = b.zeros(nl, np.int32)
        with pytest.raises(RuntimeError, match="rc=-4"):
            rt.launch("w4a8_decode_stream", 1, 1, [table, nl, rows, K, 0, 1, deltas, status] + codes.args + [other])
        rt.free(table)
        rt.free(deltas)
    for i, L in enumerate(layers):
        q = O.quant_act(L["x"])
        assert O.rel_err(host[i * rows:(i + 1) * rows], O.gemv_w4(L["wq"], L["ws"], q["q"], q["scale"], 128)["y"][0]) < REL
