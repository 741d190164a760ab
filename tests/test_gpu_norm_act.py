"""GPU tier: the operators either side of a streamed layer — RMSNorm, the SiLU gate, and their fusions with the
W4A8 activation quantiser (rmsnorm_quant_k, silu_mul_quant_k) — through the C ABI, and the MLP built from them."""
from __future__ import annotations

import numpy as np
import pytest

import cases
import w4_oracle as O
from gpu_util import Bufs
from k100lc_kernels import Int4Linear, MLP, RMSNorm, SwiGLU, Workspace
from k100lc_kernels.quant import dequant_int4_group128, pack_int4_group128

pytestmark = pytest.mark.gpu


def _judge(got, ref):
    """the reference's acceptance rule for these operators (tools/selftest_all.py judge())"""
    return np.abs(got - ref).max() <= 1e-4 + 1e-5 * max(1.0, float(np.abs(ref).max()))


@pytest.mark.parametrize("kernel", ["rmsnorm_k", "rmsnorm_fast_k", "rmsnorm_deep_k"])
def test_rmsnorm_names(rt, golden, kernel):
    arr, _ = golden
    x, w = cases.rmsnorm_case(4, 256, seed=8, gain=1.0, plain_w=True)
    with Bufs(rt) as b:
        y = b.zeros(x.size, np.float32, np.nan)
        argv = [y, b.put(x), b.put(w), 256, np.float32(1e-5)] + ([0] if kernel == "rmsnorm_k" else [])
        rt.launch(kernel, 4, 64, argv)
        got = b.get(y, x.size).reshape(x.shape)
        if kernel == "rmsnorm_k":
            with pytest.raises(RuntimeError, match="rc=-4"):            # the non-standard scaling branch is not built
                rt.launch(kernel, 4, 64, argv[:-1] + [1])
    assert _judge(got, arr["rmsnorm.y"])
    assert np.array_equal(got, O.rmsnorm(x, w, 1e-5))                   # same arithmetic as the oracle: same bits
    for rows, dim in ((1, 512), (3, 64), (2, 5120), (5, 320), (2, 17408)):   # the sizes of the reference's rmsnorm_fast_k case
        x, w = cases.rmsnorm_case(rows, dim, seed=81 + dim)
        with Bufs(rt) as b:
            y = b.zeros(x.size, np.float32, np.nan)
            rt.launch("rmsnorm_fast_k", rows, 64, [y, b.put(x), b.put(w), dim, np.float32(1e-5)])
            assert np.array_equal(b.get(y, x.size).reshape(x.shape), O.rmsnorm(x, w, 1e-5))


@pytest.mark.parametrize("rows,dim", cases.RMSNORM_QUANT_SHAPES + ((4, 17408), (1, 6144)))
def test_rmsnorm_quant_bit_exact(rt, golden, rows, dim):
    """rmsnorm_quant_k: codes, scales and group sums identical to the oracle (and, for the reference's own
    shapes, to the vectors of its host check)."""
    arr, _ = golden
    x, w = cases.rmsnorm_case(rows, dim)
    ng = dim // 128
    with Bufs(rt) as b:
        ae, ao = b.zeros(rows * dim // 2, np.int8, 99), b.zeros(rows * dim // 2, np.int8, 99)
        sc, su = b.zeros(rows * ng), b.zeros(rows * ng, np.int32)
        rt.launch("rmsnorm_quant_k", rows, 64, [ae, ao, sc, su, b.put(x), b.put(w), dim, np.float32(1e-6)])
        e, o = b.get(ae, rows * dim // 2, np.int8), b.get(ao, rows * dim // 2, np.int8)
        s, a = b.get(sc, rows * ng), b.get(su, rows * ng, np.int32)
    ref = O.rmsnorm_quant(x, w, 1e-6)
    assert np.array_equal(e.reshape(rows, -1), ref["even"]) and np.array_equal(o.reshape(rows, -1), ref["odd"])
    assert np.array_equal(s.reshape(rows, ng), ref["scale"]) and np.array_equal(a.reshape(rows, ng), ref["gsum"])
    name = f"rmsnorm_quant_{rows}x{dim}"
    if name + ".q" in arr:
        q = np.empty((rows, dim), np.int8)
        q[:, 0::2], q[:, 1::2] = e.reshape(rows, -1), o.reshape(rows, -1)
        assert np.array_equal(q, arr[name + ".q"]) and np.array_equal(s.reshape(rows, ng), arr[name + ".s"])


def test_silu_mul_and_fused_quantiser(rt, golden):
    arr, _ = golden
    gate, up = cases.silu_case()
    with Bufs(rt) as b:
        y = b.zeros(1000, np.float32, np.nan)
        rt.launch("silu_mul_k", -(-1000 // 64), 64, [y, b.put(gate), b.put(up), 1000])
        got = b.get(y, 1000)
    assert _judge(got, arr["silu_mul.y"])
    # silu_mul_quant_k == silu_mul_k followed by quant_act, bit for bit, on 1..4 rows of an MLP-sized vector
    rng = np.random.default_rng(5)
    for rows, k in ((1, 17408), (4, 5120), (3, 256)):
        g = rng.standard_normal((rows, k)).astype(np.float32) * 2
        u = rng.standard_normal((rows, k)).astype(np.float32)
        ng = k // 128
        with Bufs(rt) as b:
            pg, pu, h = b.put(g), b.put(u), b.zeros(rows * k, np.float32, np.nan)
            outs = [[b.zeros(rows * k // 2, np.int8, 99), b.zeros(rows * k // 2, np.int8, 99), b.zeros(rows * ng),
                     b.zeros(rows * ng, np.int32)] for _ in range(2)]
            rt.launch("silu_mul_k", -(-rows * k // 64), 64, [h, pg, pu, rows * k])
            rt.launch2d("quant_act", ng, rows, 32, 1, [h] + outs[0] + [rows, k])
            rt.launch2d("silu_mul_quant_k", 1, rows, 64, 1, outs[1] + [pg, pu, k])
            hv = b.get(h, rows * k).reshape(rows, k)
            for p0, p1, dt, cnt in zip(outs[0], outs[1], (np.int8, np.int8, np.float32, np.int32),
                                       (rows * k // 2, rows * k // 2, rows * ng, rows * ng)):
                assert np.array_equal(b.get(p0, cnt, dt), b.get(p1, cnt, dt))
            q1 = b.get(outs[1][0], rows * k // 2, np.int8).reshape(rows, -1)
        # against the oracle: exp() of the device and of NumPy may differ in the last place, so the codes may
        # differ by one in a few places (the reference's own criterion for its fused quantiser)
        ref = O.quant_act(O.silu_mul(g, u))
        d = np.abs(q1.astype(np.int32) - ref["even"].astype(np.int32))
        assert d.max() <= 1 and (d != 0).sum() <= max(1, d.size // 1000)
        assert _judge(hv, O.silu_mul(g, u))


def test_mlp_matches_dequantised_reference(rt):
    """RMSNorm -> MLP(gate, up, down) with W4A8 layers: the fused path (norm + quantiser, gate + quantiser) gives
    the bits of the unfused one, and both agree with the float64 product of the dequantised weights to the
    tolerance the reference states for its W4A8 path (3e-2)."""
    rng = np.random.default_rng(6)
    dim, ffn, rows = 512, 1024, 2
    mk = lambda n, k: pack_int4_group128((rng.standard_normal((n, k)) * 0.05).astype(np.float32))
    (gp, gs), (up_, us), (dp, ds) = mk(ffn, dim), mk(ffn, dim), mk(dim, ffn)
    x = rng.standard_normal((rows, dim)).astype(np.float32)
    wn = (rng.random(dim) + 0.5).astype(np.float32)
    with Workspace(rt) as ws:
        norm = RMSNorm(rt, dim, wn, 1e-6, ws, "n")
        gate = Int4Linear(rt, ffn, dim, gp, gs, "w4a8", ws, "g")
        up = Int4Linear(rt, ffn, dim, up_, us, "w4a8", ws, "u")
        down = Int4Linear(rt, dim, ffn, dp, ds, "w4a8", ws, "d")
        mlp = MLP(rt, gate, up, down, ws, "mlp")
        px = ws.upload("x", x)
        xn = norm.forward_device(px, rows)
        out = mlp.forward_device(xn, rows, sync=True)
        y_fused = rt.download(out, rows * dim, np.float32).reshape(rows, dim).copy()
        # unfused: separate gate kernel and quantiser
        h1, h2 = gate.forward_device(xn, rows), up.forward_device(xn, rows)
        act = SwiGLU(rt, ws, "sg").forward_device(h1, h2, rows * ffn)
        out2 = down.forward_device(act, rows, sync=True)
        y_plain = rt.download(out2, rows * dim, np.float32).reshape(rows, dim).copy()
        # norm + quantiser in one kernel feeding the gate projection == norm, then quantiser
        codes = norm.forward_quant_device(px, rows)
        g_a = rt.download(gate.forward_codes_device(codes, rows, sync=True), rows * ffn, np.float32).copy()
        g_b = rt.download(gate.forward_device(xn, rows, sync=True), rows * ffn, np.float32).copy()
    assert np.array_equal(y_fused, y_plain) and np.array_equal(g_a, g_b)
    W = lambda p, s, n, k: dequant_int4_group128(p, s, n, k).astype(np.float64)
    xr = O.rmsnorm(x, wn, 1e-6).astype(np.float64)
    a, bb = xr @ W(gp, gs, ffn, dim).T, xr @ W(up_, us, ffn, dim).T
    ref = (a / (1 + np.exp(-a)) * bb) @ W(dp, ds, dim, ffn).T
    assert O.rel_err(y_fused, ref) < 3e-2
