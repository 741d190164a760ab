"""GPU tier: the Python surface (Runtime, LaunchPlan, batch, W4Runner, Int4Linear,
RT4Linear, DotLinear, NVFP4Linear) end to end, plus the engine's error behaviour
(reference examples/python_w4a4_w4a8_gemv.py:68-92, examples/python_model_layer.py:214-238,
tools/selftest_all.py:1543-1557)."""
from __future__ import annotations

import numpy as np
import pytest

import w4_oracle as O
from gpu_util import Bufs
from k100lc_kernels import (DotLinear, Int4Linear, LaunchPlan, NVFP4Linear, RT4Linear, Runtime, W4Runner,
                            Workspace, run_sequence, synth)
from k100lc_kernels.quant import pack_int4_group128, dequant_int4_group128

pytestmark = pytest.mark.gpu
REL = 1e-5


def _ct_layer(n, k, seed):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    packed, scales = pack_int4_group128(w)
    return packed, scales, dequant_int4_group128(packed, scales, n, k)


@pytest.mark.parametrize("path,tol", [("w4a16", 1e-5), ("w4a8", 3e-2), ("w4a4", 3e-1)])
@pytest.mark.parametrize("m", [1, 2, 4, 7])
def test_int4linear_vs_dequant_matmul(rt, path, tol, m):
    """Against the f32 matmul of the dequantised weights, with the reference's example
    tolerances; M=7 exercises the chunks-of-4 GEMV route."""
    n, k = 320, 1024
    packed, scales, wf = _ct_layer(n, k, 3)
    x = np.random.default_rng(m).standard_normal((m, k)).astype(np.float32)
    with Workspace(rt) as ws:
        lin = Int4Linear(rt, n, k, packed, scales, path=path, ws=ws, tag="t", prefill="gemv")
        y = lin.forward(x)
    ref = x.astype(np.float64) @ wf.astype(np.float64).T
    assert O.rel_err(y, ref) < tol


def test_int4linear_w4a8_matches_oracle_exactly_defined(rt):
    """Int4Linear(w4a8) = ct->rt4 conversion + quant_act + gemv_w4a8: against the oracle
    run on the same converted bytes."""
    from k100lc_kernels.quant import ct_int4_to_rt4
    n, k, m = 256, 5120, 3
    packed, scales, _ = _ct_layer(n, k, 8)
    x = np.random.default_rng(2).standard_normal((m, k)).astype(np.float32)
    with Workspace(rt) as ws:
        y = Int4Linear(rt, n, k, packed, scales, path="w4a8", ws=ws, tag="a").forward(x)
        y4 = Int4Linear(rt, n, k, packed, scales, path="w4a4", ws=ws, tag="b").forward(x)
    q, s16 = ct_int4_to_rt4(packed, scales)
    wq = np.frombuffer(q, np.uint32).reshape(n, k // 8)
    ws16 = np.frombuffer(s16, np.float16).reshape(n, k // 128)
    qa = O.quant_act(x)
    assert O.rel_err(y, O.gemv_w4(wq, ws16, qa["q"], qa["scale"], 128)["y"]) < REL
    qa4 = O.quant_act4(x)
    assert O.rel_err(y4, O.gemv_w4(wq, ws16, qa4["q"], qa4["scale"], 32)["y"]) < REL


def test_rt4linear_run_sequence_and_plan(rt):
    """Two chained layers with one sync; then the same launches recorded in a LaunchPlan,
    replayed, patched (set_arg) and replayed again."""
    n, k = 1024, 1024
    L1, L2 = synth.rt4_layer(n, k, 1, seed=11), synth.rt4_layer(n, k, 1, seed=12)
    x = L1["x"]
    with Bufs(rt) as b:
        runner = W4Runner(rt)
        a = RT4Linear(rt, n, k, b.put(L1["wq"]), b.put(L1["ws"]), "w4a8", runner)
        c = RT4Linear(rt, n, k, b.put(L2["wq"]), b.put(L2["ws"]), "w4a8", runner)
        px, ymid, yout = b.put(x), b.zeros(n), b.zeros(n)
        out = run_sequence(rt, [lambda p: a.forward_device(p, 1, out_dev=ymid),
                                lambda p: c.forward_device(p, 1, out_dev=yout)], px)
        assert out == yout
        y1 = rt.download(ymid, n, np.float32)
        y2 = rt.download(yout, n, np.float32)
        q = O.quant_act(x)
        r1 = O.gemv_w4(L1["wq"], L1["ws"], q["q"], q["scale"], 128)["y"][0]
        assert O.rel_err(y1, r1) < REL
        q2 = O.quant_act(y1[None, :])
        r2 = O.gemv_w4(L2["wq"], L2["ws"], q2["q"], q2["scale"], 128)["y"][0]
        assert O.rel_err(y2, r2) < REL

        # record layer 1 as a plan: quant_act + gemv
        ae, ao, asc, asu, yp = b.zeros(k // 2, np.int8), b.zeros(k // 2, np.int8), b.zeros(k // 128), \
            b.zeros(k // 128, np.int32), b.zeros(n)
        calls = [("quant_act", k // 128, 32, [px, ae, ao, asc, asu, 1, k]),
                 ("gemv_w4a8<1,false,1>", n // 4, 256, [a.wq, a.ws_scale, ae, ao, asc, asu, yp, n, k])]
        plan = LaunchPlan(rt, calls)
        assert plan.kernels == ["quant_act", "gemv_w4a8<1,false,1>"]
        for _ in range(3):
            plan.run()
        rt.sync()
        assert np.array_equal(rt.download(yp, n, np.float32), y1)
        plan.set_arg(1, 0, c.wq)          # patch the weight pointers to layer 2's
        plan.set_arg(1, 1, c.ws_scale)
        plan.run()
        rt.sync()
        r3 = O.gemv_w4(L2["wq"], L2["ws"], q["q"], q["scale"], 128)["y"][0]
        assert O.rel_err(rt.download(yp, n, np.float32), r3) < REL
        plan.set_grid(1, 8)               # 8 work-groups = 32 rows only
        rt.memset(yp, 0, n * 4)
        plan.run()
        rt.sync()
        got = rt.download(yp, n, np.float32)
        assert O.rel_err(got[:32], r3[:32]) < REL and not got[32:].any()

        # batch scope: same result, one submission
        rt.memset(yp, 0, n * 4)
        with rt.batch():
            rt.launch(*calls[0])
            rt.launch(*calls[1])
        rt.sync()
        assert np.array_equal(rt.download(yp, n, np.float32), y1)
        runner.close()


def test_dotlinear_and_nvfp4linear(rt):
    L = synth.w4a16_layer(192, 2048, seed=5)
    x = np.random.default_rng(1).standard_normal((3, 2048)).astype(np.float32)
    with Workspace(rt) as ws:
        d = DotLinear(rt, 192, 2048, "int4", L["packed"].tobytes(), (L["scale_bf16"].tobytes(),), ws, "d")
        y = d.forward(x)
    assert O.rel_err(y, O.w4a16_gemv(L["packed"], L["scale_bf16"], x)) < REL
    F = synth.nvfp4_layer(192, 2048, 6, seed=6)
    with Workspace(rt) as ws:
        lin = NVFP4Linear(rt, 192, 2048, F["wq"], F["ws"], F["gscale"], ws, "f")
        y = lin.forward(F["x"])
    q = O.nvfp4_quant_act(F["x"])
    assert O.rel_err(y, O.nvfp4_gemv(F["wq"], F["ws"], q["q"], q["scale"], F["gscale"])["y"]) < REL


def test_error_codes_and_bounds(rt):
    """Unknown kernel -1, wrong arity -2, a footprint outside its allocation -4 (nothing
    is launched), a work-group size the kernel family cannot run -4, alloc failure ->
    MemoryError; the engine stays usable afterwards."""
    lib = rt._lib
    import ctypes
    argv = (ctypes.c_uint64 * 16)()
    assert lib.fm_launch(b"no_such_kernel", 1, 64, argv, 0) == -1
    assert lib.fm_launch(b"quant_act", 1, 32, argv, 3) == -2
    with Bufs(rt) as b:
        px = b.zeros(1024)                      # 4 KB
        small = b.zeros(16, np.int8)
        asc, asu = b.zeros(8), b.zeros(8, np.int32)
        with pytest.raises(RuntimeError, match="rc=-4"):
            rt.launch("quant_act", 8, 32, [px, small, small, asc, asu, 1, 1024])       # ae too small
        with pytest.raises(RuntimeError, match="rc=-4"):
            rt.launch("quant_act", 8, 32, [px + 4, small, small, asc, asu, 1, 1024])   # misaligned x
        L = synth.rt4_layer(64, 1024, 1, seed=1)
        pwq, pws = b.put(L["wq"]), b.put(L["ws"])
        with pytest.raises(RuntimeError, match="rc=-4"):
            rt.launch("gemv_w4a4<1>", 16, 512, [pwq, pws, px, asc, px, 64, 1024])      # 512 threads
        with pytest.raises(RuntimeError, match="rc=-4"):
            rt.launch("gemv_w4a4<1>", 16, 256, [pwq, pws, px, asc, px, 128, 1024])     # N beyond the weights
    with pytest.raises(MemoryError):
        rt.alloc(1 << 50)
    with pytest.raises(ValueError):
        W4Runner(rt).gemv_device("w4a8", 0, 0, np.zeros((1, 256), np.float32), 8, 256, threads=512)
    assert rt.has("gemv_w4a8<1,false,1>") and not rt.has("gemv_w4a8<9,false,1>")
    other = Runtime()                            # a second Runtime on the same image is fine
    assert other.has("quant_act")
    with pytest.raises(RuntimeError):
        Runtime(hsaco="/tmp/some_other_image.so", lib=rt.hsaco)
    rt.sync()


def test_copy_queues_beside_the_engine_stream(rt):
    """fm_upload_beside / fm_copy_beside / fm_upload_join and fm_download_beside / fm_download_join: a two-buffer
    pipeline of (upload, kernel, strided download) steps leaves every step's result in pinned host memory, and the
    argument checks hold."""
    rows, width = 64, 48                               # download `width` floats of each of `rows` rows of 256
    n = rows * 256
    host_in = rt.pinned((4, n), np.float32)
    host_in[:] = np.random.default_rng(3).standard_normal((4, n)).astype(np.float32)
    host_out = rt.pinned((4, rows, width), np.float32)
    host_out[:] = np.nan
    with Bufs(rt) as b:
        x = [b.zeros(n), b.zeros(n)]
        mid = b.zeros(n)
        y = [b.zeros(n), b.zeros(n)]
        rt.upload(x[0], host_in[0])
        for t in range(4):
            if t + 1 < 4:
                rt.upload_beside(x[(t + 1) % 2], host_in[t + 1])
            rt.download_join(1)                        # y[t % 2] was last read by the download of step t - 2
            rt.copy_dev(mid, x[t % 2], n * 4)          # the "kernel" of the step on the engine stream: two copies
            rt.copy_dev(y[t % 2], mid, n * 4)
            rt.upload_join()
            rt.download_beside(host_out, y[t % 2] + 16 * 4, width=width * 4, height=rows, dpitch=256 * 4,
                               hpitch=width * 4, host_offset=t * rows * width * 4)
        rt.sync()
        for t in range(4):
            assert np.array_equal(host_out[t], host_in[t].reshape(rows, 256)[:, 16:16 + width])
        flat = rt.pinned((n,), np.float32)
        rt.download_beside(flat, y[1])                 # plain form: all of the array
        rt.download_join(0)
        rt.sync()
        assert np.array_equal(flat, host_in[3])
        with pytest.raises(RuntimeError):
            rt.download_beside(flat, y[1] + 4)         # runs past the allocation
        with pytest.raises(RuntimeError):
            rt.download_join(7)
        with pytest.raises(ValueError):
            rt.download_beside(flat, y[1], width=4096, height=rows, dpitch=1024, hpitch=4096)
        rt.free_pinned(flat)
    rt.free_pinned(host_in)
    rt.free_pinned(host_out)
