"""GPU tier: W4A8 / W4A4 / NVFP4 decode GEMV through the C ABI.

Gates: integer accumulators identical to the oracle (dump entries), fp32 outputs within
1e-5 relative (max|d| / max|ref|) of the float64 oracle; the committed reference vectors
are checked to the reference's own tolerances as well (tools/selftest_all.py:854-910,
1087-1130)."""
from __future__ import annotations

import numpy as np
import pytest

import cases
import w4_oracle as O
from gpu_util import Bufs
from k100lc_kernels import synth
from k100lc_kernels.quant import pack_nibbles

pytestmark = pytest.mark.gpu
REL = 1e-5


def w4a8_device(rt, wq, ws, x, name=None, grid=None, dump=False):
    n, k = wq.shape[0], wq.shape[1] * 8
    m = x.shape[0]
    q = O.quant_act(x)
    with Bufs(rt) as b:
        pwq, pws = b.put(wq), b.put(ws)
        ae, ao, asc, asu = b.put(q["even"]), b.put(q["odd"]), b.put(q["scale"]), b.put(q["gsum"])
        py = b.zeros(m * n, np.float32, np.nan)
        if dump:
            pi = b.zeros(m * n * (k // 128), np.int32, -7)
            rt.launch("gemv_w4a8_iacc", -(-n // 4), 256, [pwq, pws, ae, ao, asc, asu, py, n, k, pi, m])
            return b.get(py, m * n).reshape(m, n), b.get(pi, m * n * (k // 128), np.int32).reshape(m, n, -1), q
        rpw = 1 if m == 1 else 2
        name = name or f"gemv_w4a8<{m},false,{rpw}>"
        rt.launch(name, grid if grid is not None else -(-n // (4 * rpw)), 256,
                  [pwq, pws, ae, ao, asc, asu, py, n, k])
        return b.get(py, m * n).reshape(m, n), None, q


def w4a4_device(rt, wq, ws, x, name=None, grid=None, dump=False):
    n, k = wq.shape[0], wq.shape[1] * 8
    m = x.shape[0]
    q = O.quant_act4(x)
    with Bufs(rt) as b:
        pwq, pws, aq, asc = b.put(wq), b.put(ws), b.put(q["packed"]), b.put(q["scale"])
        py = b.zeros(m * n, np.float32, np.nan)
        if dump:
            pi = b.zeros(m * n * (k // 32), np.int32, -7)
            rt.launch("gemv_w4a4_iacc", -(-n // 4), 256, [pwq, pws, aq, asc, py, n, k, pi, m])
            return b.get(py, m * n).reshape(m, n), b.get(pi, m * n * (k // 32), np.int32).reshape(m, n, -1), q
        name = name or f"gemv_w4a4<{m}>"
        rows_per_wg = 8 if "_r2" in name else 4
        rt.launch(name, grid if grid is not None else -(-n // rows_per_wg), 256, [pwq, pws, aq, asc, py, n, k])
        return b.get(py, m * n).reshape(m, n), None, q


@pytest.mark.parametrize("name,seed,m,kernel", [
    ("w4a4_m1", 60, 1, "gemv_w4a4<1>"), ("w4a4_m4", 61, 4, "gemv_w4a4<4>"),
    ("w4a4_r2_m4", 62, 4, "gemv_w4a4_r2_k"), ("w4a8_m1", 63, 1, "gemv_w4a8<1,false,1>"),
    ("w4a8_m2", 163, 2, "gemv_w4a8<2,false,2>"), ("w4a8_m3", 164, 3, "gemv_w4a8<3,false,2>"),
    ("w4a8_m4", 165, 4, "gemv_w4a8<4,false,2>"), ("w4a4_m2", 166, 2, "gemv_w4a4<2>"),
    ("w4a4_m3", 167, 3, "gemv_w4a4<3>")])
def test_w4_golden(rt, golden, name, seed, m, kernel):
    arr, _ = golden
    wv, ws, x = cases.w4_case(seed, 256, 5120, m)
    dev = w4a8_device if "w4a8" in kernel else w4a4_device
    y, _, _ = dev(rt, pack_nibbles(wv), ws, x, name=kernel)
    ref = arr[f"{name}.y"]
    assert np.abs(y - ref).max() <= 1e-4 + 1e-5 * max(1.0, float(np.abs(ref).max()))   # the tolerance of the reference's own acceptance check
    assert O.rel_err(y, ref) < REL


@pytest.mark.parametrize("m", [1, 2, 3, 4])
@pytest.mark.parametrize("n,k", [(256, 5120), (37, 1024), (130, 2176), (9, 128), (70, 6144), (45, 17408)])
def test_w4_accumulators_and_output(rt, m, n, k):
    """Ragged N, K that is / is not a multiple of 1024 (5120, 6144 and 17408 have unrolled kernels of their own
    at M = 1), every M: integer accumulators bit-exact, outputs within 1e-5."""
    L = synth.rt4_layer(n, k, m, seed=300 + m)
    for dev, grp in ((w4a8_device, 128), (w4a4_device, 32)):
        y, acc, q = dev(rt, L["wq"], L["ws"], L["x"], dump=True)
        ref = O.gemv_w4(L["wq"], L["ws"], q["q"], q["scale"], grp)
        assert np.array_equal(acc, ref["acc"]), f"integer accumulators differ (group {grp})"
        assert O.rel_err(y, ref["y"]) < REL
        y2, _, _ = dev(rt, L["wq"], L["ws"], L["x"])
        assert O.rel_err(y2, ref["y"]) < REL


def test_w4_two_row_names_and_partial_grid(rt):
    """gemv_w4a4_r2_m3_k, the SMEM=true names, and a grid that covers only part of N:
    rows beyond grid*rows_per_workgroup stay untouched, as with the reference kernels."""
    L = synth.rt4_layer(96, 5120, 3, seed=41)
    q4 = O.quant_act4(L["x"])
    ref4 = O.gemv_w4(L["wq"], L["ws"], q4["q"], q4["scale"], 32)["y"]
    y, _, _ = w4a4_device(rt, L["wq"], L["ws"], L["x"], name="gemv_w4a4_r2_m3_k")
    assert O.rel_err(y, ref4) < REL
    q8 = O.quant_act(L["x"])
    ref8 = O.gemv_w4(L["wq"], L["ws"], q8["q"], q8["scale"], 128)["y"]
    y, _, _ = w4a8_device(rt, L["wq"], L["ws"], L["x"], name="gemv_w4a8<3,true,2>")
    assert O.rel_err(y, ref8) < REL
    y, _, _ = w4a8_device(rt, L["wq"], L["ws"], L["x"], grid=5)         # 5 groups x 8 rows = 40 rows
    assert O.rel_err(y[:, :40], ref8[:, :40]) < REL and np.isnan(y[:, 40:]).all()
    y, _, _ = w4a8_device(rt, L["wq"], L["ws"], L["x"], grid=1000)      # over-provisioned grid
    assert O.rel_err(y, ref8) < REL


@pytest.mark.parametrize("kind", ["w4a8", "w4a4"])
@pytest.mark.parametrize("n,k", [(1000, 5120), (333, 6144), (17408, 5120)])
def test_quantiser_inside_the_gemv_leaves_the_same_bits(rt, kind, n, k):
    """quant_gemv_w4a8 / quant_gemv_w4a4 (one token, x fp32 in, the CTA quantises x itself): the bits of the quantiser
    launch followed by the GEMV launch, within 1e-5 of the oracle; a grid that covers fewer rows leaves the others
    alone; another K is refused."""
    L = synth.rt4_layer(n, k, 1, seed=4100 + n % 7)
    q = O.quant_act(L["x"]) if kind == "w4a8" else O.quant_act4(L["x"])
    ref = O.gemv_w4(L["wq"], L["ws"], q["q"], q["scale"], 128 if kind == "w4a8" else 32)["y"][0]
    two, _, _ = (w4a8_device if kind == "w4a8" else w4a4_device)(rt, L["wq"], L["ws"], L["x"])
    with Bufs(rt) as b:
        pwq, pws, px = b.put(L["wq"]), b.put(L["ws"]), b.put(L["x"][0])
        py = b.zeros(n, np.float32, np.nan)
        rt.launch(f"quant_gemv_{kind}", -(-n // 4), 256, [pwq, pws, px, py, n, k])
        one = b.get(py, n)
        part = b.zeros(n, np.float32, np.nan)
        rt.launch(f"quant_gemv_{kind}", 10, 256, [pwq, pws, px, part, n, k])       # 40 rows
        some = b.get(part, n)
        with pytest.raises(RuntimeError, match="rc=-4"):
            rt.launch(f"quant_gemv_{kind}", -(-n // 4), 256, [pwq, pws, px, py, n, 4096])
    assert np.array_equal(one.view(np.uint32), two[0].view(np.uint32))
    assert O.rel_err(one, ref) < REL
    assert np.array_equal(some[:40].view(np.uint32), one[:40].view(np.uint32)) and np.isnan(some[40:]).all()


@pytest.mark.parametrize("kind", ["w4a8", "w4a4"])
def test_w4_full_size(rt, kind):
    """The benchmark shape 17408 x 5120 at M=1 (seed 1): accumulators and y."""
    L = synth.rt4_layer(m=1, seed=1)
    dev, grp = (w4a8_device, 128) if kind == "w4a8" else (w4a4_device, 32)
    y, acc, q = dev(rt, L["wq"], L["ws"], L["x"], dump=True)
    ref = O.gemv_w4(L["wq"], L["ws"], q["q"], q["scale"], grp)
    assert np.array_equal(acc, ref["acc"])
    y2, _, _ = dev(rt, L["wq"], L["ws"], L["x"])
    assert O.rel_err(y, ref["y"]) < REL and O.rel_err(y2, ref["y"]) < REL
    # linearity in the weight scales: doubling ws doubles y exactly (power of two)
    y3, _, _ = dev(rt, L["wq"], (L["ws"].astype(np.float32) * 2).astype(np.float16), L["x"])
    assert np.array_equal(y3, 2 * y2)


def nvfp4_device(rt, L, x, name, grid=None, dump=False):
    n, k, m = L["n"], L["k"], x.shape[0]
    q = O.nvfp4_quant_act(x)
    with Bufs(rt) as b:
        pwq, pws = b.put(L["wq"]), b.put(L["ws"])
        qa, qb, sc = b.put(q["even"]), b.put(q["odd"]), b.put(q["scale"])
        py = b.zeros(m * n, np.float32, np.nan)
        if dump:
            pi = b.zeros(m * n * (k // 16), np.int32, -7)
            rt.launch("nvfp4_gemv_iacc", -(-n // 4), 256, [pwq, pws, qa, qb, sc, py, n, k, float(L["gscale"]), pi, m])
            return b.get(py, m * n).reshape(m, n), b.get(pi, m * n * (k // 16), np.int32).reshape(m, n, -1), q
        bw = int(name.split(",")[1].rstrip(">"))
        rt.launch(name, grid if grid is not None else -(-n // (4 * bw)), 256,
                  [pwq, pws, qa, qb, sc, py, n, k, float(L["gscale"])])
        return b.get(py, m * n).reshape(m, n), None, q


def test_nvfp4_all_variants(rt, golden):
    """All 24 template names on the reference's case (N=32, K=512, seed 202); A = tokens."""
    arr, _ = golden
    for a in (1, 2, 3, 4):
        codes, ws, x = cases.nvfp4_case(202, 32, 512, a)
        L = dict(n=32, k=512, wq=pack_nibbles(codes), ws=ws, gscale=0.75)
        q = O.nvfp4_quant_act(x)
        ref = O.nvfp4_gemv(L["wq"], ws, q["q"], q["scale"], 0.75)["y"]
        for wide, bs in ((False, (1, 2, 3, 4)), (True, (1, 2))):
            for bw in bs:
                name = f"nvfp4_gemv{'_wide' if wide else ''}<{a},{bw}>"
                y, _, _ = nvfp4_device(rt, L, x, name)
                assert O.rel_err(y, ref) < REL, name
        if a == 1:
            g = arr["nvfp4_gemv.y"]
            assert np.abs(y - g).max() <= 1e-2 + 1e-5 * float(np.abs(g).max())
        if a == 3:
            assert np.abs(y - arr["nvfp4_gemv_m3.y"]).max() <= 1e-2 + 1e-5 * float(np.abs(arr["nvfp4_gemv_m3.y"]).max())


@pytest.mark.parametrize("m", [1, 2, 3, 4])
@pytest.mark.parametrize("n,k", [(64, 5120), (19, 1056), (5, 32)])
def test_nvfp4_accumulators(rt, m, n, k):
    L = synth.nvfp4_layer(n, k, m, seed=500 + m)
    y, acc, q = nvfp4_device(rt, L, L["x"], None, dump=True)
    ref = O.nvfp4_gemv(L["wq"], L["ws"], q["q"], q["scale"], L["gscale"])
    assert np.array_equal(acc, ref["acc"])
    assert O.rel_err(y, ref["y"]) < REL
    y2, _, _ = nvfp4_device(rt, L, L["x"], f"nvfp4_gemv<{m},1>")
    assert O.rel_err(y2, ref["y"]) < REL


def test_nvfp4_all_e4m3_codes(rt):
    """Every finite E4M3 scale code, both signs, including subnormals."""
    L = synth.nvfp4_layer(16, 512, 1, seed=9)
    ws = np.arange(16 * 32, dtype=np.int64).reshape(16, 32) % 256
    ws[(ws & 0x7F) == 0x7F] = 0x3C                   # the NaN codes are unspecified in the reference
    L["ws"] = ws.astype(np.uint8)
    y, acc, q = nvfp4_device(rt, L, L["x"], None, dump=True)
    ref = O.nvfp4_gemv(L["wq"], L["ws"], q["q"], q["scale"], L["gscale"])
    assert np.array_equal(acc, ref["acc"]) and O.rel_err(y, ref["y"]) < REL


def test_nvfp4_full_size(rt):
    L = synth.nvfp4_layer(m=1, seed=2)
    y, acc, q = nvfp4_device(rt, L, L["x"], None, dump=True)
    ref = O.nvfp4_gemv(L["wq"], L["ws"], q["q"], q["scale"], L["gscale"])
    assert np.array_equal(acc, ref["acc"])
    y2, _, _ = nvfp4_device(rt, L, L["x"], "nvfp4_gemv<1,1>")
    assert O.rel_err(y, ref["y"]) < REL and O.rel_err(y2, ref["y"]) < REL


@pytest.mark.parametrize("m", [2, 3, 4])
def test_w4a8_full_size_several_tokens(rt, m):
    """17408 x 5120 at M = 2, 3, 4 (seed 1): gemv_w4a8<M,false,2> — the tensor-core kernel — with its own
    integer accumulators (the dump entry runs the same kernel source) and y."""
    L = synth.rt4_layer(m=m, seed=1)
    y, acc, q = w4a8_device(rt, L["wq"], L["ws"], L["x"], dump=True)
    ref = O.gemv_w4(L["wq"], L["ws"], q["q"], q["scale"], 128)
    assert np.array_equal(acc, ref["acc"])
    y2, _, _ = w4a8_device(rt, L["wq"], L["ws"], L["x"])
    assert O.rel_err(y, ref["y"]) < REL and O.rel_err(y2, ref["y"]) < REL


@pytest.mark.parametrize("m,name", [(2, "gemv_w4a4<2>"), (3, "gemv_w4a4<3>"), (4, "gemv_w4a4<4>"), (4, "gemv_w4a4_r2_k"),
                                    (3, "gemv_w4a4_r2_m3_k")])
def test_w4a4_full_size_several_tokens(rt, m, name):
    L = synth.rt4_layer(m=m, seed=1)
    y, acc, q = w4a4_device(rt, L["wq"], L["ws"], L["x"], dump=True)
    ref = O.gemv_w4(L["wq"], L["ws"], q["q"], q["scale"], 32)
    assert np.array_equal(acc, ref["acc"])
    y2, _, _ = w4a4_device(rt, L["wq"], L["ws"], L["x"], name=name)
    assert O.rel_err(y, ref["y"]) < REL and O.rel_err(y2, ref["y"]) < REL


@pytest.mark.parametrize("m,bw", [(2, 1), (3, 1), (4, 1), (2, 2), (4, 2)])
def test_nvfp4_full_size_several_tokens(rt, m, bw):
    """17408 x 5120 at M = 2..4 (seed 2): nvfp4_gemv<M,1> and the <M,2> variants, accumulators and y."""
    L = synth.nvfp4_layer(m=m, seed=2)
    y, acc, q = nvfp4_device(rt, L, L["x"], None, dump=True)
    ref = O.nvfp4_gemv(L["wq"], L["ws"], q["q"], q["scale"], L["gscale"])
    assert np.array_equal(acc, ref["acc"])
    y2, _, _ = nvfp4_device(rt, L, L["x"], f"nvfp4_gemv<{m},{bw}>")
    assert O.rel_err(y, ref["y"]) < REL and O.rel_err(y2, ref["y"]) < REL


def test_w4a8_mma_accumulators_small_and_ragged(rt):
    """The tensor-core GEMV's own accumulator dump on ragged shapes (N not a multiple of 16, K = 128 .. 2176)."""
    for m in (2, 3, 4):
        for n, k in ((37, 1024), (130, 2176), (9, 128), (256, 5120)):
            L = synth.rt4_layer(n, k, m, seed=640 + m)
            y, acc, q = w4a8_device(rt, L["wq"], L["ws"], L["x"], dump=True)
            ref = O.gemv_w4(L["wq"], L["ws"], q["q"], q["scale"], 128)
            assert np.array_equal(acc, ref["acc"]) and O.rel_err(y, ref["y"]) < REL


def test_zz_ring_status_clean(rt):
    """The by-name GEMVs of this file run on the bulk-copy ring at K = 5120: none of their bounded waits ran out."""
    assert rt.stream_status() == 0
