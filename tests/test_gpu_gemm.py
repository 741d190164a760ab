"""GPU tier: the tcgen05 prefill GEMM (gemm_w4a4_flat / gemm_w4a4 / gemm_w4a8) through the C
ABI.  Gates: int32 accumulators per (m, n, 128-group) identical to the oracle (dump entries),
C within 1e-5 relative of the float64 oracle, and within the reference example's 1e-3 of its
golden vector (examples/python_w4a4_gemm.py:59-83)."""
from __future__ import annotations

import numpy as np
import pytest

import cases
import w4_oracle as O
from gpu_util import Bufs
from k100lc_kernels import Int4Linear, W4Runner, Workspace, synth
from k100lc_kernels.quant import pack_int4_group128, pack_nibbles

pytestmark = pytest.mark.gpu
REL = 1e-5


def _perm8(q):
    """int8 codes [M,K] -> the (k0,k2,k4,k6,k1,k3,k5,k7) byte order of quant_rows_a8_k."""
    m, k = q.shape
    return np.ascontiguousarray(q.reshape(m, k // 8, 8)[:, :, [0, 2, 4, 6, 1, 3, 5, 7]].astype(np.int8))


def run_gemm(rt, L, a8=False, dump=False):
    m, n, k = L["m"], L["n"], L["k"]
    g = k // 128
    qa = O.quant_rows_a8(L["x"]) if a8 else O.quant_rows(L["x"])
    with Bufs(rt) as b:
        paq = b.put(_perm8(qa["q"]) if a8 else qa["words"])
        pwq, pasc, pwsc = b.put(L["wq"]), b.put(qa["scale_gf"]), b.put(L["wsc_gf"])
        pc = b.zeros(m * n, np.float32, np.nan)
        base = [paq, pwq, pasc, pwsc, pc, m, n, k]
        acc = None
        if dump:
            pi = b.zeros(m * n * g, np.int32, -7)
            rt.launch("gemm_w4a8_iacc" if a8 else "gemm_w4a4_iacc", 1, 256, base + [pi])
            acc = b.get(pi, m * n * g, np.int32).reshape(m, n, g)
        elif a8:
            rt.launch("gemm_w4a8", (n // 64) * (m // 128), 256, base)
        else:
            rt.launch("gemm_w4a4_flat", (n // 64) * (m // 128), 256, base + [n // 64, 0])
        c = b.get(pc, m * n).reshape(m, n)
        assert rt.gemm_status() == 0
    ref = O.gemm_w4(qa["q"], L["wq"], qa["scale_gf"], L["wsc_gf"])
    return c, acc, ref


@pytest.mark.parametrize("a8", [False, True])
@pytest.mark.parametrize("m,n,k", [(128, 128, 128), (128, 64, 256), (256, 192, 640), (384, 320, 1024)])
def test_gemm_accumulators_and_output(rt, a8, m, n, k):
    L = synth.gemm_layer(n, k, m, seed=900 + m + n)
    c, acc, ref = run_gemm(rt, L, a8=a8, dump=True)
    assert np.array_equal(acc, ref["acc"]), "int32 accumulators differ"
    assert O.rel_err(c, ref["c"]) < REL
    c2, _, _ = run_gemm(rt, L, a8=a8)
    assert np.array_equal(c2, c)


def test_gemm_reference_example(rt, golden):
    """The reference's own GEMM self-test: M=256, N=128, K=512, unit weight scales, through
    W4Runner.gemm (quant_rows_fast_k + gemm_w4a4_flat)."""
    arr, _ = golden
    bmat, x = cases.gemm_case()
    n, k = bmat.shape
    runner = W4Runner(rt)
    with Bufs(rt) as b:
        pwq, pwsc = b.put(pack_nibbles(bmat)), b.put(np.ones((k // 128, n), np.float32))
        y = runner.gemm(pwq, pwsc, x, n, k)
        assert rt.gemm_status() == 0
    runner.close()
    assert O.rel_err(y, arr["gemm_w4a4.c"]) < 1e-3
    q = O.quant_rows(x)
    assert O.rel_err(y, O.gemm_w4(q["q"], pack_nibbles(bmat), q["scale_gf"], np.ones((k // 128, n), np.float32))["c"]) < REL


def test_gemm_n64_uses_2d_entry_and_int4linear_prefill(rt):
    L = synth.gemm_layer(64, 256, 128, seed=77)
    runner = W4Runner(rt)
    with Bufs(rt) as b:
        y = runner.gemm(b.put(L["wq"]), b.put(L["wsc_gf"]), L["x"], 64, 256)      # N/64 == 1 -> gemm_w4a4 (2-D)
    runner.close()
    q = O.quant_rows(L["x"])
    assert O.rel_err(y, O.gemm_w4(q["q"], L["wq"], q["scale_gf"], L["wsc_gf"])["c"]) < REL
    # Int4Linear routes 128-aligned row counts to the GEMM (W4A4, or W4A8 with prefill="gemm_a8")
    rng = np.random.default_rng(4)
    n, k, m = 256, 512, 128
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    packed, scales = pack_int4_group128(w)
    x = rng.standard_normal((m, k)).astype(np.float32)
    from k100lc_kernels.quant import dequant_int4_group128
    ref = x.astype(np.float64) @ dequant_int4_group128(packed, scales, n, k).astype(np.float64).T
    with Workspace(rt) as ws:
        y4 = Int4Linear(rt, n, k, packed, scales, "w4a4", ws, "g4").forward(x)
        y8 = Int4Linear(rt, n, k, packed, scales, "w4a8", ws, "g8", prefill="gemm_a8").forward(x)
    assert rt.gemm_status() == 0
    assert O.rel_err(y4, ref) < 3e-1 and O.rel_err(y8, ref) < 3e-2


@pytest.mark.parametrize("a8", [False, True])
def test_gemm_full_size_sampled(rt, a8):
    """M=2048, N=17408, K=5120 (seed 3): C on 48 sampled token rows x 384 sampled channels
    against the oracle run on exactly those rows, plus the whole-matrix checksum property
    sum_n C[m,n] == (sum over sampled...) being finite."""
    L = synth.gemm_layer(seed=3)
    c, _, _ = run_gemm_sampled(rt, L, a8)


def run_gemm_sampled(rt, L, a8):
    m, n, k = L["m"], L["n"], L["k"]
    qa = O.quant_rows_a8(L["x"]) if a8 else O.quant_rows(L["x"])
    with Bufs(rt) as b:
        paq = b.put(_perm8(qa["q"]) if a8 else qa["words"])
        pwq, pasc, pwsc = b.put(L["wq"]), b.put(qa["scale_gf"]), b.put(L["wsc_gf"])
        pc = b.zeros(m * n, np.float32, np.nan)
        base = [paq, pwq, pasc, pwsc, pc, m, n, k]
        if a8:
            rt.launch("gemm_w4a8", (n // 64) * (m // 128), 256, base)
        else:
            rt.launch("gemm_w4a4_flat", (n // 64) * (m // 128), 256, base + [n // 64, 0])
        c = b.get(pc, m * n).reshape(m, n)
        assert rt.gemm_status() == 0
    assert np.isfinite(c).all()
    rng = np.random.default_rng(0)
    mi = np.sort(rng.choice(m, 48, replace=False))
    ni = np.sort(rng.choice(n, 384, replace=False))
    ref = O.gemm_w4(qa["q"][mi], L["wq"][ni], qa["scale_gf"][:, mi], L["wsc_gf"][:, ni])["c"]
    assert O.rel_err(c[np.ix_(mi, ni)], ref) < REL
    return c, None, None


@pytest.mark.parametrize("a8", [False, True])
def test_gemm_full_size_accumulators(rt, a8):
    """M=2048, N=17408, K=5120 (seed 3): the int32 accumulators of every 128-group, bit for bit, on three
    windows of the full-size run — the last row tile x last column tile, all row tiles across a column-tile
    boundary, and all column tiles across a row-tile boundary (so every CTA's first and last tile, every
    accumulator rotation and every ring wrap-around is sampled).  The whole GEMM runs for each window."""
    L = synth.gemm_layer(seed=3)
    m, n, k = L["m"], L["n"], L["k"]
    g = k // 128
    qa = O.quant_rows_a8(L["x"]) if a8 else O.quant_rows(L["x"])
    windows = [(m - 128, m, n - 128, n), (0, m, n // 2 - 8, n // 2 + 8), (m // 2 - 8, m // 2 + 8, 0, n)]
    with Bufs(rt) as b:
        paq = b.put(_perm8(qa["q"]) if a8 else qa["words"])
        pwq, pasc, pwsc = b.put(L["wq"]), b.put(qa["scale_gf"]), b.put(L["wsc_gf"])
        pc = b.zeros(m * n, np.float32, np.nan)
        for (m0, m1, n0, n1) in windows:
            cnt = (m1 - m0) * (n1 - n0) * g
            pi = b.zeros(cnt, np.int32, -7)
            rt.launch("gemm_w4a8_iacc_win" if a8 else "gemm_w4a4_iacc_win", 1, 256,
                      [paq, pwq, pasc, pwsc, pc, m, n, k, pi, m0, m1, n0, n1])
            acc = b.get(pi, cnt, np.int32).reshape(m1 - m0, n1 - n0, g)
            assert rt.gemm_status() == 0
            ref = O.gemm_w4(qa["q"][m0:m1], L["wq"][n0:n1], qa["scale_gf"][:, m0:m1], L["wsc_gf"][:, n0:n1])
            assert np.array_equal(acc, ref["acc"]), f"int32 accumulators differ in window {(m0, m1, n0, n1)}"
            c = b.get(pc, m * n).reshape(m, n)[m0:m1, n0:n1]
            assert O.rel_err(c, ref["c"]) < REL


def _nvfp4_gemm(rt, L, x, name="nvfp4_gemm_kernel", dump=False):
    n, k, m = L["n"], L["k"], x.shape[0]
    q = O.nvfp4_quant_act(x)
    with Bufs(rt) as b:
        args = [b.put(L["wq"]), b.put(L["ws"]), b.put(q["even"]), b.put(q["odd"]), b.put(q["scale"])]
        pc = b.zeros(m * n, np.float32, np.nan)
        args += [pc, m, n, k, float(L["gscale"])]
        acc = None
        if dump:
            pi = b.zeros(m * n * (k // 16), np.int32, -7)
            rt.launch("nvfp4_gemm_iacc", 1, 256, args + [pi])
            acc = b.get(pi, m * n * (k // 16), np.int32).reshape(m, n, -1)
        else:
            rt.launch2d(name, -(-n // 64), -(-m // 64), 256, 1, args)
        c = b.get(pc, m * n).reshape(m, n)
    return c, acc, q


@pytest.mark.parametrize("m,n,k", [(64, 128, 128), (200, 72, 512), (128, 384, 1280), (5, 19, 256)])
def test_nvfp4_gemm_accumulators_and_output(rt, m, n, k):
    """nvfp4_gemm_kernel (no reference test exists for it: parity unpinned, the oracle is nvfp4_gemv's formula on M rows):
    the int32 of every (token, row, 16-block) bit for bit, C within 1e-5, ragged M and N included."""
    L = synth.nvfp4_layer(n, k, m, seed=1700 + m)
    c, acc, q = _nvfp4_gemm(rt, L, L["x"], dump=True)
    ref = O.nvfp4_gemv(L["wq"], L["ws"], q["q"], q["scale"], L["gscale"])
    assert np.array_equal(acc, ref["acc"])
    assert O.rel_err(c, ref["y"]) < REL
    for name in ("nvfp4_gemm_kernel", "nvfp4_gemm_kernel_ng"):
        c2, _, _ = _nvfp4_gemm(rt, L, L["x"], name=name)
        assert np.array_equal(c2, c)
    # the GEMM and the GEMV agree row by row
    if m <= 8:
        with Bufs(rt) as b:
            py = b.zeros(m * n, np.float32, np.nan)
            for r0 in range(0, m, 4):
                mm = min(4, m - r0)
                rt.launch(f"nvfp4_gemv<{mm},1>", -(-n // 4), 256,
                          [b.put(L["wq"]), b.put(L["ws"]), b.put(q["even"][r0:r0 + mm]), b.put(q["odd"][r0:r0 + mm]),
                           b.put(q["scale"][r0:r0 + mm]), py + r0 * n * 4, n, k, float(L["gscale"])])
            assert O.rel_err(b.get(py, m * n).reshape(m, n), c) < 1e-6


def test_nvfp4_gemm_full_size_sampled_and_linear_prefill(rt):
    """M=2048, N=17408, K=5120 (seed 2): C on sampled token rows x sampled channels against the oracle on exactly those;
    NVFP4Linear sends row counts above 4 to the GEMM."""
    from k100lc_kernels import NVFP4Linear, Workspace
    L = synth.nvfp4_layer(m=1, seed=2)
    m = 2048
    x = np.random.default_rng(21).standard_normal((m, L["k"])).astype(np.float32)
    c, _, q = _nvfp4_gemm(rt, L, x)
    assert np.isfinite(c).all()
    rng = np.random.default_rng(0)
    mi = np.sort(rng.choice(m, 24, replace=False))
    ni = np.sort(rng.choice(L["n"], 256, replace=False))
    ref = O.nvfp4_gemv(L["wq"][ni], L["ws"][ni], q["q"][mi], q["scale"][mi], L["gscale"])["y"]
    assert O.rel_err(c[np.ix_(mi, ni)], ref) < REL
    with Workspace(rt) as ws:
        lin = NVFP4Linear(rt, L["n"], L["k"], L["wq"], L["ws"], L["gscale"], ws, "nvl")
        y = lin.forward(x[:70])
    assert np.array_equal(y, c[:70])
