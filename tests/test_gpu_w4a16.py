"""GPU tier: the W4A16 path (int4_dot_k + reduce_blocks_k + int4_dequant_k) through the
C ABI (reference cases tools/selftest_all.py:639-660, 726-770 and
tools/gen_int4_dot.py:318-418)."""
from __future__ import annotations

import numpy as np
import pytest

import cases
import w4_oracle as O
from gpu_util import Bufs
from k100lc_kernels import synth
from k100lc_kernels.model import div_magic

pytestmark = pytest.mark.gpu
REL = 1e-5


def test_int4_dequant_bit_exact(rt, golden):
    arr, _ = golden
    packed, scales = cases.int4_dequant_case()
    with Bufs(rt) as b:
        pw, ps, py = b.put(packed), b.put(scales), b.zeros(64 * 128)
        rt.launch("int4_dequant_k", (packed.size + 63) // 64, 64, [pw, ps, py, packed.size, 64])
        got = b.get(py, 64 * 128)
    assert np.array_equal(got.view(np.uint32), arr["int4_dequant.y"].view(np.uint32))


def test_reduce_blocks(rt, golden):
    arr, _ = golden
    part = cases.reduce_case()
    with Bufs(rt) as b:
        pp, py = b.put(part), b.zeros(32)
        rt.launch("reduce_blocks_k", 32, 64, [pp, py, 32, 5])
        got = b.get(py, 32)
    assert np.array_equal(got, O.reduce_blocks(part, 32, 5))          # same order of fp32 adds
    assert np.abs(got - arr["reduce_blocks.y"]).max() <= 1e-4 + 1e-5 * max(1.0, np.abs(arr["reduce_blocks.y"]).max())


def test_int4_dot_experts(rt, golden):
    """Two experts of six rows with their own activation rows (the reference's case)."""
    arr, _ = golden
    packed, scales, x = cases.int4_dot_case()
    nbpr, rpe, nexp = 8, 6, 2
    nblocks = rpe * nexp * nbpr
    with Bufs(rt) as b:
        pw, ps, px, pp = b.put(packed), b.put(scales), b.put(x), b.zeros(nblocks)
        ids = b.put(np.arange(nexp, dtype=np.uint32))
        argv = [pw, px, pp, nblocks, 64, nbpr, div_magic(nbpr, nblocks), rpe, div_magic(rpe, nblocks // nbpr + 1),
                ps, ids, rpe * nbpr * 64, rpe, div_magic(rpe, nblocks // nbpr + 1)]
        rt.launch("int4_dot_k", nblocks, 64, argv)
        got = b.get(pp, nblocks)
    ref = arr["int4_dot.partial"]
    assert np.abs(got - ref).max() <= 1e-4 + 1e-5 * max(1.0, float(np.abs(ref).max()))
    assert O.rel_err(got, O.int4_dot_partial(packed, scales, x, 12, 8, ids=[0, 1], rows_per_exp=6, rows_per_w=6)) < REL


def test_int4_dot_permuted_experts(rt):
    """ids selects weight experts out of order; the activation row follows rows_per_exp."""
    rng = np.random.default_rng(77)
    nbpr, rpw, nexp = 4, 10, 3
    packed = rng.integers(0, 1 << 32, size=(nexp * rpw, nbpr * 16), dtype=np.uint64).astype(np.uint32)
    scales = cases._bf16_trunc_bits(rng, nexp * rpw * nbpr)
    x = rng.standard_normal((2, nbpr * 128)).astype(np.float32)
    ids = np.array([2, 0], dtype=np.uint32)
    nrows, nblocks = 2 * rpw, 2 * rpw * nbpr
    with Bufs(rt) as b:
        pw, ps, px, pp, pid = b.put(packed), b.put(scales), b.put(x), b.zeros(nblocks), b.put(ids)
        rt.launch("int4_dot_k", (nblocks + 63) // 64, 64,
                  [pw, px, pp, nblocks, 64, nbpr, 0, rpw, 0, ps, pid, rpw * nbpr * 64, rpw, 0])
        got = b.get(pp, nblocks)
    ref = O.int4_dot_partial(packed, scales, x, nrows, nbpr, ids=ids, rows_per_exp=rpw, rows_per_w=rpw)
    assert O.rel_err(got, ref) < REL


@pytest.mark.parametrize("n,k", [(64, 1024), (17408, 5120)])
def test_w4a16_layer(rt, n, k):
    """Dense layer (benchmark shape, seed 0): dot + reduce against the float64 oracle."""
    L = synth.w4a16_layer(n, k, seed=0)
    nbpr, nblocks = k // 128, n * (k // 128)
    with Bufs(rt) as b:
        pw, ps, px = b.put(L["packed"]), b.put(L["scale_bf16"]), b.put(L["x"])
        pp, py, ids = b.zeros(nblocks), b.zeros(n), b.put(np.arange(n, dtype=np.uint32))
        rt.launch("int4_dot_k", (nblocks + 63) // 64, 64,
                  [pw, px, pp, nblocks, 64, nbpr, div_magic(nbpr, nblocks), n, div_magic(n, n),
                   ps, ids, nbpr * 64, n, div_magic(n, n)])
        rt.launch("reduce_blocks_k", (n + 63) // 64, 64, [pp, py, n, nbpr])
        part, y = b.get(pp, nblocks), b.get(py, n)
    assert O.rel_err(part, O.int4_dot_partial(L["packed"], L["scale_bf16"], L["x"][None, :], n, nbpr)) < REL
    assert O.rel_err(y, O.w4a16_gemv(L["packed"], L["scale_bf16"], L["x"])[0]) < REL
