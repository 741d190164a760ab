"""GPU tier: row gather / weighted combine kernels and the bucketed mixture-of-experts forward built on the
quantized linear layers (reference python/k100lc_kernels/model.py:582-720, tools/selftest_all.py:450-489)."""
from __future__ import annotations

import numpy as np
import pytest

import w4_oracle as O
from gpu_util import Bufs
from k100lc_kernels import Int4Linear, MoECombine, MoEExperts, Workspace
from k100lc_kernels.quant import pack_int4_group128

pytestmark = pytest.mark.gpu


def _judge(got, ref):
    return np.abs(got - ref).max() <= 1e-4 + 1e-5 * max(1.0, float(np.abs(ref).max()))


def test_gather_and_combine_kernels(rt):
    rng = np.random.default_rng(15)
    rows, dim = 7, 256
    src = rng.standard_normal((20, dim)).astype(np.float32)
    idx = rng.integers(0, 20, size=rows).astype(np.uint32)
    with Bufs(rt) as b:
        d = b.zeros(rows * dim, np.float32, np.nan)
        rt.launch("gather_rows_k", rows, 64, [d, b.put(src), b.put(idx), rows, dim])
        assert np.array_equal(b.get(d, rows * dim).reshape(rows, dim), src[idx])
    # the reference's two combine cases (seeds 16 and 17)
    rows, dim, n_exp = 5, 512, 3
    rng = np.random.default_rng(16)
    exp_out = rng.standard_normal((n_exp, rows, dim)).astype(np.float32)
    weights = rng.random((rows, n_exp)).astype(np.float32)
    with Workspace(rt) as ws:
        got = MoECombine(rt, rows, dim, n_exp, ws).forward(exp_out, weights)
    assert _judge(got, np.einsum("re,erd->rd", weights, exp_out))
    rows, n_sel, erows, dim = 5, 3, 8, 1024
    rng = np.random.default_rng(17)
    off = np.arange(n_sel + 1, dtype=np.uint32) * erows
    bucket = rng.standard_normal((off[-1], dim)).astype(np.float32)
    weights = rng.random((rows, n_sel)).astype(np.float32)
    base = (off[:n_sel][None, :] + rng.integers(0, erows, size=(rows, n_sel)).astype(np.uint32)).astype(np.uint32)
    with Bufs(rt) as b:
        y = b.zeros(rows * dim, np.float32, np.nan)
        rt.launch("moe_combine_gather_k", rows, 64, [y, b.put(bucket), b.put(weights), b.put(base), n_sel, rows, dim])
        got = b.get(y, rows * dim).reshape(rows, dim)
    ref = np.zeros((rows, dim), np.float32)
    for r in range(rows):
        for e in range(n_sel):
            ref[r] += weights[r, e] * bucket[base[r, e]]
    assert np.array_equal(got, ref)


@pytest.mark.parametrize("path", ["w4a8", "w4a16"])
def test_moe_experts_over_quantized_layers(rt, path):
    """Six experts, top-2 routing of 9 tokens (one pair unused, one expert with no token, one with five): the
    bucketed forward equals the weighted sum of each chosen expert applied to the token on its own."""
    rng = np.random.default_rng(31)
    n_exp, rows, dim, out_dim, topk = 6, 9, 256, 128, 2
    packs = [pack_int4_group128((rng.standard_normal((out_dim, dim)) * 0.05).astype(np.float32)) for _ in range(n_exp)]
    x = rng.standard_normal((rows, dim)).astype(np.float32)
    ids = np.array([[0, 1], [1, 2], [1, 4], [1, 0], [1, 5], [1, 2], [4, 0], [2, -1], [5, 4]])
    w = rng.random((rows, topk)).astype(np.float32)
    w[3, 1] = 0.0
    with Workspace(rt) as ws:
        experts = [Int4Linear(rt, out_dim, dim, p, s, path, ws, f"e{i}") for i, (p, s) in enumerate(packs)]
        moe = MoEExperts(rt, experts, rows, dim, out_dim, topk, ws)
        got = moe.forward(x, ids, w)
        bucket_rows, base, wz, offsets = moe.route(ids, w)
        assert offsets[-1] == 16 and offsets[4] == offsets[3]          # 18 pairs, two unused; expert 3 idle
        single = {(r, int(e)): experts[int(e)].forward(x[r:r + 1])[0].copy()
                  for r in range(rows) for e in ids[r] if 0 <= e < n_exp}
    ref = np.zeros((rows, out_dim), np.float64)
    for r in range(rows):
        for j in range(topk):
            if wz[r, j] != 0:
                ref[r] += np.float64(wz[r, j]) * single[(r, int(ids[r, j]))]
    assert O.rel_err(got, ref) < 1e-5
    # nothing routed at all: zeros
    with Workspace(rt) as ws:
        experts = [Int4Linear(rt, out_dim, dim, p, s, path, ws, f"e{i}") for i, (p, s) in enumerate(packs[:2])]
        z = MoEExperts(rt, experts, 2, dim, out_dim, 1, ws).forward(x[:2], np.array([[-1], [7]]), np.ones((2, 1), np.float32))
    assert np.array_equal(z, np.zeros((2, out_dim), np.float32))
