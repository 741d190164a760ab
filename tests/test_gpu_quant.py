"""GPU tier: activation quantisers through the C ABI, bit-exact against the oracle and
the committed reference vectors (reference cases tools/selftest_all.py:940-1016,
1071-1085)."""
from __future__ import annotations

import numpy as np
import pytest

import cases
import w4_oracle as O
from gpu_util import Bufs

pytestmark = pytest.mark.gpu


def _bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def run_quant_act(rt, x, twod=False):
    m, k = x.shape
    with Bufs(rt) as b:
        px = b.put(x)
        ae, ao = b.zeros(m * k // 2, np.int8, 77), b.zeros(m * k // 2, np.int8, 77)
        asc, asu = b.zeros(m * k // 128), b.zeros(m * k // 128, np.int32)
        if twod:
            rt.launch2d("quant_act", k // 128, m, 32, 1, [px, ae, ao, asc, asu, m, k])
        else:
            for r in range(m):
                rt.launch("quant_act", k // 128, 32, [px + r * k * 4, ae + r * k // 2, ao + r * k // 2,
                                                     asc + r * (k // 128) * 4, asu + r * (k // 128) * 4, 1, k])
        return (b.get(ae, m * k // 2, np.int8).reshape(m, -1), b.get(ao, m * k // 2, np.int8).reshape(m, -1),
                b.get(asc, m * k // 128).reshape(m, -1), b.get(asu, m * k // 128, np.int32).reshape(m, -1))


def test_quant_act_golden(rt, golden):
    arr, _ = golden
    x = cases.normal_case(72, 1, 5120)
    ae, ao, asc, asu = run_quant_act(rt, x)
    assert np.array_equal(ae[0], arr["quant_act.even"]) and np.array_equal(ao[0], arr["quant_act.odd"])
    assert np.array_equal(_bits(asc), _bits(arr["quant_act.s"]))
    assert np.array_equal(asu, arr["quant_act.gsum"])


@pytest.mark.parametrize("m,k,twod", [(1, 128, False), (3, 1024, True), (4, 5120, False), (2, 17408, True)])
def test_quant_act_oracle(rt, m, k, twod):
    rng = np.random.default_rng(1000 + m + k)
    x = (rng.standard_normal((m, k)) * rng.uniform(0.01, 30.0, (m, 1))).astype(np.float32)
    x[0, :128] = 0.0                                  # an all-zero group takes scale 1
    x[m - 1, 5] = np.float32(1e30)                    # a huge outlier: everything else rounds to 0
    r = O.quant_act(x)
    ae, ao, asc, asu = run_quant_act(rt, x, twod)
    assert np.array_equal(ae, r["even"]) and np.array_equal(ao, r["odd"])
    assert np.array_equal(_bits(asc), _bits(r["scale"])) and np.array_equal(asu, r["gsum"])


def run_quant_act4(rt, x):
    m, k = x.shape
    with Bufs(rt) as b:
        px, aq, asc = b.put(x), b.zeros(m * k // 2, np.uint8, 0xAB), b.zeros(m * k // 32)
        for r in range(m):
            rt.launch("quant_act4", k // 32, 32, [px + r * k * 4, aq + r * k // 2, asc + r * (k // 32) * 4, 1, k])
        return b.get(aq, m * k // 2, np.uint8).reshape(m, -1), b.get(asc, m * k // 32).reshape(m, -1)


def test_quant_act4(rt, golden):
    arr, _ = golden
    aq, asc = run_quant_act4(rt, cases.normal_case(71, 1, 5120))
    assert np.array_equal(aq[0], arr["quant_act4.packed"]) and np.array_equal(_bits(asc), _bits(arr["quant_act4.s"]))
    rng = np.random.default_rng(7)
    x = (rng.standard_normal((4, 5120)) * 3).astype(np.float32)
    x[2, 64:96] = 0
    r = O.quant_act4(x)
    aq, asc = run_quant_act4(rt, x)
    assert np.array_equal(aq, r["packed"]) and np.array_equal(_bits(asc), _bits(r["scale"]))
    # round-half-even: with amax = 7 the scale is exactly 1 and x.5 values are ties
    t = np.zeros((1, 32), np.float32)
    t[0, :6] = [7.0, 0.5, 1.5, 2.5, -0.5, -3.5]
    aq, _ = run_quant_act4(rt, t)
    assert list(O.int4_twos(aq.view(np.uint32))[0, :6]) == [7, 0, 2, 2, 0, -4]


def run_nvfp4_quant(rt, x):
    m, k = x.shape
    with Bufs(rt) as b:
        px, qa, qb, sc = b.put(x), b.zeros(m * k // 2, np.int8, 9), b.zeros(m * k // 2, np.int8, 9), b.zeros(m * k // 16)
        rt.launch2d("nvfp4_quant_act", k // 16, m, 64, 1, [px, qa, qb, sc, m, k])
        return (b.get(qa, m * k // 2, np.int8).reshape(m, -1), b.get(qb, m * k // 2, np.int8).reshape(m, -1),
                b.get(sc, m * k // 16).reshape(m, -1))


def test_nvfp4_quant(rt, golden):
    arr, _ = golden
    qa, qb, sc = run_nvfp4_quant(rt, cases.normal_case(90, 1, 5120, gain=3))
    assert np.array_equal(qa, arr["nvfp4_quant.a"]) and np.array_equal(qb, arr["nvfp4_quant.b"])
    assert np.array_equal(_bits(sc), _bits(arr["nvfp4_quant.s"]))
    rng = np.random.default_rng(17)
    x = (rng.standard_normal((3, 2048)) * 5).astype(np.float32)
    x[1, 16:32] = 0
    r = O.nvfp4_quant_act(x)
    qa, qb, sc = run_nvfp4_quant(rt, x)
    assert np.array_equal(qa, r["even"]) and np.array_equal(qb, r["odd"]) and np.array_equal(_bits(sc), _bits(r["scale"]))


@pytest.mark.parametrize("kernel,seed", [("quant_rows_fast_k", 70), ("quant_rows_k", 73)])
def test_quant_rows_golden(rt, golden, kernel, seed):
    arr, _ = golden
    rows, k, g = 32, 512, 128
    x = cases.normal_case(seed, rows, k)
    name = "quant_rows_fast" if kernel.endswith("fast_k") else "quant_rows"
    with Bufs(rt) as b:
        pq, psc, px = b.zeros(rows * k // 8, np.uint32), b.zeros(k // g * rows), b.put(x)
        if kernel == "quant_rows_fast_k":
            rt.launch(kernel, rows, 256, [pq, psc, px, k, g, rows, k, 0, k // g])
        else:
            rt.launch(kernel, rows, k // g, [pq, psc, px, k, g, rows, k, 0])
        assert np.array_equal(b.get(pq, rows * k // 8, np.uint32).reshape(rows, -1), arr[f"{name}.q"])
        assert np.array_equal(_bits(b.get(psc, k // g * rows)), _bits(arr[f"{name}.sc"]).reshape(-1))


def test_quant_rows_strided_and_a8(rt):
    """Input rows taken from a wider matrix (in_stride / in_off), and the int8 row
    quantiser of the W4A8 GEMM with its (k0,k2,k4,k6,k1,k3,k5,k7) byte order."""
    rng = np.random.default_rng(5)
    rows, k, stride, off = 256, 1024, 1536, 256
    big = rng.standard_normal((rows, stride)).astype(np.float32)
    x = np.ascontiguousarray(big[:, off:off + k])
    r4, r8 = O.quant_rows(x), O.quant_rows_a8(x)
    with Bufs(rt) as b:
        pq, psc, px = b.zeros(rows * k // 8, np.uint32), b.zeros(k // 128 * rows), b.put(big)
        rt.launch("quant_rows_fast_k", rows, 256, [pq, psc, px, k, 128, rows, stride, off, k // 128])
        assert np.array_equal(b.get(pq, rows * k // 8, np.uint32).reshape(rows, -1), r4["words"])
        assert np.array_equal(_bits(b.get(psc, k // 128 * rows)), _bits(r4["scale_gf"]).reshape(-1))
        p8, psc8 = b.zeros(rows * k, np.int8), b.zeros(k // 128 * rows)
        rt.launch("quant_rows_a8_k", rows, 256, [p8, 0, psc8, 0, px, k, 128, rows, stride, off])
        got = b.get(p8, rows * k, np.int8).reshape(rows, k // 8, 8)
        want = r8["q"].reshape(rows, k // 8, 8)[:, :, [0, 2, 4, 6, 1, 3, 5, 7]].astype(np.int8)
        assert np.array_equal(got, want)
        assert np.array_equal(_bits(b.get(psc8, k // 128 * rows)), _bits(r8["scale_gf"]).reshape(-1))
