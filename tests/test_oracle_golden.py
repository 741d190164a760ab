"""CPU tier: the NumPy oracle against the vectors produced by the reference's
own test oracle (tests/golden/make_golden.py).  Integer / bit-pattern outputs
must be identical; fp32 outputs agree to 1e-6 relative (both sides evaluate in
float64 and round once, only the association of the float64 sum differs)."""
from __future__ import annotations

import numpy as np
import pytest

import cases
import w4_oracle as O

F64_TOL = 1e-6


def _check_inputs(meta, name, *arrays):
    assert meta[name]["inputs_sha256"] == cases.digest(*arrays), f"{name}: seeded inputs drifted"


@pytest.mark.parametrize("name,seed,m,kind", [
    ("w4a4_m1", 60, 1, 4), ("w4a4_m4", 61, 4, 4), ("w4a4_r2_m4", 62, 4, 4),
    ("w4a8_m1", 63, 1, 8), ("w4a8_m2", 163, 2, 8), ("w4a8_m3", 164, 3, 8),
    ("w4a8_m4", 165, 4, 8), ("w4a4_m2", 166, 2, 4), ("w4a4_m3", 167, 3, 4)])
def test_w4_gemv(golden, name, seed, m, kind):
    arr, meta = golden
    wv, ws, x = cases.w4_case(seed, 256, 5120, m)
    _check_inputs(meta, name, wv, ws, x)
    qd = O.quant_act4(x) if kind == 4 else O.quant_act(x)
    assert np.array_equal(qd["q"].astype(np.int8), arr[f"{name}.qa"])
    assert np.array_equal(qd["scale"].view(np.uint32), arr[f"{name}.asc"].view(np.uint32))
    r = O.gemv_w4(O.pack_nibbles(wv), ws, qd["q"], qd["scale"], 32 if kind == 4 else 128)
    assert O.rel_err(r["y"], arr[f"{name}.y"]) < F64_TOL
    # the exact accumulators agree with a plain int64 evaluation
    g = 32 if kind == 4 else 128
    want = np.einsum("ngk,mgk->mng", wv[:8].reshape(8, -1, g).astype(np.int64),
                     qd["q"].reshape(m, -1, g).astype(np.int64))
    assert np.array_equal(r["acc"][:, :8, :], want)


def test_quantisers_bit_exact(golden):
    arr, meta = golden
    x = cases.normal_case(70, 32, 512)
    _check_inputs(meta, "quant_rows_fast", x)
    r = O.quant_rows(x)
    assert np.array_equal(r["words"], arr["quant_rows_fast.q"])
    assert np.array_equal(r["scale_gf"].view(np.uint32), arr["quant_rows_fast.sc"].view(np.uint32))
    x = cases.normal_case(73, 32, 512)
    _check_inputs(meta, "quant_rows", x)
    r = O.quant_rows(x)
    assert np.array_equal(r["words"], arr["quant_rows.q"])
    assert np.array_equal(r["scale_gf"].view(np.uint32), arr["quant_rows.sc"].view(np.uint32))

    x = cases.normal_case(71, 1, 5120)
    _check_inputs(meta, "quant_act4", x)
    r = O.quant_act4(x)
    assert np.array_equal(r["packed"].reshape(-1), arr["quant_act4.packed"])
    assert np.array_equal(r["scale"].view(np.uint32), arr["quant_act4.s"].view(np.uint32))

    x = cases.normal_case(72, 1, 5120)
    _check_inputs(meta, "quant_act", x)
    r = O.quant_act(x)
    assert np.array_equal(r["even"][0], arr["quant_act.even"])
    assert np.array_equal(r["odd"][0], arr["quant_act.odd"])
    assert np.array_equal(r["scale"].view(np.uint32), arr["quant_act.s"].view(np.uint32))
    assert np.array_equal(r["gsum"], arr["quant_act.gsum"])

    x = cases.normal_case(90, 1, 5120, gain=3)
    _check_inputs(meta, "nvfp4_quant", x)
    r = O.nvfp4_quant_act(x)
    assert np.array_equal(r["even"], arr["nvfp4_quant.a"])
    assert np.array_equal(r["odd"], arr["nvfp4_quant.b"])
    assert np.array_equal(r["scale"].view(np.uint32), arr["nvfp4_quant.s"].view(np.uint32))


def test_fp4_tables(golden):
    arr, _ = golden
    assert np.array_equal(O.e2m1_decode(np.arange(16, dtype=np.uint8)), arr["fp4_tables.e2m1"])
    assert np.array_equal(O.e4m3_decode(np.arange(256, dtype=np.uint8)).view(np.uint32),
                          arr["fp4_tables.e4m3"].view(np.uint32))
    assert np.array_equal(O.e2m1_decode_x2(np.arange(16, dtype=np.uint8)),
                          (2 * arr["fp4_tables.e2m1"]).astype(np.int32))


@pytest.mark.parametrize("name,m", [("nvfp4_gemv", 1), ("nvfp4_gemv_m3", 3)])
def test_nvfp4_gemv(golden, name, m):
    arr, meta = golden
    codes, ws, x = cases.nvfp4_case(202, 32, 512, m)
    _check_inputs(meta, name, codes, ws, x)
    wq = O.pack_nibbles(codes)
    assert np.array_equal(wq, arr[f"{name}.wq"])
    qd = O.nvfp4_quant_act(x)
    r = O.nvfp4_gemv(wq, ws, qd["q"], qd["scale"], 0.75)
    # the stored vector comes from an fp32 BLAS product (reference tolerance 1e-2 + 1e-5*max)
    ref = arr[f"{name}.y"]
    assert np.abs(r["y"] - ref).max() <= 1e-4 * max(1.0, float(np.abs(ref).max()))
    want = np.einsum("nbk,mbk->mnb", O.e2m1_decode_x2(codes).reshape(32, -1, 16).astype(np.int64),
                     qd["q"].reshape(m, -1, 16).astype(np.int64))
    assert np.array_equal(r["acc"], want)


def test_w4a16(golden):
    arr, meta = golden
    packed, scales = cases.int4_dequant_case()
    _check_inputs(meta, "int4_dequant", packed, scales)
    assert np.array_equal(O.int4_dequant(packed, scales).view(np.uint32),
                          arr["int4_dequant.y"].view(np.uint32))
    part = cases.reduce_case()
    _check_inputs(meta, "reduce_blocks", part)
    assert np.abs(O.reduce_blocks(part, 32, 5) - arr["reduce_blocks.y"]).max() < 1e-5
    packed, scales, x = cases.int4_dot_case()
    _check_inputs(meta, "int4_dot", packed, scales, x)
    got = O.int4_dot_partial(packed, scales, x, 12, 8, ids=[0, 1], rows_per_exp=6, rows_per_w=6)
    assert O.rel_err(got, arr["int4_dot.partial"]) < 1e-6
    # dense whole-layer form agrees with partial+reduce
    y = O.w4a16_gemv(packed.reshape(12, 128), scales, x[0])
    p = O.int4_dot_partial(packed, scales, x[:1], 12, 8)
    assert O.rel_err(O.reduce_blocks(p, 12, 8), y[0]) < 1e-6


def test_gemm_w4a4(golden):
    arr, meta = golden
    b, x = cases.gemm_case()
    _check_inputs(meta, "gemm_w4a4", b, x)
    qr = O.quant_rows(x)
    n, k = b.shape
    r = O.gemm_w4(qr["q"], O.pack_nibbles(b), qr["scale_gf"], np.ones((k // 128, n), np.float32))
    # reference example tolerance is 1e-3 against an fp32 matmul of dequantised operands
    assert O.rel_err(r["c"], arr["gemm_w4a4.c"]) < 1e-5
    want = np.einsum("ngk,mgk->mng", b.reshape(n, -1, 128).astype(np.int64),
                     qr["q"][:16].reshape(16, -1, 128).astype(np.int64))
    assert np.array_equal(r["acc"][:16], want)


def test_quant_edge_cases():
    """All-zero groups take scale 1; exact ties round to even; the clamp bites."""
    x = np.zeros((2, 256), np.float32)
    x[1, :128] = np.linspace(-1, 1, 128, dtype=np.float32)
    r = O.quant_act(x)
    assert r["scale"][0, 0] == 1.0 and not r["q"][0].any()
    assert r["q"][1].max() == 127 and r["q"][1].min() == -127
    t = np.zeros((1, 32), np.float32)
    t[0, :4] = [7.0, 0.5, 1.5, 2.5]
    q4 = O.quant_act4(t)["q"][0, :4]
    assert list(q4) == [7, 0, 2, 2]


@pytest.mark.parametrize("rows,dim", cases.RMSNORM_QUANT_SHAPES)
def test_rmsnorm_quant_oracle_matches_reference(golden, rows, dim):
    """oracle.rmsnorm_quant against the reference's host check of rmsnorm_quant_k (tools/gen_rmsnorm_quant.py:288-306)."""
    arr, meta = golden
    x, w = cases.rmsnorm_case(rows, dim)
    name = f"rmsnorm_quant_{rows}x{dim}"
    assert cases.digest(x, w) == meta[name]["inputs_sha256"]
    q = O.rmsnorm_quant(x, w, 1e-6)
    assert np.array_equal(q["q"], arr[name + ".q"])
    assert np.array_equal(q["scale"], arr[name + ".s"]) and np.array_equal(q["gsum"], arr[name + ".asum"])


def test_rmsnorm_and_silu_oracle_match_reference(golden):
    arr, meta = golden
    x, w = cases.rmsnorm_case(4, 256, seed=8, gain=1.0, plain_w=True)
    assert cases.digest(x, w) == meta["rmsnorm"]["inputs_sha256"]
    ref = arr["rmsnorm.y"]
    assert np.abs(O.rmsnorm(x, w, 1e-5) - ref).max() <= 1e-4 + 1e-5 * max(1.0, float(np.abs(ref).max()))
    gate, up = cases.silu_case()
    assert cases.digest(gate, up) == meta["silu_mul"]["inputs_sha256"]
    assert np.array_equal(O.silu_mul(gate, up), arr["silu_mul.y"])
