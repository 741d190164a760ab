"""Seeded input generators shared by the golden-vector script and the tests.

Each generator re-creates, draw for draw, the synthetic inputs of one test case
of the reference project (tools/selftest_all.py, examples/python_w4a4_gemm.py),
so that a fixture only has to store the SHA-256 of the inputs and the reference
outputs.  ``np.random.default_rng`` (PCG64) streams are stable across NumPy
versions for the calls used here.
"""
from __future__ import annotations

import hashlib

import numpy as np


def digest(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        a = np.ascontiguousarray(a)
        h.update(str(a.dtype).encode() + str(a.shape).encode())
        h.update(a.tobytes())
    return h.hexdigest()


def w4_case(seed: int, n: int, k: int, m: int):
    """Inputs of the reference W4 GEMV cases (tools/selftest_all.py:843-851):
    int4 values [N,K], f16 scales [N,K/128] in [0.5,1.5), x [M,K] ~ N(0,1)."""
    rng = np.random.default_rng(seed)
    wv = rng.integers(-8, 8, size=(n, k)).astype(np.int32)
    ws = rng.uniform(0.5, 1.5, size=(n, k // 128)).astype(np.float32).astype(np.float16)
    x = rng.standard_normal((m, k)).astype(np.float32)
    return wv, ws, x


def normal_case(seed: int, rows: int, k: int, gain: float = 1.0):
    """x [rows,K] ~ gain * N(0,1) (tools/selftest_all.py:940-1016,1071-1085)."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((rows, k)).astype(np.float32)
    if gain != 1.0:
        x = x * gain
    return x


def nvfp4_case(seed: int = 202, n: int = 32, k: int = 512, m: int = 1):
    """Inputs of the reference NVFP4 GEMV case (tools/selftest_all.py:1096-1104):
    codes uniform 0..15, E4M3 scale bytes uniform in [1,0x7E], x ~ 2*N(0,1)."""
    rng = np.random.default_rng(seed)
    codes = rng.integers(0, 16, size=(n, k)).astype(np.uint8)
    ws = rng.integers(1, 0x7F, size=(n, k // 16)).astype(np.uint8)
    x = rng.standard_normal((m, k)).astype(np.float32) * 2
    return codes, ws, x


def _bf16_trunc_bits(rng, count: int) -> np.ndarray:
    f = rng.uniform(1e-3, 5e-2, size=count).astype(np.float32)
    return ((f.view(np.uint32) & np.uint32(0xFFFF0000)) >> 16).astype(np.uint16)


def int4_dequant_case(seed: int = 30, nblocks: int = 64):
    """tools/selftest_all.py:639-660."""
    rng = np.random.default_rng(seed)
    packed = rng.integers(0, 1 << 32, size=nblocks * 16, dtype=np.uint64).astype(np.uint32)
    return packed, _bf16_trunc_bits(rng, nblocks)


def reduce_case(seed: int = 40, rows: int = 32, nbpr: int = 5):
    """tools/selftest_all.py:726-735."""
    rng = np.random.default_rng(seed)
    return rng.standard_normal(rows * nbpr).astype(np.float32)


def int4_dot_case(seed: int = 50, nbpr: int = 8, rows_per_exp: int = 6, n_exp: int = 2):
    """tools/selftest_all.py:738-770: two experts, six rows each."""
    rng = np.random.default_rng(seed)
    nblocks = rows_per_exp * n_exp * nbpr
    packed = rng.integers(0, 1 << 32, size=nblocks * 16, dtype=np.uint64).astype(np.uint32)
    scales = _bf16_trunc_bits(rng, nblocks)
    x = rng.standard_normal((n_exp, nbpr * 128)).astype(np.float32)
    return packed, scales, x


def gemm_case(seed: int = 3, n: int = 128, k: int = 512, m: int = 256):
    """examples/python_w4a4_gemm.py:59-66: int4 weights, unit weight scales."""
    rng = np.random.default_rng(seed)
    b = rng.integers(-8, 8, size=(n, k), dtype=np.int32)
    x = rng.standard_normal((m, k)).astype(np.float32)
    return b, x


RMSNORM_QUANT_SHAPES = ((1, 128), (2, 256), (1, 512), (3, 1280), (1, 5120))


def rmsnorm_case(rows: int, dim: int, seed: int | None = None, gain: float = 2.0, plain_w: bool = False):
    """x [rows,dim] ~ gain * N(0,1) and a weight vector: uniform [0.5,1.5) as in
    tools/gen_rmsnorm_quant.py:311-317, or N(0,1) as in tools/selftest_all.py:268-271."""
    rng = np.random.default_rng(20261012 + 1000 * rows + dim if seed is None else seed)
    x = rng.standard_normal((rows, dim)).astype(np.float32) * np.float32(gain)
    w = rng.standard_normal(dim).astype(np.float32) if plain_w else (rng.random(dim).astype(np.float32) + np.float32(0.5))
    return x, w


def silu_case(seed: int = 4, n: int = 1000):
    """tools/selftest_all.py:214-219."""
    rng = np.random.default_rng(seed)
    return rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
