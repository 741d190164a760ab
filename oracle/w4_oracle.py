"""CPU oracle for the weight-streaming quantized linear-layer path (NumPy).

TEST INFRASTRUCTURE ONLY.  This module is the checker for the CUDA kernels: the
test-suite, the smoke entry and the CPU-baseline leg of the benchmark may call
it; the product package never does and has no CPU fallback.

It restates, in vectorised NumPy, the arithmetic that the reference project
(Hong-agent/K100LC-kernels) defines for this path.  Every function names the
reference file:line it follows.  Parity of this restatement with the reference's
own NumPy test oracle is pinned by the fixtures under ``tests/golden/`` (made by
``tests/golden/make_golden.py`` from the reference's functions) — status:
PINNED for the activation quantisers, W4A8/W4A4 GEMV, NVFP4 quant/GEMV, W4A16
dot/reduce/dequant and the W4A4 GEMM; the W4A8 GEMM has no counterpart in the
reference ("parity unpinned": defined here by extension of the W4A4 GEMM).

Exact integer accumulators are computed with float32 BLAS products: every
operand is a small integer and every partial sum stays below 2**24, so each
float32 intermediate is an exact integer whatever the summation order.
"""
from __future__ import annotations

import numpy as np

GROUP_W = 128      # weight scale group (reference kernels/gemv_w4a8_core.h:15)
GROUP_A4 = 32      # int4 activation sub-group (reference kernels/gemv_w4a4_core.h:9)
BLOCK_FP4 = 16     # NVFP4 block (reference tools/selftest_all.py:1049-1059)

# E2M1 magnitudes, reference tools/selftest_all.py:1022
_E2M1_MAG = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
# the same table doubled: the device path multiplies integers and folds the 0.5
# into the block scale (reference kernels/asm/k_nvfp4/011_*.s:118-167)
_E2M1_MAG2 = np.array([0, 1, 2, 3, 4, 6, 8, 12], dtype=np.int32)


# --------------------------------------------------------------------------
# nibble containers
# --------------------------------------------------------------------------
def nibbles(words: np.ndarray) -> np.ndarray:
    """``[..., W]`` u32 words -> ``[..., 8W]`` raw 4-bit codes, nibble j of word w
    is element 8w+j (reference python/k100lc_kernels/rt4.py:6-8, quant.py:9-10)."""
    w = np.ascontiguousarray(words, dtype=np.uint32)
    sh = np.arange(8, dtype=np.uint32) * np.uint32(4)
    out = (w[..., None] >> sh) & np.uint32(0xF)
    return out.reshape(*w.shape[:-1], w.shape[-1] * 8).astype(np.uint8)


def int4_twos(words: np.ndarray) -> np.ndarray:
    """Two's-complement int4 values (RT4 weights, packed activations).
    Reference tools/selftest_all.py:783-792."""
    c = nibbles(words).astype(np.int8)
    return np.where(c >= 8, c - 16, c).astype(np.int8)


def int4_offset(words: np.ndarray) -> np.ndarray:
    """Offset-binary int4 values (compressed-tensors: value = code - 8).
    Reference python/k100lc_kernels/quant.py:59-67, tools/ct_int4.py:98-105."""
    return (nibbles(words).astype(np.int8) - np.int8(8)).astype(np.int8)


def pack_nibbles(values: np.ndarray) -> np.ndarray:
    """``[R, K]`` integers -> ``[R, K/8]`` u32, low nibble = lower k.
    Reference tools/selftest_all.py:776-781."""
    v = np.asarray(values).astype(np.int64) & 0xF
    r, k = v.shape
    v = v.reshape(r, k // 8, 8).astype(np.uint32)
    sh = np.arange(8, dtype=np.uint32) * np.uint32(4)
    return np.bitwise_or.reduce(v << sh, axis=2).astype(np.uint32)


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    """bf16 bit pattern -> f32 (reference python/k100lc_kernels/quant.py:27-30)."""
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# --------------------------------------------------------------------------
# activation quantisers
# --------------------------------------------------------------------------
def _absmax_quant(x: np.ndarray, group: int, qmax: float, lo: int, hi: int):
    """Shared body: per (row, group) ``s = amax/qmax`` (1 when the group is all
    zero), ``q = clip(rint(x / s))`` with IEEE fp32 division and round-half-even."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    m, k = x.shape
    if k % group:
        raise ValueError(f"K={k} is not a multiple of {group}")
    xg = x.reshape(m, k // group, group)
    amax = np.abs(xg).max(axis=2)
    s = np.ones_like(amax, dtype=np.float32)
    nz = amax > 0
    s[nz] = (amax[nz] / np.float32(qmax)).astype(np.float32)
    q = np.rint(xg / s[:, :, None]).astype(np.int32)
    np.clip(q, lo, hi, out=q)
    return q.reshape(m, k), s


def quant_act(x: np.ndarray) -> dict:
    """``quant_act``: int8, group 128 (reference kernels/gemv_w4a8_core.h:34-66,
    oracle tools/selftest_all.py:806-814).  Returns q ``[M,K]`` int32, the even-k
    and odd-k int8 streams, the scales ``[M,K/128]`` and the group sums."""
    q, s = _absmax_quant(x, GROUP_W, 127.0, -128, 127)
    m, k = q.shape
    return dict(q=q, even=q[:, 0::2].astype(np.int8), odd=q[:, 1::2].astype(np.int8),
                scale=s, gsum=q.reshape(m, k // GROUP_W, GROUP_W).sum(axis=2).astype(np.int32))


def quant_act4(x: np.ndarray) -> dict:
    """``quant_act4``: int4, group 32, two nibbles per byte, low nibble = even k
    (reference kernels/gemv_w4a4_core.h:26-45, oracle tools/selftest_all.py:795-803)."""
    q, s = _absmax_quant(x, GROUP_A4, 7.0, -8, 7)
    packed = pack_nibbles(q).view(np.uint8).reshape(q.shape[0], -1)
    return dict(q=q, packed=packed, scale=s)


def quant_rows(x: np.ndarray, group: int = GROUP_W) -> dict:
    """``quant_rows_fast_k`` / ``quant_rows_k``: int4 per (row, group) for the
    prefill GEMM; codes ``[rows,K/8]`` u32, scales GROUP-FIRST ``[K/group, rows]``
    (reference tools/gen_quant_fast.py:187-205, tools/selftest_all.py:916-937)."""
    q, s = _absmax_quant(x, group, 7.0, -8, 7)
    return dict(q=q, words=pack_nibbles(q), scale_gf=np.ascontiguousarray(s.T))


def quant_rows_a8(x: np.ndarray, group: int = GROUP_W) -> dict:
    """int8 row quantiser for the W4A8 prefill GEMM.  No reference kernel is
    verified for it (parity unpinned); arithmetic = ``quant_act`` per
    (row, 128-group) with group-first scales like ``quant_rows``."""
    q, s = _absmax_quant(x, group, 127.0, -128, 127)
    return dict(q=q, scale_gf=np.ascontiguousarray(s.T))


def nvfp4_quant_act(x: np.ndarray) -> dict:
    """``nvfp4_quant_act``: int8 per 16-block (reference
    tools/selftest_all.py:1049-1059; device kernels/asm/k_nvfp4/001_*.s)."""
    q, s = _absmax_quant(x, BLOCK_FP4, 127.0, -128, 127)
    return dict(q=q, even=q[:, 0::2].astype(np.int8), odd=q[:, 1::2].astype(np.int8), scale=s)


# --------------------------------------------------------------------------
# exact integer accumulators
# --------------------------------------------------------------------------
def group_acc(wv: np.ndarray, qa: np.ndarray, group: int) -> np.ndarray:
    """``I[m, n, g] = sum_{k in g} wv[n,k] * qa[m,k]`` as int32, exact.

    This is the per-group integer accumulator the device kernels hold before any
    scale is applied (reference kernels/gemv_w4a8_core.h:157-206 group 128,
    kernels/gemv_w4a4_core.h:105-121 group 32, kernels/gemm_core.h:144-188,
    kernels/asm/k_nvfp4/011_*.s:117-184 group 16)."""
    n, k = wv.shape
    m = qa.shape[0]
    ng = k // group
    wf = np.ascontiguousarray(wv.astype(np.float32).reshape(n, ng, group).transpose(1, 0, 2))
    qf = np.ascontiguousarray(qa.astype(np.float32).reshape(m, ng, group).transpose(1, 2, 0))
    lim = float(np.abs(wf).max(initial=0.0)) * float(np.abs(qf).max(initial=0.0)) * group
    if lim >= 2 ** 24:
        raise ValueError("integer accumulator would not be exact in float32")
    acc = np.matmul(wf, qf)                      # [ng, n, m]
    return np.ascontiguousarray(acc.transpose(2, 1, 0)).astype(np.int32)


# --------------------------------------------------------------------------
# W4A8 / W4A4 decode GEMV
# --------------------------------------------------------------------------
def gemv_w4(wq_words: np.ndarray, ws_f16: np.ndarray, qa: np.ndarray,
            asc: np.ndarray, grp_a: int) -> dict:
    """``gemv_w4a8`` (grp_a=128) / ``gemv_w4a4`` (grp_a=32).

    ``y[m,n] = sum_g f16(ws[n,g]) * sum_{s in g} asc[m,s] * I[m,n,s]`` evaluated
    in float64 and cast to f32, as the reference oracle does
    (tools/selftest_all.py:817-840; device math kernels/gemv_w4a8_core.h:199-204,
    kernels/gemv_w4a4_core.h:105-121).  ``wq_words`` ``[N,K/8]`` u32 two's
    complement, ``ws_f16`` ``[N,K/128]`` float16, ``qa`` ``[M,K]`` integer codes,
    ``asc`` ``[M,K/grp_a]`` f32."""
    wv = int4_twos(wq_words)
    n, k = wv.shape
    acc = group_acc(wv, qa, grp_a)                              # [M,N,K/grp_a]
    sub = GROUP_W // grp_a
    t = acc.astype(np.float64) * asc.astype(np.float64)[:, None, :]
    t = t.reshape(t.shape[0], n, k // GROUP_W, sub).sum(axis=3)
    y = (t * np.asarray(ws_f16).view(np.float16).astype(np.float64)[None, :, :]).sum(axis=2)
    return dict(acc=acc, y=y.astype(np.float32))


# --------------------------------------------------------------------------
# NVFP4
# --------------------------------------------------------------------------
def e2m1_decode(codes: np.ndarray) -> np.ndarray:
    """4-bit E2M1 code -> f32; bit 3 is the sign (reference tools/selftest_all.py:1025-1029)."""
    c = np.asarray(codes, dtype=np.uint8)
    mag = _E2M1_MAG[c & 7]
    return np.where((c & 8) != 0, -mag, mag).astype(np.float32)


def e2m1_decode_x2(codes: np.ndarray) -> np.ndarray:
    """4-bit E2M1 code -> the integer 2*value in {0,+-1,...,+-12}."""
    c = np.asarray(codes, dtype=np.uint8)
    mag = _E2M1_MAG2[c & 7]
    return np.where((c & 8) != 0, -mag, mag).astype(np.int32)


def e4m3_decode(bits: np.ndarray) -> np.ndarray:
    """OCP E4M3 byte -> f32: bias 7, subnormals m/8 * 2**-6; codes 0x7F/0xFF are
    decoded arithmetically like every other code, as the reference oracle does
    (tools/selftest_all.py:1032-1037)."""
    b = np.asarray(bits, dtype=np.uint8).astype(np.int64)
    e, mant = (b >> 3) & 0xF, (b & 7).astype(np.float64)
    mag = np.where(e == 0, mant / 8.0 * 2.0 ** -6, (1.0 + mant / 8.0) * np.exp2((e - 7).astype(np.float64)))
    return np.where((b >> 7) == 1, -mag, mag).astype(np.float32)


def nvfp4_gemv(wq_words: np.ndarray, ws_e4m3: np.ndarray, qa: np.ndarray,
               asc: np.ndarray, gscale: float) -> dict:
    """``nvfp4_gemv<A,B>`` / ``nvfp4_gemv_wide<A,B>`` for A = qa.shape[0] tokens.

    ``I[m,n,b] = sum_{16} (2*E2M1(w)) * q`` exact; then
    ``y[m,n] = sum_b I * (0.5*gscale*E4M3(ws[n,b])) * asc[m,b]`` in float64
    (reference formula tools/selftest_all.py:1108-1114; device
    kernels/asm/k_nvfp4/011_*.s:11-62,117-184)."""
    w2 = e2m1_decode_x2(nibbles(wq_words))
    acc = group_acc(w2, qa, BLOCK_FP4)                          # [M,N,K/16]
    bs = e4m3_decode(ws_e4m3).astype(np.float64) * (0.5 * float(np.float32(gscale)))
    y = (acc.astype(np.float64) * bs[None, :, :] * asc.astype(np.float64)[:, None, :]).sum(axis=2)
    return dict(acc=acc, y=y.astype(np.float32))


# --------------------------------------------------------------------------
# W4A16 (compressed-tensors INT4): int4_dot_k + reduce_blocks_k + int4_dequant_k
# --------------------------------------------------------------------------
def int4_dequant(words: np.ndarray, scale_bf16: np.ndarray) -> np.ndarray:
    """``int4_dequant_k``: ``(code-8) * bf16(scale)`` per element, one scale per
    16 words, result f32 and bit-exact (reference tools/gen_int4_dot.py:162-223,
    python/k100lc_kernels/quant.py:59-67)."""
    w = np.ascontiguousarray(words, dtype=np.uint32).reshape(-1)
    v = int4_offset(w.reshape(-1, 16)).astype(np.float32)          # [blocks,128]
    s = bf16_to_f32(np.asarray(scale_bf16).reshape(-1))[: v.shape[0]]
    return (v * s[:, None]).reshape(-1)


def int4_dot_partial(wbuf: np.ndarray, sbuf: np.ndarray, x: np.ndarray, nrows: int,
                     nbpr: int, ids=None, rows_per_exp=None, rows_per_w=None) -> np.ndarray:
    """``int4_dot_k``: ``partial[row*nbpr+b] = bf16(scale) * sum_{128}(code-8)*x``.

    Index algebra of the reference (tools/gen_gemv_qdot.py:152-167,189-196,
    tools/gen_int4_dot.py:96-117,229-251): ``ew = row // rows_per_w`` selects the
    weight expert ``ids[ew]`` (weights of expert e start at row ``e*rows_per_w`` of
    ``wbuf``), ``e = row // rows_per_exp`` selects the activation row.  Evaluated
    in float64 (the device accumulates in fp32; gate is 1e-5 relative)."""
    rows_per_exp = nrows if rows_per_exp is None else rows_per_exp
    rows_per_w = nrows if rows_per_w is None else rows_per_w
    vals = int4_offset(np.asarray(wbuf, dtype=np.uint32).reshape(-1, nbpr * 16))
    vals = vals.astype(np.float64).reshape(-1, nbpr, GROUP_W)
    sc = bf16_to_f32(np.asarray(sbuf).reshape(-1)).astype(np.float64).reshape(-1, nbpr)
    xb = np.ascontiguousarray(x, dtype=np.float32).astype(np.float64).reshape(-1, nbpr, GROUP_W)
    row = np.arange(nrows)
    ew, er = row // rows_per_w, row % rows_per_w
    src = row if ids is None else np.asarray(ids)[ew] * rows_per_w + er
    e = row // rows_per_exp
    out = (vals[src] * xb[e]).sum(axis=2) * sc[src]
    return out.reshape(-1).astype(np.float32)


def reduce_blocks(partial: np.ndarray, nrows: int, nbpr: int) -> np.ndarray:
    """``reduce_blocks_k``: ``y[r] = sum_j partial[r*nbpr+j]``, added in order j=0,1,…
    in fp32 (reference tools/gen_gemv_qdot.py:207-308)."""
    p = np.ascontiguousarray(partial, dtype=np.float32).reshape(nrows, nbpr)
    y = np.zeros(nrows, dtype=np.float32)
    for j in range(nbpr):
        y = (y + p[:, j]).astype(np.float32)
    return y


def w4a16_gemv(words: np.ndarray, scale_bf16: np.ndarray, x: np.ndarray) -> np.ndarray:
    """Whole W4A16 layer ``y[m,n] = sum_k (code-8)*bf16(scale[n,k//128])*x[m,k]`` in
    float64 (reference dequantise-then-matmul python/k100lc_kernels/quant.py:59-67
    and tools/bench_model_paths.py:54-55)."""
    n = words.shape[0]
    v = int4_offset(words).astype(np.float64)
    s = bf16_to_f32(np.asarray(scale_bf16).reshape(n, -1)).astype(np.float64)
    w = v * np.repeat(s, GROUP_W, axis=1)
    x = np.atleast_2d(np.asarray(x, dtype=np.float32)).astype(np.float64)
    return (x @ w.T).astype(np.float32)


# --------------------------------------------------------------------------
# prefill GEMM
# --------------------------------------------------------------------------
def gemm_w4(a_codes: np.ndarray, b_words: np.ndarray, sa_gf: np.ndarray,
            sb_gf: np.ndarray, group: int = GROUP_W) -> dict:
    """``gemm_w4a4`` / ``gemm_w4a4_flat`` (and, with int8 ``a_codes``, the W4A8
    GEMM): ``I[m,n,g]`` exact; ``C[m,n] = sum_g float(I) * (sa[g,m]*sb[g,n])`` with
    the scale product rounded to fp32 first and the terms added for g = 0,1,… by
    fused multiply-add, as reference kernels/gemm_core.h:176-188 does.  The fma
    chain is evaluated in float64 and cast to f32 once (gate: 1e-5 relative).
    ``a_codes`` ``[M,K]`` integers; ``b_words`` ``[N,K/8]`` two's-complement nibbles;
    ``sa_gf`` ``[K/group, M]``; ``sb_gf`` ``[K/group, N]`` (group-first f32)."""
    wv = int4_twos(b_words)
    acc = group_acc(wv, a_codes, group)                         # [M,N,G]
    sa = np.asarray(sa_gf, dtype=np.float32)
    sb = np.asarray(sb_gf, dtype=np.float32)
    prod = (sa.T[:, None, :] * sb.T[None, :, :]).astype(np.float32)   # [M,N,G] fp32-rounded
    c = (acc.astype(np.float64) * prod.astype(np.float64)).sum(axis=2)
    return dict(acc=acc, c=c.astype(np.float32))


def rel_err(got: np.ndarray, ref: np.ndarray) -> float:
    """``max|got-ref| / max|ref|`` — the reference's own definition
    (tools/bench_model_paths.py:39-40)."""
    ref = np.asarray(ref, dtype=np.float64)
    den = float(np.abs(ref).max()) or 1.0
    return float(np.abs(np.asarray(got, dtype=np.float64) - ref).max()) / den


# --------------------------------------------------------------------------
# the operators either side of the layer
# --------------------------------------------------------------------------
def rmsnorm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """``y = (x * rs) * w`` with ``rs = float32(1 / sqrt(mean(x^2) + eps))``, the mean taken in
    float64 — the arithmetic of the reference's host check of its fused kernel
    (tools/gen_rmsnorm_quant.py:288-296); python/k100lc_kernels/model.py:480-481 states the operator."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    ms = (x.astype(np.float64) ** 2).mean(axis=1, keepdims=True)
    rs = (1.0 / np.sqrt(ms + eps)).astype(np.float32)
    return (x * rs).astype(np.float32) * w[None, :]


def rmsnorm_quant(x: np.ndarray, w: np.ndarray, eps: float) -> dict:
    """``quant_act(rmsnorm(x))``: reference tools/gen_rmsnorm_quant.py:16-33, 288-306."""
    return quant_act(rmsnorm(x, w, eps))


def silu_mul(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """``gate / (1 + exp(-gate)) * up`` in float32 (reference tools/selftest_all.py:205-223)."""
    g = np.ascontiguousarray(gate, dtype=np.float32)
    return (g / (np.float32(1.0) + np.exp(-g)) * np.ascontiguousarray(up, dtype=np.float32)).astype(np.float32)
