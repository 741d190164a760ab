"""Host-side packing and conversion of INT4 / NVFP4 weights (NumPy only).

Same functions and byte layouts as the reference's python/k100lc_kernels/quant.py:
compressed-tensors INT4 is group-128, offset-binary (``code = round(w/scale) + 8``,
``w = (code - 8) * scale``), eight codes per little-endian u32 with the lowest k in the
lowest nibble, one bf16 scale per (row, 128 k).  RT4 keeps the nibble positions but
stores two's-complement values and f16 scales; the prefill GEMM wants f32 scales laid
out group-first ``[K/128, N]``.
"""
from __future__ import annotations

import numpy as np

GROUP = 128
_SHIFTS = np.arange(8, dtype=np.uint32) * np.uint32(4)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns (uint16), round to nearest even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    """bf16 bit patterns (uint16) -> float32 (exact: bf16 is the top half of f32)."""
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def pack_nibbles(values: np.ndarray) -> np.ndarray:
    """``[R, K]`` integers -> ``[R, K/8]`` u32, nibble j of word w = element 8w+j (mod 16)."""
    a = np.asarray(values)
    r, k = a.shape
    # bytes first (two nibbles each, low nibble = even k), then four bytes per little-endian word
    v = (a.astype(np.uint8) if a.dtype.itemsize == 1 else (a.astype(np.int64) & 0xF).astype(np.uint8)) & np.uint8(0xF)
    b = v[:, 0::2] | (v[:, 1::2] << np.uint8(4))
    return np.ascontiguousarray(b).view("<u4").reshape(r, k // 8)


def unpack_nibbles(words: np.ndarray) -> np.ndarray:
    """``[R, K/8]`` u32 -> ``[R, K]`` raw codes 0..15."""
    w = np.ascontiguousarray(words, dtype=np.uint32)
    return ((w[..., None] >> _SHIFTS) & np.uint32(0xF)).reshape(w.shape[0], -1).astype(np.uint8)


def pack_int4_group128(w: np.ndarray) -> tuple[bytes, bytes]:
    """f32 weights ``[N, K]`` -> ``(packed_bytes, scale_bf16_bytes)``; ``K % 128 == 0``.
    The scale of a group is ``max|w| / 7`` (1.0 for an all-zero group)."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    if w.ndim != 2:
        raise ValueError("pack_int4_group128 expects a 2-D [N, K] weight")
    n, k = w.shape
    if k % GROUP:
        raise ValueError(f"K={k} is not a multiple of {GROUP}")
    g = w.reshape(n, k // GROUP, GROUP)
    amax = np.abs(g).max(axis=2)
    scale = np.where(amax > 0, amax / 7.0, 1.0).astype(np.float32)
    codes = np.clip(np.rint(g / scale[:, :, None]) + 8.0, 0.0, 15.0).astype(np.uint32)
    return pack_nibbles(codes.reshape(n, k)).tobytes(), f32_to_bf16_bits(scale).tobytes()


def dequant_int4_group128(packed: bytes, scales: bytes, n: int, k: int) -> np.ndarray:
    """Packed bytes -> f32 ``[N, K]`` with the kernels' definition ``(code - 8) * scale``."""
    codes = unpack_nibbles(np.frombuffer(packed, dtype=np.uint32).reshape(n, k // 8)).astype(np.int32)
    s = bf16_bits_to_f32(np.frombuffer(scales, dtype=np.uint16)).reshape(n, k // GROUP)
    return (codes - 8).astype(np.float32) * np.repeat(s, GROUP, axis=1)


def ct_int4_to_twos_complement(packed: bytes) -> bytes:
    """Offset-binary codes -> two's-complement nibbles, nibble positions unchanged:
    ``value = code - 8`` and the two's-complement nibble of ``value`` is ``code ^ 8``."""
    raw = np.frombuffer(packed, dtype=np.uint8)
    return (raw ^ np.uint8(0x88)).tobytes()


def ct_int4_to_rt4(packed: bytes, scales_bf16: bytes) -> tuple[bytes, bytes]:
    """compressed-tensors INT4 -> RT4 ``(q_bytes, f16_scale_bytes)`` for the W4A8 / W4A4
    kernels; done once per layer."""
    s = bf16_bits_to_f32(np.frombuffer(scales_bf16, dtype=np.uint16))
    return ct_int4_to_twos_complement(packed), s.astype(np.float16).tobytes()


def int4_scale_group_first_f32(scales_bf16: bytes, n: int, k: int) -> np.ndarray:
    """bf16 scales ``[N, K/128]`` -> f32 ``[K/128, N]`` (the layout of the W4 GEMM)."""
    s = bf16_bits_to_f32(np.frombuffer(scales_bf16, dtype=np.uint16)).reshape(n, k // GROUP)
    return np.ascontiguousarray(s.T, dtype=np.float32)


# ---- NVFP4 helpers (the reference has them only inside its self-test) ---------------
_E4M3_VALUES = None


def e4m3_values() -> np.ndarray:
    """The 256 OCP E4M3 code points as f32 (bias 7; 0x7F/0xFF decoded arithmetically)."""
    global _E4M3_VALUES
    if _E4M3_VALUES is None:
        b = np.arange(256, dtype=np.int64)
        e, m = (b >> 3) & 0xF, (b & 7).astype(np.float64)
        mag = np.where(e == 0, m / 8.0 * 2.0 ** -6, (1.0 + m / 8.0) * np.exp2((e - 7).astype(np.float64)))
        _E4M3_VALUES = np.where(b >= 128, -mag, mag).astype(np.float32)
    return _E4M3_VALUES


def f32_to_e4m3_bits(x: np.ndarray) -> np.ndarray:
    """Positive f32 -> nearest positive finite E4M3 code (ties to the even code), never
    the NaN code 0x7F; values above 448 saturate to 0x7E."""
    x = np.ascontiguousarray(x, dtype=np.float32).astype(np.float64)
    tab = e4m3_values()[:0x7F].astype(np.float64)           # ascending 0 .. 448
    hi = np.clip(np.searchsorted(tab, x, side="left"), 1, len(tab) - 1)
    lo = hi - 1
    dlo, dhi = x - tab[lo], tab[hi] - x
    pick_hi = (dhi < dlo) | ((dhi == dlo) & (hi % 2 == 0))
    return np.where(pick_hi, hi, lo).astype(np.uint8)
