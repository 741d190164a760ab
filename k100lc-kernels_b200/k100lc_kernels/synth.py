"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations of this path (17408 x 5120 layers, group 128).  No checkpoint is needed:
weights are uniform int4 / E2M1 codes, scales and activations follow the stated
distributions, and every array is a pure function of (seed, shape), so the device
harness and the CPU oracle see identical bits.  Draw order inside each generator is
part of the contract — do not reorder the ``rng`` calls.

The generators only produce inputs; nothing here computes a reference result.
"""
from __future__ import annotations

import numpy as np

from .quant import f32_to_bf16_bits, f32_to_e4m3_bits, pack_nibbles

N_DEFAULT, K_DEFAULT, GROUP = 17408, 5120, 128


def _scale_values(rng, shape) -> np.ndarray:
    """|N(0,1)| * 0.01 + 1e-3, f32."""
    return (np.abs(rng.standard_normal(shape)) * 0.01 + 1e-3).astype(np.float32)


def w4a16_layer(n=N_DEFAULT, k=K_DEFAULT, seed=0) -> dict:
    """compressed-tensors INT4 layer for ``int4_dot_k``: offset-binary codes (value+8)
    ``[N,K/8]`` u32, bf16 scale bits ``[N,K/128]`` u16, x ``[K]`` f32."""
    rng = np.random.default_rng(seed)
    w = rng.integers(-8, 8, size=(n, k), dtype=np.int8)
    scale = f32_to_bf16_bits(_scale_values(rng, (n, k // GROUP)))
    x = rng.standard_normal(k).astype(np.float32)
    return dict(n=n, k=k, w=w, packed=pack_nibbles(w.astype(np.int16) + 8), scale_bf16=scale, x=x)


def rt4_layer(n=N_DEFAULT, k=K_DEFAULT, m=1, seed=1) -> dict:
    """RT4 layer for the W4A8 / W4A4 GEMV: two's-complement nibbles ``[N,K/8]`` u32,
    f16 scales ``[N,K/128]``, x ``[M,K]`` f32."""
    rng = np.random.default_rng(seed)
    w = rng.integers(-8, 8, size=(n, k), dtype=np.int8)
    ws = _scale_values(rng, (n, k // GROUP)).astype(np.float16)
    x = rng.standard_normal((m, k)).astype(np.float32)
    return dict(n=n, k=k, m=m, w=w, wq=pack_nibbles(w), ws=ws, x=x)


def nvfp4_layer(n=N_DEFAULT, k=K_DEFAULT, m=1, seed=2) -> dict:
    """NVFP4 layer: E2M1 codes uniform over the 16 values ``[N,K/8]`` u32, E4M3 block
    scales per 16 weights drawn from 2**U(-4,2) ``[N,K/16]`` u8, global scale 0.05,
    x ``[M,K]`` f32."""
    rng = np.random.default_rng(seed)
    codes = rng.integers(0, 16, size=(n, k), dtype=np.uint8)
    ws = f32_to_e4m3_bits(np.exp2(rng.uniform(-4.0, 2.0, size=(n, k // 16))).astype(np.float32))
    x = rng.standard_normal((m, k)).astype(np.float32)
    return dict(n=n, k=k, m=m, codes=codes, wq=pack_nibbles(codes), ws=ws, gscale=0.05, x=x)


def gemm_layer(n=N_DEFAULT, k=K_DEFAULT, m=2048, seed=3) -> dict:
    """Prefill GEMM inputs: int4 weights as ``rt4_layer``, f32 group-first scales
    ``[K/128, N]`` (bf16-representable values), x ``[M,K]`` f32."""
    rng = np.random.default_rng(seed)
    w = rng.integers(-8, 8, size=(n, k), dtype=np.int8)
    sbits = f32_to_bf16_bits(_scale_values(rng, (n, k // GROUP)))
    wsc = np.ascontiguousarray(((sbits.astype(np.uint32) << 16).view(np.float32)).T)
    x = rng.standard_normal((m, k)).astype(np.float32)
    return dict(n=n, k=k, m=m, w=w, wq=pack_nibbles(w), wsc_gf=wsc, x=x)


STREAM_ROW_BLOCKS = 8        # a layer is generated in 8 independent row blocks


def stream_layer_block(layer: int, block: int, n=N_DEFAULT, k=K_DEFAULT, seed=4) -> dict:
    """Row block ``block`` (of ``STREAM_ROW_BLOCKS``) of layer ``layer`` of the decode
    weight stream: ``n/8`` rows of packed two's-complement nibbles (uniform bytes = two
    uniform int4 values each) and their f16 scales.  Blocks are independent draws from
    ``default_rng([seed, layer, block])`` so that a rank holding any row shard
    (1/2/4/8-way) generates exactly its own rows and the global layer is the same for
    every sharding."""
    rows = n // STREAM_ROW_BLOCKS
    rng = np.random.default_rng([seed, layer, block])
    wq = rng.integers(0, 256, size=(rows, k // 2), dtype=np.uint8)
    ws = _scale_values(rng, (rows, k // GROUP)).astype(np.float16)
    return dict(wq=wq, ws=ws)


def stream_layer_x(layer: int, k=K_DEFAULT, seed=4) -> np.ndarray:
    """The fixed input row of layer ``layer`` of the stream, f32 ``[K]`` ~ N(0,1)."""
    return np.random.default_rng([seed, layer, 1 << 20]).standard_normal(k).astype(np.float32)
