"""k100lc_kernels on B200: the weight-streaming quantized linear-layer path of
Hong-agent/K100LC-kernels (W4A16 / W4A8 / W4A4 / NVFP4 decode GEMV with their
activation quantisers and the W4 prefill GEMM) as hand-written sm_100a CUDA kernels
behind the reference's Python surface (python/k100lc_kernels/__init__.py:2-22)."""
from .catalog import info, kernels
from .model import (Attention, DotLinear, F32Linear, FlashAttention, Int4Linear, KVCache, MLP,
                    MoECombine, MoEExperts, NVFP4Linear, RMSNorm, RoPE, RT4Linear, Sampler, SwiGLU,
                    TransformerLayer, Workspace, div_magic, run_sequence)
from .quant import (ct_int4_to_rt4, ct_int4_to_twos_complement, dequant_int4_group128,
                    int4_scale_group_first_f32, pack_int4_group128)
from .rt4 import RT4File, RT4Tensor, W4Runner
from .runtime import LaunchPlan, Runtime

__all__ = [
    "Runtime", "LaunchPlan", "kernels", "info", "RT4File", "RT4Tensor", "W4Runner", "Workspace",
    "DotLinear", "F32Linear", "RT4Linear", "Int4Linear", "NVFP4Linear", "Attention", "FlashAttention",
    "TransformerLayer", "RMSNorm", "SwiGLU", "MLP", "MoECombine", "MoEExperts", "RoPE", "KVCache",
    "Sampler", "div_magic", "run_sequence", "pack_int4_group128", "dequant_int4_group128",
    "ct_int4_to_rt4", "ct_int4_to_twos_complement", "int4_scale_group_first_f32",
]
