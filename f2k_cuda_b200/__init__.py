"""B200-native joint attention for the FLUX.2-klein MMDiT path.

A drop-in for ONE path of chrisjhebert1973/F2K_CUDA: per-head QK-RMSNorm, 4-axis RoPE and
non-causal attention over text||image tokens, written as CUDA for sm_100a (TMA, mbarrier
pipelines, tcgen05 MMA with accumulators in tensor memory) behind the C ABI declared in
`include/f2k_attn.h`. This package is the thin host side: it loads the in-tree library and
mirrors the reference's call surface. Importing it fails when the library is missing; there
is no fallback implementation.
"""
from .api import (  # noqa: F401
    Attention, JointAttention, build_rope_4axis_tables, rmsnorm_bf16, rope_4axis_inplace_bf16,
)
from .inputs import WORKLOADS, Workload, make_problem  # noqa: F401

__all__ = ["Attention", "JointAttention", "build_rope_4axis_tables", "rmsnorm_bf16",
           "rope_4axis_inplace_bf16", "WORKLOADS", "Workload", "make_problem"]
