"""B200-native joint attention for the FLUX.2-klein MMDiT path.

A drop-in for ONE path of chrisjhebert1973/F2K_CUDA: per-head QK-RMSNorm, 4-axis RoPE and
non-causal attention over text||image tokens, written as CUDA for sm_100a (TMA, mbarrier
pipelines, tcgen05 MMA with accumulators in tensor memory) behind the C ABI declared in
`include/f2k_attn.h`. This package is the thin host side: it loads the in-tree library and
mirrors the reference's call surface. There is no fallback implementation: the first use of any
attention entry point loads `libf2k_attn.so` and fails loudly when it is missing and cannot be
built. (`f2k_cuda_b200.inputs`, the seeded workload generator, is plain numpy and can be imported
without the library.)
"""
from .inputs import WORKLOADS, Workload, make_problem  # noqa: F401

_API = ("Attention", "JointAttention", "build_rope_4axis_tables", "rmsnorm_bf16", "rope_4axis_inplace_bf16")
__all__ = [*_API, "WORKLOADS", "Workload", "make_problem"]


def __getattr__(name):
    if name in _API:
        from . import api          # loads the library (and builds it first when it is stale)
        return getattr(api, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
