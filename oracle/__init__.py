"""CPU oracle of the joint-attention path (TEST INFRASTRUCTURE).

Only tests/, `__graft_entry__.smoke()` and the cpu_baseline / reference legs of
`bench.py` may import this package; the product (`f2k_cuda_b200`) never does.
See `f2k_oracle.c` for what it restates and how it is pinned.
"""
from .oracle import (  # noqa: F401
    IDEAL, REF_ROUND, Oracle, RefLib, bf16_to_f32, f32_to_bf16, load_oracle, load_ref,
)
