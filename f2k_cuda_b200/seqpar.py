"""Sequence-parallel joint attention across the GPUs of one box (host side).

One process per GPU. Rank r holds the queries, keys and values of its `seq_local` tokens of the
text||image sequence; `SequenceParallelAttention.forward` gives it the attention output of its
queries over every rank's keys and values. The K/V shards of the other ranks are pulled into
local memory by the copy engines over NVLink while the attention kernel already works on what
has arrived (see csrc/seqpar.cu). torch.distributed is used once, to hand the 64-byte IPC handles
of the shard buffers around; a step runs no collective (the ranks tell each other "my K/V are
written" through words in those buffers).

`plan_ring` and `shard_bounds` are pure host logic (tested on CPU with gloo ranks).
"""
from __future__ import annotations

import ctypes as C

from . import _lib
from ._lib import SeqParConfig, lib


def shard_bounds(seq: int, world: int, rank: int) -> tuple[int, int]:
    """Token range [begin, end) of `rank` when `seq` tokens are dealt out in equal contiguous
    shards (the last shard is shorter when world does not divide seq)."""
    per = -(-seq // world)
    return min(rank * per, seq), min((rank + 1) * per, seq)


def plan_ring(world: int, rank: int) -> list[int]:
    """Order in which `rank` consumes the K/V shards: its own, then rank+1, rank+2, ... (mod
    world). Every rank starts on a different shard, so at step i the N pulls hit N different
    source GPUs."""
    return [(rank + i) % world for i in range(world)]


class SequenceParallelAttention:
    """One rank's end of the sequence-parallel attention.

    ranks_in_process: for tests on a single GPU, a list of the objects of all ranks living in
    this process (their buffers are attached by pointer instead of through CUDA IPC).
    """

    def __init__(self, batch: int, seq_local: int, n_heads: int, head_dim: int, world: int, rank: int,
                 scale: float = 0.0):
        self.world, self.rank = world, rank
        self.batch, self.seq_local, self.n_heads, self.head_dim = batch, seq_local, n_heads, head_dim
        self._h = C.c_void_p()
        cfg = SeqParConfig(batch, seq_local, n_heads, head_dim, world, rank, scale)
        self._rc = lib.f2k_seqpar_create(C.byref(cfg), C.byref(self._h))
        self._opened = []

    def __del__(self):
        if lib is None:          # interpreter shutdown
            return
        for base in getattr(self, "_opened", []):
            lib.f2k_ipc_close(base)
        h, self._h = getattr(self, "_h", None), None
        if h:
            lib.f2k_seqpar_destroy(h)

    def ok(self) -> bool:
        return self._rc == _lib.F2K_OK

    def last_error(self) -> str:
        return lib.f2k_seqpar_last_error(self._h).decode() if self._h else "no handle"

    def buffer(self) -> tuple[int, int]:
        base, n = C.c_void_p(), C.c_size_t()
        lib.f2k_seqpar_buffer(self._h, C.byref(base), C.byref(n))
        return base.value, n.value

    # ---- wiring the ranks together ------------------------------------------------------
    def attach_in_process(self, ranks: list["SequenceParallelAttention"]) -> bool:
        bases = (C.c_void_p * self.world)(*[r.buffer()[0] for r in ranks])
        return lib.f2k_seqpar_attach(self._h, bases) == _lib.F2K_OK

    def attach_distributed(self, group=None) -> bool:
        """Exchange IPC handles over torch.distributed (any backend) and map every peer's buffer."""
        import torch.distributed as dist
        handle = (C.c_ubyte * 64)()
        if lib.f2k_ipc_export(C.c_void_p(self.buffer()[0]), handle) != _lib.F2K_OK:
            return False
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=group)
        bases = (C.c_void_p * self.world)()
        for r, hb in enumerate(handles):
            if r == self.rank:
                bases[r] = self.buffer()[0]
                continue
            base = C.c_void_p()
            if lib.f2k_ipc_open((C.c_ubyte * 64).from_buffer_copy(hb), C.byref(base)) != _lib.F2K_OK:
                return False
            self._opened.append(base)
            bases[r] = base.value
        return lib.f2k_seqpar_attach(self._h, bases) == _lib.F2K_OK

    # ---- per step -------------------------------------------------------------------------
    def local_kv(self):
        """(k, v) torch views [batch, seq_local, n_heads, 128] of where this rank's K and V for the
        next forward() go."""
        k, v = C.c_void_p(), C.c_void_p()
        lib.f2k_seqpar_local_kv(self._h, C.byref(k), C.byref(v))
        shape = (self.batch, self.seq_local, self.n_heads, self.head_dim)
        return _tensor_from_ptr(k.value, shape), _tensor_from_ptr(v.value, shape)

    def forward(self, q_local, o_local, overlap: bool = True, stream=None) -> bool:
        """Attention of this rank's queries over all ranks' keys/values. `stream` is the compute
        stream this rank wrote its K/V on; the pulls run on a copy stream owned by the handle."""
        import torch
        if stream is None:
            stream = torch.cuda.current_stream()
        rc = lib.f2k_seqpar_forward(self._h, C.c_void_p(q_local.data_ptr()), C.c_void_p(o_local.data_ptr()),
                                    int(overlap), C.c_void_p(stream.cuda_stream), None)
        return rc == _lib.F2K_OK

    def device_status(self) -> int:
        st = C.c_int(0)
        lib.f2k_seqpar_device_status(self._h, C.byref(st))
        return st.value

    def set_wait_limits(self, in_cta_clk: int = 0, peer_clk: int = 0) -> bool:
        """Limits of the kernels' bounded waits in SM clock cycles (0 = default)."""
        return lib.f2k_seqpar_set_wait_limits(self._h, in_cta_clk, peer_clk) == _lib.F2K_OK

    def abort(self) -> bool:
        """Releases the copy stream of the current step when a peer never announced its K/V."""
        return lib.f2k_seqpar_abort(self._h) == _lib.F2K_OK


def qk_norm_rope(x, y, gamma, cos_table, sin_table, eps: float, stream=None) -> bool:
    """y = RoPE(RMSNorm(x) * gamma) per head row of x [batch, seq, heads, 128]; position = token
    index, so a sequence shard passes its own rows of the tables."""
    import torch
    if stream is None:
        stream = torch.cuda.current_stream()
    b, s, h, _ = x.shape
    p = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
    return lib.f2k_qk_norm_rope_bf16(p(x), p(y), p(gamma), p(cos_table), p(sin_table), b, s, h, eps,
                                     C.c_void_p(stream.cuda_stream)) == _lib.F2K_OK


def _tensor_from_ptr(ptr: int, shape):
    """A torch.bfloat16 CUDA tensor over memory owned by the library (no copy)."""
    import numpy as np
    import torch

    class _Holder:
        pass

    n = int(np.prod(shape))
    holder = _Holder()
    holder.__cuda_array_interface__ = {"shape": (n,), "typestr": "<i2", "data": (ptr, False), "version": 3,
                                       "strides": None}
    return torch.as_tensor(holder, device="cuda").view(torch.bfloat16).view(*shape)
