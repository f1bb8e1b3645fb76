"""Sequence-parallel attention by head exchange (host side).

One process per GPU. Rank r holds the raw Q, K, V of its `seq_local` tokens (all heads) and gets
the attention output of those tokens; inside, every rank attends n_heads / world heads over all
tokens. The exchange is done by the kernels themselves with stores into peer memory (see
csrc/headswap.cu). torch.distributed is used once, to hand the IPC handles around.
"""
from __future__ import annotations

import ctypes as C

from . import _lib
from ._lib import SeqParConfig, lib
from .seqpar import _tensor_from_ptr


def head_exchange_plan(seq_local: int, n_heads: int, world: int, rank: int) -> dict:
    """Where `rank`'s rows go, as the kernels compute it (pure host logic, tested on CPU).

    Inbound: head h of local token t is stored on rank h // heads_per_rank, in that rank's
    [world * seq_local, heads_per_rank, 128] buffers, at token rank * seq_local + t, head
    h % heads_per_rank. Outbound: the attention output of query segment s (the tokens of rank s)
    is stored on rank s, in its [seq_local, n_heads, 128] buffer, in head columns
    [rank * heads_per_rank, (rank + 1) * heads_per_rank)."""
    if world <= 0 or n_heads % world != 0 or not 0 <= rank < world:
        raise ValueError("world must divide n_heads and 0 <= rank < world")
    hpr = n_heads // world
    return {
        "heads_per_rank": hpr,
        "send": [{"to": d, "heads": (d * hpr, (d + 1) * hpr), "token_offset": rank * seq_local} for d in range(world)],
        "return": [{"to": s, "tokens_of_rank": s, "head_columns": (rank * hpr, (rank + 1) * hpr)} for s in range(world)],
    }


def peer_failures(failed_words, step: int) -> list[int]:
    """Ranks whose attention kernel gave up during `step`: rank s stores the step number into word
    s of every peer's "failed" words before it publishes "done" (csrc/headswap.cu), so a rank that
    sees all "done" words and no marker knows that every row it received was written. Words of
    earlier steps hold older numbers and do not count. Pure host logic (tested on CPU)."""
    return [s for s, wd in enumerate(failed_words) if step > 0 and int(wd) == step]


class HeadExchangeAttention:
    def __init__(self, seq_local: int, n_heads: int, head_dim: int, world: int, rank: int, scale: float = 0.0):
        self.world, self.rank = world, rank
        self.seq_local, self.n_heads, self.head_dim = seq_local, n_heads, head_dim
        self._h = C.c_void_p()
        cfg = SeqParConfig(1, seq_local, n_heads, head_dim, world, rank, scale)
        self._rc = lib.f2k_hx_create(C.byref(cfg), C.byref(self._h))
        self._opened = []

    def __del__(self):
        if lib is None:          # interpreter shutdown
            return
        for base in getattr(self, "_opened", []):
            lib.f2k_ipc_close(base)
        h, self._h = getattr(self, "_h", None), None
        if h:
            lib.f2k_hx_destroy(h)

    def ok(self) -> bool:
        return self._rc == _lib.F2K_OK

    def last_error(self) -> str:
        return lib.f2k_hx_last_error(self._h).decode() if self._h else "no handle"

    def buffer(self):
        base, n = C.c_void_p(), C.c_size_t()
        lib.f2k_hx_buffer(self._h, C.byref(base), C.byref(n))
        return base.value, n.value

    def attach_in_process(self, ranks) -> bool:
        """All ranks live in this process on one GPU (tests): attach their buffers by pointer."""
        bases = (C.c_void_p * self.world)(*[r.buffer()[0] for r in ranks])
        return lib.f2k_hx_attach(self._h, bases) == _lib.F2K_OK

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
        return lib.f2k_hx_attach(self._h, bases) == _lib.F2K_OK

    # ---- per step, all on one stream ------------------------------------------------------
    @staticmethod
    def _stream(stream):
        import torch
        return C.c_void_p((stream or torch.cuda.current_stream()).cuda_stream)

    def exchange_in(self, q_raw, k_raw, v, gamma_q, gamma_k, cos_local, sin_local, eps: float, stream=None) -> bool:
        """q_raw, k_raw, v: [1, seq_local, n_heads, 128] bf16; cos_local/sin_local: this rank's rows
        of the RoPE tables. Normalises + rotates Q and K and sends every head to its rank."""
        p = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
        return lib.f2k_hx_exchange_in(self._h, p(q_raw), p(k_raw), p(v), p(gamma_q), p(gamma_k), p(cos_local),
                                      p(sin_local), eps, self._stream(stream)) == _lib.F2K_OK

    def exchange_in_copy(self, q_raw, k_raw, v, gamma_q, gamma_k, cos_local, sin_local, eps: float, stream=None) -> bool:
        """exchange_in with the copy engines doing the transfers (one local prologue kernel, then
        strided copies per destination on streams of the handle): the attention that attend()
        launches behind it runs while the copies are on their way."""
        p = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
        return lib.f2k_hx_exchange_in_copy(self._h, p(q_raw), p(k_raw), p(v), p(gamma_q), p(gamma_k), p(cos_local),
                                           p(sin_local), eps, self._stream(stream)) == _lib.F2K_OK

    def forward(self, q_raw, k_raw, v, gamma_q, gamma_k, cos_local, sin_local, eps: float, stream=None) -> bool:
        """exchange_in + attend as one kernel (the exchange runs on the attention kernel's spare
        warps and hides under the attention). One process per GPU, or world == 1."""
        p = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
        return lib.f2k_hx_forward(self._h, p(q_raw), p(k_raw), p(v), p(gamma_q), p(gamma_k), p(cos_local),
                                  p(sin_local), eps, self._stream(stream)) == _lib.F2K_OK

    def attend(self, stream=None) -> bool:
        return lib.f2k_hx_attend(self._h, self._stream(stream)) == _lib.F2K_OK

    def output(self, stream=None):
        """Makes the stream wait for every rank's contribution; returns this rank's
        [1, seq_local, n_heads, 128] output (a view into the exchange buffer)."""
        o = C.c_void_p()
        if lib.f2k_hx_output(self._h, C.byref(o), self._stream(stream)) != _lib.F2K_OK:
            return None
        return _tensor_from_ptr(o.value, (1, self.seq_local, self.n_heads, self.head_dim))

    def device_status(self) -> int:
        st = C.c_int(0)
        lib.f2k_hx_device_status(self._h, C.byref(st))
        return st.value

    def set_wait_limits(self, in_cta_clk: int = 0, peer_clk: int = 0) -> bool:
        """Limits of the kernels' bounded waits in SM clock cycles (0 = default)."""
        return lib.f2k_hx_set_wait_limits(self._h, in_cta_clk, peer_clk) == _lib.F2K_OK

    def abort(self) -> bool:
        """Releases the stream waits of output() when a peer never delivered."""
        return lib.f2k_hx_abort(self._h) == _lib.F2K_OK
