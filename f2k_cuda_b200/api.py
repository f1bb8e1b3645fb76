"""Host-side mirror of the reference's attention call surface over the C ABI.

Names, argument meaning and error behaviour follow the reference's C++ classes
(F2K_CUDA src/backend/cuda/attention.h:29-54, joint_attention.h:21-54,
kernels/rmsnorm.h:23-29, kernels/rope_4axis.h:31-50): objects are configured once,
never raise from `forward` (it returns False and `last_error()` explains), tensors are
bf16 `[batch, seq, n_heads, head_dim]` on the GPU. torch is used for device memory and
streams only; all arithmetic happens inside libf2k_attn.so.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib
from ._lib import AttnConfig, lib


def _p(t):
    """Device (or host) address of a tensor, None -> NULL."""
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream(stream):
    if stream is None:
        stream = torch.cuda.current_stream()
    return C.c_void_p(stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream))


def _check_bf16(*tensors):
    for t in tensors:
        if t is None:
            continue
        if t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise TypeError("tensors must be contiguous bfloat16")


class _Module:
    def __init__(self, batch, seq_txt, seq_img, n_heads, head_dim, scale):
        self._h = C.c_void_p()
        cfg = AttnConfig(batch, seq_txt, seq_img, n_heads, head_dim, scale)
        self._rc = lib.f2k_attn_create(C.byref(cfg), C.byref(self._h))
        self.batch, self.seq_txt, self.seq_img = batch, seq_txt, seq_img
        self.n_heads, self.head_dim = n_heads, head_dim

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and lib is not None:
            lib.f2k_attn_destroy(h)

    def ok(self) -> bool:
        return self._rc == _lib.F2K_OK

    def last_error(self) -> str:
        return lib.f2k_attn_last_error(self._h).decode() if self._h else "no handle"

    def device_status(self) -> int:
        """Synchronises; 0 means every kernel of this module ran clean."""
        st = C.c_int(0)
        lib.f2k_attn_device_status(self._h, C.byref(st))
        return st.value

    def set_wait_limits(self, in_cta_clk: int = 0, peer_clk: int = 0) -> bool:
        """Limits of the kernels' bounded waits in SM clock cycles (0 = default)."""
        return lib.f2k_attn_set_wait_limits(self._h, in_cta_clk, peer_clk) == _lib.F2K_OK

    # ---- fused calls (no counterpart in the reference classes); a module without a text stream
    # ---- passes None for every *_txt argument
    def fused_workspace_size_bytes(self) -> int:
        return int(lib.f2k_attn_fused_workspace_bytes(self._h)) if self.ok() else 0

    def forward_fused(self, Q_txt, K_txt, V_txt, Q_img, K_img, V_img, gammas, tables, eps,
                      O_txt, O_img, workspace, stream=None) -> bool:
        """Raw projections in; per-head RMSNorm + RoPE + attention in one call.
        gammas = (gq_txt, gk_txt, gq_img, gk_img) bf16 [128];
        tables = (cos_txt, sin_txt, cos_img, sin_img) fp32 [seq, 64]."""
        if not self.ok():
            return False
        _check_bf16(Q_txt, K_txt, V_txt, Q_img, K_img, V_img, O_txt, O_img, *gammas)
        ws_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
        return lib.f2k_attn_forward_fused(
            self._h, _p(Q_txt), _p(K_txt), _p(V_txt), _p(Q_img), _p(K_img), _p(V_img),
            *[_p(g) for g in gammas], *[_p(t) for t in tables], eps, _p(O_txt), _p(O_img),
            _p(workspace), ws_bytes, _stream(stream)) == _lib.F2K_OK

    def forward_fused_strided(self, Q_txt, K_txt, V_txt, Q_img, K_img, V_img, gammas, tables, eps,
                              O_txt, O_img, workspace, stream=None) -> bool:
        """forward_fused on views: every tensor is a [batch, seq, n_heads, 128] view whose token
        rows may be slices of wider rows (e.g. columns of a fused projection output viewed with
        as_strided); rows of all batch elements must be consecutive. The strides are read off the
        views."""
        if not self.ok():
            return False
        st = _lib.AttnStrides()
        for name, t in (("q_txt", Q_txt), ("k_txt", K_txt), ("v_txt", V_txt), ("o_txt", O_txt),
                        ("q_img", Q_img), ("k_img", K_img), ("v_img", V_img), ("o_img", O_img)):
            if t is None:
                continue
            if t.dtype != torch.bfloat16 or t.dim() != 4 or t.stride(3) != 1 or t.stride(2) != t.shape[3] \
                    or (t.shape[0] > 1 and t.stride(0) != t.shape[1] * t.stride(1)):
                raise TypeError("tensors must be bfloat16 [batch, seq, heads, 128] views with dense heads and "
                                "consecutive token rows")
            setattr(st, name, t.stride(1))
        _check_bf16(*gammas)
        ws_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
        return lib.f2k_attn_forward_fused_strided(
            self._h, _p(Q_txt), _p(K_txt), _p(V_txt), _p(Q_img), _p(K_img), _p(V_img),
            *[_p(g) for g in gammas], *[_p(t) for t in tables], eps, _p(O_txt), _p(O_img),
            C.byref(st), _p(workspace), ws_bytes, _stream(stream)) == _lib.F2K_OK

    def forward_fused_host(self, hQ_txt, hK_txt, hV_txt, hQ_img, hK_img, hV_img, gammas, tables,
                           eps, hO_txt, hO_img, stream=None) -> bool:
        """Same as forward_fused with q, k, v, o in (pinned) host memory; gammas and tables on
        the GPU. Asynchronous on the stream."""
        if not self.ok():
            return False
        return lib.f2k_attn_forward_fused_host(
            self._h, _p(hQ_txt), _p(hK_txt), _p(hV_txt), _p(hQ_img), _p(hK_img), _p(hV_img),
            *[_p(g) for g in gammas], *[_p(t) for t in tables], eps, _p(hO_txt), _p(hO_img),
            _stream(stream)) == _lib.F2K_OK


class Attention(_Module):
    """Mirror of f2k::cuda::Attention: softmax(scale * Q K^T) V per head, non-causal."""

    @dataclass
    class Config:
        batch: int = 0
        seq: int = 0
        n_heads: int = 0
        head_dim: int = 0
        scale: float = 0.0  # 0 => 1/sqrt(head_dim)

    def __init__(self, cfg: "Attention.Config"):
        super().__init__(cfg.batch, 0, cfg.seq, cfg.n_heads, cfg.head_dim, cfg.scale)

    def forward(self, Q, K, V, O, stream=None) -> bool:
        if not self.ok():
            return False
        _check_bf16(Q, K, V, O)
        return lib.f2k_attn_forward(self._h, None, None, None, _p(Q), _p(K), _p(V), None, _p(O),
                                    None, 0, _stream(stream)) == _lib.F2K_OK

    def forward_fused_single(self, Q, K, V, gamma_q, gamma_k, cos, sin, eps, O, workspace, stream=None,
                             strided: bool = False) -> bool:
        """Raw projections of one combined stream in (the single-stream block's call):
        per-head RMSNorm + RoPE + attention. strided=True takes [batch, seq, heads, 128] views
        whose token rows are slices of wider rows."""
        call = self.forward_fused_strided if strided else self.forward_fused
        return call(None, None, None, Q, K, V, (None, None, gamma_q, gamma_k), (None, None, cos, sin), eps,
                    None, O, workspace, stream)


class JointAttention(_Module):
    """Mirror of f2k::cuda::JointAttention: attention over text tokens followed by image tokens."""

    @dataclass
    class Config:
        batch: int = 0
        seq_txt: int = 0
        seq_img: int = 0
        n_heads: int = 0
        head_dim: int = 0
        scale: float = 0.0

    def __init__(self, cfg: "JointAttention.Config"):
        # The reference refuses an empty text stream; 0 would mean "plain attention" to the C ABI.
        super().__init__(cfg.batch, cfg.seq_txt if cfg.seq_txt > 0 else -1, cfg.seq_img,
                         cfg.n_heads, cfg.head_dim, cfg.scale)

    def workspace_size_bytes(self) -> int:
        return int(lib.f2k_attn_workspace_bytes(self._h)) if self.ok() else 0

    def forward(self, Q_txt, K_txt, V_txt, Q_img, K_img, V_img, O_txt, O_img,
                workspace=None, workspace_size=0, stream=None) -> bool:
        if not self.ok():
            return False
        _check_bf16(Q_txt, K_txt, V_txt, Q_img, K_img, V_img, O_txt, O_img)
        return lib.f2k_attn_forward(self._h, _p(Q_txt), _p(K_txt), _p(V_txt), _p(Q_img), _p(K_img),
                                    _p(V_img), _p(O_txt), _p(O_img), _p(workspace), workspace_size,
                                    _stream(stream)) == _lib.F2K_OK


def rmsnorm_bf16(x, gamma, y, batch_rows: int, dim: int, eps: float, stream=None) -> bool:
    """Mirror of f2k::cuda::rmsnorm_bf16 (y may be x)."""
    return lib.f2k_rmsnorm_bf16(_p(x), _p(gamma), _p(y), batch_rows, dim, eps, _stream(stream)) == _lib.F2K_OK


def rope_4axis_inplace_bf16(x, cos_table, sin_table, pos_ids, batch_rows: int, head_dim: int,
                            seq_max: int, stream=None) -> bool:
    """Mirror of f2k::cuda::rope_4axis_inplace_bf16."""
    return lib.f2k_rope_4axis_inplace_bf16(_p(x), _p(cos_table), _p(sin_table), _p(pos_ids),
                                           batch_rows, head_dim, seq_max, _stream(stream)) == _lib.F2K_OK


def build_rope_4axis_tables(axes_dim, token_positions, theta: float):
    """Mirror of f2k::cuda::build_rope_4axis_tables; returns (cos, sin) float32 [seq, sum(axes)/2]."""
    axes = np.ascontiguousarray(axes_dim, dtype=np.int32)
    pos = np.ascontiguousarray(token_positions, dtype=np.int32).reshape(-1, len(axes))
    half = int(axes.sum()) // 2
    cos = np.zeros((pos.shape[0], half), np.float32)
    sin = np.zeros_like(cos)
    rc = lib.f2k_build_rope_4axis_tables(axes.ctypes.data_as(C.c_void_p), len(axes),
                                         pos.ctypes.data_as(C.c_void_p), pos.shape[0], theta,
                                         cos.ctypes.data_as(C.c_void_p), sin.ctypes.data_as(C.c_void_p))
    if rc != _lib.F2K_OK:
        raise ValueError("build_rope_4axis_tables: invalid arguments")
    return cos, sin
