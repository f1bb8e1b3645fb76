"""ctypes bindings of the oracle libraries (TEST INFRASTRUCTURE, see f2k_oracle.c).

`load_oracle()` -> Oracle: the CPU restatement, numpy in / numpy out.
`load_ref()`    -> RefLib or None: the reference's own CUDA code rebuilt for sm_100a
                   (oracle/_ref/libf2k_ref.so), device pointers in / out.
Both libraries are built by `make -C oracle` (the GPU machine only ever sees the
prebuilt files; the reference checkout does not exist there).
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ORACLE_LIB = HERE / "_build" / "libf2k_oracle.so"
REF_LIB = HERE / "_ref" / "libf2k_ref.so"

IDEAL, REF_ROUND = 0, 1


def build(ref: bool = True) -> None:
    """(Re)build the checker libraries; `ref` also rebuilds oracle/_ref (the reference's attention
    path and the block-level test programs) when the reference checkout is present."""
    subprocess.run(["make", "-C", str(HERE), "oracle"] + (["ref", "blocks"] if ref else []),
                   check=True, capture_output=True)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns (uint16), round to nearest even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + np.uint32(0x7FFF)
    return ((u + r) >> 16).astype(np.uint16)


def bf16_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


class _Problem(C.Structure):
    _fields_ = [
        ("mode", C.c_int), ("apply_prologue", C.c_int),
        ("batch", C.c_int), ("seq_txt", C.c_int), ("seq_img", C.c_int),
        ("n_heads", C.c_int), ("head_dim", C.c_int),
        ("head_begin", C.c_int), ("head_end", C.c_int),
        ("scale", C.c_float), ("eps", C.c_float),
        ("q_txt", C.c_void_p), ("k_txt", C.c_void_p), ("v_txt", C.c_void_p),
        ("q_img", C.c_void_p), ("k_img", C.c_void_p), ("v_img", C.c_void_p),
        ("gamma_q_txt", C.c_void_p), ("gamma_k_txt", C.c_void_p),
        ("gamma_q_img", C.c_void_p), ("gamma_k_img", C.c_void_p),
        ("cos_txt", C.c_void_p), ("sin_txt", C.c_void_p),
        ("cos_img", C.c_void_p), ("sin_img", C.c_void_p),
    ]


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _u16(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.uint16)


def _f32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


class Oracle:
    def __init__(self, path: Path = ORACLE_LIB):
        if not path.exists():
            build(ref=False)
        self.lib = C.CDLL(str(path))
        L = self.lib
        L.f2k_oracle_joint_path.restype = C.c_int
        L.f2k_oracle_joint_path.argtypes = [C.POINTER(_Problem), C.c_void_p, C.c_void_p]
        L.f2k_oracle_joint_rows.restype = C.c_int
        L.f2k_oracle_joint_rows.argtypes = [C.POINTER(_Problem), C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p]
        L.f2k_oracle_attention_f32.restype = C.c_int
        L.f2k_oracle_attention_f32.argtypes = [C.c_void_p] * 4 + [C.c_int] * 4 + [C.c_float, C.c_int, C.c_int]
        L.f2k_oracle_rmsnorm_ideal.argtypes = [C.c_void_p] * 3 + [C.c_long, C.c_int, C.c_float]
        L.f2k_oracle_rmsnorm_bf16.argtypes = [C.c_void_p] * 3 + [C.c_long, C.c_int, C.c_float]
        L.f2k_oracle_build_rope_tables.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_float,
                                                   C.c_void_p, C.c_void_p]
        L.f2k_oracle_rope_bf16.argtypes = [C.c_void_p] * 4 + [C.c_long, C.c_int, C.c_int]
        L.f2k_oracle_num_threads.restype = C.c_int

    @property
    def threads(self) -> int:
        return int(self.lib.f2k_oracle_num_threads())

    def _problem(self, q_img, k_img, v_img, q_txt, k_txt, v_txt, gammas, tables, eps, scale, mode):
        q_img, k_img, v_img = _u16(q_img), _u16(k_img), _u16(v_img)
        B, Si, H, D = q_img.shape
        St = 0 if q_txt is None else q_txt.shape[1]
        q_txt, k_txt, v_txt = _u16(q_txt), _u16(k_txt), _u16(v_txt)
        pro = gammas is not None
        keep = [q_img, k_img, v_img, q_txt, k_txt, v_txt]
        pr = _Problem()
        pr.mode, pr.apply_prologue = mode, int(pro)
        pr.batch, pr.seq_txt, pr.seq_img, pr.n_heads, pr.head_dim = B, St, Si, H, D
        pr.head_begin, pr.head_end = 0, H
        pr.scale, pr.eps = scale, eps
        pr.q_txt, pr.k_txt, pr.v_txt = _ptr(q_txt), _ptr(k_txt), _ptr(v_txt)
        pr.q_img, pr.k_img, pr.v_img = _ptr(q_img), _ptr(k_img), _ptr(v_img)
        if pro:
            g = [_u16(x) for x in gammas]
            t = [_f32(x) for x in tables]
            keep += g + t
            pr.gamma_q_txt, pr.gamma_k_txt, pr.gamma_q_img, pr.gamma_k_img = map(_ptr, g)
            pr.cos_txt, pr.sin_txt, pr.cos_img, pr.sin_img = map(_ptr, t)
        return pr, keep

    def joint_rows(self, rows, *, batch=0, head=0, q_img, k_img, v_img, q_txt=None, k_txt=None, v_txt=None,
                   gammas=None, tables=None, eps=1e-6, scale=0.0, mode=IDEAL):
        """The joint path for selected query rows (indices into the text||image sequence) of one
        (batch, head): float32 [len(rows), D]. All threads work on the one head, so long
        sequences are checked in seconds."""
        pr, keep = self._problem(q_img, k_img, v_img, q_txt, k_txt, v_txt, gammas, tables, eps, scale, mode)
        rows = np.ascontiguousarray(rows, dtype=np.int32)
        out = np.zeros((len(rows), pr.head_dim), np.float32)
        rc = self.lib.f2k_oracle_joint_rows(C.byref(pr), batch, head, _ptr(rows), len(rows), _ptr(out))
        if rc != 0:
            raise RuntimeError("oracle: bad problem, bad row index or out of memory")
        del keep
        return out

    def joint_path(self, *, q_img, k_img, v_img, q_txt=None, k_txt=None, v_txt=None,
                   gammas=None, tables=None, eps=1e-6, scale=0.0, mode=IDEAL,
                   heads=None):
        """Tensors: uint16 bf16 bit patterns [B, S, H, D]. gammas = (gq_txt, gk_txt, gq_img,
        gk_img) and tables = (cos_txt, sin_txt, cos_img, sin_img) switch the prologue on.
        Returns (o_txt or None, o_img) as float32; only heads[0]:heads[1] are computed."""
        q_img, k_img, v_img = _u16(q_img), _u16(k_img), _u16(v_img)
        B, Si, H, D = q_img.shape
        St = 0 if q_txt is None else q_txt.shape[1]
        q_txt, k_txt, v_txt = _u16(q_txt), _u16(k_txt), _u16(v_txt)
        pro = gammas is not None
        keep = [q_img, k_img, v_img, q_txt, k_txt, v_txt]
        pr = _Problem()
        pr.mode, pr.apply_prologue = mode, int(pro)
        pr.batch, pr.seq_txt, pr.seq_img, pr.n_heads, pr.head_dim = B, St, Si, H, D
        pr.head_begin, pr.head_end = (0, H) if heads is None else heads
        pr.scale, pr.eps = scale, eps
        pr.q_txt, pr.k_txt, pr.v_txt = _ptr(q_txt), _ptr(k_txt), _ptr(v_txt)
        pr.q_img, pr.k_img, pr.v_img = _ptr(q_img), _ptr(k_img), _ptr(v_img)
        if pro:
            g = [_u16(x) for x in gammas]
            t = [_f32(x) for x in tables]
            keep += g + t
            pr.gamma_q_txt, pr.gamma_k_txt, pr.gamma_q_img, pr.gamma_k_img = map(_ptr, g)
            pr.cos_txt, pr.sin_txt, pr.cos_img, pr.sin_img = map(_ptr, t)
        o_txt = np.zeros((B, St, H, D), np.float32) if St else None
        o_img = np.zeros((B, Si, H, D), np.float32)
        rc = self.lib.f2k_oracle_joint_path(C.byref(pr), _ptr(o_txt), _ptr(o_img))
        if rc != 0:
            raise RuntimeError("oracle: bad problem or out of memory")
        return o_txt, o_img

    def attention_f32(self, q, k, v, scale=0.0, heads=None):
        q, k, v = _u16(q), _u16(k), _u16(v)
        B, S, H, D = q.shape
        o = np.zeros((B, S, H, D), np.float32)
        h0, h1 = (0, H) if heads is None else heads
        rc = self.lib.f2k_oracle_attention_f32(_ptr(q), _ptr(k), _ptr(v), _ptr(o), B, S, H, D,
                                               scale, h0, h1)
        if rc != 0:
            raise RuntimeError("oracle: attention_f32 failed")
        return o

    def rmsnorm_ideal(self, x, gamma, eps):
        x, gamma = _u16(x), _u16(gamma)
        y = np.zeros(x.shape, np.float32)
        self.lib.f2k_oracle_rmsnorm_ideal(_ptr(x), _ptr(gamma), _ptr(y), x.size // x.shape[-1], x.shape[-1], eps)
        return y

    def rmsnorm_bf16(self, x, gamma, eps):
        x, gamma = _u16(x), _u16(gamma)
        y = np.zeros(x.shape, np.uint16)
        self.lib.f2k_oracle_rmsnorm_bf16(_ptr(x), _ptr(gamma), _ptr(y), x.size // x.shape[-1], x.shape[-1], eps)
        return y

    def build_rope_tables(self, axes_dim, positions, theta):
        axes = np.ascontiguousarray(axes_dim, dtype=np.int32)
        pos = np.ascontiguousarray(positions, dtype=np.int32).reshape(-1, len(axes))
        half = int(axes.sum()) // 2
        cos = np.zeros((pos.shape[0], half), np.float32)
        sin = np.zeros_like(cos)
        self.lib.f2k_oracle_build_rope_tables(_ptr(axes), len(axes), _ptr(pos), pos.shape[0], theta,
                                              _ptr(cos), _ptr(sin))
        return cos, sin

    def rope_bf16(self, x, cos, sin, pos_ids, seq_max):
        y = _u16(x).copy()
        cos, sin = _f32(cos), _f32(sin)
        pos = np.ascontiguousarray(pos_ids, dtype=np.int32)
        self.lib.f2k_oracle_rope_bf16(_ptr(y), _ptr(cos), _ptr(sin), _ptr(pos), y.size // y.shape[-1],
                                      y.shape[-1], seq_max)
        return y


class RefLib:
    """The reference's own CUDA attention path (device pointers as ints)."""

    def __init__(self, path: Path = REF_LIB):
        self.lib = C.CDLL(str(path))
        L = self.lib
        vp = C.c_void_p
        L.f2k_ref_joint_create.restype = vp
        L.f2k_ref_joint_create.argtypes = [C.c_int] * 5 + [C.c_float]
        L.f2k_ref_joint_ok.argtypes = [vp]
        L.f2k_ref_joint_last_error.restype = C.c_char_p
        L.f2k_ref_joint_last_error.argtypes = [vp]
        L.f2k_ref_joint_workspace_bytes.restype = C.c_size_t
        L.f2k_ref_joint_workspace_bytes.argtypes = [vp]
        L.f2k_ref_joint_forward.argtypes = [vp] * 10 + [C.c_size_t, vp]
        L.f2k_ref_joint_destroy.argtypes = [vp]
        L.f2k_ref_attn_create.restype = vp
        L.f2k_ref_attn_create.argtypes = [C.c_int] * 4 + [C.c_float]
        L.f2k_ref_attn_ok.argtypes = [vp]
        L.f2k_ref_attn_last_error.restype = C.c_char_p
        L.f2k_ref_attn_last_error.argtypes = [vp]
        L.f2k_ref_attn_forward.argtypes = [vp] * 6
        L.f2k_ref_attn_destroy.argtypes = [vp]
        L.f2k_ref_rmsnorm_bf16.argtypes = [vp, vp, vp, C.c_int, C.c_int, C.c_float, vp]
        L.f2k_ref_rope_4axis_inplace_bf16.argtypes = [vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, vp]
        L.f2k_ref_build_rope_4axis_tables.argtypes = [vp, C.c_int, vp, C.c_int, C.c_float, vp, vp]

    def build_rope_tables(self, axes_dim, positions, theta):
        axes = np.ascontiguousarray(axes_dim, dtype=np.int32)
        pos = np.ascontiguousarray(positions, dtype=np.int32).reshape(-1, len(axes))
        half = int(axes.sum()) // 2
        cos = np.zeros((pos.shape[0], half), np.float32)
        sin = np.zeros_like(cos)
        self.lib.f2k_ref_build_rope_4axis_tables(_ptr(axes), len(axes), _ptr(pos), pos.shape[0], theta,
                                                 _ptr(cos), _ptr(sin))
        return cos, sin


_oracle = None


def load_oracle() -> Oracle:
    global _oracle
    if _oracle is None:
        _oracle = Oracle()
    return _oracle


def load_ref():
    """RefLib, or None when oracle/_ref was never built (no reference checkout)."""
    return RefLib() if REF_LIB.exists() else None
