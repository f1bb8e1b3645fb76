"""ctypes view of libf2k_attn.so - exactly the entry points include/f2k_attn.h declares.

Importing this module loads the in-tree library and raises if it is missing: the package
has no other implementation to fall back on.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

from .build import LIB_PATH, build

F2K_OK, F2K_ERR_INVALID, F2K_ERR_UNSUPPORTED, F2K_ERR_WORKSPACE, F2K_ERR_CUDA, F2K_ERR_DEVICE = range(6)


class SeqParConfig(C.Structure):
    """struct f2k_seqpar_config"""
    _fields_ = [("batch", C.c_int), ("seq_local", C.c_int), ("n_heads", C.c_int), ("head_dim", C.c_int),
                ("world", C.c_int), ("rank", C.c_int), ("scale", C.c_float)]


class AttnConfig(C.Structure):
    """struct f2k_attn_config"""
    _fields_ = [("batch", C.c_int), ("seq_txt", C.c_int), ("seq_img", C.c_int),
                ("n_heads", C.c_int), ("head_dim", C.c_int), ("scale", C.c_float)]


class AttnStrides(C.Structure):
    """struct f2k_attn_strides: token strides in elements, 0 = dense"""
    _fields_ = [(n, C.c_longlong) for n in ("q_txt", "k_txt", "v_txt", "o_txt", "q_img", "k_img", "v_img", "o_img")]


def _declare(lib: C.CDLL) -> None:
    vp, i, f, sz = C.c_void_p, C.c_int, C.c_float, C.c_size_t
    lib.f2k_attn_create.restype = i
    lib.f2k_attn_create.argtypes = [C.POINTER(AttnConfig), C.POINTER(vp)]
    lib.f2k_attn_destroy.restype = None
    lib.f2k_attn_destroy.argtypes = [vp]
    lib.f2k_attn_last_error.restype = C.c_char_p
    lib.f2k_attn_last_error.argtypes = [vp]
    lib.f2k_attn_workspace_bytes.restype = sz
    lib.f2k_attn_workspace_bytes.argtypes = [vp]
    lib.f2k_attn_fused_workspace_bytes.restype = sz
    lib.f2k_attn_fused_workspace_bytes.argtypes = [vp]
    lib.f2k_attn_forward.restype = i
    lib.f2k_attn_forward.argtypes = [vp] * 10 + [sz, vp]
    lib.f2k_attn_forward_fused.restype = i
    lib.f2k_attn_forward_fused.argtypes = [vp] * 15 + [f, vp, vp, vp, sz, vp]
    lib.f2k_attn_forward_fused_strided.restype = i
    lib.f2k_attn_forward_fused_strided.argtypes = [vp] * 15 + [f, vp, vp, C.POINTER(AttnStrides), vp, sz, vp]
    lib.f2k_attn_forward_fused_host.restype = i
    lib.f2k_attn_forward_fused_host.argtypes = [vp] * 15 + [f, vp, vp, vp]
    lib.f2k_attn_forward_fused_noalloc.restype = i
    lib.f2k_attn_forward_fused_noalloc.argtypes = [C.POINTER(AttnConfig)] + [vp] * 14 + [f, vp, vp, vp, C.c_char_p, sz]
    lib.f2k_attn_noalloc_device_status.restype = i
    lib.f2k_attn_noalloc_device_status.argtypes = [C.POINTER(i), C.c_char_p, sz]
    lib.f2k_attn_set_wait_limits.restype = i
    lib.f2k_attn_set_wait_limits.argtypes = [vp, C.c_longlong, C.c_longlong]
    lib.f2k_seqpar_set_wait_limits.restype = i
    lib.f2k_seqpar_set_wait_limits.argtypes = [vp, C.c_longlong, C.c_longlong]
    lib.f2k_seqpar_abort.restype = i
    lib.f2k_seqpar_abort.argtypes = [vp]
    lib.f2k_hx_set_wait_limits.restype = i
    lib.f2k_hx_set_wait_limits.argtypes = [vp, C.c_longlong, C.c_longlong]
    lib.f2k_hx_abort.restype = i
    lib.f2k_hx_abort.argtypes = [vp]
    lib.f2k_attn_device_status.restype = i
    lib.f2k_attn_device_status.argtypes = [vp, C.POINTER(i)]
    lib.f2k_rmsnorm_bf16.restype = i
    lib.f2k_rmsnorm_bf16.argtypes = [vp, vp, vp, i, i, f, vp]
    lib.f2k_rope_4axis_inplace_bf16.restype = i
    lib.f2k_rope_4axis_inplace_bf16.argtypes = [vp, vp, vp, vp, i, i, i, vp]
    lib.f2k_build_rope_4axis_tables.restype = i
    lib.f2k_build_rope_4axis_tables.argtypes = [vp, i, vp, i, f, vp, vp]
    lib.f2k_seqpar_create.restype = i
    lib.f2k_seqpar_create.argtypes = [C.POINTER(SeqParConfig), C.POINTER(vp)]
    lib.f2k_seqpar_destroy.restype = None
    lib.f2k_seqpar_destroy.argtypes = [vp]
    lib.f2k_seqpar_last_error.restype = C.c_char_p
    lib.f2k_seqpar_last_error.argtypes = [vp]
    lib.f2k_seqpar_buffer.restype = i
    lib.f2k_seqpar_buffer.argtypes = [vp, C.POINTER(vp), C.POINTER(sz)]
    lib.f2k_seqpar_attach.restype = i
    lib.f2k_seqpar_attach.argtypes = [vp, C.POINTER(vp)]
    lib.f2k_seqpar_local_kv.restype = i
    lib.f2k_seqpar_local_kv.argtypes = [vp, C.POINTER(vp), C.POINTER(vp)]
    lib.f2k_seqpar_forward.restype = i
    lib.f2k_seqpar_forward.argtypes = [vp, vp, vp, i, vp, vp]
    lib.f2k_seqpar_device_status.restype = i
    lib.f2k_seqpar_device_status.argtypes = [vp, C.POINTER(i)]
    lib.f2k_hx_create.restype = i
    lib.f2k_hx_create.argtypes = [C.POINTER(SeqParConfig), C.POINTER(vp)]
    lib.f2k_hx_destroy.restype = None
    lib.f2k_hx_destroy.argtypes = [vp]
    lib.f2k_hx_last_error.restype = C.c_char_p
    lib.f2k_hx_last_error.argtypes = [vp]
    lib.f2k_hx_buffer.restype = i
    lib.f2k_hx_buffer.argtypes = [vp, C.POINTER(vp), C.POINTER(sz)]
    lib.f2k_hx_attach.restype = i
    lib.f2k_hx_attach.argtypes = [vp, C.POINTER(vp)]
    lib.f2k_hx_exchange_in.restype = i
    lib.f2k_hx_exchange_in.argtypes = [vp] * 8 + [f, vp]
    lib.f2k_hx_exchange_in_copy.restype = i
    lib.f2k_hx_exchange_in_copy.argtypes = [vp] * 8 + [f, vp]
    lib.f2k_hx_forward.restype = i
    lib.f2k_hx_forward.argtypes = [vp] * 8 + [f, vp]
    lib.f2k_hx_attend.restype = i
    lib.f2k_hx_attend.argtypes = [vp, vp]
    lib.f2k_hx_output.restype = i
    lib.f2k_hx_output.argtypes = [vp, C.POINTER(vp), vp]
    lib.f2k_hx_device_status.restype = i
    lib.f2k_hx_device_status.argtypes = [vp, C.POINTER(i)]
    lib.f2k_ipc_export.restype = i
    lib.f2k_ipc_export.argtypes = [vp, vp]
    lib.f2k_ipc_open.restype = i
    lib.f2k_ipc_open.argtypes = [vp, C.POINTER(vp)]
    lib.f2k_ipc_close.restype = i
    lib.f2k_ipc_close.argtypes = [vp]
    lib.f2k_qk_norm_rope_bf16.restype = i
    lib.f2k_qk_norm_rope_bf16.argtypes = [vp, vp, vp, vp, vp, i, i, i, f, vp]
    lib.f2k_attn_version.restype = C.c_char_p
    lib.f2k_attn_version.argtypes = []


def load(path: Path | None = None) -> C.CDLL:
    path = Path(path) if path else LIB_PATH
    if path == LIB_PATH:
        build()          # returns at once when the library is newer than every source it is built from
    if not path.exists():
        raise ImportError(f"{path} is missing and could not be built; f2k_cuda_b200 has no fallback path")
    lib = C.CDLL(str(path))
    try:
        _declare(lib)
    except AttributeError:
        # a library from an older source tree: rebuild it once and bind the fresh file
        if path != LIB_PATH:
            raise
        build(force=True)
        import shutil
        import tempfile
        fresh = Path(tempfile.mkdtemp(prefix="f2k_attn_")) / path.name   # dlopen caches by path
        shutil.copy2(path, fresh)
        lib = C.CDLL(str(fresh))
        _declare(lib)
    return lib


lib = load()
