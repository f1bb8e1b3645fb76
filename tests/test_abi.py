"""The C ABI without a GPU: the library loads, exports what the header declares, validates
its arguments like the reference does, and the C++ call surface compiles."""
import ctypes as C
import re
import subprocess
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "f2k_attn.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(f2k_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    syms = declared_symbols()
    for s in ("f2k_attn_create", "f2k_attn_destroy", "f2k_attn_forward", "f2k_attn_forward_fused",
              "f2k_attn_last_error", "f2k_attn_workspace_bytes", "f2k_rmsnorm_bf16",
              "f2k_rope_4axis_inplace_bf16", "f2k_build_rope_4axis_tables"):
        assert s in syms


def test_library_exports_every_declared_symbol():
    from f2k_cuda_b200.build import build
    lib = C.CDLL(str(build()))
    for s in declared_symbols():
        assert hasattr(lib, s), f"libf2k_attn.so does not export {s}"


def test_library_is_sm100a_only_and_self_contained():
    from f2k_cuda_b200.build import LIB_PATH, build
    build()
    needed = subprocess.run(["ldd", str(LIB_PATH)], capture_output=True, text=True).stdout
    assert "libcuda.so" not in needed      # driver entry points are fetched at run time
    assert "libtorch" not in needed and "libpython" not in needed


def test_create_refuses_bad_shapes_with_reference_wording():
    import f2k_cuda_b200 as f
    a = f.Attention(f.Attention.Config(batch=0, seq=64, n_heads=4, head_dim=128))
    assert not a.ok() and a.last_error() == "Attention: zero/negative dim"
    j = f.JointAttention(f.JointAttention.Config(batch=1, seq_txt=0, seq_img=64, n_heads=4, head_dim=128))
    assert not j.ok() and j.last_error() == "JointAttention: zero/negative dim"
    j = f.JointAttention(f.JointAttention.Config(batch=1, seq_txt=8, seq_img=64, n_heads=4, head_dim=-1))
    assert not j.ok() and j.last_error() == "JointAttention: zero/negative dim"
    # documented deviation: only head_dim 128 exists, and the refusal says why
    a = f.Attention(f.Attention.Config(batch=1, seq=64, n_heads=1, head_dim=512))
    assert not a.ok() and "head_dim must be 128" in a.last_error()
    # a failed module refuses to run and keeps its message
    assert a.forward(None, None, None, None, stream=0) is False
    assert "head_dim must be 128" in a.last_error()


def test_kernel_wrappers_refuse_like_the_reference():
    from f2k_cuda_b200._lib import F2K_ERR_INVALID, lib
    one = C.c_void_p(16)
    # rmsnorm_bf16: rows/dim <= 0, dim % 8 != 0 (kernels/rmsnorm.cu:76-77)
    assert lib.f2k_rmsnorm_bf16(one, one, one, 0, 128, 1e-6, None) == F2K_ERR_INVALID
    assert lib.f2k_rmsnorm_bf16(one, one, one, 4, 0, 1e-6, None) == F2K_ERR_INVALID
    assert lib.f2k_rmsnorm_bf16(one, one, one, 4, 132, 1e-6, None) == F2K_ERR_INVALID
    # rope: odd or > 512 head_dim, rows <= 0 (kernels/rope_4axis.cu:48-49)
    assert lib.f2k_rope_4axis_inplace_bf16(one, one, one, one, 4, 127, 8, None) == F2K_ERR_INVALID
    assert lib.f2k_rope_4axis_inplace_bf16(one, one, one, one, 4, 1024, 8, None) == F2K_ERR_INVALID
    assert lib.f2k_rope_4axis_inplace_bf16(one, one, one, one, 0, 128, 8, None) == F2K_ERR_INVALID


def test_misaligned_pointers_are_refused_on_the_host():
    """The kernels use 16-byte loads and stores, so a pointer that is not 16-byte aligned would be
    a misaligned-address fault on the GPU. Every entry point that takes no handle refuses it before
    it touches CUDA at all (so this runs without a GPU); the handle-based ones are covered by the
    GPU tests. Nothing is launched by any call here."""
    from f2k_cuda_b200._lib import AttnConfig, F2K_ERR_INVALID, lib
    ok, odd, four = C.c_void_p(256), C.c_void_p(258), C.c_void_p(260)
    for bad in range(3):     # x, gamma, y
        args = [ok, ok, ok]
        args[bad] = odd
        assert lib.f2k_rmsnorm_bf16(*args, 4, 128, 1e-6, None) == F2K_ERR_INVALID
    for bad in range(3):     # x, cos, sin at head_dim 128
        args = [ok, ok, ok]
        args[bad] = four
        assert lib.f2k_rope_4axis_inplace_bf16(*args, ok, 4, 128, 8, None) == F2K_ERR_INVALID
    # other head dims read x four bytes at a time and the tables one float at a time
    assert lib.f2k_rope_4axis_inplace_bf16(odd, ok, ok, ok, 4, 64, 8, None) == F2K_ERR_INVALID
    assert lib.f2k_rope_4axis_inplace_bf16(ok, odd, ok, ok, 4, 64, 8, None) == F2K_ERR_INVALID
    assert lib.f2k_rope_4axis_inplace_bf16(ok, ok, ok, odd, 4, 64, 8, None) == F2K_ERR_INVALID
    for bad in range(5):     # x, y, gamma, cos, sin
        args = [ok] * 5
        args[bad] = odd
        assert lib.f2k_qk_norm_rope_bf16(*args, 1, 8, 4, 1e-6, None) == F2K_ERR_INVALID
    err = C.create_string_buffer(256)
    cfg = AttnConfig(1, 8, 64, 4, 128, 0.0)
    for bad in range(16):    # q, k, v per stream, four gains, four tables, two outputs
        args = [ok] * 16
        args[bad] = odd
        rc = lib.f2k_attn_forward_fused_noalloc(C.byref(cfg), *args[:14], 1e-6, args[14], args[15], None, err, len(err))
        assert rc == F2K_ERR_INVALID and b"16-byte aligned" in err.value, (bad, err.value)


def test_table_builder_matches_oracle_and_reference_golden(orc):
    import f2k_cuda_b200 as f
    g = np.load(ROOT / "tests" / "golden" / "rope_tables.npz")
    for tag in ("small", "flux_img", "flux_txt", "edit_img"):
        cos, sin = f.build_rope_4axis_tables(g[f"{tag}_axes"], g[f"{tag}_pos"], float(g[f"{tag}_theta"]))
        assert np.array_equal(cos, g[f"{tag}_cos"]) and np.array_equal(sin, g[f"{tag}_sin"]), tag
    from f2k_cuda_b200.inputs import WORKLOADS, token_positions
    pt, pi = token_positions(WORKLOADS["s8704_edit"])
    assert pi[:4096, 0].max() == 0 and pi[4096:, 0].min() == 1 and pi.shape == (8192, 4)
    c1, s1 = f.build_rope_4axis_tables((32,) * 4, pi, 2000.0)
    c2, s2 = orc.build_rope_tables((32,) * 4, pi, 2000.0)
    assert np.array_equal(c1, c2) and np.array_equal(s1, s2)


def test_cpp_call_surface_compiles_against_compat_headers(tmp_path):
    """A translation unit written against the reference's headers (same include paths, same
    class and function names) must compile against ours."""
    src = tmp_path / "user.cpp"
    src.write_text(r'''
#include "backend/cuda/attention.h"
#include "backend/cuda/joint_attention.h"
#include "backend/cuda/kernels/rmsnorm.h"
#include "backend/cuda/kernels/rope_4axis.h"
#include <memory>
#include <vector>
int main() {
    f2k::cuda::Attention::Config ac{}; ac.batch = 1; ac.seq = 64; ac.n_heads = 4; ac.head_dim = 128;
    f2k::cuda::Attention att(ac);
    f2k::cuda::JointAttention::Config jc{}; jc.batch = 1; jc.seq_txt = 8; jc.seq_img = 64; jc.n_heads = 4; jc.head_dim = 128;
    auto ja = std::make_unique<f2k::cuda::JointAttention>(jc);
    size_t ws = ja->workspace_size_bytes();
    bool ok = att.ok() && ja->ok();
    ok &= att.forward(nullptr, nullptr, nullptr, nullptr);
    ok &= ja->forward(nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, ws);
    ok &= f2k::cuda::rmsnorm_bf16(nullptr, nullptr, nullptr, 4, 128, 1e-6f);
    ok &= f2k::cuda::rope_4axis_inplace_bf16(nullptr, nullptr, nullptr, nullptr, 4, 128, 8);
    std::vector<float> c, s;
    f2k::cuda::build_rope_4axis_tables({32, 32, 32, 32}, {{0, 1, 2, 3}, {0, 0, 0, 1}}, 2000.0f, c, s);
    const char* e = att.last_error(); (void)e;
    return (ok || c.size() == 128) ? 0 : 1;
}
''')
    from f2k_cuda_b200.build import LIB_PATH, build
    build()
    exe = tmp_path / "user"
    cmd = ["/usr/bin/g++", "-std=c++17", "-I", str(ROOT / "f2k_cuda_b200/csrc/compat"), str(src), "-o", str(exe),
           str(LIB_PATH), f"-Wl,-rpath,{LIB_PATH.parent}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    # runs without a GPU too: every call fails cleanly (no device), the host table builder works
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
