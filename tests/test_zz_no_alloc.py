"""The allocation-free entry point against the regular fused entry point.

f2k_attn_forward_fused_noalloc serves callers that may not allocate device memory (a
real-time loop, a plug-in under a host application's no-allocation rule, a process whose
device memory is fully assigned): it takes no handle and no workspace and keeps its scratch in
a fixed 32 MiB array inside the library. Here it is called through the C ABI twice in a row,
on different inputs, and each result is compared with what f2k_attn_forward_fused (handle +
caller workspace) gives for the same inputs; the array is shared by all calls, so the second
call also shows that nothing stale from the first one leaks through. Every result is also held
against the ideal oracle, the status word is read through f2k_attn_noalloc_device_status, and
the shapes cover a module without a text stream and the largest shape the array takes (256
bytes below its size; the next larger one is refused with a message). A last test, in a
process of its own, shows when device memory is taken: by the first call on the device and
never after.

The file name sorts last on purpose: a run that stops at the first failure has then already
gone through every other test.
"""
import ctypes as C

import numpy as np
import pytest

from tests._util import assert_parity, dev_bf16, host_f32

pytestmark = pytest.mark.gpu


def _problem(seed, B, St, grid, H):
    from f2k_cuda_b200.inputs import Workload, make_problem
    w = Workload("noalloc", B, St, (grid,), n_heads=H, seed=seed)
    return w, make_problem(w)


def _run_both(f2k, w, p):
    import torch
    from f2k_cuda_b200._lib import AttnConfig, F2K_OK, lib
    tabs = (*f2k.build_rope_4axis_tables((32,) * 4, p.pos_txt, 2000.0),
            *f2k.build_rope_4axis_tables((32,) * 4, p.pos_img, 2000.0))
    d = [dev_bf16(x) for x in (p.q_txt, p.k_txt, p.v_txt, p.q_img, p.k_img, p.v_img)]
    dg = [dev_bf16(g) for g in p.gammas]
    dtab = [torch.from_numpy(t).cuda() for t in tabs]
    ptr = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731

    # the existing entry point: handle + caller-provided workspace
    ja = (f2k.JointAttention(f2k.JointAttention.Config(w.batch, w.seq_txt, w.seq_img, w.n_heads, w.head_dim))
          if w.seq_txt else f2k.Attention(f2k.Attention.Config(w.batch, w.seq_img, w.n_heads, w.head_dim)))
    assert ja.ok(), ja.last_error()
    ws = torch.empty(ja.fused_workspace_size_bytes(), dtype=torch.uint8, device="cuda")
    ref_t, ref_i = torch.full_like(d[0], float("nan")), torch.full_like(d[3], float("nan"))
    assert ja.forward_fused(*d, dg, dtab, 1e-6, ref_t, ref_i, ws), ja.last_error()
    assert ja.device_status() == 0

    # the new entry point: config by value, no handle, no workspace
    cfg = AttnConfig(w.batch, w.seq_txt, w.seq_img, w.n_heads, w.head_dim, 0.0)
    err = C.create_string_buffer(256)
    got_t, got_i = torch.full_like(d[0], float("nan")), torch.full_like(d[3], float("nan"))
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.f2k_attn_forward_fused_noalloc(C.byref(cfg), *map(ptr, d), *map(ptr, dg), *map(ptr, dtab), 1e-6,
                                            ptr(got_t), ptr(got_i), stream, err, len(err))
    assert rc == F2K_OK, err.value.decode()
    st = C.c_int(-1)
    assert lib.f2k_attn_noalloc_device_status(C.byref(st), err, len(err)) == F2K_OK, err.value.decode()
    assert st.value == 0
    return (host_f32(got_t), host_f32(got_i)), (host_f32(ref_t), host_f32(ref_i)), tabs


def _check_against_oracle(orc, w, p, tabs, got_t, got_i, what):
    kw = dict(q_txt=p.q_txt, k_txt=p.k_txt, v_txt=p.v_txt) if w.seq_txt else {}
    if w.seq * w.n_heads <= 40000:
        ideal_t, ideal_i = orc.joint_path(q_img=p.q_img, k_img=p.k_img, v_img=p.v_img, gammas=p.gammas, tables=tabs,
                                          eps=1e-6, **kw)
        if w.seq_txt:
            assert_parity(got_t, ideal_t, f"{what} txt vs ideal oracle")
        assert_parity(got_i, ideal_i, f"{what} img vs ideal oracle")
        return
    rows = np.arange(w.seq)            # larger shapes: every row of the first and the last head
    for h in (0, w.n_heads - 1):
        cut = {k: v[:, :, h:h + 1] for k, v in dict(q_img=p.q_img, k_img=p.k_img, v_img=p.v_img, **kw).items()}
        ideal = orc.joint_rows(rows, gammas=p.gammas, tables=tabs, eps=1e-6, **cut)
        got = np.concatenate([got_t[0, :, h], got_i[0, :, h]], 0) if w.seq_txt else got_i[0, :, h]
        assert_parity(got, ideal, f"{what} head {h} vs ideal oracle")


def test_noalloc_matches_fused_on_two_calls_in_a_row(orc):
    import torch
    assert torch.cuda.is_available()
    import f2k_cuda_b200 as f2k
    # first call: the 1152-token generation shape, 32 heads; second call: a smaller, ragged shape
    # with other data, reusing the same array; third: no text stream (the single-stream block's
    # call); fourth: the largest shape the array takes: 65535 head rows of Q and of K, 256 bytes
    # below the 32 MiB (15 heads also take the prologue's one-row-at-a-time path)
    for seed, B, St, grid, H in ((0xA110C, 1, 128, (32, 32), 32), (0xA110D, 2, 77, (9, 13), 4),
                                 (0xA110E, 1, 0, (20, 17), 8), (0xA110F, 1, 257, (16, 257), 15)):
        w, p = _problem(seed, B, St, grid, H)
        (got_t, got_i), (ref_t, ref_i), tabs = _run_both(f2k, w, p)
        if St:
            assert_parity(got_t, ref_t, f"noalloc txt (seed {seed:#x})")
        assert_parity(got_i, ref_i, f"noalloc img (seed {seed:#x})")
        # same kernels on the same values: not just close, identical
        assert np.array_equal(got_t, ref_t) and np.array_equal(got_i, ref_i)
        _check_against_oracle(orc, w, p, tabs, got_t, got_i, f"noalloc (seed {seed:#x})")


def test_noalloc_refuses_what_does_not_fit():
    import torch
    assert torch.cuda.is_available()
    from f2k_cuda_b200._lib import AttnConfig, F2K_ERR_INVALID, F2K_ERR_UNSUPPORTED, F2K_ERR_WORKSPACE, lib
    err = C.create_string_buffer(256)
    one = C.c_void_p(256)          # never dereferenced: every call below is refused before any launch
    args = [one] * 14

    def call(cfg):
        return lib.f2k_attn_forward_fused_noalloc(C.byref(cfg), *args, 1e-6, one, one, None, err, len(err))

    # 4608 tokens x 32 heads needs 75.5 MB of scratch: more than the 32 MiB array
    assert call(AttnConfig(1, 512, 4096, 32, 128, 0.0)) == F2K_ERR_WORKSPACE
    assert b"32 MiB" in err.value and b"f2k_attn_forward_fused" in err.value
    # 65536 head rows of Q and of K: 256 bytes more than the array holds
    assert call(AttnConfig(1, 0, 4096, 16, 128, 0.0)) == F2K_ERR_WORKSPACE
    assert b"33554688 bytes" in err.value
    assert call(AttnConfig(1, 8, 64, 4, 64, 0.0)) == F2K_ERR_UNSUPPORTED
    assert call(AttnConfig(0, 8, 64, 4, 128, 0.0)) == F2K_ERR_INVALID


def test_noalloc_takes_its_memory_in_the_first_call_and_none_after():
    """In a fresh process (fresh CUDA context): free device memory before the first call of this
    file's entry points, after it, and after a forward call and a second status read. The
    array's 32 MiB (and the kernels' code) are taken by the first call; later calls take nothing.
    The figures are printed for the record."""
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    code = r"""
import ctypes as C, json, sys
sys.path.insert(0, %r)
import torch
torch.cuda.init(); torch.cuda.set_device(0)
torch.empty(1, device="cuda")
import f2k_cuda_b200 as f2k
from f2k_cuda_b200._lib import AttnConfig, lib
B, St, Si, H = 1, 64, 256, 4
mk = lambda n: torch.randn(B, n, H, 128, device="cuda").to(torch.bfloat16)
d = [mk(St), mk(St), mk(St), mk(Si), mk(Si), mk(Si)]
g = [torch.ones(128, device="cuda", dtype=torch.bfloat16) for _ in range(4)]
t = [torch.zeros(n, 64, device="cuda") for n in (St, St, Si, Si)]
o = [torch.empty_like(d[0]), torch.empty_like(d[3])]
torch.cuda.synchronize()
free = lambda: torch.cuda.mem_get_info()[0]
err = C.create_string_buffer(256)
p = lambda x: C.c_void_p(x.data_ptr())
f0 = free()
rc1 = lib.f2k_attn_noalloc_device_status(None, err, len(err))
f1 = free()
cfg = AttnConfig(B, St, Si, H, 128, 0.0)
rc2 = lib.f2k_attn_forward_fused_noalloc(C.byref(cfg), *map(p, d), *map(p, g), *map(p, t), 1e-6, p(o[0]), p(o[1]),
                                         None, err, len(err))
st = C.c_int(-1)
rc3 = lib.f2k_attn_noalloc_device_status(C.byref(st), err, len(err))
f2 = free()
print(json.dumps({"rc": [rc1, rc2, rc3], "status": st.value, "first_call_bytes": f0 - f1, "later_bytes": f1 - f2}))
""" % str(root)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    import json
    rec = json.loads(r.stdout.strip().splitlines()[-1])
    print("allocation-free entry point, device memory:", rec)
    assert rec["rc"] == [0, 0, 0] and rec["status"] == 0
    assert rec["later_bytes"] == 0, rec
    assert rec["first_call_bytes"] >= 0, rec
