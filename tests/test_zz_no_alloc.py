"""The allocation-free entry point against the regular fused entry point.

f2k_attn_forward_fused_noalloc serves callers that may not allocate device memory (a
real-time loop, a plug-in under a host application's no-allocation rule, a process whose
device memory is fully assigned): it takes no handle and no workspace and keeps its scratch in
a fixed 32 MiB array inside the library. Here it is called through the C ABI twice in a row,
on different inputs, and each result is compared with what f2k_attn_forward_fused (handle +
caller workspace) gives for the same inputs; the array is shared by all calls, so the second
call also shows that nothing stale from the first one leaks through. Shapes beyond the array
must be refused with a message.

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
    ja = f2k.JointAttention(f2k.JointAttention.Config(w.batch, w.seq_txt, w.seq_img, w.n_heads, w.head_dim))
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
    torch.cuda.synchronize()
    return (host_f32(got_t), host_f32(got_i)), (host_f32(ref_t), host_f32(ref_i))


def test_noalloc_matches_fused_on_two_calls_in_a_row():
    import torch
    assert torch.cuda.is_available()
    import f2k_cuda_b200 as f2k
    # first call: the largest generation shape that fits the built-in array (1152 tokens, 32 heads)
    # second call: a smaller, ragged shape with other data, reusing the same array
    for seed, B, St, grid, H in ((0xA110C, 1, 128, (32, 32), 32), (0xA110D, 2, 77, (9, 13), 4)):
        w, p = _problem(seed, B, St, grid, H)
        (got_t, got_i), (ref_t, ref_i) = _run_both(f2k, w, p)
        assert_parity(got_t, ref_t, f"noalloc txt (seed {seed:#x})")
        assert_parity(got_i, ref_i, f"noalloc img (seed {seed:#x})")
        # same kernels on the same values: not just close, identical
        assert np.array_equal(got_t, ref_t) and np.array_equal(got_i, ref_i)


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
    assert call(AttnConfig(1, 8, 64, 4, 64, 0.0)) == F2K_ERR_UNSUPPORTED
    assert call(AttnConfig(0, 8, 64, 4, 128, 0.0)) == F2K_ERR_INVALID
