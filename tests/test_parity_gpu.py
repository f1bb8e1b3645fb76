"""Parity of the CUDA path with the oracle, through the C ABI, on a B200.

Gate: bf16 output against the ideal oracle, max-abs <= 2e-2 and cosine >= 0.9999
(tests/_util.py). Shapes: the reference's own test shapes (tests/test_attention.cu:109-114,
tests/test_joint_attention.cu:167-170) with head_dim 128, ragged lengths around the
128-token tile, the 1152-token generation shape in full, and the 4608-token shape through
size-independent properties plus a head subset against the oracle.
"""
import ctypes as C

import numpy as np
import pytest

import oracle
from tests._util import (assert_parity, dev_bf16, host_bits, host_f32, metrics, normal_bits,
                         uniform_bits)

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def f2k():
    import torch
    assert torch.cuda.is_available(), "these tests need a GPU"
    import f2k_cuda_b200
    return f2k_cuda_b200


def run_attention(f2k, q, k, v):
    import torch
    B, S, H, D = q.shape
    att = f2k.Attention(f2k.Attention.Config(B, S, H, D))
    assert att.ok(), att.last_error()
    dq, dk, dv = dev_bf16(q), dev_bf16(k), dev_bf16(v)
    do = torch.full_like(dq, float("nan"))
    assert att.forward(dq, dk, dv, do), att.last_error()
    assert att.device_status() == 0
    return host_f32(do)


def run_joint(f2k, t, im, fused=None):
    """t, im: (q, k, v) bit arrays per stream. fused = (gammas, tables) switches the prologue on."""
    import torch
    B, St, H, D = t[0].shape
    Si = im[0].shape[1]
    ja = f2k.JointAttention(f2k.JointAttention.Config(B, St, Si, H, D))
    assert ja.ok(), ja.last_error()
    dt, di = [dev_bf16(x) for x in t], [dev_bf16(x) for x in im]
    keep = [x.clone() for x in dt + di]
    o_t, o_i = torch.full_like(dt[0], float("nan")), torch.full_like(di[0], float("nan"))
    if fused is None:
        assert ja.workspace_size_bytes() == 0
        assert ja.forward(*dt, *di, o_t, o_i, None, 0), ja.last_error()
    else:
        gammas, tables = fused
        dg = [dev_bf16(g) for g in gammas]
        dtab = [torch.from_numpy(x).cuda() for x in tables]
        ws = torch.empty(ja.fused_workspace_size_bytes(), dtype=torch.uint8, device="cuda")
        assert ja.forward_fused(*dt, *di, dg, dtab, 1e-6, o_t, o_i, ws), ja.last_error()
        small = torch.empty(16, dtype=torch.uint8, device="cuda")
        assert not ja.forward_fused(*dt, *di, dg, dtab, 1e-6, o_t, o_i, small)
        assert ja.last_error() == "workspace too small"
    assert ja.device_status() == 0
    for a, b in zip(keep, dt + di):     # inputs are never modified
        assert torch.equal(a, b)
    return host_f32(o_t), host_f32(o_i)


@pytest.mark.parametrize("B,S,H", [(2, 128, 4), (1, 512, 8), (1, 1024, 4), (1, 130, 2), (1, 1, 1),
                                   (1, 127, 1), (1, 129, 3), (3, 257, 2), (1, 384, 1)])
def test_attention_reference_shapes(f2k, orc, B, S, H):
    q, k, v = (uniform_bits(0xA77E, i, (B, S, H, 128)) for i in range(3))
    got = run_attention(f2k, q, k, v)
    _, ref = orc.joint_path(q_img=q, k_img=k, v_img=v)
    assert_parity(got, ref, f"attention B{B} S{S} H{H}")


@pytest.mark.parametrize("B,St,Si,H", [(1, 64, 128, 4), (2, 32, 256, 8), (1, 64, 512, 8), (1, 1, 1, 1),
                                       (1, 100, 200, 2), (2, 128, 130, 2), (1, 129, 127, 1)])
def test_joint_reference_shapes(f2k, orc, B, St, Si, H):
    t = [uniform_bits(0xABCD, i, (B, St, H, 128)) for i in range(3)]
    im = [uniform_bits(0xABCD, 3 + i, (B, Si, H, 128)) for i in range(3)]
    o_t, o_i = run_joint(f2k, t, im)
    r_t, r_i = orc.joint_path(q_txt=t[0], k_txt=t[1], v_txt=t[2], q_img=im[0], k_img=im[1], v_img=im[2])
    assert_parity(o_t, r_t, f"joint txt B{B} {St}+{Si} H{H}")
    assert_parity(o_i, r_i, f"joint img B{B} {St}+{Si} H{H}")


def test_large_scores_and_moving_maximum(f2k, orc):
    """Scores that grow along the key axis force the running maximum (and the lazy rescale
    of the accumulator) to move on every tile; N(0,1)*4 inputs give |scale*q.k| up to ~50."""
    B, S, H = 1, 640, 2
    q = normal_bits(5, 0, (B, S, H, 128))
    kf = np.random.default_rng(5).standard_normal((B, S, H, 128)).astype(np.float32)
    ramp = np.linspace(0.2, 4.0, S, dtype=np.float32)[None, :, None, None]
    from f2k_cuda_b200.inputs import from_bf16_bits, to_bf16_bits
    k = to_bf16_bits(from_bf16_bits(q) * ramp * 0.5 + kf * 0.5)
    v = normal_bits(5, 2, (B, S, H, 128))
    got = run_attention(f2k, q, k, v)
    _, ref = orc.joint_path(q_img=q, k_img=k, v_img=v)
    assert_parity(got, ref, "moving maximum", max_abs_tol=3e-2)


def test_generation_shape_1152_full_path(f2k, orc):
    """128 text + 32x32 image tokens, 32 heads, QK-norm + 4-axis RoPE + attention, every head."""
    from f2k_cuda_b200.inputs import WORKLOADS, make_problem
    w = WORKLOADS["s1152"]
    p = make_problem(w)
    tabs = (*f2k.build_rope_4axis_tables((32,) * 4, p.pos_txt, 2000.0),
            *f2k.build_rope_4axis_tables((32,) * 4, p.pos_img, 2000.0))
    o_t, o_i = run_joint(f2k, (p.q_txt, p.k_txt, p.v_txt), (p.q_img, p.k_img, p.v_img), fused=(p.gammas, tabs))
    r_t, r_i = orc.joint_path(q_txt=p.q_txt, k_txt=p.k_txt, v_txt=p.v_txt, q_img=p.q_img, k_img=p.k_img,
                              v_img=p.v_img, gammas=p.gammas, tables=tabs, eps=1e-6)
    assert_parity(o_t, r_t, "s1152 txt")
    assert_parity(o_i, r_i, "s1152 img")


def test_fused_prologue_equals_separate_kernels(f2k, orc):
    """forward_fused against rmsnorm_bf16 -> rope_4axis_inplace_bf16 -> forward (the reference's
    call sequence) on the same inputs: the only difference is one bf16 rounding fewer."""
    import torch
    B, St, Si, H, D = 2, 96, 160, 4, 128
    t = [normal_bits(31, i, (B, St, H, D)) for i in range(3)]
    im = [normal_bits(31, 3 + i, (B, Si, H, D)) for i in range(3)]
    from f2k_cuda_b200.inputs import to_bf16_bits, uniform01
    gam = [to_bf16_bits((1 + 0.2 * (uniform01(31, 50 + i, D) - 0.5)).astype(np.float32)) for i in range(4)]
    pt = np.zeros((St, 4), np.int32); pt[:, 3] = np.arange(St)
    pi = np.zeros((Si, 4), np.int32); pi[:, 1] = np.arange(Si) // 16; pi[:, 2] = np.arange(Si) % 16
    tabs = (*f2k.build_rope_4axis_tables((32,) * 4, pt, 2000.0), *f2k.build_rope_4axis_tables((32,) * 4, pi, 2000.0))
    f_t, f_i = run_joint(f2k, t, im, fused=(gam, tabs))

    def prep(x, g, cos, sin, seq):
        dx, dg = dev_bf16(x), dev_bf16(g)
        rows = B * seq * H
        assert f2k.rmsnorm_bf16(dx, dg, dx, rows, D, 1e-6)
        pos = ((torch.arange(rows, device="cuda") // H) % seq).to(torch.int32)
        assert f2k.rope_4axis_inplace_bf16(dx, torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda(),
                                           pos, rows, D, seq)
        torch.cuda.synchronize()
        return host_bits(dx)

    qt, kt = prep(t[0], gam[0], tabs[0], tabs[1], St), prep(t[1], gam[1], tabs[0], tabs[1], St)
    qi, ki = prep(im[0], gam[2], tabs[2], tabs[3], Si), prep(im[1], gam[3], tabs[2], tabs[3], Si)
    s_t, s_i = run_joint(f2k, (qt, kt, t[2]), (qi, ki, im[2]))
    assert_parity(f_t, s_t, "fused vs separate txt")
    assert_parity(f_i, s_i, "fused vs separate img")
    # and the separate kernels reproduce the oracle's reference-rounding statement of them
    ref_q = orc.rope_bf16(orc.rmsnorm_bf16(im[0].reshape(-1, D), gam[2], 1e-6), tabs[2], tabs[3],
                          ((np.arange(B * Si * H) // H) % Si).astype(np.int32), Si).reshape(qi.shape)
    assert np.mean(ref_q != qi) < 0.01
    from f2k_cuda_b200.inputs import from_bf16_bits
    assert np.max(np.abs(from_bf16_bits(ref_q) - from_bf16_bits(qi))) < 0.04


@pytest.mark.parametrize("rows,dim", [(1, 128), (36864, 128), (8, 1024), (32, 3072), (5, 8)])
def test_rmsnorm_kernel(f2k, orc, rows, dim):
    import torch
    from f2k_cuda_b200.inputs import from_bf16_bits, to_bf16_bits, uniform01
    x = to_bf16_bits((4 * uniform01(0xC0FFEE, 0, rows * dim) - 2).astype(np.float32)).reshape(rows, dim)
    g = to_bf16_bits((uniform01(0xC0FFEE, 1, dim) + 0.5).astype(np.float32))
    dx, dg = dev_bf16(x), dev_bf16(g)
    dy = torch.empty_like(dx)
    assert f2k.rmsnorm_bf16(dx, dg, dy, rows, dim, 1e-6)
    torch.cuda.synchronize()
    ideal = orc.rmsnorm_ideal(x, g, 1e-6)
    got = host_f32(dy)
    # the reference's thresholds (tests/test_rmsnorm.cu:87-90) ...
    assert np.max(np.abs(got - ideal)) < 0.05 and np.mean(np.abs(got - ideal)) < 0.005
    # ... and agreement with the reference-rounding statement up to summation order
    assert np.mean(host_bits(dy) != orc.rmsnorm_bf16(x, g, 1e-6)) < 0.01
    assert f2k.rmsnorm_bf16(dx, dg, dx, rows, dim, 1e-6)       # in place, as the blocks call it
    torch.cuda.synchronize()
    assert torch.equal(dx, dy)


@pytest.mark.parametrize("seq,H,D", [(256, 32, 128), (16, 4, 16), (64, 2, 512)])
def test_rope_kernel(f2k, orc, seq, H, D):
    import torch
    pos = np.zeros((seq, 4), np.int32)
    s = np.arange(seq); W = int(np.sqrt(seq))
    pos[:, 0], pos[:, 1], pos[:, 2], pos[:, 3] = s % 7, s // W, s % W, s
    cos, sin = f2k.build_rope_4axis_tables((D // 4,) * 4, pos, 2000.0 if D == 128 else 100.0)
    x = normal_bits(0xCAFE, 0, (seq * H, D))
    pos_ids = (np.arange(seq * H) // H).astype(np.int32)
    pos_ids[0], pos_ids[-1] = -3, seq + 5                       # clamped like the reference does
    dx = dev_bf16(x)
    assert f2k.rope_4axis_inplace_bf16(dx, torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda(),
                                       torch.from_numpy(pos_ids).cuda(), seq * H, D, seq)
    torch.cuda.synchronize()
    # bit for bit: kernel and oracle spell out the same fused multiply-adds
    assert np.array_equal(host_bits(dx), orc.rope_bf16(x, cos, sin, pos_ids, seq))


def test_against_the_reference_kernels_on_this_gpu(f2k, reflib):
    """The reference's own CUDA path, rebuilt for sm_100a, on identical device buffers."""
    if reflib is None:
        pytest.skip("oracle/_ref/libf2k_ref.so was not built")
    import torch
    B, St, Si, H, D = 1, 128, 1024, 8, 128
    t = [normal_bits(77, i, (B, St, H, D)) for i in range(3)]
    im = [normal_bits(77, 3 + i, (B, Si, H, D)) for i in range(3)]
    o_t, o_i = run_joint(f2k, t, im)
    L = reflib.lib
    p = lambda x: C.c_void_p(x.data_ptr())  # noqa: E731
    dt, di = [dev_bf16(x) for x in t], [dev_bf16(x) for x in im]
    r_t, r_i = torch.empty_like(dt[0]), torch.empty_like(di[0])
    h = L.f2k_ref_joint_create(B, St, Si, H, D, 0.0)
    assert L.f2k_ref_joint_ok(h)
    nbytes = L.f2k_ref_joint_workspace_bytes(h)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    assert L.f2k_ref_joint_forward(h, *map(p, dt), *map(p, di), p(r_t), p(r_i), p(ws), nbytes, None)
    torch.cuda.synchronize()
    L.f2k_ref_joint_destroy(h)
    assert_parity(o_t, host_f32(r_t), "vs reference kernel txt")
    assert_parity(o_i, host_f32(r_i), "vs reference kernel img")


def test_norm_and_rope_kernels_match_the_reference_kernels_bit_for_bit(f2k, reflib):
    """rmsnorm_bf16 and rope_4axis_inplace_bf16 keep the reference's rounding points, so on the
    same GPU they should reproduce the reference kernels' bits (1M elements each)."""
    if reflib is None:
        pytest.skip("oracle/_ref/libf2k_ref.so was not built")
    import torch
    L = reflib.lib
    p = lambda x: C.c_void_p(x.data_ptr())  # noqa: E731
    seq, H, D = 256, 32, 128
    rows = seq * H
    x = normal_bits(0xBEEF, 0, (rows, D))
    from f2k_cuda_b200.inputs import to_bf16_bits, uniform01
    g = to_bf16_bits((uniform01(0xBEEF, 1, D) + 0.5).astype(np.float32))
    mine, ref = dev_bf16(x), dev_bf16(x)
    dg = dev_bf16(g)
    assert f2k.rmsnorm_bf16(mine, dg, mine, rows, D, 1e-6)
    assert L.f2k_ref_rmsnorm_bf16(p(ref), p(dg), p(ref), rows, D, 1e-6, None)
    torch.cuda.synchronize()
    # the reference reduces the sum of squares in another order: the same up to the last bit
    assert (mine != ref).float().mean().item() < 2e-3
    pos = np.zeros((seq, 4), np.int32)
    s_ = np.arange(seq)
    pos[:, 0], pos[:, 1], pos[:, 2], pos[:, 3] = s_ % 7, s_ // 16, s_ % 16, s_
    cos, sin = f2k.build_rope_4axis_tables((32,) * 4, pos, 2000.0)
    dc, ds = torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda()
    pos_ids = ((torch.arange(rows, device="cuda") // H) % seq).to(torch.int32)
    ref.copy_(mine)
    assert f2k.rope_4axis_inplace_bf16(mine, dc, ds, pos_ids, rows, D, seq)
    assert L.f2k_ref_rope_4axis_inplace_bf16(p(ref), p(dc), p(ds), p(pos_ids), rows, D, seq, None)
    torch.cuda.synchronize()
    assert torch.equal(mine, ref)


# ---------------------------------------------------------------- full-size properties (S = 4608)
@pytest.fixture(scope="module")
def big(f2k):
    from f2k_cuda_b200.inputs import WORKLOADS, make_problem
    w = WORKLOADS["s4608"]
    p = make_problem(w)
    tabs = (*f2k.build_rope_4axis_tables((32,) * 4, p.pos_txt, 2000.0),
            *f2k.build_rope_4axis_tables((32,) * 4, p.pos_img, 2000.0))
    return w, p, tabs


def test_4608_head_subset_against_oracle(f2k, orc, big):
    w, p, tabs = big
    o_t, o_i = run_joint(f2k, (p.q_txt, p.k_txt, p.v_txt), (p.q_img, p.k_img, p.v_img), fused=(p.gammas, tabs))
    heads = (30, 32)     # the oracle needs ~20 s per head at this length
    r_t, r_i = orc.joint_path(q_txt=p.q_txt, k_txt=p.k_txt, v_txt=p.v_txt, q_img=p.q_img, k_img=p.k_img,
                              v_img=p.v_img, gammas=p.gammas, tables=tabs, eps=1e-6, heads=heads)
    assert_parity(o_t[:, :, 30:32], r_t[:, :, 30:32], "s4608 txt heads 30-31")
    assert_parity(o_i[:, :, 30:32], r_i[:, :, 30:32], "s4608 img heads 30-31")


def test_4608_properties(f2k, big):
    """No oracle needed: (1) constant V rows come back unchanged (softmax rows sum to 1);
    (2) attention is linear in V; (3) permuting the keys (K and V rows together) changes
    nothing; (4) two runs are bitwise identical."""
    import torch
    from f2k_cuda_b200.inputs import from_bf16_bits, to_bf16_bits
    w, p, tabs = big
    t, im = (p.q_txt, p.k_txt, p.v_txt), (p.q_img, p.k_img, p.v_img)
    base_t, base_i = run_joint(f2k, t, im)
    again_t, again_i = run_joint(f2k, t, im)
    assert np.array_equal(base_t, again_t) and np.array_equal(base_i, again_i)
    # (1)
    c = normal_bits(99, 0, (1, 1, w.n_heads, 128))
    vt, vi = np.broadcast_to(c, p.v_txt.shape).copy(), np.broadcast_to(c, p.v_img.shape).copy()
    o_t, o_i = run_joint(f2k, (p.q_txt, p.k_txt, vt), (p.q_img, p.k_img, vi))
    cf = from_bf16_bits(c)
    assert np.max(np.abs(o_t - cf)) < 2e-2 and np.max(np.abs(o_i - cf)) < 2e-2
    # (2) V2 = 2 V is exact in bf16, so O must double up to one rounding
    v2t, v2i = to_bf16_bits(2 * from_bf16_bits(p.v_txt)), to_bf16_bits(2 * from_bf16_bits(p.v_img))
    d_t, d_i = run_joint(f2k, (p.q_txt, p.k_txt, v2t), (p.q_img, p.k_img, v2i))
    assert np.array_equal(d_t, 2 * base_t) and np.array_equal(d_i, 2 * base_i)
    # (3)
    perm = np.random.default_rng(1).permutation(w.seq_img)
    k2, v2 = p.k_img[:, perm].copy(), p.v_img[:, perm].copy()
    q_t, q_i = run_joint(f2k, t, (p.q_img, k2, v2))
    assert_parity(q_t, base_t, "key permutation txt", max_abs_tol=1e-2, cos_tol=0.99999)
    assert_parity(q_i, base_i, "key permutation img", max_abs_tol=1e-2, cos_tol=0.99999)


# (batch, heads, pipeline): None = the library's choice. Batch 1 and large enough: chunks of query
# rows; "heads": groups of heads (4 groups of 2, 2 groups of 3); small problems: one pass.
@pytest.mark.parametrize("batch,heads,mode", [(1, 4, None), (1, 8, None), (1, 4, "rows"), (1, 8, "heads"),
                                              (1, 6, "heads"), (2, 8, None)])
def test_host_buffer_entry_point(f2k, orc, monkeypatch, batch, heads, mode):
    import torch
    from f2k_cuda_b200.inputs import Workload, make_problem
    if mode:
        monkeypatch.setenv("F2K_HOST_PIPELINE", mode)
    else:
        monkeypatch.delenv("F2K_HOST_PIPELINE", raising=False)
    w = Workload("host", batch, 128, ((32, 32),), seed=0x4057)
    p = make_problem(w, heads=heads)
    tabs = (*f2k.build_rope_4axis_tables((32,) * 4, p.pos_txt, 2000.0),
            *f2k.build_rope_4axis_tables((32,) * 4, p.pos_img, 2000.0))
    ja = f2k.JointAttention(f2k.JointAttention.Config(w.batch, w.seq_txt, w.seq_img, heads, 128))
    assert ja.ok(), ja.last_error()
    pin = lambda b: torch.from_numpy(b.view(np.int16)).view(torch.bfloat16).pin_memory()  # noqa: E731
    hin = [pin(x) for x in (p.q_txt, p.k_txt, p.v_txt, p.q_img, p.k_img, p.v_img)]
    ho_t, ho_i = torch.empty_like(hin[0]).pin_memory(), torch.empty_like(hin[3]).pin_memory()
    dg = [dev_bf16(g) for g in p.gammas]
    dtab = [torch.from_numpy(x).cuda() for x in tabs]
    for _ in range(2):       # second call reuses the staging buffers
        ho_t.fill_(float("nan")); ho_i.fill_(float("nan"))
        assert ja.forward_fused_host(*hin, dg, dtab, 1e-6, ho_t, ho_i), ja.last_error()
        torch.cuda.synchronize()
    assert ja.device_status() == 0
    d_t, d_i = run_joint(f2k, (p.q_txt, p.k_txt, p.v_txt), (p.q_img, p.k_img, p.v_img), fused=(p.gammas, tabs))
    assert np.array_equal(host_f32(ho_t), d_t) and np.array_equal(host_f32(ho_i), d_i)


@pytest.mark.parametrize("batch,seq_txt,heads", [(1, 0, 8), (2, 64, 4)])
def test_strided_rows_read_the_projection_output_in_place(f2k, orc, batch, seq_txt, heads):
    """Q, K, V as column slices of one wide projection buffer (the reference's fused QKV+MLP
    output, which it first splits) and O as a column slice of the [attn | mlp] buffer: inside the
    gate against the ideal oracle, same bits as the dense call on contiguous copies, and nothing
    outside the O columns is written."""
    import torch
    from f2k_cuda_b200.inputs import Workload, make_problem
    w = Workload("strided", batch, seq_txt, ((16, 24),), seed=0x57D1)
    p = make_problem(w, heads=heads)
    hd = heads * 128
    wide, out_w = 3 * hd + 520, hd + 264            # row widths, multiples of 8
    tabs = (*f2k.build_rope_4axis_tables((32,) * 4, p.pos_txt, 2000.0),
            *f2k.build_rope_4axis_tables((32,) * 4, p.pos_img, 2000.0))
    dg = [dev_bf16(g) for g in p.gammas]
    dtab = [torch.from_numpy(x).cuda() for x in tabs]
    ja = (f2k.JointAttention(f2k.JointAttention.Config(batch, seq_txt, w.seq_img, heads, 128)) if seq_txt
          else f2k.Attention(f2k.Attention.Config(batch, w.seq_img, heads, 128)))
    assert ja.ok(), ja.last_error()
    ws = torch.empty(ja.fused_workspace_size_bytes(), dtype=torch.uint8, device="cuda")

    def stream_views(q, k, v):
        S = q.shape[1]
        proj = torch.full((batch * S, wide), 7.0, dtype=torch.bfloat16, device="cuda")
        out = torch.full((batch * S, out_w), -3.0, dtype=torch.bfloat16, device="cuda")
        views = []
        for i, x in enumerate((q, k, v)):
            proj[:, i * hd:(i + 1) * hd] = dev_bf16(x).reshape(batch * S, hd)
            views.append(proj[:, i * hd:(i + 1) * hd].unflatten(0, (batch, S)).unflatten(2, (heads, 128)))
        o = out[:, 8:8 + hd].unflatten(0, (batch, S)).unflatten(2, (heads, 128))
        return views, o, out

    (vi, o_i, out_i) = stream_views(p.q_img, p.k_img, p.v_img)
    if seq_txt:
        (vt, o_t, out_t) = stream_views(p.q_txt, p.k_txt, p.v_txt)
    else:
        vt, o_t, out_t = [None] * 3, None, None
    g = dg if seq_txt else [None, None, dg[2], dg[3]]
    t = dtab if seq_txt else [None, None, dtab[2], dtab[3]]
    assert ja.forward_fused_strided(*vt, *vi, g, t, 1e-6, o_t, o_i, ws), ja.last_error()
    torch.cuda.synchronize()
    assert ja.device_status() == 0
    # dense call on contiguous copies
    di = [dev_bf16(x) for x in (p.q_img, p.k_img, p.v_img)]
    dt = [dev_bf16(x) for x in (p.q_txt, p.k_txt, p.v_txt)] if seq_txt else [None] * 3
    r_i = torch.empty_like(di[0])
    r_t = torch.empty_like(dt[0]) if seq_txt else None
    assert ja.forward_fused(*dt, *di, g, t, 1e-6, r_t, r_i, ws), ja.last_error()
    torch.cuda.synchronize()
    kw = dict(q_txt=p.q_txt, k_txt=p.k_txt, v_txt=p.v_txt) if seq_txt else {}
    ideal_t, ideal_i = orc.joint_path(q_img=p.q_img, k_img=p.k_img, v_img=p.v_img, gammas=p.gammas, tables=tabs,
                                      eps=1e-6, **kw)
    assert_parity(host_f32(o_i.contiguous()), ideal_i, "strided rows img vs ideal oracle")
    if seq_txt:
        assert_parity(host_f32(o_t.contiguous()), ideal_t, "strided rows txt vs ideal oracle")
    assert torch.equal(o_i, r_i)
    assert bool((out_i[:, :8] == -3.0).all()) and bool((out_i[:, 8 + hd:] == -3.0).all())
    if seq_txt:
        assert torch.equal(o_t, r_t)
        assert bool((out_t[:, :8] == -3.0).all()) and bool((out_t[:, 8 + hd:] == -3.0).all())
    # refusals: a stride that is not a multiple of 8, or smaller than a dense row
    import ctypes as C
    from f2k_cuda_b200 import _lib
    bad = _lib.AttnStrides(q_img=hd + 4)
    rc = _lib.lib.f2k_attn_forward_fused_strided(
        ja._h, *[None if x is None else C.c_void_p(x.data_ptr()) for x in (*dt, *di)],
        *[None if x is None else C.c_void_p(x.data_ptr()) for x in (*g, *t)], 1e-6,
        None if r_t is None else C.c_void_p(r_t.data_ptr()), C.c_void_p(r_i.data_ptr()), C.byref(bad),
        C.c_void_p(ws.data_ptr()), ws.numel(), None)
    assert rc == _lib.F2K_ERR_INVALID and "stride" in ja.last_error()
