"""Parity at the full size of every benchmark configuration, all heads, on a B200.

For each of the five configurations (1152, 4608, 4608 x batch 4, 8704 image-edit, 16896 tokens; 32
heads x 128) the fused call of this library runs beside the REFERENCE'S OWN path on the same
device buffers: its CUDA sources rebuilt unmodified for sm_100a (oracle/_ref), driven in its
blocks' order - rmsnorm_bf16 on Q and K of each stream, rope_4axis_inplace_bf16 with position =
token index, JointAttention::forward (src/backend/cuda/double_stream_block.cu:341-379,
tests/test_joint_attention.cu:72-157). Gate on the whole bf16 output: max-abs <= 2e-2 and
cosine >= 0.9999.

The second check is against fp32/double host math (the ideal oracle) on a head subset: every
query row of one head where the oracle finishes in seconds, a spread of rows (all of the first
and last tile, then every 29th) for the long shapes.

Inputs: the seeded generator of f2k_cuda_b200.inputs for the two generation shapes; for the
three large shapes Q, K, V are drawn N(0,1) on the device from a seeded torch generator (the
host generator needs half a minute per shape), gains and positions still come from
f2k_cuda_b200.inputs - the image-edit shape puts its second image at t = 1.
"""
import ctypes as C

import numpy as np
import pytest

from tests._util import COSINE_TOL, MAX_ABS_TOL, assert_parity, dev_bf16, host_bits, host_f32

pytestmark = pytest.mark.gpu

CONFIGS = ["s1152", "s4608", "s4608_b4", "s8704_edit", "s16896"]


def _inputs(f2k, name):
    """Device tensors q_txt, k_txt, v_txt, q_img, k_img, v_img, the four gains, the four tables."""
    import torch
    from f2k_cuda_b200.inputs import WORKLOADS, make_problem, token_positions
    w = WORKLOADS[name]
    B, St, Si, H, D = w.batch, w.seq_txt, w.seq_img, w.n_heads, w.head_dim
    if name in ("s1152", "s4608"):
        p = make_problem(w)
        d = [dev_bf16(x) for x in (p.q_txt, p.k_txt, p.v_txt, p.q_img, p.k_img, p.v_img)]
        gammas, pt, pi = p.gammas, p.pos_txt, p.pos_img
    else:
        gen = torch.Generator(device="cuda").manual_seed(w.seed & 0x7FFFFFFF)
        d = [torch.randn(B, n, H, D, device="cuda", generator=gen).to(torch.bfloat16) for n in (St, St, St, Si, Si, Si)]
        gammas = make_problem(WORKLOADS["s1152"], heads=1).gammas
        pt, pi = token_positions(w)
    tabs = (*f2k.build_rope_4axis_tables((32,) * 4, pt, 2000.0), *f2k.build_rope_4axis_tables((32,) * 4, pi, 2000.0))
    return w, d, gammas, tabs


def reference_path(reflib, w, d, dg, dtab):
    """The reference's block sequence on copies of the raw tensors; returns (o_txt, o_img)."""
    import torch
    L = reflib.lib
    B, St, Si, H, D = w.batch, w.seq_txt, w.seq_img, w.n_heads, w.head_dim
    P = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
    r = [x.clone() for x in d]                  # it normalises and rotates in place
    pos_t = ((torch.arange(B * St * H, device="cuda") // H) % St).to(torch.int32)
    pos_i = ((torch.arange(B * Si * H, device="cuda") // H) % Si).to(torch.int32)
    for x, g, (c_, s_), pos, seq in ((r[0], dg[0], dtab[0:2], pos_t, St), (r[1], dg[1], dtab[0:2], pos_t, St),
                                     (r[3], dg[2], dtab[2:4], pos_i, Si), (r[4], dg[3], dtab[2:4], pos_i, Si)):
        rows = B * seq * H
        assert L.f2k_ref_rmsnorm_bf16(P(x), P(g), P(x), rows, D, 1e-6, None)
        assert L.f2k_ref_rope_4axis_inplace_bf16(P(x), P(c_), P(s_), P(pos), rows, D, seq, None)
    h = L.f2k_ref_joint_create(B, St, Si, H, D, 0.0)
    assert L.f2k_ref_joint_ok(h), L.f2k_ref_joint_last_error(h)
    nbytes = L.f2k_ref_joint_workspace_bytes(h)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    o_t, o_i = torch.empty_like(d[0]), torch.empty_like(d[3])
    assert L.f2k_ref_joint_forward(h, *map(P, r), P(o_t), P(o_i), P(ws), nbytes, None)
    torch.cuda.synchronize()
    L.f2k_ref_joint_destroy(h)
    return o_t, o_i


def device_metrics(got, ref):
    """max-abs and cosine of two bf16 device tensors, computed on the device in fp64."""
    a, b = got.double().flatten(), ref.double().flatten()
    max_abs = float((a - b).abs().max())
    cos = float((a @ b) / ((a @ a).sqrt() * (b @ b).sqrt()))
    return max_abs, cos


@pytest.mark.parametrize("name", CONFIGS)
def test_config_at_full_size(name, reflib, orc):
    import torch
    assert torch.cuda.is_available(), "these tests need a GPU"
    import f2k_cuda_b200 as f2k
    w, d, gammas, tabs = _inputs(f2k, name)
    B, St, Si, H, D = w.batch, w.seq_txt, w.seq_img, w.n_heads, w.head_dim
    dg = [dev_bf16(g) for g in gammas]
    dtab = [torch.from_numpy(t).cuda() for t in tabs]
    ja = f2k.JointAttention(f2k.JointAttention.Config(B, St, Si, H, D))
    assert ja.ok(), ja.last_error()
    ws = torch.empty(ja.fused_workspace_size_bytes(), dtype=torch.uint8, device="cuda")
    o_t, o_i = torch.full_like(d[0], float("nan")), torch.full_like(d[3], float("nan"))
    assert ja.forward_fused(*d, dg, dtab, 1e-6, o_t, o_i, ws), ja.last_error()
    assert ja.device_status() == 0
    assert bool(torch.isfinite(o_t).all()) and bool(torch.isfinite(o_i).all())

    # (1) fp32/double host math on a head subset (last batch element, two heads)
    S = St + Si
    rows = np.arange(S) if S <= 4608 else np.unique(np.concatenate([np.arange(128), np.arange(128, S - 128, 29),
                                                                    np.arange(S - 128, S)]))
    b = B - 1
    for h in (0, H - 1):
        cut = [host_bits(x[b:b + 1, :, h:h + 1]) for x in d]
        ideal = orc.joint_rows(rows, q_txt=cut[0], k_txt=cut[1], v_txt=cut[2], q_img=cut[3], k_img=cut[4],
                               v_img=cut[5], gammas=gammas, tables=tabs, eps=1e-6)
        got = np.concatenate([host_f32(o_t[b, :, h]), host_f32(o_i[b, :, h])], 0)[rows]
        assert_parity(got, ideal, f"{name} head {h} vs ideal oracle ({len(rows)} rows)")

    # (2) every head, every row against the reference's own kernels on the same buffers
    if reflib is None:
        pytest.skip("oracle/_ref/libf2k_ref.so was not built")
    r_t, r_i = reference_path(reflib, w, d, dg, dtab)
    for what, got, ref in (("txt", o_t, r_t), ("img", o_i, r_i)):
        max_abs, cos = device_metrics(got, ref)
        assert max_abs <= MAX_ABS_TOL and cos >= COSINE_TOL, \
            f"{name} {what} vs reference kernels: max_abs={max_abs:.4g} cos={cos:.6f}"
