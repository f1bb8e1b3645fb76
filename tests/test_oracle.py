"""The oracle against independent statements of the same math and against the reference.

No GPU needed: numpy restatements at tiny sizes, closed-form properties, the reference's
own host-side table builder (golden vectors generated from it), and the outputs of the
reference's CUDA kernels recorded on a B200 (tests/golden/, see make_golden.py there).
"""
from pathlib import Path

import numpy as np
import pytest

import oracle
from f2k_cuda_b200.inputs import from_bf16_bits, to_bf16_bits
from tests._util import metrics, normal_bits, uniform_bits

GOLDEN = Path(__file__).resolve().parent / "golden"


def np_attention(q, k, v, scale):
    """float64 numpy softmax attention on [S, D] arrays."""
    s = (q @ k.T) * scale
    s = s - s.max(axis=1, keepdims=True)
    p = np.exp(s)
    return (p @ v) / p.sum(axis=1, keepdims=True)


def test_bf16_round_trip_and_rounding():
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.140625, 0.0], np.float32)
    b = oracle.f32_to_bf16(x)
    assert np.array_equal(b, to_bf16_bits(x))
    # 1.00390625 = 1 + 2^-8 is a tie between 1.0 and 1 + 2^-7: goes to even (1.0)
    assert oracle.bf16_to_f32(b)[1] == 1.0
    # 1.01171875 = 1 + 3*2^-8 is a tie between 1+2^-7 (odd) and 1+2^-6 (even)
    assert oracle.bf16_to_f32(b)[2] == 1.015625
    assert np.array_equal(oracle.bf16_to_f32(b), from_bf16_bits(b))


@pytest.mark.parametrize("B,S,H,D", [(1, 64, 1, 64), (2, 128, 4, 128), (1, 130, 2, 128)])
def test_attention_matches_numpy(orc, B, S, H, D):
    # shapes of the reference's attention test (tests/test_attention.cu:109-114)
    q, k, v = (uniform_bits(0xA77E, i, (B, S, H, D)) for i in range(3))
    _, o = orc.joint_path(q_img=q, k_img=k, v_img=v)
    qf, kf, vf = (from_bf16_bits(x).astype(np.float64) for x in (q, k, v))
    for b in range(B):
        for h in range(H):
            ref = np_attention(qf[b, :, h], kf[b, :, h], vf[b, :, h], 1.0 / np.sqrt(D))
            assert np.max(np.abs(o[b, :, h] - ref)) < 1e-6


@pytest.mark.parametrize("B,St,Si,H,D", [(1, 32, 64, 4, 64), (1, 64, 128, 4, 128), (2, 32, 256, 8, 128)])
def test_joint_is_concat_attention_split(orc, B, St, Si, H, D):
    # shapes of the reference's joint test (tests/test_joint_attention.cu:167-170)
    t = [uniform_bits(0xABCD, i, (B, St, H, D)) for i in range(3)]
    im = [uniform_bits(0xABCD, 3 + i, (B, Si, H, D)) for i in range(3)]
    o_t, o_i = orc.joint_path(q_txt=t[0], k_txt=t[1], v_txt=t[2], q_img=im[0], k_img=im[1], v_img=im[2])
    cat = [np.concatenate([a, b], axis=1) for a, b in zip(t, im)]
    _, o_c = orc.joint_path(q_img=cat[0], k_img=cat[1], v_img=cat[2])
    assert np.array_equal(o_c[:, :St], o_t) and np.array_equal(o_c[:, St:], o_i)


def test_fast_f32_attention_agrees_with_double(orc):
    q, k, v = (normal_bits(7, i, (1, 300, 3, 128)) for i in range(3))
    _, o = orc.joint_path(q_img=q, k_img=k, v_img=v)
    o32 = orc.attention_f32(q, k, v)
    max_abs, cos, _ = metrics(o32, o)
    assert max_abs < 2e-5 and cos > 0.999999


def test_reference_rounding_mode_is_close_to_ideal(orc):
    q, k, v = (normal_bits(9, i, (1, 200, 2, 128)) for i in range(3))
    _, ideal = orc.joint_path(q_img=q, k_img=k, v_img=v, mode=oracle.IDEAL)
    _, rr = orc.joint_path(q_img=q, k_img=k, v_img=v, mode=oracle.REF_ROUND)
    max_abs, cos, _ = metrics(rr, ideal)
    assert max_abs < 2e-2 and cos > 0.9999
    # and its output is exactly representable in bf16
    assert np.array_equal(from_bf16_bits(to_bf16_bits(rr)), rr)


def test_softmax_rows_sum_to_one_constant_v(orc):
    q, k = (normal_bits(11, i, (1, 150, 2, 128)) for i in range(2))
    v = np.broadcast_to(normal_bits(11, 5, (1, 1, 2, 128)), (1, 150, 2, 128)).copy()
    _, o = orc.joint_path(q_img=q, k_img=k, v_img=v)
    assert np.max(np.abs(o - from_bf16_bits(v))) < 1e-6


@pytest.mark.parametrize("rows,dim", [(1, 128), (8, 1024), (32, 3072)])
def test_rmsnorm_matches_numpy(orc, rows, dim):
    # distributions of tests/test_rmsnorm.cu:32-36
    from f2k_cuda_b200.inputs import uniform01
    x = to_bf16_bits((4 * uniform01(0xC0FFEE, 0, rows * dim) - 2).astype(np.float32)).reshape(rows, dim)
    g = to_bf16_bits((uniform01(0xC0FFEE, 1, dim) + 0.5).astype(np.float32))
    xf, gf = from_bf16_bits(x).astype(np.float64), from_bf16_bits(g).astype(np.float64)
    ref = xf / np.sqrt((xf * xf).mean(axis=1, keepdims=True) + 1e-6) * gf
    y = orc.rmsnorm_ideal(x, g, 1e-6)
    assert np.max(np.abs(y - ref)) < 1e-6
    yb = from_bf16_bits(orc.rmsnorm_bf16(x, g, 1e-6))
    # reference thresholds (tests/test_rmsnorm.cu:87-90)
    assert np.max(np.abs(yb - ref)) < 0.05 and np.mean(np.abs(yb - ref)) < 0.005


def _test_positions(seq, n_axes):
    # the position pattern of tests/test_rope_4axis.cu:33-41 (non-zero T axis)
    W = int(np.sqrt(seq))
    pos = np.zeros((seq, n_axes), np.int32)
    s = np.arange(seq)
    pos[:, 0] = s % 7
    if n_axes > 1: pos[:, 1] = s // W
    if n_axes > 2: pos[:, 2] = s % W
    if n_axes > 3: pos[:, 3] = s
    return pos


@pytest.mark.parametrize("seq,axes,theta", [(16, (4, 4, 4, 4), 100.0), (256, (32, 32, 32, 32), 2000.0)])
def test_rope_tables_and_rotation(orc, seq, axes, theta):
    pos = _test_positions(seq, len(axes))
    cos, sin = orc.build_rope_tables(axes, pos, theta)
    # independent numpy statement
    off = 0
    for a, d in enumerate(axes):
        k = np.arange(d // 2)
        ang = pos[:, a:a + 1].astype(np.float64) * np.power(float(theta), -2.0 * k / d)[None, :]
        assert np.array_equal(cos[:, off:off + d // 2], np.cos(ang).astype(np.float32))
        assert np.array_equal(sin[:, off:off + d // 2], np.sin(ang).astype(np.float32))
        off += d // 2
    # rotation vs fp32 numpy (tests/test_rope_4axis.cu:57-68), H heads per token
    H, D = 4, sum(axes)
    x = normal_bits(0xCAFE, 0, (seq * H, D))
    pos_ids = (np.arange(seq * H) // H).astype(np.int32)
    y = from_bf16_bits(orc.rope_bf16(x, cos, sin, pos_ids, seq))
    xf = from_bf16_bits(x)
    c, s_ = cos[pos_ids], sin[pos_ids]
    ref = np.empty_like(xf)
    ref[:, 0::2] = xf[:, 0::2] * c - xf[:, 1::2] * s_
    ref[:, 1::2] = xf[:, 0::2] * s_ + xf[:, 1::2] * c
    assert np.max(np.abs(y - ref)) < 0.05 and np.mean(np.abs(y - ref)) < 0.01
    # the oracle fuses the multiply-adds the way the reference kernel's compiled code does, so a
    # plain fp32 evaluation may differ in the last bf16 bit of a few elements in 10^5
    assert np.mean(to_bf16_bits(ref) != to_bf16_bits(y)) < 1e-3


def test_rope_position_clamp(orc):
    cos, sin = orc.build_rope_tables((4, 4), np.array([[0, 0], [1, 2], [2, 5]]), 10.0)
    x = normal_bits(3, 0, (3, 8))
    a = orc.rope_bf16(x, cos, sin, np.array([-4, 1, 99], np.int32), 3)
    b = orc.rope_bf16(x, cos, sin, np.array([0, 1, 2], np.int32), 3)
    assert np.array_equal(a, b)


def test_prologue_composition_matches_stepwise(orc):
    """norm -> RoPE -> attention in one oracle call == the three oracle steps chained
    with the reference's rounding points."""
    B, St, Si, H, D = 1, 24, 40, 2, 128
    t = [normal_bits(21, i, (B, St, H, D)) for i in range(3)]
    im = [normal_bits(21, 3 + i, (B, Si, H, D)) for i in range(3)]
    from f2k_cuda_b200.inputs import uniform01
    gam = [to_bf16_bits((1 + 0.2 * (uniform01(21, 50 + i, D) - 0.5)).astype(np.float32)) for i in range(4)]
    pt = np.zeros((St, 4), np.int32); pt[:, 3] = np.arange(St)
    pi = np.zeros((Si, 4), np.int32); pi[:, 1] = np.arange(Si) // 8; pi[:, 2] = np.arange(Si) % 8
    tab_t = orc.build_rope_tables((32,) * 4, pt, 2000.0)
    tab_i = orc.build_rope_tables((32,) * 4, pi, 2000.0)
    o_t, o_i = orc.joint_path(q_txt=t[0], k_txt=t[1], v_txt=t[2], q_img=im[0], k_img=im[1], v_img=im[2],
                              gammas=gam, tables=(*tab_t, *tab_i), eps=1e-6, mode=oracle.REF_ROUND)

    def prep(x, g, tab, seq):
        y = orc.rmsnorm_bf16(x.reshape(-1, D), g, 1e-6)
        pos_ids = ((np.arange(B * seq * H) // H) % seq).astype(np.int32)
        return orc.rope_bf16(y, tab[0], tab[1], pos_ids, seq).reshape(B, seq, H, D)

    qt, kt = prep(t[0], gam[0], tab_t, St), prep(t[1], gam[1], tab_t, St)
    qi, ki = prep(im[0], gam[2], tab_i, Si), prep(im[1], gam[3], tab_i, Si)
    s_t, s_i = orc.joint_path(q_txt=qt, k_txt=kt, v_txt=t[2], q_img=qi, k_img=ki, v_img=im[2],
                              mode=oracle.REF_ROUND)
    assert np.array_equal(s_t, o_t) and np.array_equal(s_i, o_i)


# ------------------------------------------------------------------ golden vectors
def test_golden_rope_tables_from_reference_builder(orc):
    """Tables produced by the reference's own build_rope_4axis_tables (host code of
    src/backend/cuda/kernels/rope_4axis.cu:56-97, run through oracle/_ref)."""
    f = GOLDEN / "rope_tables.npz"
    g = np.load(f)
    for tag in ("small", "flux_img", "flux_txt", "edit_img"):
        pos, axes, theta = g[f"{tag}_pos"], g[f"{tag}_axes"], float(g[f"{tag}_theta"])
        cos, sin = orc.build_rope_tables(axes, pos, theta)
        assert np.array_equal(cos, g[f"{tag}_cos"]) and np.array_equal(sin, g[f"{tag}_sin"]), tag


def _golden_cases():
    f = GOLDEN / "ref_kernels_b200.npz"
    return np.load(f) if f.exists() else None


@pytest.mark.skipif(_golden_cases() is None, reason="golden file from the B200 run not recorded yet")
def test_golden_reference_kernel_outputs(orc):
    """Outputs of the reference's CUDA kernels (rebuilt for sm_100a) on seeded inputs;
    the oracle must agree within the reference's own test thresholds, and far tighter
    in its reference-rounding mode."""
    from tests.golden.make_golden import gpu_cases, regenerate_inputs
    g = _golden_cases()
    report = {}
    for case in gpu_cases():
        inp = regenerate_inputs(case)
        tag = case["tag"]
        if case["kind"] == "rmsnorm":
            got = from_bf16_bits(orc.rmsnorm_bf16(inp["x"], inp["gamma"], 1e-6))
            ref = from_bf16_bits(g[f"{tag}_y"])
            assert np.max(np.abs(got - ref)) <= 0.0625 * np.max(np.abs(ref)) * 2 ** -6, tag  # <= 1 bf16 ulp
            assert np.mean(got != ref) < 0.01, tag
        elif case["kind"] == "rope":
            cos, sin = orc.build_rope_tables((32,) * 4, inp["pos"], 2000.0)
            got = orc.rope_bf16(inp["x"], cos, sin, inp["pos_ids"], case["seq"])
            assert np.array_equal(got, g[f"{tag}_y"]), tag      # bit for bit
            assert np.max(np.abs(from_bf16_bits(got) - from_bf16_bits(g[f"{tag}_y"]))) < 0.04, tag
        else:
            kw = dict(q_img=inp["q_img"], k_img=inp["k_img"], v_img=inp["v_img"])
            if case["seq_txt"]:
                kw.update(q_txt=inp["q_txt"], k_txt=inp["k_txt"], v_txt=inp["v_txt"])
            if case["prologue"]:
                from tests.golden.make_golden import path_tables
                tab_t, tab_i = path_tables(case, orc.build_rope_tables)
                kw.update(gammas=inp["gammas"], tables=(*tab_t, *tab_i), eps=1e-6)
            for mode, tol in ((oracle.IDEAL, 2e-2), (oracle.REF_ROUND, 8e-3)):
                o_t, o_i = orc.joint_path(mode=mode, **kw)
                max_abs, cos, rel = metrics(o_i, from_bf16_bits(g[f"{tag}_o_img"]))
                assert cos > 0.9999 and rel < 0.05 and max_abs < tol, (tag, mode, max_abs, cos)
                if case["seq_txt"]:
                    max_abs, cos, rel = metrics(o_t, from_bf16_bits(g[f"{tag}_o_txt"]))
                    assert cos > 0.9999 and rel < 0.05 and max_abs < tol, (tag, mode, max_abs, cos)
