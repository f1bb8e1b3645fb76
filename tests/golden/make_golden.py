"""Generates the golden vectors under tests/golden/ from the reference's own code.

  python -m tests.golden.make_golden tables   (any machine with oracle/_ref built)
      -> tests/golden/rope_tables.npz: outputs of the reference's host-side
         build_rope_4axis_tables (src/backend/cuda/kernels/rope_4axis.cu:56-97).

  python -m tests.golden.make_golden kernels OUTDIR   (on a B200, oracle/_ref prebuilt)
      -> OUTDIR/ref_kernels_b200.npz: outputs of the reference's CUDA kernels rebuilt
         unmodified for sm_100a (rmsnorm_bf16, rope_4axis_inplace_bf16, Attention::forward,
         JointAttention::forward, and the three chained as the blocks chain them) on the
         seeded inputs `regenerate_inputs` recreates. The file is then committed here.

Inputs are never stored: they are a pure function of the case (f2k_cuda_b200.inputs).
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from f2k_cuda_b200.inputs import normal, to_bf16_bits, uniform01  # noqa: E402

SEED = 0x601D


def table_cases():
    s = np.arange(256)
    small = np.zeros((16, 4), np.int32)
    t = np.arange(16)
    small[:, 0], small[:, 1], small[:, 2], small[:, 3] = t % 7, t // 4, t % 4, t
    img = np.zeros((256, 4), np.int32); img[:, 1], img[:, 2] = s // 16, s % 16
    txt = np.zeros((77, 4), np.int32); txt[:, 3] = np.arange(77)
    edit = np.concatenate([img, img + np.array([1, 0, 0, 0], np.int32)], 0)
    return {
        "small": (small, (4, 4, 4, 4), 100.0),
        "flux_img": (img, (32, 32, 32, 32), 2000.0),
        "flux_txt": (txt, (32, 32, 32, 32), 2000.0),
        "edit_img": (edit, (32, 32, 32, 32), 2000.0),
    }


def gpu_cases():
    return [
        dict(tag="rms_128", kind="rmsnorm", rows=64, dim=128),
        dict(tag="rms_1024", kind="rmsnorm", rows=8, dim=1024),
        dict(tag="rope_128", kind="rope", seq=64, heads=4, dim=128),
        dict(tag="attn_130", kind="attn", batch=1, seq_txt=0, seq_img=130, heads=2, dim=128, prologue=False),
        dict(tag="attn_2x128", kind="attn", batch=2, seq_txt=0, seq_img=128, heads=4, dim=128, prologue=False),
        dict(tag="joint_64_128", kind="attn", batch=1, seq_txt=64, seq_img=128, heads=4, dim=128, prologue=False),
        dict(tag="joint_32_256", kind="attn", batch=1, seq_txt=32, seq_img=256, heads=4, dim=128, prologue=False),
        dict(tag="path_40_64", kind="attn", batch=1, seq_txt=40, seq_img=64, heads=4, dim=128, prologue=True),
    ]


def _bits(stream, shape, dist="uniform"):
    n = int(np.prod(shape))
    x = normal(SEED, stream, n) if dist == "normal" else (uniform01(SEED, stream, n) - 0.5).astype(np.float32)
    return to_bf16_bits(x).reshape(shape)


def path_tables(case, builder):
    St, Si = case["seq_txt"], case["seq_img"]
    W = int(np.sqrt(Si))
    pt = np.zeros((St, 4), np.int32); pt[:, 3] = np.arange(St)
    pi = np.zeros((Si, 4), np.int32); pi[:, 1] = np.arange(Si) // W; pi[:, 2] = np.arange(Si) % W
    return builder((32,) * 4, pt, 2000.0), builder((32,) * 4, pi, 2000.0)


def regenerate_inputs(case):
    k = case["kind"]
    base = 1000 * (1 + [c["tag"] for c in gpu_cases()].index(case["tag"]))
    if k == "rmsnorm":
        x = to_bf16_bits((4 * uniform01(SEED, base, case["rows"] * case["dim"]) - 2).astype(np.float32))
        g = to_bf16_bits((uniform01(SEED, base + 1, case["dim"]) + 0.5).astype(np.float32))
        return dict(x=x.reshape(case["rows"], case["dim"]), gamma=g)
    if k == "rope":
        seq, H, D = case["seq"], case["heads"], case["dim"]
        W = int(np.sqrt(seq))
        pos = np.zeros((seq, 4), np.int32)
        s = np.arange(seq)
        pos[:, 0], pos[:, 1], pos[:, 2], pos[:, 3] = s % 7, s // W, s % W, s
        return dict(x=_bits(base, (seq * H, D), "normal"), pos=pos,
                    pos_ids=(np.arange(seq * H) // H).astype(np.int32))
    B, St, Si, H, D = case["batch"], case["seq_txt"], case["seq_img"], case["heads"], case["dim"]
    dist = "normal" if case["prologue"] else "uniform"
    out = dict(q_img=_bits(base + 3, (B, Si, H, D), dist), k_img=_bits(base + 4, (B, Si, H, D), dist),
               v_img=_bits(base + 5, (B, Si, H, D), dist))
    if St:
        out.update(q_txt=_bits(base, (B, St, H, D), dist), k_txt=_bits(base + 1, (B, St, H, D), dist),
                   v_txt=_bits(base + 2, (B, St, H, D), dist))
    if case["prologue"]:
        out["gammas"] = [to_bf16_bits((1 + 0.2 * (uniform01(SEED, base + 10 + i, D) - 0.5)).astype(np.float32))
                         for i in range(4)]
    return out


def make_tables():
    import oracle
    ref = oracle.load_ref()
    if ref is None:
        raise SystemExit("oracle/_ref is not built (needs the reference checkout): make -C oracle ref")
    out = {}
    for tag, (pos, axes, theta) in table_cases().items():
        cos, sin = ref.build_rope_tables(axes, pos, theta)
        out[f"{tag}_pos"], out[f"{tag}_axes"], out[f"{tag}_theta"] = pos, np.array(axes, np.int32), np.float32(theta)
        out[f"{tag}_cos"], out[f"{tag}_sin"] = cos, sin
    np.savez_compressed(HERE / "rope_tables.npz", **out)
    print("wrote", HERE / "rope_tables.npz")


def make_kernels(outdir: Path):
    import ctypes as C

    import torch

    import oracle
    from tests._util import dev_bf16, host_bits
    ref = oracle.load_ref()
    if ref is None:
        raise SystemExit("oracle/_ref/libf2k_ref.so missing")
    L = ref.lib
    p = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
    out = {}
    for case in gpu_cases():
        inp, tag = regenerate_inputs(case), case["tag"]
        if case["kind"] == "rmsnorm":
            x, g = dev_bf16(inp["x"]), dev_bf16(inp["gamma"])
            y = torch.empty_like(x)
            assert L.f2k_ref_rmsnorm_bf16(p(x), p(g), p(y), case["rows"], case["dim"], 1e-6, None)
            torch.cuda.synchronize()
            out[f"{tag}_y"] = host_bits(y)
        elif case["kind"] == "rope":
            cos, sin = ref.build_rope_tables((32,) * 4, inp["pos"], 2000.0)
            x = dev_bf16(inp["x"])
            dc, ds = torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda()
            dp = torch.from_numpy(inp["pos_ids"]).cuda()
            assert L.f2k_ref_rope_4axis_inplace_bf16(p(x), p(dc), p(ds), p(dp), x.shape[0], case["dim"],
                                                     case["seq"], None)
            torch.cuda.synchronize()
            out[f"{tag}_y"] = host_bits(x)
        else:
            B, St, Si, H, D = case["batch"], case["seq_txt"], case["seq_img"], case["heads"], case["dim"]
            d = {k: dev_bf16(v) for k, v in inp.items() if k != "gammas"}
            if case["prologue"]:
                (ct, st), (ci, si) = path_tables(case, ref.build_rope_tables)
                gam = [dev_bf16(g) for g in inp["gammas"]]
                for name, g, (c_, s_), seq in (("q_txt", gam[0], (ct, st), St), ("k_txt", gam[1], (ct, st), St),
                                               ("q_img", gam[2], (ci, si), Si), ("k_img", gam[3], (ci, si), Si)):
                    x = d[name]
                    rows = B * seq * H
                    assert L.f2k_ref_rmsnorm_bf16(p(x), p(g), p(x), rows, D, 1e-6, None)
                    dc, ds = torch.from_numpy(c_).cuda(), torch.from_numpy(s_).cuda()
                    pos_ids = ((torch.arange(rows, device="cuda") // H) % seq).to(torch.int32)
                    assert L.f2k_ref_rope_4axis_inplace_bf16(p(x), p(dc), p(ds), p(pos_ids), rows, D, seq, None)
                    torch.cuda.synchronize()
            o_i = torch.empty_like(d["q_img"])
            if St:
                h = L.f2k_ref_joint_create(B, St, Si, H, D, 0.0)
                assert L.f2k_ref_joint_ok(h)
                ws_bytes = L.f2k_ref_joint_workspace_bytes(h)
                ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
                o_t = torch.empty_like(d["q_txt"])
                assert L.f2k_ref_joint_forward(h, p(d["q_txt"]), p(d["k_txt"]), p(d["v_txt"]), p(d["q_img"]),
                                               p(d["k_img"]), p(d["v_img"]), p(o_t), p(o_i), p(ws), ws_bytes, None)
                torch.cuda.synchronize()
                L.f2k_ref_joint_destroy(h)
                out[f"{tag}_o_txt"] = host_bits(o_t)
            else:
                h = L.f2k_ref_attn_create(B, Si, H, D, 0.0)
                assert L.f2k_ref_attn_ok(h)
                assert L.f2k_ref_attn_forward(h, p(d["q_img"]), p(d["k_img"]), p(d["v_img"]), p(o_i), None)
                torch.cuda.synchronize()
                L.f2k_ref_attn_destroy(h)
            out[f"{tag}_o_img"] = host_bits(o_i)
    outdir.mkdir(parents=True, exist_ok=True)
    np.savez_compressed(outdir / "ref_kernels_b200.npz", **out)
    print("wrote", outdir / "ref_kernels_b200.npz")


if __name__ == "__main__":
    if len(sys.argv) >= 2 and sys.argv[1] == "tables":
        make_tables()
    elif len(sys.argv) >= 3 and sys.argv[1] == "kernels":
        make_kernels(Path(sys.argv[2]))
    else:
        raise SystemExit(__doc__)
