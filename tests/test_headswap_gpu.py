"""Sequence-parallel attention by head exchange on the GPU.

One GPU: all ranks live in this process on cuda:0; their exchange buffers are attached by pointer,
so the scatter kernel's "peer" stores, the per-source-rank arrival words the attention kernel
waits on, the output rows written into the token owner's buffer and the "done" words all run as
they do across GPUs. Every rank's exchange kernel has finished before the first attention kernel
starts (a kernel never waits for SM work of another rank on the same GPU).
Two or more GPUs: child processes, one per GPU, over CUDA IPC.
"""
import os
import socket
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from tests._util import assert_parity, dev_bf16, host_f32

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def reference_output(orc, w, p):
    """Ideal fused path (QK-norm, RoPE, attention) of the whole sequence as one image stream."""
    import f2k_cuda_b200 as f2k
    cos, sin = f2k.build_rope_4axis_tables((32,) * 4, p.pos_img, 2000.0)
    _, ref = orc.joint_path(q_img=p.q_img, k_img=p.k_img, v_img=p.v_img, gammas=(None, None, p.gammas[2], p.gammas[3]),
                            tables=(None, None, cos, sin), eps=1e-6)
    return cos, sin, ref


# (world, tokens per rank, heads): ragged shards (200, 136: not multiples of 128), an odd number of
# tiles per shard, one head per rank, world 1
@pytest.mark.parametrize("copy_engines", [False, True])
@pytest.mark.parametrize("world,per,H", [(2, 256, 4), (4, 200, 4), (8, 136, 8), (4, 128, 8), (1, 300, 2), (2, 384, 8)])
@pytest.mark.timeout(120, method="thread")
def test_all_ranks_in_one_process(orc, world, per, H, copy_engines):
    import torch
    from f2k_cuda_b200.headswap import HeadExchangeAttention
    from f2k_cuda_b200.inputs import Workload, make_problem
    S, D = world * per, 128
    side = int(round(S ** 0.5))
    grid = (side, S // side) if side * (S // side) == S else (1, S)
    w = Workload("hx", 1, 0, (grid,), seed=0x4EAD + world)
    p = make_problem(w, heads=H)
    cos, sin, ref = reference_output(orc, w, p)
    ranks = [HeadExchangeAttention(per, H, D, world, r) for r in range(world)]
    for r in ranks:
        assert r.ok(), r.last_error()
    for r in ranks:
        assert r.attach_in_process(ranks)
    gq, gk = dev_bf16(p.gammas[2]), dev_bf16(p.gammas[3])
    dcos, dsin = torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda()
    shard = lambda x, r: dev_bf16(np.ascontiguousarray(x[:, r * per:(r + 1) * per]))  # noqa: E731
    for step in range(3):                           # both buffer sets, then the first again
        keep = []                                   # the copy engines read the inputs after the call returns
        for r, hx in enumerate(ranks):
            args = (shard(p.q_img, r), shard(p.k_img, r), shard(p.v_img, r), gq, gk,
                    dcos[r * per:(r + 1) * per].contiguous(), dsin[r * per:(r + 1) * per].contiguous(), 1e-6)
            keep.append(args)
            # the exchange as a scatter kernel, or as a prologue kernel + copy-engine transfers
            assert (hx.exchange_in_copy if copy_engines else hx.exchange_in)(*args), hx.last_error()
        torch.cuda.synchronize()                    # all exchanges done before any attention starts
        for hx in ranks:
            assert hx.attend(), hx.last_error()
        torch.cuda.synchronize()
        for r, hx in enumerate(ranks):
            o = hx.output()
            assert o is not None, hx.last_error()
            torch.cuda.synchronize()
            assert hx.device_status() == 0, hx.last_error()
            assert_parity(host_f32(o), ref[:, r * per:(r + 1) * per], f"world {world} rank {r} step {step}")


@pytest.mark.parametrize("per,H", [(300, 2), (1088, 4), (129, 5)])
@pytest.mark.timeout(120, method="thread")
def test_exchange_inside_the_attention_kernel_world_1(orc, per, H):
    """The fused form (f2k_hx_forward): the attention kernel's spare warps normalise, rotate and
    deliver Q, K, V while its other warps wait for the arrival words and attend. With one rank the
    whole mechanism (chunk queue, per-destination counters, arrival words for K/V and for Q, head-
    fastest CTA numbering) runs on one GPU in one kernel. Three steps: both buffer sets, then the
    first again; heads not a multiple of four take the exchange's narrower path."""
    import torch
    from f2k_cuda_b200.headswap import HeadExchangeAttention
    from f2k_cuda_b200.inputs import Workload, make_problem
    w = Workload("hxf", 1, 0, ((1, per),), seed=0xF05E + per)
    p = make_problem(w, heads=H)
    cos, sin, ref = reference_output(orc, w, p)
    hx = HeadExchangeAttention(per, H, 128, 1, 0)
    assert hx.ok(), hx.last_error()
    assert hx.attach_in_process([hx])
    gq, gk = dev_bf16(p.gammas[2]), dev_bf16(p.gammas[3])
    dcos, dsin = torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda()
    q, k, v = dev_bf16(p.q_img), dev_bf16(p.k_img), dev_bf16(p.v_img)
    keep = [x.clone() for x in (q, k, v)]
    for step in range(3):
        assert hx.forward(q, k, v, gq, gk, dcos, dsin, 1e-6), hx.last_error()
        o = hx.output()
        assert o is not None, hx.last_error()
        torch.cuda.synchronize()
        assert hx.device_status() == 0, hx.last_error()
        assert_parity(host_f32(o), ref, f"fused exchange step {step}")
    assert all(torch.equal(a, b) for a, b in zip(keep, (q, k, v)))        # the raw tensors are only read
    fused_bits = o.clone()
    # the same arithmetic as the two-kernel form: identical bits
    assert hx.exchange_in(q, k, v, gq, gk, dcos, dsin, 1e-6) and hx.attend(), hx.last_error()
    o2 = hx.output()
    torch.cuda.synchronize()
    assert hx.device_status() == 0
    assert torch.equal(o2, fused_bits), "fused and two-kernel forms must agree bit for bit"


def test_equals_the_single_gpu_fused_call_bit_for_bit(orc):
    """Same kernels, same arithmetic: the exchanged result must equal the one-GPU fused call."""
    import torch
    import f2k_cuda_b200 as f2k
    from f2k_cuda_b200.headswap import HeadExchangeAttention
    from f2k_cuda_b200.inputs import Workload, make_problem
    world, per, H, D = 4, 256, 8, 128
    w = Workload("hx", 1, 0, ((32, 32),), seed=0xB17)
    p = make_problem(w, heads=H)
    cos, sin = f2k.build_rope_4axis_tables((32,) * 4, p.pos_img, 2000.0)
    dcos, dsin = torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda()
    gq, gk = dev_bf16(p.gammas[2]), dev_bf16(p.gammas[3])
    att = f2k.Attention(f2k.Attention.Config(1, world * per, H, D))
    q, k, v = dev_bf16(p.q_img), dev_bf16(p.k_img), dev_bf16(p.v_img)
    o = torch.empty_like(q)
    ws = torch.empty(att.fused_workspace_size_bytes(), dtype=torch.uint8, device="cuda")
    assert att.forward_fused_single(q, k, v, gq, gk, dcos, dsin, 1e-6, o, ws), att.last_error()
    ranks = [HeadExchangeAttention(per, H, D, world, r) for r in range(world)]
    for r in ranks:
        assert r.ok() and r.attach_in_process(ranks)
    for r, hx in enumerate(ranks):
        sl = slice(r * per, (r + 1) * per)
        assert hx.exchange_in(q[:, sl].contiguous(), k[:, sl].contiguous(), v[:, sl].contiguous(), gq, gk,
                              dcos[sl].contiguous(), dsin[sl].contiguous(), 1e-6)
    torch.cuda.synchronize()
    for hx in ranks:
        assert hx.attend()
    torch.cuda.synchronize()
    for r, hx in enumerate(ranks):
        out = hx.output()
        torch.cuda.synchronize()
        assert torch.equal(out, o[:, r * per:(r + 1) * per])


def test_refusals():
    from f2k_cuda_b200.headswap import HeadExchangeAttention
    bad = HeadExchangeAttention(128, 6, 128, 4, 0)          # 4 ranks do not divide 6 heads
    assert not bad.ok() and "divide" in bad.last_error()
    hx = HeadExchangeAttention(128, 4, 128, 2, 0)
    assert hx.ok()
    assert not hx.attend() and "exchange_in" in hx.last_error()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_one_process_per_gpu(world):
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()), NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", env["MASTER_PORT"],
           str(ROOT / "tests" / "headswap_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "HEADSWAP_OK" in r.stdout
