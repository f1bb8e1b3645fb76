"""Sequence-parallel attention on the GPU.

One GPU: all ranks live in this process on cuda:0 and their shard buffers are attached by
pointer; the copy stream still moves every remote shard and writes its arrival word while the
attention kernel of the consuming rank is already running, so the whole data path (pulls,
arrival words, per-segment waits in the kernel, ragged shards) runs as it does across GPUs.
Two or more GPUs: child processes, one per GPU, wired through CUDA IPC and NCCL.
No test here waits on another kernel: a kernel only ever waits (bounded) for copy-engine work.
"""
import os
import socket
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from tests._util import assert_parity, dev_bf16, host_f32, normal_bits

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


_STREAMS = []


def _rank_streams(world):
    """Eight distinct streams, made once: torch hands streams out of a small pool round-robin, and
    two ranks must never end up on the same underlying stream."""
    import torch
    while len(_STREAMS) < 8:
        _STREAMS.append(torch.cuda.Stream())
    assert len({s.cuda_stream for s in _STREAMS}) == 8
    return _STREAMS[:world]


# groups: 0 = the library's own choice (whole slots at these sizes), else the number of head
# groups a slot is pulled in (one 3-D copy per group)
@pytest.mark.parametrize("world,per,H,B,overlap,groups",
                         [(2, 256, 4, 1, True, 0), (4, 200, 2, 1, True, 0), (4, 200, 2, 1, False, 0),
                          (8, 136, 2, 2, True, 0), (3, 128, 1, 1, True, 0), (1, 300, 2, 1, True, 0),
                          (2, 256, 4, 1, True, 4), (4, 200, 2, 2, True, 2), (8, 136, 8, 1, True, 8)])
@pytest.mark.timeout(120, method="thread")      # a stream wait that never ends must end the run
def test_all_ranks_in_one_process(orc, monkeypatch, world, per, H, B, overlap, groups):
    import torch
    from f2k_cuda_b200.seqpar import SequenceParallelAttention, shard_bounds
    if groups:
        monkeypatch.setenv("F2K_SEQPAR_GROUPS", str(groups))
    else:
        monkeypatch.delenv("F2K_SEQPAR_GROUPS", raising=False)
    S, D = world * per, 128
    q, k, v = (normal_bits(0x5E9, i, (B, S, H, D)) for i in range(3))
    _, ref = orc.joint_path(q_img=q, k_img=k, v_img=v)
    ranks = [SequenceParallelAttention(B, per, H, D, world, r) for r in range(world)]
    for r in ranks:
        assert r.ok(), r.last_error()
    for r in ranks:
        assert r.attach_in_process(ranks)
    streams = _rank_streams(world)              # every rank has its own compute stream
    for step in range(2):                       # twice: both buffer sets, fresh arrival values
        outs = []
        for r, sp in enumerate(ranks):          # every rank's inputs first (ranks share this GPU:
            b, e = shard_bounds(S, world, r)    # a rank's kernel must never wait for SM work of another)
            with torch.cuda.stream(streams[r]):
                ks, vs = sp.local_kv()
                ks.copy_(dev_bf16(k[:, b:e])); vs.copy_(dev_bf16(v[:, b:e]))
                dq = dev_bf16(q[:, b:e])
                outs.append((dq, torch.full_like(dq, float("nan"))))
        torch.cuda.synchronize()
        for r, sp in enumerate(ranks):
            # no barrier between the ranks: they tell each other through words in their shard buffers
            assert sp.forward(outs[r][0], outs[r][1], overlap=overlap, stream=streams[r]), sp.last_error()
        torch.cuda.synchronize()
        for r, sp in enumerate(ranks):
            assert sp.device_status() == 0, sp.last_error()
            b, e = shard_bounds(S, world, r)
            assert_parity(host_f32(outs[r][1]), ref[:, b:e], f"world {world} rank {r} step {step}")


def test_prologue_entry_point_matches_fused_path(orc):
    """qk_norm_rope on a sequence shard == the prologue of the fused call on those tokens."""
    import torch
    import f2k_cuda_b200 as f2k
    from f2k_cuda_b200.inputs import Workload, make_problem, to_bf16_bits
    from f2k_cuda_b200.seqpar import qk_norm_rope
    w = Workload("p", 1, 0, ((16, 16),), n_heads=4, seed=0x9109)
    p = make_problem(w)
    cos, sin = f2k.build_rope_4axis_tables((32,) * 4, p.pos_img, 2000.0)
    lo, hi = 64, 192                                        # a shard in the middle of the sequence
    x = dev_bf16(p.q_img[:, lo:hi])
    y = torch.empty_like(x)
    assert qk_norm_rope(x, y, dev_bf16(p.gammas[2]), torch.from_numpy(cos[lo:hi]).cuda(),
                        torch.from_numpy(sin[lo:hi]).cuda(), 1e-6)
    torch.cuda.synchronize()
    # ideal statement: RMSNorm in double, rotation in double, one rounding
    from f2k_cuda_b200.inputs import from_bf16_bits
    xf = from_bf16_bits(p.q_img[:, lo:hi]).astype(np.float64)
    g = from_bf16_bits(p.gammas[2]).astype(np.float64)
    n = xf / np.sqrt((xf * xf).mean(-1, keepdims=True) + 1e-6) * g
    c, s = cos[lo:hi][None, :, None, :].astype(np.float64), sin[lo:hi][None, :, None, :].astype(np.float64)
    ref = np.empty_like(n)
    ref[..., 0::2] = n[..., 0::2] * c - n[..., 1::2] * s
    ref[..., 1::2] = n[..., 0::2] * s + n[..., 1::2] * c
    got = host_f32(y)
    assert np.max(np.abs(got - ref)) < 0.02 and np.mean(to_bf16_bits(ref.astype(np.float32)) != to_bf16_bits(got)) < 0.01


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
           str(ROOT / "tests" / "seqpar_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "SEQPAR_OK" in r.stdout
