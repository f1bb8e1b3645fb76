"""Host-side logic that needs no GPU: workloads, seeded inputs, sharding plans, and the
multi-rank plumbing with gloo ranks on CPU."""
import os
import socket

import numpy as np
import pytest

from f2k_cuda_b200 import inputs
from f2k_cuda_b200.seqpar import plan_ring, shard_bounds


def test_workloads_match_the_five_configurations():
    w = inputs.WORKLOADS
    assert [w[k].seq for k in ("s1152", "s4608", "s4608_b4", "s8704_edit", "s16896")] == [1152, 4608, 4608, 8704, 16896]
    assert w["s4608_b4"].batch == 4 and all(v.n_heads == 32 and v.head_dim == 128 for v in w.values())
    # 4 * B * H * S^2 * D
    assert w["s4608"].flops == pytest.approx(3.479e11, rel=1e-3)
    assert w["s16896"].flops == pytest.approx(4.677e12, rel=1e-3)


def test_inputs_are_a_pure_function_of_seed_and_index():
    a = inputs.normal(123, 4, 1000)
    assert np.array_equal(a, inputs.normal(123, 4, 1000))
    assert np.array_equal(a[:10], inputs.normal(123, 4, 10))          # prefix-stable
    assert not np.array_equal(a, inputs.normal(124, 4, 1000))
    big = inputs.normal(7, 0, 200000)
    assert abs(big.mean()) < 0.01 and abs(big.std() - 1) < 0.01
    u = inputs.uniform01(7, 1, 200000)
    assert 0 < u.min() and u.max() < 1 and abs(u.mean() - 0.5) < 0.005
    # a head subset draws the same values as the full problem
    w = inputs.Workload("t", 1, 8, ((4, 4),), n_heads=4, seed=99)
    full, part = inputs.make_problem(w), inputs.make_problem(w, heads=2)
    assert np.array_equal(full.q_img[:, :, :2], part.q_img) and np.array_equal(full.v_txt[:, :, :2], part.v_txt)
    g = inputs.from_bf16_bits(full.gammas[0])
    assert 0.89 < g.min() and g.max() < 1.11


def test_positions_follow_the_reference_layout():
    pt, pi = inputs.token_positions(inputs.WORKLOADS["s4608"])
    assert pt.shape == (512, 4) and np.array_equal(pt[:, 3], np.arange(512)) and not pt[:, :3].any()
    assert pi.shape == (4096, 4) and np.array_equal(pi[65], [0, 1, 1, 0]) and not pi[:, 3].any()


@pytest.mark.parametrize("seq,world", [(16896, 8), (8704, 4), (4608, 2), (10, 4), (7, 8)])
def test_shards_cover_the_sequence_once(seq, world):
    b = [shard_bounds(seq, world, r) for r in range(world)]
    assert b[0][0] == 0 and b[-1][1] == seq
    assert all(b[i][1] == b[i + 1][0] for i in range(world - 1))
    assert all(0 <= e - s <= -(-seq // world) for s, e in b)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_ring_plan_is_a_latin_square(world):
    plans = [plan_ring(world, r) for r in range(world)]
    for r, p in enumerate(plans):
        assert p[0] == r and sorted(p) == list(range(world))
    # at every step the ranks pull from pairwise different sources
    for step in range(world):
        assert sorted(p[step] for p in plans) == list(range(world))


def np_attention_by_segments(q, k_segs, v_segs, scale):
    """Online-softmax over key/value segments in the given order (what the kernel does per row)."""
    m = np.full(q.shape[0], -np.inf)
    l = np.zeros(q.shape[0])
    o = np.zeros((q.shape[0], v_segs[0].shape[1]))
    for k, v in zip(k_segs, v_segs):
        s = (q @ k.T) * scale
        m_new = np.maximum(m, s.max(axis=1))
        f = np.exp(m - m_new)
        p = np.exp(s - m_new[:, None])
        l = l * f + p.sum(axis=1)
        o = o * f[:, None] + p @ v
        m = m_new
    return o / l[:, None]


def test_segment_order_does_not_change_attention(orc):
    """Each rank walks the shards in its own ring order; the result must be the full attention."""
    from tests._util import normal_bits
    world, per, H, D = 4, 50, 1, 128
    S = world * per
    q, k, v = (normal_bits(77, i, (1, S, H, D)) for i in range(3))
    _, full = orc.joint_path(q_img=q, k_img=k, v_img=v)
    qf, kf, vf = (inputs.from_bf16_bits(x)[0, :, 0].astype(np.float64) for x in (q, k, v))
    for r in range(world):
        b, e = shard_bounds(S, world, r)
        order = plan_ring(world, r)
        ks = [kf[slice(*shard_bounds(S, world, s))] for s in order]
        vs = [vf[slice(*shard_bounds(S, world, s))] for s in order]
        got = np_attention_by_segments(qf[b:e], ks, vs, 1 / np.sqrt(D))
        assert np.max(np.abs(got - full[0, b:e, 0])) < 1e-6


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _gloo_worker(rank, world, port, seq, out):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # the exchange attach_distributed performs: every rank publishes 64 opaque bytes and
        # must receive everybody's, in rank order
        handle = bytes([rank]) * 64
        got = [None] * world
        dist.all_gather_object(got, handle)
        plans = [None] * world
        dist.all_gather_object(plans, (plan_ring(world, rank), shard_bounds(seq, world, rank)))
        # the benchmark's only collective: a tiny all-reduce of the measured time (a step has none)
        import torch
        t = torch.ones(1)
        dist.all_reduce(t)
        out[rank] = (got == [bytes([r]) * 64 for r in range(world)], plans, float(t.item()))
    finally:
        dist.destroy_process_group()


def test_rank_plumbing_with_two_gloo_ranks():
    import torch.multiprocessing as mp
    world, seq = 2, 8704
    mgr = mp.Manager()
    out = mgr.dict()
    port = _free_port()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_gloo_worker, args=(r, world, port, seq, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    for r in range(world):
        ok, plans, total = out[r]
        assert ok and total == world
        assert [p[0] for p in plans] == [plan_ring(world, k) for k in range(world)]
        assert plans[1][1] == (4352, 8704)


def test_bench_rank_problem_shards_heads_not_work():
    import bench
    for n in (1, 2, 4, 8):
        assert 32 % n == 0
    # per-GPU units stay at 32 (batch n x 32/n heads): weak scaling without data-path traffic
    from f2k_cuda_b200.inputs import Workload
    for n in (1, 2, 4, 8):
        w = Workload("s4608", n, 512, ((64, 64),), n_heads=32 // n)
        assert w.batch * w.n_heads == 32


def _head_exchange_worker(rank, world, port, out):
    """One rank of the head exchange with numpy standing in for the kernels: scatter the rank's
    normalised rows by head (an object all-gather stands in for the peer stores), attend the
    rank's heads over all tokens, send every output row back to the rank that owns the token."""
    import torch.distributed as dist
    import oracle
    from f2k_cuda_b200.headswap import head_exchange_plan
    from tests._util import normal_bits
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        orc = oracle.load_oracle()
        per, H, D = 48, 4, 128
        S = world * per
        q, k, v = (normal_bits(0x4EAD, i, (1, S, H, D)) for i in range(3))      # every rank draws the whole problem
        plan = head_exchange_plan(per, H, world, rank)
        hpr = plan["heads_per_rank"]
        mine = slice(rank * per, (rank + 1) * per)
        # inbound: what this rank would store into each destination's buffers
        parcels = {}
        for dst in plan["send"]:
            h0, h1 = dst["heads"]
            parcels[dst["to"]] = (dst["token_offset"], q[:, mine, h0:h1], k[:, mine, h0:h1], v[:, mine, h0:h1])
        everyone = [None] * world
        dist.all_gather_object(everyone, parcels)
        qh = np.zeros((1, S, hpr, D), np.uint16); kh = np.zeros_like(qh); vh = np.zeros_like(qh)
        for src in range(world):
            off, pq, pk, pv = everyone[src][rank]
            qh[:, off:off + per], kh[:, off:off + per], vh[:, off:off + per] = pq, pk, pv
        _, oh = orc.joint_path(q_img=qh, k_img=kh, v_img=vh)                  # this rank's heads, all tokens
        # outbound: rows of segment s go to rank s, into this rank's head columns
        back = {r["to"]: (r["head_columns"], oh[:, r["tokens_of_rank"] * per:(r["tokens_of_rank"] + 1) * per])
                for r in plan["return"]}
        everyone = [None] * world
        dist.all_gather_object(everyone, back)
        o = np.zeros((1, per, H, D), np.float32)
        for src in range(world):
            (c0, c1), rows = everyone[src][rank]
            o[:, :, c0:c1] = rows
        _, full = orc.joint_path(q_img=q, k_img=k, v_img=v)
        err = float(np.max(np.abs(o - full[:, mine])))
        # a second step in which rank 0's "kernel" gives up: it sends no rows back, and marks the
        # step number in everybody's failed words before "done". Every rank must find the marker.
        from f2k_cuda_b200.headswap import peer_failures
        step = 2
        failed_words = [1] * world                      # what the (clean) first step could have left: older numbers
        note = {"done": step, "failed": step if rank == 0 else None}
        everyone = [None] * world
        dist.all_gather_object(everyone, note)
        for src in range(world):
            assert everyone[src]["done"] == step         # "done" always arrives: nobody hangs
            if everyone[src]["failed"] is not None:
                failed_words[src] = everyone[src]["failed"]
        out[rank] = (err, peer_failures(failed_words, step), peer_failures(failed_words, step + 1))
    finally:
        dist.destroy_process_group()


def test_head_exchange_with_two_gloo_ranks():
    import torch.multiprocessing as mp
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    port = _free_port()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_head_exchange_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    assert all(out[r][0] == 0.0 for r in range(world)), dict(out)   # same arithmetic per head: identical
    # the failed step is seen by both ranks, as rank 0's, and only for that step
    assert all(out[r][1] == [0] and out[r][2] == [] for r in range(world)), dict(out)


def test_head_exchange_plan_covers_every_head_once():
    from f2k_cuda_b200.headswap import head_exchange_plan
    for world in (1, 2, 4, 8):
        seen = []
        for rank in range(world):
            plan = head_exchange_plan(2112, 32, world, rank)
            assert [d["heads"] for d in plan["send"]] == [(d * 32 // world, (d + 1) * 32 // world) for d in range(world)]
            assert all(d["token_offset"] == rank * 2112 for d in plan["send"])
            seen += [r["head_columns"] for r in plan["return"] if r["to"] == 0]
        assert sorted(seen) == [(r * 32 // world, (r + 1) * 32 // world) for r in range(world)]
    with pytest.raises(ValueError):
        head_exchange_plan(128, 6, 4, 0)
