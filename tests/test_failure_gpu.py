"""Failure detection on the GPU without a GPU fault.

Every wait inside the kernels is bounded; when one runs out the kernel leaves through its normal
exit, sets a status word and the context stays usable. These tests make a wait run out by the
only means allowed on shared GPUs: a word that nothing writes (a rank that is late or never
comes, in the one-process emulation of the ranks), with the limits shortened to a millisecond
through the C ABI. No trap, no bad address, no endless loop.

 * sequence-parallel attention: a peer never announces its K/V. The kernel gives up after the
   limit and reports it; the copy stream, parked on a stream wait for the peer's word, is
   released by f2k_seqpar_abort; the handles then run a normal step correctly.
 * head exchange: a rank that starts a step too late. The early rank's kernel gives up; the late
   rank would otherwise take the early rank's unwritten output rows for valid ones - it finds the
   failure marker in its control words. A rank that never comes is handled with f2k_hx_abort.
"""
import time

import numpy as np
import pytest

from tests._util import assert_parity, dev_bf16, host_f32, normal_bits

pytestmark = pytest.mark.gpu

MS = 2_000_000          # about one millisecond of SM clock cycles


def _streams(n):
    import torch
    out = []
    while len({s.cuda_stream for s in out}) < n:
        out.append(torch.cuda.Stream())
    seen, uniq = set(), []
    for s in out:
        if s.cuda_stream not in seen:
            seen.add(s.cuda_stream)
            uniq.append(s)
    return uniq[:n]


@pytest.mark.timeout(120, method="thread")
def test_seqpar_peer_never_announces(orc):
    import torch
    from f2k_cuda_b200 import _lib
    from f2k_cuda_b200.seqpar import SequenceParallelAttention
    world, per, H, B, D = 2, 256, 2, 1, 128
    S = world * per
    q, k, v = (normal_bits(0xFA11, i, (B, S, H, D)) for i in range(3))
    _, ref = orc.joint_path(q_img=q, k_img=k, v_img=v)
    ranks = [SequenceParallelAttention(B, per, H, D, world, r) for r in range(world)]
    for r in ranks:
        assert r.ok(), r.last_error()
    for r in ranks:
        assert r.attach_in_process(ranks)
    streams = _streams(world)

    def put_inputs(r):
        with torch.cuda.stream(streams[r]):
            ks, vs = ranks[r].local_kv()
            ks.copy_(dev_bf16(k[:, r * per:(r + 1) * per])); vs.copy_(dev_bf16(v[:, r * per:(r + 1) * per]))
            dq = dev_bf16(q[:, r * per:(r + 1) * per])
            return dq, torch.full_like(dq, float("nan"))

    # ---- step 1: rank 1 never calls forward. Rank 0's kernel waits for the arrival word of rank
    # 1's shard, which can only come after rank 1's "written" word: it gives up after ~1 ms.
    assert ranks[0].set_wait_limits(MS, MS)
    io0 = put_inputs(0)
    streams[0].synchronize()
    t0 = time.perf_counter()
    assert ranks[0].forward(io0[0], io0[1], overlap=True, stream=streams[0]), ranks[0].last_error()
    streams[0].synchronize()                 # the kernel returns by itself (the copy stream is still parked)
    assert time.perf_counter() - t0 < 5.0
    assert ranks[0].abort(), ranks[0].last_error()        # host-side release of the parked stream waits
    st = ranks[0].device_status()            # synchronises the device: returns only because of the abort
    assert st & 1, "the expired wait must be reported"
    assert st & 4, "the abort must be reported"
    assert "abort" in ranks[0].last_error()
    assert ranks[0].device_status() == 0     # reported once, then clean

    # ---- rank 1 catches up with step 1 (rank 0's word and shard of that step are there)
    io1 = put_inputs(1)
    streams[1].synchronize()
    assert ranks[1].forward(io1[0], io1[1], overlap=True, stream=streams[1]), ranks[1].last_error()
    torch.cuda.synchronize()
    assert ranks[1].device_status() == 0, ranks[1].last_error()
    assert_parity(host_f32(io1[1]), ref[:, per:], "late rank, step 1")

    # ---- step 2: a normal step on the same handles, default limits again
    assert ranks[0].set_wait_limits(0, 0)
    ios = [put_inputs(r) for r in range(world)]
    torch.cuda.synchronize()
    for r in range(world):
        assert ranks[r].forward(ios[r][0], ios[r][1], overlap=True, stream=streams[r]), ranks[r].last_error()
    torch.cuda.synchronize()
    for r in range(world):
        assert ranks[r].device_status() == 0, ranks[r].last_error()
        assert_parity(host_f32(ios[r][1]), ref[:, r * per:(r + 1) * per], f"rank {r} after the failed step")
    assert _lib.lib.f2k_seqpar_abort(None) == _lib.F2K_ERR_INVALID


@pytest.mark.timeout(120, method="thread")
def test_attention_handle_is_usable_after_an_expired_wait(orc):
    """The single-GPU handle: same kernel, same exit path. The wait is made to expire through a
    world-2 sequence-parallel handle (the plain handle has no word to wait for); afterwards a plain
    attention call in the same context must be bit-identical to one made before."""
    import torch
    import f2k_cuda_b200 as f2k
    from f2k_cuda_b200.seqpar import SequenceParallelAttention
    B, S, H, D = 1, 384, 2, 128
    q, k, v = (dev_bf16(normal_bits(0xFA12, i, (B, S, H, D))) for i in range(3))
    att = f2k.Attention(f2k.Attention.Config(B, S, H, D))
    assert att.ok(), att.last_error()
    before, after = torch.empty_like(q), torch.empty_like(q)
    assert att.forward(q, k, v, before)
    assert att.device_status() == 0
    ranks = [SequenceParallelAttention(B, 128, H, D, 2, r) for r in range(2)]
    for r in ranks:
        assert r.ok() and r.attach_in_process(ranks)
    assert ranks[0].set_wait_limits(MS, MS)
    s0 = _streams(1)[0]
    o = torch.empty(B, 128, H, D, dtype=torch.bfloat16, device="cuda")
    assert ranks[0].forward(q[:, :128].contiguous(), o, overlap=True, stream=s0)
    s0.synchronize()
    assert ranks[0].abort()
    assert ranks[0].device_status() & 1
    assert att.forward(q, k, v, after)
    assert att.device_status() == 0
    assert torch.equal(before, after)


def _hx_ranks(world, per, H):
    from f2k_cuda_b200.headswap import HeadExchangeAttention
    ranks = [HeadExchangeAttention(per, H, 128, world, r) for r in range(world)]
    for r in ranks:
        assert r.ok(), r.last_error()
    for r in ranks:
        assert r.attach_in_process(ranks)
    return ranks


@pytest.mark.timeout(120, method="thread")
def test_head_exchange_marks_rows_a_failed_peer_did_not_write(orc):
    import torch
    import f2k_cuda_b200 as f2k
    from f2k_cuda_b200.inputs import Workload, make_problem
    world, per, H = 2, 256, 4
    w = Workload("hxf", 1, 0, ((16, 32),), seed=0xFA13)
    p = make_problem(w, heads=H)
    cos, sin = f2k.build_rope_4axis_tables((32,) * 4, p.pos_img, 2000.0)
    _, ref = orc.joint_path(q_img=p.q_img, k_img=p.k_img, v_img=p.v_img, gammas=(None, None, p.gammas[2], p.gammas[3]),
                            tables=(None, None, cos, sin), eps=1e-6)
    ranks = _hx_ranks(world, per, H)
    gq, gk = dev_bf16(p.gammas[2]), dev_bf16(p.gammas[3])
    dcos, dsin = torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda()
    shard = lambda x, r: dev_bf16(np.ascontiguousarray(x[:, r * per:(r + 1) * per]))  # noqa: E731

    def exchange(r):
        hx = ranks[r]
        assert hx.exchange_in(shard(p.q_img, r), shard(p.k_img, r), shard(p.v_img, r), gq, gk,
                              dcos[r * per:(r + 1) * per].contiguous(), dsin[r * per:(r + 1) * per].contiguous(),
                              1e-6), hx.last_error()

    # a call out of order is refused on the host
    assert not ranks[0].attend() and "without exchange_in" in ranks[0].last_error()
    exchange(0)
    assert not ranks[0].exchange_in(shard(p.q_img, 0), shard(p.k_img, 0), shard(p.v_img, 0), gq, gk, dcos, dsin, 1e-6)
    assert "previous step" in ranks[0].last_error()

    # ---- step 1: rank 0 is a millisecond too early for rank 1. Its kernel gives up on rank 1's
    # rows, skips the output rows it owed and says so in rank 1's control words before "done".
    assert ranks[0].set_wait_limits(MS, MS)
    torch.cuda.synchronize()
    assert ranks[0].attend(), ranks[0].last_error()
    torch.cuda.current_stream().synchronize()
    exchange(1)                                   # the late rank
    torch.cuda.synchronize()
    assert ranks[1].attend(), ranks[1].last_error()
    o0, o1 = ranks[0].output(), ranks[1].output()
    assert o0 is not None and o1 is not None
    torch.cuda.synchronize()
    assert ranks[0].device_status() & 1, "the early rank's expired wait"
    st1 = ranks[1].device_status()
    assert st1 == 2 and "peer" in ranks[1].last_error(), "the late rank must learn that rows it got are stale"

    # ---- step 2: normal, on the same handles
    assert ranks[0].set_wait_limits(0, 0)
    for r in range(world):
        exchange(r)
    torch.cuda.synchronize()
    for hx in ranks:
        assert hx.attend(), hx.last_error()
    torch.cuda.synchronize()
    for r, hx in enumerate(ranks):
        o = hx.output()
        torch.cuda.synchronize()
        assert hx.device_status() == 0, hx.last_error()
        assert_parity(host_f32(o), ref[:, r * per:(r + 1) * per], f"rank {r} after the failed step")


@pytest.mark.timeout(120, method="thread")
def test_head_exchange_abort_releases_the_output_wait():
    import torch
    world, per, H = 2, 128, 2
    ranks = _hx_ranks(world, per, H)
    mk = lambda: torch.randn(1, per, H, 128, device="cuda").to(torch.bfloat16)  # noqa: E731
    g = torch.ones(128, dtype=torch.bfloat16, device="cuda")
    tab = torch.zeros(per, 64, device="cuda")
    one = torch.ones(per, 64, device="cuda")
    s0 = _streams(1)[0]
    assert ranks[0].set_wait_limits(MS, MS)
    assert ranks[0].exchange_in(mk(), mk(), mk(), g, g, one, tab, 1e-6, stream=s0)
    assert ranks[0].attend(stream=s0)
    assert ranks[0].output(stream=s0) is not None          # parks s0 on rank 1's "done" word: rank 1 never comes
    time.sleep(0.2)
    assert not s0.query()
    assert ranks[0].abort(), ranks[0].last_error()
    s0.synchronize()
    st = ranks[0].device_status()
    assert st & 4 and st & 1
    assert ranks[0].device_status() == 0
