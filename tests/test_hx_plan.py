"""Host-side planning of the in-kernel head exchange, checked on CPU through the C ABI.

Two pieces of arithmetic decide whether the fused form (f2k_hx_forward) can work at all:
 * the chunk queue: every 16-token block of Q and of K/V for every destination must be sent
   exactly once, and the rows the first wave of CTAs needs must come first;
 * the K/V walk: every destination walks K/V as two pieces of the whole buffer and waits, per
   128-token tile of that walk, for a count of delivered blocks; the senders must count in
   exactly those tiles, ceil(tokens of the tile / 16) times in total.
Shapes: the benchmark's long jobs over 2, 4 and 8 ranks, and ragged small ones.
"""
import ctypes as C

import numpy as np
import pytest

TILE, BLOCK = 128, 16


@pytest.fixture(scope="module")
def lib():
    from f2k_cuda_b200.build import build
    L = C.CDLL(str(build()))
    L.f2k_hx_exchange_plan.argtypes = [C.c_int] * 4 + [C.POINTER(C.c_int), C.c_int, C.POINTER(C.c_int)]
    L.f2k_hx_kv_walk_tile.argtypes = [C.c_int] * 4 + [C.POINTER(C.c_int)]
    return L


def walk_tile(lib, world, seq_local, dst, token):
    t = C.c_int(-1)
    assert lib.f2k_hx_kv_walk_tile(world, seq_local, dst, token, C.byref(t)) == 0
    return t.value


def plan(lib, world, seq_local, hpr, sms=148):
    buf = (C.c_int * (4 * 64))()
    n = C.c_int(0)
    assert lib.f2k_hx_exchange_plan(world, seq_local, hpr, sms, buf, 64, C.byref(n)) == 0
    assert 0 < n.value <= 32, n.value
    return np.array(buf[:4 * n.value]).reshape(n.value, 4)


SHAPES = [(8, 2112, 4), (4, 4224, 8), (2, 8448, 16), (8, 1088, 4), (2, 4352, 16), (1, 4608, 32), (1, 384, 2),
          (2, 256, 2), (4, 200, 1), (8, 16, 4), (3, 1000, 2)]


@pytest.mark.parametrize("world,seq_local,hpr", SHAPES)
def test_queue_sends_every_block_once(lib, world, seq_local, hpr):
    r = plan(lib, world, seq_local, hpr)
    n_sub = -(-seq_local // BLOCK)
    seen = np.zeros((2, world, n_sub), dtype=int)
    for kind, step, sub0, n in r:
        assert kind in (0, 1) and 0 <= step < world and sub0 >= 0 and n > 0 and sub0 + n <= n_sub
        seen[kind, step, sub0:sub0 + n] += 1
    assert (seen == 1).all()
    assert r[:, 3].sum() == 2 * world * n_sub


@pytest.mark.parametrize("world,seq_local,hpr", SHAPES)
def test_queue_starts_with_the_first_waves_query_rows(lib, world, seq_local, hpr):
    sms = 148
    r = plan(lib, world, seq_local, hpr, sms)
    tiles_per_seg = -(-seq_local // TILE)
    first_tiles = min(2 * -(-sms // hpr), world * tiles_per_seg)
    # the leading Q ranges cover exactly the query tiles of the first `sms` CTAs, in ring order
    lead = []
    for kind, step, sub0, n in r:
        if kind != 0:
            break
        lead.append((step, sub0, n))
    assert lead and [s for s, _, _ in lead] == list(range(len(lead)))
    covered = 0
    for step, sub0, n in lead:
        assert sub0 == 0
        covered += min(tiles_per_seg, -(-n * BLOCK // TILE))
    assert covered == first_tiles
    # K/V of the rank's own tokens (ring step 0) comes right after them
    assert tuple(r[len(lead)][:3]) == (1, 0, 0)


@pytest.mark.parametrize("world,seq_local", [(8, 2112), (4, 4224), (2, 8448), (8, 1088), (2, 256), (8, 16), (3, 1008),
                                              (1, 4608)])
def test_walk_counters_get_what_the_consumer_waits_for(lib, world, seq_local):
    assert seq_local % BLOCK == 0            # the walk is used only then
    total = world * seq_local
    for dst in range(world):
        start = dst * seq_local
        pieces = [n for n in (total - start, start) if n > 0]
        expected = []                        # blocks the consumer waits for, per tile of its walk
        for n in pieces:
            for t in range(-(-n // TILE)):
                expected.append(-(-min(TILE, n - t * TILE) // BLOCK))
        got = np.zeros(len(expected), dtype=int)
        for src in range(world):
            for tok0 in range(0, seq_local, BLOCK):
                t = walk_tile(lib, world, seq_local, dst, src * seq_local + tok0)
                assert 0 <= t < len(expected)
                # a block never straddles two tiles of the walk
                assert t == walk_tile(lib, world, seq_local, dst, src * seq_local + tok0 + BLOCK - 1)
                got[t] += 1
        assert (got == np.array(expected)).all(), (dst, got, expected)
        # the walk starts with the destination's own tokens
        assert walk_tile(lib, world, seq_local, dst, start) == 0


def test_plan_refuses_bad_arguments(lib):
    buf, n, t = (C.c_int * 8)(), C.c_int(0), C.c_int(0)
    assert lib.f2k_hx_exchange_plan(0, 128, 4, 148, buf, 2, C.byref(n)) != 0
    assert lib.f2k_hx_exchange_plan(9, 128, 4, 148, buf, 2, C.byref(n)) != 0
    assert lib.f2k_hx_exchange_plan(2, 128, 4, 148, None, 2, C.byref(n)) != 0
    assert lib.f2k_hx_exchange_plan(2, 128, 4, 148, buf, 2, None) != 0
    assert lib.f2k_hx_exchange_plan(2, 128, 4, 148, None, 0, C.byref(n)) == 0 and n.value > 0     # count only
    assert lib.f2k_hx_kv_walk_tile(2, 128, 2, 0, C.byref(t)) != 0
    assert lib.f2k_hx_kv_walk_tile(2, 128, 0, 256, C.byref(t)) != 0
    assert lib.f2k_hx_kv_walk_tile(2, 128, 0, 0, None) != 0
