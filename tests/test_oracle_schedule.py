"""The oracle's tile schedule is an exact cover of the eager mask, and the library's C schedule
(host arithmetic behind the C ABI) agrees with the oracle number for number."""

import itertools
import random

import pytest

from oracle import schedule as S

WINDOWS = [[0, 256, 0, 0], [0, 0, 0, 256], [0, 1024, 0, 0], [64, 94, 188, 256], [64, 94, 0, 256], [0, 300, 100, 200],
           [40, 100, 37, 77]]
SHAPES = [(1024, 1024), (987, 1024), (300, 1024)]
TILES = [(64, 64), (128, 128), (128, 64), (64, 128)]


def _cover_fwd(sq, sk, window, tm, tn, causal, local, ns, split, gpack=1):
    seen = {}
    m_blocks = -(-sq * gpack // tm)
    for mb in range(m_blocks):
        for sp in range(ns):
            sched = S.fwd_schedule(sq, sk, mb, sp, window, ns, tn, tm, causal, local, split, gpack)
            if sched.is_empty():
                continue
            for n, mode in S.fwd_tiles(sched, causal, local):
                for r in range(tm):
                    qi = (mb * tm + r) // gpack
                    g = (mb * tm + r) % gpack
                    if qi >= sq:
                        continue
                    for kk in range(n * tn, min((n + 1) * tn, sk)):
                        if S.visible(qi, kk, sq, sk, window, mode):
                            key = (qi, g, kk)
                            seen[key] = seen.get(key, 0) + 1
    return seen


def _expected(sq, sk, window, causal, local, gpack=1):
    exp = set()
    for qi in range(sq):
        for kk in range(sk):
            if S.allowed(qi, kk, sq, sk, window, causal, local):
                for g in range(gpack):
                    exp.add((qi, g, kk))
    return exp


@pytest.mark.parametrize("window", WINDOWS[:4])
@pytest.mark.parametrize("ns", [1, 3])
def test_fwd_exact_cover_local(window, ns):
    # small sizes keep the pure-Python brute force to seconds; windows scaled down with them
    scale = 8
    w = [x // scale for x in window]
    for (sq, sk), (tm, tn) in itertools.product([(128, 128), (123, 128), (37, 128)], [(16, 16), (32, 16), (16, 32)]):
        seen = _cover_fwd(sq, sk, w, tm, tn, True, True, ns, ns > 1)
        assert set(seen) == _expected(sq, sk, w, True, True), (sq, sk, tm, tn, w, ns)
        assert all(v == 1 for v in seen.values())


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("ns", [1, 2, 5])
def test_fwd_exact_cover_nonlocal(causal, ns):
    for (sq, sk), (tm, tn) in itertools.product([(128, 128), (123, 128), (37, 128), (128, 100)], [(16, 16), (32, 16)]):
        if causal and sq > sk:
            continue
        seen = _cover_fwd(sq, sk, [0, 0, 0, 0], tm, tn, causal, False, ns, ns > 1)
        assert set(seen) == _expected(sq, sk, [0, 0, 0, 0], causal, False)
        assert all(v == 1 for v in seen.values())


def test_fwd_exact_cover_pack_gqa():
    for gpack in (2, 4):
        seen = _cover_fwd(60, 96, [0, 0, 0, 0], 16, 16, True, False, 1, False, gpack)
        assert set(seen) == _expected(60, 96, [0, 0, 0, 0], True, False, gpack)
        assert all(v == 1 for v in seen.values())


@pytest.mark.parametrize("local", [False, True])
@pytest.mark.parametrize("ns", [1, 3])
def test_bwd_exact_cover(local, ns):
    window = [8, 12, 23, 32] if local else [0, 0, 0, 0]
    for (sq, sk), (tm, tn), causal in itertools.product([(128, 128), (123, 128), (37, 128)], [(16, 16), (32, 16), (16, 32)],
                                                        [True, False]):
        if local and not causal:
            continue
        seen = {}
        for nb in range(-(-sk // tn)):
            for sp in range(ns):
                sched = S.bwd_schedule(sq, sk, nb, sp, window, ns, tn, tm, causal, local, ns > 1)
                if sched.is_empty():
                    continue
                for m, mode in S.bwd_tiles(sched, causal, local):
                    for qi in range(m * tm, min((m + 1) * tm, sq)):
                        for kk in range(nb * tn, min((nb + 1) * tn, sk)):
                            if S.visible(qi, kk, sq, sk, window, mode):
                                seen[(qi, kk)] = seen.get((qi, kk), 0) + 1
        exp = {(qi, kk) for qi in range(sq) for kk in range(sk) if S.allowed(qi, kk, sq, sk, window, causal, local)}
        assert set(seen) == exp, (sq, sk, tm, tn, causal, local, ns)
        assert all(v == 1 for v in seen.values())


def test_bwd_tiles_stay_inside_the_query_range():
    """A short query against a long causal key sequence: the reference's unclamped m_min_no_mask
    (scheduler.py:1028-1043) points past the last query tile; the listed tiles must not."""
    for sq, sk in [(77, 300), (128, 300), (5, 1000), (129, 700)]:
        for nb in range(-(-sk // 128)):
            sched = S.bwd_schedule(sq, sk, nb, 0, [0, 0, 0, 0], 1, 128, 128, True, False, False)
            tiles = [m for m, _ in S.bwd_tiles(sched, True, False)]
            assert all(0 <= m < -(-sq // 128) for m in tiles), (sq, sk, nb, tiles)
            assert len(set(tiles)) == len(tiles)
    # the case that motivated this: the raw schedule value really is out of range
    raw = S.bwd_schedule(77, 300, 2, 0, [0, 0, 0, 0], 1, 128, 128, True, False, False)
    assert raw.m_min_no_mask == 2 and raw.m_max == 1


def _decode_cover(sk, window, tn, nsub, gpack, cover):
    seen = {}
    for sp in range(nsub):
        sc = S.fwd_schedule(1, sk, 0, sp, window, nsub, tn, 16, False, True, True, gpack, cover_single_query=cover)
        if sc.is_empty():
            continue
        for n, mode in S.fwd_tiles(sc, True, True):
            for kk in range(n * tn, min((n + 1) * tn, sk)):
                if S.visible(0, kk, 1, sk, window, mode):
                    seen[kk] = seen.get(kk, 0) + 1
    exp = {kk for kk in range(sk) if S.allowed(0, kk, 1, sk, window, False, True)}
    return seen, exp


def test_decode_schedule_cover():
    """Single query position + local window + split-KV. With the reference's rounding the first partial
    tile of the near band is not visited when the band is not tile aligned (a property of the reference,
    recorded here); the decode kernel's variant covers the mask exactly once."""
    for window in ([32, 200, 100, 160], [0, 300, 0, 64], [64, 128, 256, 1024]):
        for tn, nsub, gpack in itertools.product((16, 64), (1, 4, 12), (1, 16)):
            seen, exp = _decode_cover(1500, window, tn, nsub, gpack, cover=True)
            assert set(seen) == exp and all(v == 1 for v in seen.values()), (window, tn, nsub, gpack)
    # the forward kernel's tile size with one query position (flash_*_attn_func called with Sq = 1)
    for window in ([1, 128, 128, 260], [32, 200, 100, 160]):
        for nsub in (2, 3, 5):
            seen, exp = _decode_cover(1100, window, 128, nsub, 1, cover=True)
            assert set(seen) == exp and all(v == 1 for v in seen.values()), (window, nsub)
    seen, exp = _decode_cover(1500, [32, 200, 100, 160], 16, 4, 16, cover=False)
    assert sorted(exp - set(seen)) == [1340, 1341, 1342, 1343]


def test_c_schedule_matches_oracle():
    from flash_sparse_attn import _lib

    rng = random.Random(0)
    for _ in range(3000):
        tm, tn = rng.choice(TILES)
        sk = rng.randint(1, 3000)
        sq = rng.choice([1, sk, rng.randint(1, sk)])
        local = rng.random() < 0.6
        causal = rng.random() < 0.6
        window = [rng.choice([0, 17, 64, 130]), rng.randint(0, 600), rng.randint(0, 400), rng.randint(0, 700)]
        ns = rng.choice([1, 1, 2, 3, 7])
        split = ns > 1 or rng.random() < 0.2
        gpack = rng.choice([1, 1, 2, 4, 8])
        mb = rng.randint(0, max(0, -(-sq * gpack // tm) - 1))
        sp = rng.randint(0, ns - 1)
        cover = rng.random() < 0.3
        ref = S.fwd_schedule(sq, sk, mb, sp, window, ns, tn, tm, causal, local, split, gpack, cover).as_list()
        got = _lib.debug_fwd_schedule(sq, sk, mb, sp, window, ns, tn, tm, causal, local, split, gpack, cover)
        assert got == ref, ("fwd", sq, sk, mb, sp, window, ns, tn, tm, causal, local, split, gpack, cover)
        nb = rng.randint(0, max(0, -(-sk // tn) - 1))
        ref = S.bwd_schedule(sq, sk, nb, sp, window, ns, tn, tm, causal, local, split).as_list()
        got = _lib.debug_bwd_schedule(sq, sk, nb, sp, window, ns, tn, tm, causal, local, split)
        assert got == ref, ("bwd", sq, sk, nb, sp, window, ns, tn, tm, causal, local, split)


# --------------------------------------------------------------------------------------------------
# pinned to the reference's own integers: golden/schedule.npz holds what block_info.py and the three
# `create` schedulers of scheduler.py return when their Triton source runs on the CPU interpreter
# (tests/golden/make_schedule_golden.py); everything below is compared with ==
# --------------------------------------------------------------------------------------------------
def _golden():
    import numpy as np
    import os

    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "schedule.npz"))


def test_oracle_block_ranges_equal_reference():
    z = _golden()
    for a, r in zip(z["fwd_args"].tolist(), z["fwd_out"].tolist()):
        sq, sk, mb, sp, s_, l_, r_, n_, ns, tn, tm, causal, local, split, gpack = a
        got = S.n_block_min_max(sq, sk, mb, sp, [s_, l_, r_, n_], ns, tn, tm, bool(causal), bool(local), bool(split), gpack)
        assert list(got) == r, ("n_block_min_max", a)
    for a, r in zip(z["bwd_args"].tolist(), z["bwd_out"].tolist()):
        sq, sk, nb, sp, s_, l_, r_, n_, ns, tn, tm, causal, local, split = a
        got = S.m_block_min_max(sq, sk, nb, sp, [s_, l_, r_, n_], ns, tn, tm, bool(causal), bool(local), bool(split))
        assert list(got) == r, ("m_block_min_max", a)
    for a, r in zip(z["edges_n_args"].tolist(), z["edges_n_out"].tolist()):
        sq, sk, mb, n_min, l_, r_, n_, tn, tm, local, gpack = a
        got = [S._n_min_causal_local_mask(sq, sk, mb, n_min, r_, n_, tn, tm, bool(local), gpack),
               S._n_min_before_local_mask(sq, sk, mb, n_min, [0, l_, r_, n_], tn, tm, bool(local), gpack)]
        assert got == r, ("edges_n", a)
    for a, r in zip(z["edges_m_args"].tolist(), z["edges_m_out"].tolist()):
        sq, sk, nb, m_lim, l_, r_, n_, tn, tm, causal, local = a
        got = [S._m_min_causal_local_mask(sq, sk, nb, m_lim, r_, n_, tn, tm, bool(causal), bool(local)),
               S._m_max_before_local_mask(sq, sk, nb, m_lim, [0, l_, r_, n_], tn, tm, bool(local))]
        assert got == r, ("edges_m", a)
    for a, r in zip(z["topk_args"].tolist(), z["topk_out"].tolist()):
        topk, sp, ns, tn = a
        sc = S.topk_schedule(topk, sp, ns, tn)
        assert [sc.n_min, sc.n_max] == r, ("topk", a)


def test_oracle_and_library_schedules_equal_reference_schedulers():
    """The nine numbers of AttnFwdBlockScheduler.create / AttnBwdBlockScheduler.create / AttnDecBlockScheduler.create:
    oracle/schedule.py and the C schedule behind fsa_debug_*_schedule both reproduce them exactly."""
    from flash_sparse_attn import _lib

    z = _golden()
    for a, r in zip(z["fwd_args"].tolist(), z["fwd_create"].tolist()):
        sq, sk, mb, sp, s_, l_, r_, n_, ns, tn, tm, causal, local, split, gpack = a
        w = [s_, l_, r_, n_]
        assert S.fwd_schedule(sq, sk, mb, sp, w, ns, tn, tm, bool(causal), bool(local), bool(split), gpack).as_list() == r, a
        assert _lib.debug_fwd_schedule(sq, sk, mb, sp, w, ns, tn, tm, causal, local, split, gpack) == r, ("C fwd", a)
    for a, r in zip(z["bwd_args"].tolist(), z["bwd_create"].tolist()):
        sq, sk, nb, sp, s_, l_, r_, n_, ns, tn, tm, causal, local, split = a
        w = [s_, l_, r_, n_]
        assert S.bwd_schedule(sq, sk, nb, sp, w, ns, tn, tm, bool(causal), bool(local), bool(split)).as_list() == r, a
        assert _lib.debug_bwd_schedule(sq, sk, nb, sp, w, ns, tn, tm, causal, local, split) == r, ("C bwd", a)
    for a, r in zip(z["dec_args"].tolist(), z["dec_create"].tolist()):
        sk, sp, s_, l_, r_, n_, ns, topk, tn, tm, local, gather, gpack = a
        if gather:
            got = S.topk_schedule(topk, sp, ns, tn).as_list()
        else:
            w = [s_, l_, r_, n_]
            got = S.fwd_schedule(1, sk, 0, sp, w, ns, tn, tm, False, bool(local), True, gpack).as_list()
            assert _lib.debug_fwd_schedule(1, sk, 0, sp, w, ns, tn, tm, 0, local, 1, gpack) == r, ("C dec", a)
        assert got == r, ("dec", a)
