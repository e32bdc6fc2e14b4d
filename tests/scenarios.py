"""Cache-semantics scenarios ported from the reference's own unit tests
(Tests/MLXLMTests/KVCacheTests.swift, KVCacheRoundTests.swift). Each scenario is
written once against a small backend interface and runs twice: on the numpy
oracle (CPU suite, pins the oracle to the reference's expectations) and on the
CUDA library through its C ABI (GPU suite).
"""
from __future__ import annotations

import numpy as np


class OracleBackend:
    name = "oracle"

    def __init__(self, oracle):
        self.o = oracle

    def arr(self, a: np.ndarray):
        return np.ascontiguousarray(a, dtype=np.float32)

    def to_np(self, a) -> np.ndarray:
        return np.asarray(a)

    def rotating(self, max_size, keep=0, step=256):
        return self.o.RotatingKVCache(max_size, keep, step)

    def simple(self, step=256):
        return self.o.KVCacheSimple(step)

    def quantized(self, group_size=64, bits=8):
        return self.o.QuantizedKVCache(group_size, bits)

    def begin_round(self, cache, width=8):
        return _OracleRound(self.o, cache, width)

    def rewind(self, cache, count):
        r = getattr(cache, "_last_restore", None)
        valid = getattr(cache, "_restore_valid", False)
        n = self.o.rewind_last_round(cache, r if valid else None, count)
        cache._restore_valid = False
        return n

    def invalidate(self, cache):
        cache._restore_valid = False


class _OracleRound:
    def __init__(self, o, cache, width):
        self.r = o.StagedRound(cache, width)
        self.cache = cache
        cache._restore_valid = False

    def update(self, k, v):
        return self.r.update(k, v)

    def commit(self, accepted):
        self.cache._last_restore = self.r.commit(accepted)
        self.cache._restore_valid = self.cache._last_restore is not None

    def rollback(self):
        self.commit(0)


class GpuBackend:
    name = "gpu"

    def __init__(self, kvc, device):
        self.k = kvc
        self.device = device

    def arr(self, a: np.ndarray):
        import torch
        return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(self.device)

    def to_np(self, a) -> np.ndarray:
        return a.detach().float().cpu().numpy()

    def rotating(self, max_size, keep=0, step=256):
        return self.k.RotatingKVCache(max_size, keep, step)

    def simple(self, step=256):
        return self.k.KVCacheSimple(step)

    def quantized(self, group_size=64, bits=8):
        return self.k.QuantizedKVCache(group_size, bits)

    def begin_round(self, cache, width=8):
        return _GpuRound(self.k, cache, width)

    def rewind(self, cache, count):
        if isinstance(cache, self.k.RotatingKVCache):
            return cache.rewind_last_round(count)
        return cache.trim(count)

    def invalidate(self, cache):
        pass


class _GpuRound:
    def __init__(self, k, cache, width):
        self.r = k.StagedRound(cache, width)

    def update(self, k, v):
        return self.r.update(k, v)

    def commit(self, accepted):
        self.r.commit(accepted)

    def rollback(self):
        self.r.rollback()


# ---------------------------------------------------------------------------
# fixtures of the reference tests
# ---------------------------------------------------------------------------

def positioned_kv(be, positions, head_dim=2):
    """Keys carry +p, values -p in every element (KVCacheTests.swift:1282-1293)."""
    pos = np.asarray(list(positions), dtype=np.float32)
    k = np.repeat(pos[:, None], head_dim, axis=1)[None, None]
    return be.arr(k), be.arr(-k)


def encoded_positions(be, keys):
    a = be.to_np(keys)
    return [int(round(x)) for x in a[0, 0, :, 0]]


def fill_one_at_a_time(be, cache, positions):
    for p in positions:
        k, v = positioned_kv(be, range(p, p + 1))
        cache.update(k, v)


# ---------------------------------------------------------------------------
# scenarios (each returns nothing and asserts)
# ---------------------------------------------------------------------------

def logical_view_is_none_before_first_write(be):
    assert be.rotating(8, 0).logical_view(8) is None  # KVCacheTests.swift:1308-1310


def logical_view_chronological_tail_past_wrap(be):
    cache = be.rotating(8, 0)
    fill_one_at_a_time(be, cache, range(20))
    assert cache.offset == 20
    full = cache.logical_view(8)
    assert encoded_positions(be, full[0]) == list(range(12, 20))  # KVCacheTests.swift:1320-1323
    assert [-p for p in encoded_positions(be, full[1])] == list(range(12, 20))
    short = cache.logical_view(3)
    assert encoded_positions(be, short[0]) == [17, 18, 19]


def logical_view_clamps_tail(be):
    cache = be.rotating(8, 0)
    fill_one_at_a_time(be, cache, range(5))
    assert encoded_positions(be, cache.logical_view(99)[0]) == list(range(5))
    assert encoded_positions(be, cache.logical_view(5)[0]) == list(range(5))
    assert cache.logical_view(0)[0].shape[2] == 0
    assert cache.logical_view(-1)[0].shape[2] == 0


def logical_view_leaves_ring_untouched(be):
    cache = be.rotating(8, 0)
    fill_one_at_a_time(be, cache, range(20))
    before = [be.to_np(a).copy() for a in cache.state]
    before_off, before_meta = cache.offset, list(cache.meta_state)
    cache.logical_view(7)
    cache.logical_view(3)
    after = [be.to_np(a) for a in cache.state]
    assert len(before) == len(after)
    for b, a in zip(before, after):
        assert b.shape == a.shape and np.array_equal(a, b)
    assert cache.offset == before_off and list(cache.meta_state) == before_meta


def logical_view_pinned_prefix(be):
    cache = be.rotating(8, 2)
    fill_one_at_a_time(be, cache, range(20))
    pos = encoded_positions(be, cache.logical_view(5)[0])
    assert len(pos) == 5 and pos[:2] == [0, 1] and pos[2:] == sorted(pos[2:])
    for tail in range(3):
        v = cache.logical_view(tail)
        assert encoded_positions(be, v[0]) == [0, 1]
        assert [-p for p in encoded_positions(be, v[1])] == [0, 1]
    pos3 = encoded_positions(be, cache.logical_view(3)[0])
    assert len(pos3) == 3 and pos3[:2] == [0, 1]
    small = be.rotating(8, 4)
    fill_one_at_a_time(be, small, range(2))
    assert encoded_positions(be, small.logical_view(0)[0]) == [0, 1]
    assert encoded_positions(be, small.logical_view(9)[0]) == [0, 1]


def logical_view_plus_new_rows_equals_write_presentation(be):
    window, staged = 8, 4
    cache = be.rotating(window, 0)
    fill_one_at_a_time(be, cache, range(20))
    view = cache.logical_view(window - 1)
    view_k, view_v = be.to_np(view[0]).copy(), be.to_np(view[1]).copy()
    mask = cache.make_mask(staged, window, False)
    nk, nv = positioned_kv(be, range(20, 20 + staged))
    pk, pv = cache.update(nk, nv)
    ck = np.concatenate([view_k, be.to_np(nk)], axis=2)
    cv = np.concatenate([view_v, be.to_np(nv)], axis=2)
    assert np.array_equal(be.to_np(pk), ck) and np.array_equal(be.to_np(pv), cv)
    assert not isinstance(mask, str), "expected an array mask once offset + n exceeds the window"
    assert mask.shape[-1] == ck.shape[2] and mask.shape[-2] == staged


def trimmable_boundary(be):
    c = be.rotating(8)
    c.offset = 3
    assert c.is_trimmable_after(4) and not c.is_trimmable_after(5)  # KVCacheTests.swift:136-142
    c.offset = 8
    assert not c.is_trimmable and not c.is_trimmable_after(0)
    c.offset = 9
    assert not c.is_trimmable
    assert be.simple().is_trimmable_after(1000)


def quantized_meta_state(be):
    c = be.quantized()
    c.meta_state = ["256", "11", "32", "4"]  # KVCacheTests.swift:503-512
    assert c.offset == 11 and c.group_size == 32 and c.bits == 4
    assert list(c.meta_state) == ["256", "11", "32", "4"]
    c2 = be.quantized()
    c2.meta_state = ["256", "5", "32", "4"]
    cp = c2.copy()
    assert cp.offset == 5 and cp.group_size == 32 and cp.bits == 4 and list(cp.meta_state) == list(c2.meta_state)
    s = be.simple()
    s.offset = 7
    q = s.to_quantized(128, 4)  # KVCacheTests.swift:526-536
    assert q.offset == 7 and q.group_size == 128 and q.bits == 4
    assert list(q.meta_state) == ["256", "7", "128", "4"]


def rotating_meta_state_roundtrip(be):
    c = be.rotating(8, 2, 4)
    fill_one_at_a_time(be, c, range(11))
    m = list(c.meta_state)
    assert m[:3] == ["2", "8", "4"] and m[3] == "11" and m[5] == "modelNative"
    cp = c.copy()
    assert list(cp.meta_state) == m
    assert [np.array_equal(be.to_np(a), be.to_np(b)) for a, b in zip(c.state, cp.state)] == [True, True]


def ring_one_at_a_time_trace(be):
    """Single-token growth: 256 rows, then 512 with idx = prev, first wrap at offset 512."""
    c = be.rotating(512, 0, 256)
    fill_one_at_a_time(be, c, range(256))
    assert c.state[0].shape[2] == 256 and list(c.meta_state)[3:5] == ["256", "256"]
    fill_one_at_a_time(be, c, range(256, 257))
    assert list(c.meta_state)[3:5] == ["257", "257"]
    fill_one_at_a_time(be, c, range(257, 512))
    assert c.state[0].shape[2] == 512 and list(c.meta_state)[3:5] == ["512", "512"]
    fill_one_at_a_time(be, c, range(512, 513))
    assert list(c.meta_state)[3:5] == ["513", "1"]
    assert encoded_positions(be, c.state[0])[:3] == [512, 1, 2]


def ring_prefill_then_decode_trace(be, chunk=8, window=8, chunks=4):
    """The sliding-window benchmark shape in miniature: chunked prefill
    (buffer lengths window, 2*window-1, ...), hand-over trim at the first
    single-token write, then in-place wraparound."""
    c = be.rotating(window, 0)
    lengths = []
    for i in range(chunks):
        k, v = positioned_kv(be, range(i * chunk, (i + 1) * chunk))
        pk, _ = c.update(k, v)
        lengths.append(pk.shape[2])
    assert lengths == [chunk] + [window + chunk - 1] * (chunks - 1)
    total = chunk * chunks
    assert c.offset == total and list(c.meta_state)[4] == str(window + chunk - 1)
    k, v = positioned_kv(be, range(total, total + 1))
    pk, _ = c.update(k, v)
    assert pk.shape[2] == window
    expect = [total] + list(range(total - window + 1, total))
    assert encoded_positions(be, pk) == expect
    assert list(c.meta_state)[3:5] == [str(total + 1), "1"]
    for p in range(total + 1, total + 1 + 2 * window):
        k, v = positioned_kv(be, range(p, p + 1))
        pk, _ = c.update(k, v)
    last = total + 2 * window
    assert sorted(encoded_positions(be, pk)) == list(range(last - window + 1, last + 1))


def overlay_leaves_ring_untouched(be):
    live = be.rotating(8, 0)
    fill_one_at_a_time(be, live, range(20))
    snap = ([be.to_np(a).copy() for a in live.state], live.offset, list(live.meta_state))
    rnd = be.begin_round(live)
    rnd.update(*positioned_kv(be, range(20, 24)))
    assert all(np.array_equal(be.to_np(a), b) for a, b in zip(live.state, snap[0]))
    assert live.offset == snap[1] and list(live.meta_state) == snap[2]
    rnd.rollback()
    assert all(np.array_equal(be.to_np(a), b) for a, b in zip(live.state, snap[0]))
    assert live.offset == snap[1] and list(live.meta_state) == snap[2]


def overlay_write_through_rollback(be):
    live = be.simple()
    fill_one_at_a_time(be, live, range(6))
    rnd = be.begin_round(live)
    rnd.update(*positioned_kv(be, range(6, 10)))
    assert live.offset == 10
    rnd.rollback()
    assert live.offset == 6


def overlay_presentation_equals_live_write(be):
    staged, written = be.rotating(8, 0), be.rotating(8, 0)
    for c in (staged, written):
        fill_one_at_a_time(be, c, range(20))
    rnd = be.begin_round(staged)
    m1 = staged.make_mask(4, 8, False)
    m2 = written.make_mask(4, 8, False)
    nk, nv = positioned_kv(be, range(20, 24))
    pk, pv = rnd.update(nk, nv)
    rk, rv = written.update(nk, nv)
    assert np.array_equal(be.to_np(pk), be.to_np(rk)) and np.array_equal(be.to_np(pv), be.to_np(rv))
    assert not isinstance(m1, str) and tuple(m1.shape) == tuple(m2.shape)
    assert m1.shape[-1] == pk.shape[2]
    assert np.array_equal(be.to_np(m1) != 0, be.to_np(m2) != 0)


def commit_equivalence(be, window, rounds, prefill, keep=0):
    live, ref = be.rotating(window, keep), be.rotating(window, keep)
    if prefill > 0:
        k, v = positioned_kv(be, range(prefill))
        live.update(k, v)
        ref.update(k, v)
    nxt = prefill
    for i, (written, accepted) in enumerate(rounds):
        rnd = be.begin_round(live)
        rnd.update(*positioned_kv(be, range(nxt, nxt + written)))
        rnd.commit(accepted)
        if accepted > 0:
            ref.update(*positioned_kv(be, range(nxt, nxt + accepted)))
        nxt += accepted
        assert live.offset == ref.offset, f"round {i}"
        lw, rw = live.logical_view(window), ref.logical_view(window)
        if lw is None or rw is None:
            assert lw is None and rw is None
            continue
        assert encoded_positions(be, lw[0]) == encoded_positions(be, rw[0]), f"round {i}"
        assert [-p for p in encoded_positions(be, lw[1])] == encoded_positions(be, rw[0])


COMMIT_CASES = [
    dict(window=8, rounds=[(4, 0)] * 3, prefill=6),
    dict(window=8, rounds=[(4, 4)] * 6, prefill=6),
    dict(window=8, rounds=[(4, 1), (4, 4), (4, 0), (4, 2), (4, 3), (4, 1), (4, 4), (4, 2), (4, 0), (4, 3)], prefill=7),
    dict(window=8, keep=2, rounds=[(4, 2), (4, 4), (4, 1), (4, 3), (4, 0), (4, 4)], prefill=6),
    dict(window=8, rounds=[(4, 3), (4, 4), (4, 1), (4, 4), (4, 2)], prefill=0),
    dict(window=4, rounds=[(6, 2), (6, 6), (6, 0), (6, 3)], prefill=3),
    dict(window=4, rounds=[(8, 5), (8, 8), (8, 1)], prefill=0),
]


def rewind_matches_emitted_only_replay(be, window, prefill, written, retaining, rewinding, keep=0):
    live, ref = be.rotating(window, keep), be.rotating(window, keep)
    k, v = positioned_kv(be, range(prefill))
    live.update(k, v)
    ref.update(k, v)
    rnd = be.begin_round(live, written)
    rnd.update(*positioned_kv(be, range(prefill, prefill + written)))
    rnd.commit(retaining)
    assert be.rewind(live, rewinding) == rewinding
    survive = retaining - rewinding
    if survive > 0:
        ref.update(*positioned_kv(be, range(prefill, prefill + survive)))
    assert live.offset == ref.offset
    lw, rw = live.logical_view(window), ref.logical_view(window)
    assert encoded_positions(be, lw[0]) == encoded_positions(be, rw[0])
    assert list(live.meta_state) == list(ref.meta_state)


REWIND_CASES = ([dict(window=8, prefill=20, written=4, retaining=4, rewinding=r) for r in (1, 2, 3, 4)] +
                [dict(window=32, prefill=4, written=4, retaining=4, rewinding=r) for r in (1, 2, 3)] +
                [dict(window=8, keep=2, prefill=20, written=4, retaining=3, rewinding=2),
                 dict(window=8, prefill=20, written=4, retaining=3, rewinding=3)])


def rewind_refused_after_another_write(be):
    live = be.rotating(8, 0)
    live.update(*positioned_kv(be, range(20)))
    rnd = be.begin_round(live, 4)
    rnd.update(*positioned_kv(be, range(20, 24)))
    rnd.commit(4)
    live.update(*positioned_kv(be, range(24, 25)))
    be.invalidate(live)
    assert be.rewind(live, 2) == 0  # KVCacheRoundTests.swift:756-768
    assert live.offset == 25


ALL_SIMPLE = [
    logical_view_is_none_before_first_write,
    logical_view_chronological_tail_past_wrap,
    logical_view_clamps_tail,
    logical_view_leaves_ring_untouched,
    logical_view_pinned_prefix,
    logical_view_plus_new_rows_equals_write_presentation,
    trimmable_boundary,
    quantized_meta_state,
    rotating_meta_state_roundtrip,
    ring_one_at_a_time_trace,
    ring_prefill_then_decode_trace,
    overlay_leaves_ring_untouched,
    overlay_write_through_rollback,
    overlay_presentation_equals_live_write,
    rewind_refused_after_another_write,
]
