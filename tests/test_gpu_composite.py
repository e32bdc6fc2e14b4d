"""ChunkedKVCache, CacheList and the batch-length masks (KVCache.swift:1213-1304, :1556-1726, :253-275)
against the oracle on the GPU: contents and metadata bit-exact, attention within tolerance, prompt-cache
files round-tripped."""
import numpy as np
import pytest
import torch

from helpers import TOL, bits_equal, max_abs_diff, seeded, to_oracle

pytestmark = pytest.mark.gpu


def _same(g, o, what=""):
    gs, os_ = g.state, o.state
    assert len(gs) == len(os_), what
    for i, (a, b) in enumerate(zip(gs, os_)):
        assert tuple(a.shape) == tuple(b.shape), f"{what}: state[{i}] {tuple(a.shape)} vs {tuple(b.shape)}"
        assert bits_equal(a, np.ascontiguousarray(b)), f"{what}: state[{i}]"
    assert list(g.meta_state) == list(o.meta_state), what
    assert g.offset == o.offset, what


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("chunk,step", [(96, 64), (256, 256), (None, 32)])
def test_chunked_cache_walk(kvc, oracle, cuda, dtype, chunk, step):
    """A walk of updates of ragged lengths, front trims, trims and attention calls; after every move the
    state (buffer rows up to the absolute offset, zero padding included), metaState [chunkSize, startPosition]
    and offset agree with the oracle."""
    B, Hq, Hkv, D = 2, 4, 2, 64
    g, o = kvc.ChunkedKVCache(chunk, step=step), oracle.ChunkedKVCache(chunk, step=step)
    assert list(g.meta_state) == list(o.meta_state) and g.state == []
    rng = np.random.default_rng(3)
    for move in range(40):
        S = int(rng.choice([1, 1, 1, 5, 17, 64, 100]))
        k, v = seeded((B, Hkv, S, D), 10 + move, dtype), seeded((B, Hkv, S, D), 100 + move, dtype)
        if move % 3 == 0:
            q = seeded((B, Hq, S, D), 200 + move, dtype)
            mask = "causal" if S > 1 else "none"
            out = g.attention(q.to(cuda), k.to(cuda), v.to(cuda), D ** -0.5, mask)
            ok_, ov_ = o.update(to_oracle(k), to_oracle(v))
            ref = oracle.sdpa(to_oracle(q), ok_, ov_, D ** -0.5, mask)
            assert max_abs_diff(out, ref) <= TOL[dtype], f"move {move}"
        else:
            gk, gv = g.update(k.to(cuda), v.to(cuda))
            ok_, ov_ = o.update(to_oracle(k), to_oracle(v))
            assert bits_equal(gk, np.ascontiguousarray(ok_)) and bits_equal(gv, np.ascontiguousarray(ov_)), f"move {move}"
        _same(g, o, f"after update {move}")
        # a front trim that would move startPosition past the fill (a buffer mostly made of zero padding) is
        # outside what the reference can do (its next update would index the buffer negatively); the
        # library refuses that state with KVC_ERR_INVALID_STATE, the walk stays inside the valid domain
        drop = 0 if (o.keys is None or chunk is None or o.keys.shape[2] < chunk) else o.keys.shape[2] - chunk
        if move % 4 == 1 and o.offset - o.start_position >= drop:
            g.maybe_trim_front()
            o.maybe_trim_front()
            assert g.start_position == o.start_position
            _same(g, o, f"after front trim {move}")
        if move % 7 == 2:
            n = int(rng.integers(0, 40))
            assert g.trim(n) == o.trim(n)
            _same(g, o, f"after trim {move}")
    c2, o2 = g.copy(), o.copy()
    _same(c2, o2, "copy")
    k, v = seeded((B, Hkv, 3, D), 900, dtype), seeded((B, Hkv, 3, D), 901, dtype)
    if o2.offset >= o2.start_position:
        c2.update(k.to(cuda), v.to(cuda))
        o2.update(to_oracle(k), to_oracle(v))
        _same(c2, o2, "copy after an update")
    else:
        # the reference's copy() adopts the state rows as its offset but keeps startPosition (KVCache.swift:
        # 1278-1287): after a front trim the copy's offset lies before startPosition and its next update would
        # index negatively; the library refuses instead
        with pytest.raises(kvc.KVCError) as e:
            c2.update(k.to(cuda), v.to(cuda))
        assert e.value.status == kvc.ERR_INVALID_STATE
    _same(g, o, "the original is untouched by the copy")


def test_cache_list_semantics_and_prompt_cache(kvc, oracle, cuda, tmp_path):
    """CacheList: state is the concatenation of the children's, trim returns the last child's count,
    isTrimmable(after:) needs every child, metaState is [count, (class, stateCount, metaCount, meta...)*],
    update on the list is refused; a file with a list (nested once) beside plain caches loads back equal."""
    B, Hkv, D = 1, 2, 64
    dtype = torch.bfloat16

    def fill(g, o, n, seed):
        k, v = seeded((B, Hkv, n, D), seed, dtype), seeded((B, Hkv, n, D), seed + 1, dtype)
        if isinstance(o, oracle.QuantizedKVCache):
            g.update_quantized(k.to(cuda), v.to(cuda))
            o.update_quantized(to_oracle(k), to_oracle(v))
        else:
            g.update(k.to(cuda), v.to(cuda))
            o.update(to_oracle(k), to_oracle(v))

    gs = [kvc.KVCacheSimple(), kvc.RotatingKVCache(max_size=16, keep=2), kvc.QuantizedKVCache(64, 4), kvc.ChunkedKVCache(32)]
    os_ = [oracle.KVCacheSimple(), oracle.RotatingKVCache(16, keep=2), oracle.QuantizedKVCache(64, 4), oracle.ChunkedKVCache(32)]
    for i, (g, o) in enumerate(zip(gs, os_)):
        fill(g, o, 5 + i, 10 * i)
    inner_g = kvc.CacheList(gs[2], gs[3])
    inner_o = oracle.CacheList(os_[2], os_[3])
    lg = kvc.CacheList(gs[0], gs[1], inner_g)
    lo = oracle.CacheList(os_[0], os_[1], inner_o)
    assert len(lg) == 3 and len(lg[2]) == 2
    assert list(lg.meta_state) == list(lo.meta_state)
    assert len(lg.state) == len(lo.state) == 2 + 2 + 6 + 2
    for a, b in zip(lg.state, lo.state):
        assert bits_equal(a, np.ascontiguousarray(b))
    assert lg.is_trimmable_after(3) == lo.is_trimmable_after(3) and lg.is_trimmable_after(12) == lo.is_trimmable_after(12)
    with pytest.raises(kvc.KVCError):
        lg.update(torch.zeros((B, Hkv, 1, D), dtype=dtype, device=cuda), torch.zeros((B, Hkv, 1, D), dtype=dtype, device=cuda))
    # work goes through the children
    fill(lg[0], lo[0], 3, 77)
    fill(lg[2][0], lo[2][0], 2, 79)
    assert lg.trim(2) == lo.trim(2)
    assert list(lg.meta_state) == list(lo.meta_state)
    for a, b in zip(lg.state, lo.state):
        assert tuple(a.shape) == tuple(b.shape) and bits_equal(a, np.ascontiguousarray(b))
    cp = lg.copy()
    assert list(cp.meta_state) == list(lg.meta_state)
    fill(cp[0], oracle.KVCacheSimple(), 1, 5)            # the copy is independent
    assert lg[0].offset == lo[0].offset and cp[0].offset == lg[0].offset + 1
    # prompt-cache file: a plain cache beside the list
    plain = kvc.KVCacheSimple()
    fill(plain, oracle.KVCacheSimple(), 4, 91)
    path = str(tmp_path / "list.safetensors")
    kvc.save_prompt_cache(path, [plain, lg], {"note": "composite"})
    loaded, meta = kvc.load_prompt_cache(path)
    assert meta == {"note": "composite"} and len(loaded) == 2
    assert isinstance(loaded[1], kvc.CacheList) and len(loaded[1]) == 3 and len(loaded[1][2]) == 2
    assert list(loaded[1].meta_state) == list(lg.meta_state)
    for a, b in zip(loaded[1].state, lg.state):
        assert tuple(a.shape) == tuple(b.shape) and torch.equal(a, b)
    assert loaded[1][1].offset == lg[1].offset and loaded[1][2][1].start_position == lg[2][1].start_position
    # and the restored children keep working
    fill(loaded[1][2][1], lo[2][1], 6, 123)
    fill(lg[2][1], oracle.ChunkedKVCache(32), 6, 123)
    for a, b in zip(loaded[1][2][1].state, lg[2][1].state):
        assert torch.equal(a, b)


def test_causal_mask_with_prepared_lengths(kvc, oracle, cuda):
    """createCausalMask(n:offset:windowSize:lengths:): the per-entry length cut on top of the causal and
    window conditions; prepare(lengths:) / finalize() are accepted and change nothing on these caches."""
    for n, offset, window, lengths in ((5, 0, None, [5, 3, 1]), (4, 9, None, [13, 10, 2, 0]), (6, 20, 8, [26, 21]), (3, 2, 2, [1])):
        got = kvc.create_causal_mask(n, offset, window, lengths, device=cuda)
        want = oracle.create_causal_mask(n, offset, window, lengths)
        assert tuple(got.shape) == want.shape == (len(lengths), 1, n, offset + n)
        assert np.array_equal(got.cpu().numpy(), want)
        plain = kvc.create_causal_mask(n, offset, window, device=cuda)
        assert np.array_equal(plain.cpu().numpy(), oracle.create_causal_mask(n, offset, window))
    # the mask drives attention like any other array mask
    B, Hq, Hkv, D, T = 3, 4, 2, 64, 7
    q, k, v = seeded((B, Hq, T, D), 1), seeded((B, Hkv, T, D), 2), seeded((B, Hkv, T, D), 3)
    lengths = [7, 4, 2]
    m = kvc.create_causal_mask(T, 0, None, lengths, device=cuda)
    out = kvc.scaled_dot_product_attention(q.to(cuda), k.to(cuda), v.to(cuda), 0.125, m)
    ref = oracle.sdpa(to_oracle(q), to_oracle(k), to_oracle(v), 0.125, oracle.create_causal_mask(T, 0, None, lengths))
    for b, n in enumerate(lengths):     # rows at or past an entry's length see no key at all: compare the defined rows
        assert max_abs_diff(out[b, :, :n], ref[b, :, :n]) <= 1e-4
    c = kvc.KVCacheSimple()
    c.prepare(lengths)
    c.update(k.to(cuda), v.to(cuda))
    c.finalize()
    assert c.offset == T and list(c.meta_state) == [""]
    lst = kvc.CacheList(kvc.KVCacheSimple(), kvc.RotatingKVCache(max_size=8))
    lst.prepare(lengths)
    lst.finalize()
