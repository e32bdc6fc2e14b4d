"""The benchmark configurations as they are worded, against the oracle.

Each test drives the library through the schedule one configuration names (prefill, decode
steps, trims, verify chunks) at the configuration's own head layout, dtype and lengths, and
checks what the configuration asks to be checked: cache contents, ring indices, packed codes,
scales and biases bit-exact; attention outputs within the stated tolerance (1e-4 for float32,
2e-2 for bfloat16). Where a dimension is reduced so that the CPU oracle finishes in seconds
(the layer count of configurations 3 and 4, the context of configuration 5), the docstring says
which; every other number is the configuration's.

Inputs are seeded N(0, 1) draws (a Philox stream on the host); no dataset is involved.
"""
import numpy as np
import pytest
import torch

from helpers import TOL, bits_equal, max_abs_diff, seeded, to_oracle, worst_excess

pytestmark = pytest.mark.gpu


def _same_state(g, o, what=""):
    gs, os_ = g.state, o.state
    assert len(gs) == len(os_), what
    for i, (a, b) in enumerate(zip(gs, os_)):
        assert tuple(a.shape) == tuple(b.shape), f"{what} state[{i}] shape {tuple(a.shape)} vs {tuple(b.shape)}"
        assert bits_equal(a, np.ascontiguousarray(b)), f"{what} state[{i}] differs"
    assert list(g.meta_state) == list(o.meta_state), what


def _new_rows_equal(g, o, rows, what=""):
    """Bit-exact comparison of the last `rows` token rows of every state array."""
    for i, (a, b) in enumerate(zip(g.state, o.state)):
        assert a.shape[2] == b.shape[2], what
        assert bits_equal(a[:, :, -rows:].contiguous(), np.ascontiguousarray(b[:, :, -rows:])), f"{what} state[{i}] new rows differ"


def test_config1_quantized_8bit_llama32_1b_whole(kvc, oracle, cuda):
    """Configuration 1 as worded: 16 layers, 32 query heads, 8 KV heads, head dim 64, batch 1, float32;
    one 1024-token prefill into QuantizedKVCache(groupSize 64, bits 8) with a causal mask, then 256
    decode steps (append one token, quantized SDPA, scale 1/8). Every step: the appended codes, scales
    and biases bit-exact and the outputs within 1e-4 in every layer; the whole state and metaState after
    the prefill and at the end."""
    layers, B, Hq, Hkv, D, P, steps = 16, 1, 32, 8, 64, 1024, 256
    scale = 1.0 / 8.0
    dtype = torch.float32
    pairs = [(kvc.QuantizedKVCache(64, 8), oracle.QuantizedKVCache(64, 8)) for _ in range(layers)]
    for i, (g, o) in enumerate(pairs):
        q, k, v = seeded((B, Hq, P, D), 100 + i, dtype), seeded((B, Hkv, P, D), 200 + i, dtype), seeded((B, Hkv, P, D), 300 + i, dtype)
        out = g.attention(q.to(cuda), k.to(cuda), v.to(cuda), scale, "causal")
        ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, scale, "causal")
        assert max_abs_diff(out, ref) <= 1e-4, f"prefill, layer {i}"
        _same_state(g, o, f"after prefill, layer {i}")
        assert g.offset == P
    worst = 0.0
    # one seeded draw per layer for all 256 steps (row s is step s)
    qs = [seeded((steps, B, Hq, 1, D), 1000 + i, dtype) for i in range(layers)]
    ks = [seeded((steps, B, Hkv, 1, D), 2000 + i, dtype) for i in range(layers)]
    vs = [seeded((steps, B, Hkv, 1, D), 3000 + i, dtype) for i in range(layers)]
    for s in range(steps):
        for i, (g, o) in enumerate(pairs):
            q, k, v = qs[i][s], ks[i][s], vs[i][s]
            out = g.attention(q.to(cuda), k.to(cuda), v.to(cuda), scale)
            ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, scale)
            d = max_abs_diff(out, ref)
            worst = max(worst, d)
            assert d <= 1e-4, f"step {s}, layer {i}: {d}"
            if i in (0, layers - 1) or s % 32 == 31:
                _new_rows_equal(g, o, 1, f"step {s}, layer {i}")
    for i, (g, o) in enumerate(pairs):
        assert g.offset == o.offset == P + steps
        _same_state(g, o, f"end, layer {i}")
        assert list(g.meta_state) == ["256", str(P + steps), "64", "8"]
    assert kvc.device_status() == 0


def test_config2_simple_bf16_llama3_8b_chunked_prefill_then_decode(kvc, oracle, cuda):
    """Configuration 2 as worded: KVCacheSimple (step 256), 32 query heads, 8 KV heads, head dim 128,
    bfloat16; prefill 8192 tokens in 512-token chunks with causal SDPA, then decode steps. Reduced so
    that the oracle finishes in seconds: 2 layers of 32, batch 2 of 8, 64 decode steps of 512, and
    the oracle computes the chunk attention for the first, one middle and the last prefill chunk only
    (the other chunks are appended with `update` on the oracle side; the library runs attention on
    every chunk). Cache rows bit-exact after every chunk and at the end, outputs within 2e-2."""
    layers, B, Hq, Hkv, D, P, C, steps = 2, 2, 32, 8, 128, 8192, 512, 64
    scale = D ** -0.5
    dtype = torch.bfloat16
    pairs = [(kvc.KVCacheSimple(), oracle.KVCacheSimple()) for _ in range(layers)]
    checked = {0, 7, P // C - 1}
    for i, (g, o) in enumerate(pairs):
        for c in range(P // C):
            q = seeded((B, Hq, C, D), 10_000 * i + 3 * c, dtype)
            k, v = seeded((B, Hkv, C, D), 10_000 * i + 3 * c + 1, dtype), seeded((B, Hkv, C, D), 10_000 * i + 3 * c + 2, dtype)
            out = g.attention(q.to(cuda), k.to(cuda), v.to(cuda), scale, "causal")
            if c in checked:
                ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, scale, "causal")
                assert max_abs_diff(out, ref) <= TOL[dtype], f"layer {i}, chunk {c}"
            else:
                o.update(to_oracle(k), to_oracle(v))
            assert g.offset == o.offset == (c + 1) * C
            _new_rows_equal(g, o, C, f"layer {i}, chunk {c}")
        _same_state(g, o, f"after prefill, layer {i}")
    for s in range(steps):
        for i, (g, o) in enumerate(pairs):
            q = seeded((B, Hq, 1, D), 500_000 + 10 * s + i, dtype)
            k, v = seeded((B, Hkv, 1, D), 600_000 + 10 * s + i, dtype), seeded((B, Hkv, 1, D), 700_000 + 10 * s + i, dtype)
            out = g.attention(q.to(cuda), k.to(cuda), v.to(cuda), scale)
            ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, scale)
            assert max_abs_diff(out, ref) <= TOL[dtype], f"step {s}, layer {i}"
    for i, (g, o) in enumerate(pairs):
        assert g.offset == o.offset == P + steps
        _same_state(g, o, f"end, layer {i}")
    assert kvc.device_status() == 0


def test_config3_rotating_gemma3_schedule(kvc, oracle, cuda):
    """Configuration 3 as worded, on one sliding-window layer and one global layer of its 26 (the other
    local / global layers repeat these two): 4 query heads, 1 KV head, head dim 256, batch 4, bfloat16;
    RotatingKVCache(maxSize 512, keep 0) beside KVCacheSimple(step 1024) (Gemma3Text.swift:409-428);
    prefill 2048 tokens in 512-token chunks with the masks makeMask hands out, then 4096 single-token
    decode steps, and trimPromptCache(64) over the layer list every 1024 steps. The ring has wrapped
    long before the first trim, so the list-level trim returns 0 and changes nothing
    (KVCache.swift:2293-2306, :817-823). Ring contents (the physical buffer), idx, offset and metaState
    are compared bit-exact after every prefill chunk and every 64th decode step (and at every trim
    point); the appended row of the global layer every step; outputs within 2e-2 every step."""
    B, Hq, Hkv, D, W = 4, 4, 1, 256, 512
    dtype = torch.bfloat16
    scale = D ** -0.5
    g_loc, o_loc = kvc.RotatingKVCache(max_size=W, keep=0), oracle.RotatingKVCache(W, keep=0)
    g_glb, o_glb = kvc.KVCacheSimple(step=1024), oracle.KVCacheSimple(step=1024)
    layers = [(g_loc, o_loc, W), (g_glb, o_glb, None)]
    seed = 0
    for chunk in range(4):
        for li, (g, o, window) in enumerate(layers):
            seed += 1
            q, k, v = seeded((B, Hq, 512, D), seed, dtype), seeded((B, Hkv, 512, D), seed + 7000, dtype), seeded((B, Hkv, 512, D), seed + 14000, dtype)
            gm, om = g.make_mask(512, window_size=window), o.make_mask(512, window_size=window)
            if isinstance(om, str):
                assert gm == om, (chunk, li)
            else:
                assert not isinstance(gm, str) and np.array_equal(gm.cpu().numpy(), om), (chunk, li)
            out = g.attention(q.to(cuda), k.to(cuda), v.to(cuda), scale, gm)
            ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, scale, om)
            assert max_abs_diff(out, ref) <= TOL[dtype], f"prefill chunk {chunk}, layer {li}"
            _same_state(g, o, f"prefill chunk {chunk}, layer {li}")
    assert list(g_loc.meta_state) == list(o_loc.meta_state) and g_loc.offset == 2048
    # one seeded draw per layer for all 4096 decode steps (row s is step s)
    dq = [seeded((4096, B, Hq, 1, D), 31 + li, dtype) for li in range(2)]
    dk = [seeded((4096, B, Hkv, 1, D), 41 + li, dtype) for li in range(2)]
    dv = [seeded((4096, B, Hkv, 1, D), 51 + li, dtype) for li in range(2)]
    for s in range(4096):
        if s and s % 1024 == 0:
            glist, olist = [g_loc, g_glb], [o_loc, o_glb]
            can = all(o.is_trimmable_after(64) if hasattr(o, "is_trimmable_after") else o.is_trimmable for o in olist)
            trimmed = kvc.trim_prompt_cache(glist, 64)
            assert not can and trimmed == 0, "the wrapped ring makes the list untrimmable"
            assert not kvc.can_trim_prompt_cache(glist) or not g_loc.is_trimmable_after(64)
            _same_state(g_loc, o_loc, f"after the trim attempt at step {s}")
            assert g_glb.offset == o_glb.offset
        for li, (g, o, window) in enumerate(layers):
            q, k, v = dq[li][s], dk[li][s], dv[li][s]
            gm, om = g.make_mask(1, window_size=window), o.make_mask(1, window_size=window)
            assert isinstance(om, str) and gm == om == "none"       # maxSize == window: no rolled mask (KVCache.swift:855)
            out = g.attention(q.to(cuda), k.to(cuda), v.to(cuda), scale, gm)
            ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, scale, om)
            assert max_abs_diff(out, ref) <= TOL[dtype], f"decode step {s}, layer {li}"
            if li == 0:
                assert list(g.meta_state) == list(o.meta_state), f"step {s}"
                if s % 64 == 63 or s < 4:
                    _same_state(g, o, f"decode step {s}, ring")
            else:
                assert g.offset == o.offset
                _new_rows_equal(g, o, 1, f"decode step {s}, global layer")
    _same_state(g_loc, o_loc, "end, ring")
    _same_state(g_glb, o_glb, "end, global layer")
    assert g_loc.offset == 2048 + 4096 and g_glb.offset == 2048 + 4096
    assert kvc.device_status() == 0


def test_config4_ragged_quantized_qwen2(kvc, oracle, cuda):
    """Configuration 4 as worded, on 2 of its 28 layers and 6 of its 256 decode steps: 28 query heads,
    4 KV heads, head dim 128, bfloat16, 32 sequences with prompt lengths drawn uniformly from
    [2048, 32768] (numpy default_rng(4), the draw bench.py uses), K/V ~ N(0, 1) with 1 % of the channels
    scaled by 20, QuantizedKVCache(groupSize 64, bits 4) filled with 512-token updateQuantized chunks.
    The reference keeps one cache object per sequence (a cache has one offset); the library appends and
    attends all 32 in one var-len call per layer. Codes, scales and biases of every sequence bit-exact
    after the fill and after the steps; outputs within 2e-2 plus the rounding of the bfloat16 store
    (outlier channels make some outputs larger than 1, see helpers.worst_excess)."""
    layers, n, Hq, Hkv, D, steps = 2, 32, 28, 4, 128, 6
    dtype = torch.bfloat16
    scale = D ** -0.5
    rng = np.random.default_rng(4)
    lengths = [int(x) for x in rng.integers(2048, 32768 + 1, size=n)]
    assert min(lengths) >= 2048 and max(lengths) <= 32768
    chunk_k = seeded((1, Hkv, 512, D), 41, dtype, outlier_frac=0.01)
    chunk_v = seeded((1, Hkv, 512, D), 42, dtype, outlier_frac=0.01)
    dk, dv = chunk_k.to(cuda), chunk_v.to(cuda)
    ok_, ov_ = to_oracle(chunk_k), to_oracle(chunk_v)
    caches = []
    for layer in range(layers):
        row = []
        for t in lengths:
            g, o = kvc.QuantizedKVCache(64, 4), oracle.QuantizedKVCache(64, 4)
            left = t
            while left > 0:
                m = min(left, 512)
                g.update_quantized(dk[:, :, :m], dv[:, :, :m])
                o.update_quantized(ok_[:, :, :m], ov_[:, :, :m])
                left -= m
            row.append((g, o))
        caches.append(row)
    for layer in range(layers):
        for i in (0, 7, 31):
            _same_state(*caches[layer][i], f"after the fill, layer {layer}, sequence {i}")
    for s in range(steps):
        for layer in range(layers):
            seed = 500 + 10 * s + layer
            q = seeded((n, Hq, 1, D), seed, dtype)
            k = seeded((n, Hkv, 1, D), seed + 100, dtype, outlier_frac=0.01)
            v = seeded((n, Hkv, 1, D), seed + 200, dtype, outlier_frac=0.01)
            dq, dk1, dv1 = q.to(cuda), k.to(cuda), v.to(cuda)
            out = torch.empty((n, Hq, 1, D), dtype=dtype, device=cuda)
            plan = kvc.DecodeStep([g for g, _ in caches[layer]], [dq[i:i + 1] for i in range(n)],
                                  [dk1[i:i + 1] for i in range(n)], [dv1[i:i + 1] for i in range(n)],
                                  [out[i:i + 1] for i in range(n)], scale)
            plan.run_varlen()
            torch.cuda.synchronize()
            for i, (g, o) in enumerate(caches[layer]):
                ref = oracle.attention_with_cache_update(to_oracle(q[i:i + 1]), to_oracle(k[i:i + 1]), to_oracle(v[i:i + 1]),
                                                         o, scale)
                assert worst_excess(out[i:i + 1], ref, dtype) <= 0, f"step {s}, layer {layer}, sequence {i} (length {lengths[i]})"
                assert g.offset == o.offset == lengths[i] + s + 1
    for layer in range(layers):
        for i, (g, o) in enumerate(caches[layer]):
            _same_state(g, o, f"end, layer {layer}, sequence {i}")
    assert kvc.device_status() == 0


@pytest.mark.parametrize("affine_values", [False, True], ids=["turbo-values", "affine-values"])
def test_config5_turbo_llama3_70b_decode_and_verify(kvc, oracle, cuda, affine_values):
    """Configuration 5 as worded except for the context (2 048 instead of 32 768 tokens, so that the CPU
    oracle finishes in seconds) and the layer count (2 of 80): 64 query heads, 8 KV heads, head dim 128,
    batch 16, bfloat16; keys rotated by the seeded random-sign Walsh-Hadamard transform and quantised to
    3-bit codebook indices, values 4-bit -- both as the reference's codebook values and as the "4-bit
    affine, group 64" values the configuration words; the cache filled in the compressed domain in
    512-token chunks (encodeNewToken); then decode steps and 6-row speculative verify chunks (5 draft
    tokens + the bonus token, causal), of which 4 rows are rejected (trim) each round. Packed indices,
    norms (codes, scales, biases) bit-exact; outputs within 2e-2."""
    layers, B, Hq, Hkv, D, T0 = 2, 16, 64, 8, 128, 2048
    dtype = torch.bfloat16
    scale = D ** -0.5
    kw = dict(bits=4, key_bits=3, value_bits=4, affine_values=affine_values)
    pairs = [(kvc.TurboQuantKVCache(**kw), oracle.TurboQuantKVCache(**kw)) for _ in range(layers)]
    for li, (g, o) in enumerate(pairs):
        for c in range(T0 // 512):
            k, v = seeded((B, Hkv, 512, D), 10 * li + c, dtype), seeded((B, Hkv, 512, D), 1000 + 10 * li + c, dtype)
            g.encode_new_token(k.to(cuda), v.to(cuda))
            o.encode_new_token(to_oracle(k), to_oracle(v))
        _same_state(g, o, f"after the fill, layer {li}")
    seed = 5000
    rounds = 2
    for rnd in range(rounds):
        for L, mask in ((1, "none"), (6, "causal")):
            for li, (g, o) in enumerate(pairs):
                seed += 1
                q, k, v = seeded((B, Hq, L, D), seed, dtype), seeded((B, Hkv, L, D), seed + 300, dtype), seeded((B, Hkv, L, D), seed + 600, dtype)
                out = g.attention(q.to(cuda), k.to(cuda), v.to(cuda), scale, mask)
                ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, scale, mask)
                assert max_abs_diff(out, ref) <= TOL[dtype], f"round {rnd}, L {L}, layer {li}"
                _new_rows_equal(g, o, L, f"round {rnd}, L {L}, layer {li}")
        glist = [g for g, _ in pairs]
        assert kvc.trim_prompt_cache(glist, 4) == 4           # 2 of the 6 verify rows accepted
        for _, o in pairs:
            assert o.trim(4) == 4
    for li, (g, o) in enumerate(pairs):
        assert g.offset == o.offset == T0 + rounds * (1 + 6 - 4)
        _same_state(g, o, f"end, layer {li}")
    assert kvc.device_status() == 0
