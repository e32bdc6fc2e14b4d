"""The caller's side of the cache path: rotary positions at the cache's ropeOffset ahead of
attentionWithCacheUpdate (MLXLLM/Models/Llama.swift:58-69, MLXLMCommon/RoPEApplication.swift:58-69) and
the cache traffic of a speculative round over a model's layer list (Evaluate.swift:1179-1286,
KVCachePlan.swift:219-300), against the oracle."""
import numpy as np
import pytest
import torch

from helpers import TOL, bits_equal, max_abs_diff, seeded, to_oracle

pytestmark = pytest.mark.gpu

# one bf16 / f16 spacing at |x| <= 8 (rotated N(0, 1) inputs): the rotation itself is float32 on both sides
ROPE_TOL = {torch.float32: 2e-5, torch.bfloat16: 2 ** -5, torch.float16: 2 ** -8}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("D,dims,traditional,base,scale", [(128, 128, False, 10000.0, 1.0), (128, 128, True, 500000.0, 1.0),
                                                           (64, 32, False, 10000.0, 0.25), (256, 64, True, 1000000.0, 1.0)])
def test_rope_matches_oracle(kvc, oracle, cuda, dtype, D, dims, traditional, base, scale):
    x = seeded((2, 3, 7, D), 5, dtype)
    for offset in (0, 1, 4096, 131071):
        got = kvc.rope(x.to(cuda), offset, dims, traditional, base, scale)
        want = oracle.rope(to_oracle(x), offset, dims, traditional, base, scale)
        # large positions: float32 angles lose absolute precision on both sides alike (p * f is rounded once);
        # what remains is the sin/cos implementation, a few float32 spacings of the angle
        tol = ROPE_TOL[dtype] + (2e-3 if offset > 100000 else (1e-4 if offset > 1000 else 0.0))
        assert max_abs_diff(got, want) <= tol, (offset, max_abs_diff(got, want))
        if dims < D:
            assert torch.equal(got[..., dims:].cpu(), x[..., dims:])            # pass-through features untouched
    # in place and strided (the [B, L, H, D] storage of a projection output)
    xs = x.to(cuda).transpose(1, 2).contiguous().transpose(1, 2)
    got = kvc.rope(xs, 3, dims, traditional, base, scale, out=xs)
    assert max_abs_diff(got, oracle.rope(to_oracle(x), 3, dims, traditional, base, scale)) <= ROPE_TOL[dtype]


@pytest.mark.parametrize("kind", ["simple", "rotating", "quantized", "turbo", "none"])
def test_attention_block_step_with_rope(kvc, oracle, cuda, kind):
    """Prefill in two chunks, then decode steps: every call rotates q and k at the cache offset before the
    fused update + attention; the cache ends up holding rotated keys (bit-exact where both sides agree on
    the rotated values to the bit is not required: rotated keys are compared at the store tolerance)."""
    B, Hq, Hkv, D = 2, 8, 2, 128
    dtype = torch.bfloat16
    cfg = dict(dims=D, traditional=False, base=500000.0, scale=1.0)
    scale = D ** -0.5
    if kind == "simple":
        g, o = kvc.KVCacheSimple(), oracle.KVCacheSimple()
    elif kind == "rotating":
        g, o = kvc.RotatingKVCache(max_size=96, keep=4), oracle.RotatingKVCache(96, keep=4)
    elif kind == "quantized":
        g, o = kvc.QuantizedKVCache(64, 8), oracle.QuantizedKVCache(64, 8)
    elif kind == "turbo":
        g, o = kvc.TurboQuantKVCache(bits=4), oracle.TurboQuantKVCache(bits=4)
    else:
        g = o = None
    seed = 0
    for S in ((70, 50) + (1,) * 6 if g is not None else (33,)):
        seed += 1
        q, k, v = seeded((B, Hq, S, D), seed, dtype), seeded((B, Hkv, S, D), seed + 50, dtype), seeded((B, Hkv, S, D), seed + 90, dtype)
        if g is not None and S > 1:
            gm, om = g.make_mask(S), o.make_mask(S)
            om_ = om if isinstance(om, str) else om
            gm_ = gm if isinstance(gm, str) else gm
        else:
            gm_, om_ = ("causal", "causal") if S > 1 else ("none", "none")
        out = kvc.attention_rope(q.to(cuda), k.to(cuda), v.to(cuda), g, cfg, scale, gm_)
        ref = oracle.attention_rope(to_oracle(q), to_oracle(k), to_oracle(v), o, cfg, scale, om_)
        # rotated operands may differ by one bf16 spacing between the two sides (float32 sin/cos of the
        # device and of numpy are not the same bits), which moves scores by ~1e-2 at worst
        assert max_abs_diff(out, ref) <= 2 * TOL[dtype], (kind, S)
        if g is not None:
            assert g.offset == o.offset
    if kind == "simple":
        gk, ok_ = g.state[0], o.state[0]
        assert max_abs_diff(gk, np.ascontiguousarray(ok_)) <= 2 ** -5           # rotated keys, one bf16 spacing at |x| < 8


def test_speculative_rounds_over_a_layer_list(kvc, oracle, cuda):
    """A four-layer list (simple, sliding window past its wrap, affine-quantised, TurboQuant): rounds of
    5 draft tokens + 1 through KVCacheStorage-style staged rounds with a scripted number of accepted
    tokens per round; after every commit each layer's state equals the oracle's, where the oracle is
    driven the reference's way (one StagedRound per cache, commit(retaining)). The sliding-window layer is
    also compared with an emitted-only replay (what the cache would hold had only the kept tokens ever
    been written)."""
    B, Hq, Hkv, D, L = 1, 8, 2, 128, 6
    dtype = torch.bfloat16
    scale = D ** -0.5

    def make():
        gs = [kvc.KVCacheSimple(), kvc.RotatingKVCache(max_size=48, keep=0), kvc.QuantizedKVCache(64, 4), kvc.TurboQuantKVCache(bits=4)]
        os_ = [oracle.KVCacheSimple(), oracle.RotatingKVCache(48, keep=0), oracle.QuantizedKVCache(64, 4), oracle.TurboQuantKVCache(bits=4)]
        return gs, os_

    gs, os_ = make()
    replay = oracle.RotatingKVCache(48, keep=0)
    P = 60                                        # prefill past the window: the ring has wrapped
    for i, (g, o) in enumerate(zip(gs, os_)):
        q, k, v = seeded((B, Hq, P, D), 10 + i, dtype), seeded((B, Hkv, P, D), 20 + i, dtype), seeded((B, Hkv, P, D), 30 + i, dtype)
        gm, om = g.make_mask(P, window_size=48 if i == 1 else None), o.make_mask(P, window_size=48 if i == 1 else None)
        g.attention(q.to(cuda), k.to(cuda), v.to(cuda), scale, gm)
        oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, scale, om)
        if i == 1:
            replay.update(to_oracle(k), to_oracle(v))
    accepted_script = [5, 0, 2, 5, 1, 3]
    for rnd, accepted in enumerate(accepted_script):
        retaining = accepted + 1                  # the accepted drafts plus the token verified before them
        qs = [seeded((B, Hq, L, D), 100 + 10 * rnd + i, dtype) for i in range(4)]
        ks = [seeded((B, Hkv, L, D), 200 + 10 * rnd + i, dtype) for i in range(4)]
        vs = [seeded((B, Hkv, L, D), 300 + 10 * rnd + i, dtype) for i in range(4)]
        outs = [torch.empty((B, Hq, L, D), dtype=dtype, device=cuda) for _ in range(4)]
        rd = kvc.StorageRound(gs, L)
        rd.attention([t.to(cuda) for t in qs], [t.to(cuda) for t in ks], [t.to(cuda) for t in vs], scale, outs, "causal")
        for i, o in enumerate(os_):
            if isinstance(o, (oracle.KVCacheSimple, oracle.RotatingKVCache)):
                ro = oracle.StagedRound(o, L)
                ko, vo = ro.update(to_oracle(ks[i]), to_oracle(vs[i]))
                ref = oracle.sdpa(to_oracle(qs[i]), ko, vo, scale, "causal")
                ro.commit(retaining)
            else:
                # packed caches take the rows through their normal update path and give the rejected ones back
                ref = oracle.attention_with_cache_update(to_oracle(qs[i]), to_oracle(ks[i]), to_oracle(vs[i]), o, scale, "causal")
                if L > retaining:
                    assert o.trim(L - retaining) == L - retaining
            assert max_abs_diff(outs[i], ref) <= TOL[dtype], f"round {rnd}, layer {i}"
        rd.commit(retaining)
        replay.update(to_oracle(ks[1][:, :, :retaining]), to_oracle(vs[1][:, :, :retaining]))
        for i, (g, o) in enumerate(zip(gs, os_)):
            assert g.offset == o.offset, f"round {rnd}, layer {i}"
            for a, b in zip(g.state, o.state):
                assert tuple(a.shape) == tuple(b.shape) and bits_equal(a, np.ascontiguousarray(b)), f"round {rnd}, layer {i}"
            assert list(g.meta_state) == list(o.meta_state)
    # the sliding-window layer holds what an emitted-only history would have left (same logical window)
    tail = min(replay.offset, 47)
    gv = gs[1].logical_view(tail)
    rv = replay.logical_view(tail)
    assert gv is not None and rv is not None
    assert bits_equal(gv[0], np.ascontiguousarray(rv[0])) and bits_equal(gv[1], np.ascontiguousarray(rv[1]))
    assert kvc.device_status() == 0


def test_speculate_rewind_rule(kvc, oracle, cuda):
    """Without staged rounds the main caches give back numDraft - accepted positions and the draft caches
    max(numDraft - accepted - 1, 0) (Evaluate.swift:1262-1264), all or nothing over the list."""
    B, Hkv, D = 1, 2, 64
    caches = [kvc.KVCacheSimple(), kvc.QuantizedKVCache(64, 8)]
    k = seeded((B, Hkv, 20, D), 1, torch.bfloat16).to(cuda)
    caches[0].update(k, k)
    caches[1].update_quantized(k, k)
    assert kvc.speculate_rewind(caches, 5, 2) == 3 and [c.offset for c in caches] == [17, 17]
    assert kvc.speculate_rewind(caches, 5, 5) == 0 and [c.offset for c in caches] == [17, 17]
    assert kvc.speculate_rewind(caches, 5, 2, is_draft=True) == 2 and [c.offset for c in caches] == [15, 15]
    assert kvc.speculate_rewind(caches, 5, 4, is_draft=True) == 0
    ring = kvc.RotatingKVCache(max_size=8)
    kk = seeded((B, Hkv, 12, D), 2, torch.bfloat16).to(cuda)
    ring.update(kk, kk)                                         # wrapped: not trimmable, so the list refuses
    assert kvc.speculate_rewind([caches[0], ring], 5, 1) == 0 and caches[0].offset == 15
    with pytest.raises(kvc.KVCError):
        kvc.speculate_rewind(caches, 3, 4)
