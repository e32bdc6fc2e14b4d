"""GPU parity: cache contents, ring indices, metaState and packed affine codes
produced by the CUDA library through its C ABI must be bit-identical to the CPU
oracle on the same seeded inputs."""
import numpy as np
import pytest
import torch

import scenarios as sc
from helpers import bits_equal, from_oracle, seeded, to_oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be(kvc, cuda):
    return sc.GpuBackend(kvc, cuda)


@pytest.mark.parametrize("scenario", sc.ALL_SIMPLE, ids=lambda f: f.__name__)
def test_reference_cache_semantics(be, scenario):
    scenario(be)


@pytest.mark.parametrize("case", sc.COMMIT_CASES, ids=lambda c: f"w{c['window']}p{c['prefill']}k{c.get('keep', 0)}")
def test_commit_equivalence(be, case):
    sc.commit_equivalence(be, **case)


@pytest.mark.parametrize("case", sc.REWIND_CASES, ids=lambda c: f"w{c['window']}p{c['prefill']}r{c['rewinding']}k{c.get('keep', 0)}")
def test_rewind(be, case):
    sc.rewind_matches_emitted_only_replay(be, **case)


def _same_state(gpu_cache, ora_cache):
    gs, os_ = gpu_cache.state, ora_cache.state
    assert len(gs) == len(os_)
    for g, o in zip(gs, os_):
        assert tuple(g.shape) == tuple(o.shape), (g.shape, o.shape)
        assert bits_equal(g, np.ascontiguousarray(o))
    assert gpu_cache.offset == ora_cache.offset
    assert list(gpu_cache.meta_state) == list(ora_cache.meta_state)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_simple_cache_append_growth_trim(kvc, oracle, cuda, dtype):
    B, H, D = 2, 3, 64
    g, o = kvc.KVCacheSimple(step=16), oracle.KVCacheSimple(step=16)
    seed = 0
    for S in (5, 1, 1, 16, 40, 1, 7):
        k, v = seeded((B, H, S, D), seed, dtype), seeded((B, H, S, D), seed + 1, dtype)
        seed += 2
        gk, gv = g.update(k.to(cuda), v.to(cuda))
        ok, ov = o.update(to_oracle(k), to_oracle(v))
        assert bits_equal(gk, np.ascontiguousarray(ok)) and bits_equal(gv, np.ascontiguousarray(ov))
        _same_state(g, o)
    assert g.trim(9) == o.trim(9)
    k, v = seeded((B, H, 3, D), 99, dtype), seeded((B, H, 3, D), 100, dtype)
    g.update(k.to(cuda), v.to(cuda))
    o.update(to_oracle(k), to_oracle(v))
    _same_state(g, o)
    assert g.trim(10_000) == o.trim(10_000) and g.offset == 0
    cp = g.copy()
    _same_state(cp, o)


def test_simple_cache_accepts_strided_inputs(kvc, oracle, cuda):
    # models hand over keys as a transposed [B, S, H, D] projection
    B, H, S, D = 2, 4, 6, 32
    base_k, base_v = seeded((B, S, H, D), 1, torch.bfloat16), seeded((B, S, H, D), 2, torch.bfloat16)
    k, v = base_k.to(cuda).transpose(1, 2), base_v.to(cuda).transpose(1, 2)
    assert not k.is_contiguous()
    g, o = kvc.KVCacheSimple(), oracle.KVCacheSimple()
    g.update(k, v)
    o.update(to_oracle(base_k.transpose(1, 2).contiguous()), to_oracle(base_v.transpose(1, 2).contiguous()))
    _same_state(g, o)
    # and an inner stride != 1 (element-wise path)
    wide = seeded((B, H, S, 2 * D), 3, torch.float32).to(cuda)
    g2, o2 = kvc.KVCacheSimple(), oracle.KVCacheSimple()
    g2.update(wide[..., ::2], wide[..., 1::2])
    o2.update(to_oracle(wide[..., ::2].contiguous()), to_oracle(wide[..., 1::2].contiguous()))
    _same_state(g2, o2)


@pytest.mark.parametrize("keep", [0, 3])
def test_rotating_cache_random_walk(kvc, oracle, cuda, keep):
    """Mixed single/multi-token writes and pre-wrap trims: physical ring, idx,
    offset and metaState identical after every step."""
    rng = np.random.default_rng(keep)
    B, H, D, W = 2, 2, 32, 24
    g, o = kvc.RotatingKVCache(W, keep, step=8), oracle.RotatingKVCache(W, keep, step=8)
    seed = 10
    for step in range(60):
        S = int(rng.choice([1, 1, 1, 2, 5, 30]))
        k, v = seeded((B, H, S, D), seed, torch.bfloat16), seeded((B, H, S, D), seed + 1, torch.bfloat16)
        seed += 2
        gk, gv = g.update(k.to(cuda), v.to(cuda))
        ok, ov = o.update(to_oracle(k), to_oracle(v))
        assert tuple(gk.shape) == tuple(ok.shape)
        assert bits_equal(gk, np.ascontiguousarray(ok)) and bits_equal(gv, np.ascontiguousarray(ov))
        _same_state(g, o)
        assert g.idx == o.idx
        if o.is_trimmable_after(0) and o.offset > 2 and rng.random() < 0.3 and o.idx >= 2:
            assert g.trim(2) == o.trim(2)
            _same_state(g, o)
        for n, w in ((1, None), (1, 8), (4, None), (4, 8)):
            gm, om = g.make_mask(n, w), o.make_mask(n, w)
            if isinstance(om, str):
                assert gm == om
            else:
                assert np.array_equal(gm.cpu().numpy(), om)


def test_rotating_window_config_shape(kvc, oracle, cuda):
    """Sliding-window benchmark shape scaled down: chunked prefill past the
    window, then decode with wraparound, head_dim 256, bf16."""
    B, H, D, W = 2, 1, 256, 64
    g, o = kvc.RotatingKVCache(W), oracle.RotatingKVCache(W)
    seed = 0
    for _ in range(4):
        k, v = seeded((B, H, 64, D), seed, torch.bfloat16), seeded((B, H, 64, D), seed + 1, torch.bfloat16)
        seed += 2
        g.update(k.to(cuda), v.to(cuda))
        o.update(to_oracle(k), to_oracle(v))
        _same_state(g, o)
    for _ in range(2 * W + 5):
        k, v = seeded((B, H, 1, D), seed, torch.bfloat16), seeded((B, H, 1, D), seed + 1, torch.bfloat16)
        seed += 2
        g.update(k.to(cuda), v.to(cuda))
        o.update(to_oracle(k), to_oracle(v))
    _same_state(g, o)
    # the list-level trim is all-or-nothing and refuses a wrapped ring (KVCache.swift:2302-2306)
    simple = kvc.KVCacheSimple()
    simple.update(k.to(cuda), v.to(cuda))
    assert not kvc.can_trim_prompt_cache([simple, g])
    assert kvc.trim_prompt_cache([simple, g], 64) == 0 and simple.offset == 1
    assert kvc.trim_prompt_cache([simple], 64) == 1


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("bits", [8, 4, 2])
@pytest.mark.parametrize("D,group", [(64, 64), (128, 64), (128, 32), (256, 128), (32, 64), (96, 32)])
def test_affine_codes_bit_exact(kvc, oracle, cuda, dtype, bits, D, group):
    B, H = 2, 2
    g, o = kvc.QuantizedKVCache(group, bits), oracle.QuantizedKVCache(group, bits)
    seed = 0
    for S in (9, 1, 1, 300, 1):
        k = seeded((B, H, S, D), seed, dtype, outlier_frac=0.05)
        v = seeded((B, H, S, D), seed + 1, dtype)
        if S == 9:
            k[:, :, 0] = 0          # degenerate all-equal group
            v[:, :, 1] = 1.5
            k[:, :, 2] = -k[:, :, 2].abs()
        seed += 2
        gq = g.update_quantized(k.to(cuda), v.to(cuda))
        oq = o.update_quantized(to_oracle(k), to_oracle(v))
        for gt, ot in zip(gq[0] + gq[1], oq[0] + oq[1]):
            assert bits_equal(gt, np.ascontiguousarray(ot))
    assert g.group_size == o.group_size
    _same_state(g, o)
    cp = g.copy()
    _same_state(cp, o)
    g.trim(7); o.trim(7)
    _same_state(g, o)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("bits,D,group", [(4, 128, 64), (8, 128, 32), (2, 64, 64), (4, 256, 128), (8, 64, 32), (2, 128, 64)])
def test_affine_codes_bit_exact_prefill_chunk(kvc, oracle, cuda, dtype, bits, D, group):
    """A prefill-sized chunk (the launcher keeps several rows per warp in flight), an odd-sized one, and
    a strided (transposed-projection) source that must take the element-wise path."""
    B, H = 2, 4
    g, o = kvc.QuantizedKVCache(group, bits), oracle.QuantizedKVCache(group, bits)
    for i, S in enumerate((1100, 3, 1031)):
        k = seeded((B, H, S, D), 40 + i, dtype, outlier_frac=0.05)
        v = seeded((B, H, S, D), 50 + i, dtype)
        kd, vd = k.to(cuda), v.to(cuda)
        if i == 2:   # [B, S, H, D] storage viewed as [B, H, S, D]
            kd = kd.transpose(1, 2).contiguous().transpose(1, 2)
            vd = vd.transpose(1, 2).contiguous().transpose(1, 2)
        gq = g.update_quantized(kd, vd)
        oq = o.update_quantized(to_oracle(k), to_oracle(v))
        for gt, ot in zip(gq[0] + gq[1], oq[0] + oq[1]):
            assert bits_equal(gt, np.ascontiguousarray(ot))
    _same_state(g, o)


def test_quantized_cache_rejects_what_the_reference_rejects(kvc, cuda):
    q = kvc.QuantizedKVCache()
    x = torch.zeros(1, 2, 4, 64, dtype=torch.bfloat16, device=cuda)
    with pytest.raises(kvc.KVCError) as e:
        q.update(x, x)  # KVCache.swift:1106-1110
    assert e.value.status == kvc.ERR_INVALID_STATE
    bad = torch.zeros(1, 2, 4, 5, dtype=torch.float32, device=cuda)
    with pytest.raises(kvc.KVCError):
        q.update_quantized(bad, bad)
    s = kvc.KVCacheSimple()
    s.state = [bad, bad]
    with pytest.raises(kvc.KVCError):
        s.to_quantized(64, 4)  # KVCacheTests.swift:538-551
    with pytest.raises(kvc.KVCError):
        kvc.RotatingKVCache(32).to_quantized()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_to_quantized_and_back(kvc, oracle, cuda, dtype):
    B, H, T, D = 2, 2, 37, 128
    k, v = seeded((B, H, T, D), 5, dtype), seeded((B, H, T, D), 6, dtype)
    g, o = kvc.KVCacheSimple(), oracle.KVCacheSimple()
    g.update(k.to(cuda), v.to(cuda))
    o.update(to_oracle(k), to_oracle(v))
    gq, oq = g.to_quantized(64, 4), o.to_quantized(64, 4)
    _same_state(gq, oq)
    gu, ou = gq.to_unquantized(), oq.to_unquantized()
    _same_state(gu, ou)
    codes, scales, biases = kvc.quantized(k.to(cuda), 64, 4)
    oc, os_, ob = oracle.affine_quantize(to_oracle(k), 64, 4)
    assert bits_equal(codes, oc) and bits_equal(scales, os_) and bits_equal(biases, ob)
    deq = kvc.dequantized(codes, scales, biases, 64, 4)
    assert bits_equal(deq, oracle.affine_dequantize(oc, os_, ob, 64, 4))


def test_state_round_trip_and_export(kvc, oracle, cuda):
    B, H, T, D = 2, 2, 20, 64
    k, v = seeded((B, H, T, D), 7, torch.bfloat16), seeded((B, H, T, D), 8, torch.bfloat16)
    g = kvc.KVCacheSimple()
    g.update(k.to(cuda), v.to(cuda))
    host = g.export_state(0)
    assert host.shape == (B, H, T, D) and torch.equal(host, k)
    fresh = kvc.KVCacheSimple()
    fresh.state = g.state
    assert fresh.offset == T and torch.equal(fresh.export_state(1), v)
    r = kvc.RotatingKVCache(8)
    for t in range(11):
        r.update(k[:, :, t:t + 1].to(cuda), v[:, :, t:t + 1].to(cuda))
    r2 = kvc.RotatingKVCache(8)
    r2.state = r.state
    r2.meta_state = r.meta_state
    assert list(r2.meta_state) == list(r.meta_state)
    assert torch.equal(r2.export_state(0), r.export_state(0))
    assert g.memory_bytes > 0


def test_list_level_dynamic_conversion(kvc, cuda):
    """maybeTurboQuantizeKVCache / maybeAffineQuantizeKVCache over a layer list: boundary layers get
    8-bit affine protection, the others the requested scheme, rotating layers and layers below the
    start threshold are left alone; converted layers equal the per-cache conversions."""
    B, H, D = 1, 2, 128

    def layers():
        out = []
        for i in range(7):
            c = kvc.KVCacheSimple()
            n = 5 if i == 3 else 40 + i
            c.update(seeded((B, H, n, D), 10 + i, torch.bfloat16).to(cuda), seeded((B, H, n, D), 50 + i, torch.bfloat16).to(cuda))
            out.append(c)
        rot = kvc.RotatingKVCache(max_size=16)
        rot.update(seeded((B, H, 30, D), 99, torch.bfloat16).to(cuda), seeded((B, H, 30, D), 98, torch.bfloat16).to(cuda))
        out.insert(2, rot)
        return out

    caches, twins = layers(), layers()
    done = kvc.maybe_turbo_quantize_kv_cache(caches, 4, 4, quantized_kv_start=10)
    assert done is False                                  # one simple layer (5 tokens) still waits
    kinds = [type(c).__name__ for c in caches]
    assert kinds == ["QuantizedKVCache", "QuantizedKVCache", "RotatingKVCache", "TurboQuantKVCache", "KVCacheSimple",
                     "TurboQuantKVCache", "QuantizedKVCache", "QuantizedKVCache"]
    for i, c in enumerate(caches):
        assert c.offset == twins[i].offset
        if isinstance(c, kvc.QuantizedKVCache):
            ref = twins[i].to_quantized(64, 8)
            assert c.group_size == 64 and c.bits == 8
            for x, y in zip(c.state, ref.state):
                assert torch.equal(x, y)
        elif isinstance(c, kvc.TurboQuantKVCache):
            assert not c.is_compressed
            for x, y in zip(c.state, twins[i].state):
                assert torch.equal(x, y)                  # raw phase: the live rows were adopted
    # decode still works on every converted layer
    for c in caches:
        if isinstance(c, kvc.RotatingKVCache):
            continue
        q, k, v = (seeded((B, 4, 1, D), 1, torch.bfloat16).to(cuda), seeded((B, H, 1, D), 2, torch.bfloat16).to(cuda),
                   seeded((B, H, 1, D), 3, torch.bfloat16).to(cuda))
        assert torch.isfinite(c.attention(q, k, v, 0.09).float()).all()

    caches2 = layers()
    assert kvc.maybe_affine_quantize_kv_cache(caches2, 4, 64, compression_start=0) is True
    assert [type(c).__name__ for c in caches2] == ["QuantizedKVCache"] * 2 + ["RotatingKVCache"] + ["QuantizedKVCache"] * 5
    assert all(c.bits == 4 for c in caches2 if isinstance(c, kvc.QuantizedKVCache))


def _filled(kvc, oracle, cuda, dtype):
    """Four caches (library, oracle) over the same seeded tokens: simple, rotating past its window,
    affine-quantized, turbo in its compressed phase."""
    B, H, D = 1, 2, 64
    g = [kvc.KVCacheSimple(), kvc.RotatingKVCache(max_size=16, keep=2), kvc.QuantizedKVCache(32, 4),
         kvc.TurboQuantKVCache(bits=4, key_bits=3, value_bits=4, seed=11)]
    o = [oracle.KVCacheSimple(), oracle.RotatingKVCache(max_size=16, keep=2), oracle.QuantizedKVCache(32, 4),
         oracle.TurboQuantKVCache(bits=4, key_bits=3, value_bits=4, seed=11,
                                  key_codebook=np.array(kvc.turbo_codebook(D, 3)[0], dtype=np.float32),
                                  value_codebook=np.array(kvc.turbo_codebook(D, 4)[0], dtype=np.float32))]
    seed = 300
    for S in (12, 1, 1, 9, 1):
        k, v = seeded((B, H, S, D), seed, dtype), seeded((B, H, S, D), seed + 1, dtype)
        q = seeded((B, 2 * H, S, D), seed + 2, dtype)
        seed += 3
        for gc, oc in zip(g, o):
            kvc.attention_with_cache_update(q.to(cuda), k.to(cuda), v.to(cuda), gc, D ** -0.5, "causal" if S > 1 else "none")
            oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), oc, D ** -0.5,
                                               "causal" if S > 1 else "none")
    return g, o


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_prompt_cache_file_round_trip(kvc, oracle, cuda, tmp_path, dtype):
    """savePromptCache / loadPromptCache (KVCache.swift:1797-1913): a file written by the library holds
    exactly the oracle caches' state arrays and metaState strings; loading it back (and loading the
    oracle's own file) rebuilds caches whose state is bit-identical and whose next decode step
    matches the original cache's bit for bit."""
    import prompt_cache_oracle as pco
    g, o = _filled(kvc, oracle, cuda, dtype)
    assert g[3].is_compressed
    path = str(tmp_path / "prompt.safetensors")
    kvc.save_prompt_cache(path, g, {"tokens": "24"})
    entries, user = pco.load(path)
    assert user == {"tokens": "24"}
    for e, oc in zip(entries, o):
        want = pco.entry_of(oc, bf16=dtype == torch.bfloat16)
        assert (e.class_name, e.meta_state) == (want.class_name, want.meta_state)
        assert len(e.state) == len(want.state)
        for a, b, abf, bbf in zip(e.state, want.state, e.bf16, want.bf16):
            assert a.shape == b.shape and a.dtype == b.dtype and abf == bbf
            assert a.tobytes() == b.tobytes()

    opath = str(tmp_path / "oracle.safetensors")
    pco.save(opath, [pco.entry_of(oc, bf16=dtype == torch.bfloat16) for oc in o], {"tokens": "24"})
    B, H, D = 1, 2, 64
    k, v = seeded((B, H, 1, D), 900, dtype).to(cuda), seeded((B, H, 1, D), 901, dtype).to(cuda)
    q = seeded((B, 2 * H, 1, D), 902, dtype).to(cuda)
    want_out = [kvc.attention_with_cache_update(q, k, v, c.copy(), D ** -0.5, "none") for c in g]
    for p in (path, opath):
        loaded, meta = kvc.load_prompt_cache(p)
        assert meta == {"tokens": "24"}
        assert [type(c) for c in loaded] == [type(c) for c in g]
        for lc, gc, w in zip(loaded, g, want_out):
            assert lc.offset == gc.offset and list(lc.meta_state) == list(gc.meta_state)
            ls, gs = lc.state, gc.state
            assert len(ls) == len(gs)
            for a, b in zip(ls, gs):
                assert a.shape == b.shape and a.dtype == b.dtype and torch.equal(a, b)
            got = kvc.attention_with_cache_update(q, k, v, lc, D ** -0.5, "none")
            assert torch.equal(got, w)
    assert kvc.lib().kvc_device_status() == 0


def test_prompt_cache_legacy_rotating_metadata(kvc, cuda, tmp_path):
    """KVCacheTests.swift:590-603: a five-field RotatingKVCache metaState (files written before the
    capacity origin existed) loads, and reads back with the model-native origin appended."""
    import prompt_cache_oracle as pco
    p = str(tmp_path / "legacy.safetensors")
    pco.save(p, [pco.Entry("RotatingKVCache", [np.zeros((1, 1, 1, 1), np.float32)] * 2, ["0", "32", "256", "1", "1"])])
    (rot,), _ = kvc.load_prompt_cache(p)
    assert isinstance(rot, kvc.RotatingKVCache)
    assert list(rot.meta_state) == ["0", "32", "256", "1", "1", "modelNative"]
