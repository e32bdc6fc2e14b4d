"""Pins the CPU oracle to what the reference itself asserts or ships as data:
the cache-semantics expectations of the reference's unit tests (ported in
scenarios.py), its packing known-answers, its codebook table, and the
properties its codec tests check. Runs without a GPU."""
import json
import os

import numpy as np
import pytest

import scenarios as sc

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def be(oracle):
    return sc.OracleBackend(oracle)


@pytest.mark.parametrize("scenario", sc.ALL_SIMPLE, ids=lambda f: f.__name__)
def test_reference_cache_semantics(be, scenario):
    scenario(be)


@pytest.mark.parametrize("case", sc.COMMIT_CASES, ids=lambda c: f"w{c['window']}p{c['prefill']}k{c.get('keep', 0)}")
def test_commit_equivalence(be, case):
    sc.commit_equivalence(be, **case)


@pytest.mark.parametrize("case", sc.REWIND_CASES, ids=lambda c: f"w{c['window']}p{c['prefill']}r{c['rewinding']}k{c.get('keep', 0)}")
def test_rewind(be, case):
    sc.rewind_matches_emitted_only_replay(be, **case)


def test_packed_width_known_answers(oracle):
    # TurboQuantTests.swift:80-84
    assert oracle.packed_width(128, 4) == 16
    assert oracle.packed_width(128, 3) == 12
    assert oracle.packed_width(128, 1) == 4


@pytest.mark.parametrize("bits,idx", [(3, [0, 1, 2, 3, 4, 5, 6, 7, 7, 6, 5, 4]), (1, [0, 1, 0, 1, 1, 0, 1, 0]),
                                      (4, [0, 5, 10, 15, 3, 7, 11, 14])])
def test_pack_unpack_round_trip(oracle, bits, idx):
    # TurboQuantTests.swift:86-111
    a = np.array([idx], dtype=np.uint32)
    packed = oracle.pack_low_bit(a, bits)
    assert packed.shape == (1, oracle.packed_width(len(idx), bits))
    assert oracle.unpack_low_bit(packed, bits, len(idx)).tolist() == [idx]


def test_pack_layout_low_bits_first_with_straddle(oracle):
    # TurboQuantKVCache.swift:361-394: code d sits at bit d*bits, spilling into the next word.
    idx = np.arange(12, dtype=np.uint32)[None] % 8
    w = oracle.pack_low_bit(idx, 3)[0]
    bits = sum(int(v) << (3 * d) for d, v in enumerate(idx[0]))
    assert int(w[0]) == bits & 0xFFFFFFFF and int(w[1]) == bits >> 32


def test_codebook_matches_reference_table(oracle):
    table = json.load(open(os.path.join(GOLDEN, "turbo_codebooks.json")))["centroids"]
    worst = 0.0
    for dim, per_bits in table.items():
        for bits, vals in per_bits.items():
            got = oracle.generate_centroids(int(dim), int(bits))
            worst = max(worst, float(np.max(np.abs(got - np.array(vals, dtype=np.float32)))))
            assert np.all(np.diff(got) > 0)
    # the shipped table is a float32 k-means snapshot (visibly asymmetric in the 5th decimal)
    assert worst < 2e-4, worst


def test_default_codebook_is_the_reference_table(oracle, kvc):
    """TurboQuantCodebook.codebook(dim:bits:) reads the shipped table first (TurboQuantKVCache.swift:134-147):
    for its nine (head dim, bits) pairs both the oracle's and the library's default centroids are those
    floats exactly, and the boundaries are the float32 midpoints (:164-167)."""
    table = json.load(open(os.path.join(GOLDEN, "turbo_codebooks.json")))["centroids"]
    assert sorted(table) == ["128", "256", "64"]
    for dim, per_bits in table.items():
        assert sorted(per_bits) == ["2", "3", "4"]
        for bits, vals in per_bits.items():
            want = np.array(vals, dtype=np.float32)
            assert np.array_equal(oracle.codebook(int(dim), int(bits)), want)
            assert np.array_equal(oracle.MSECodec(int(dim), int(bits)).codebook, want)
            c, b = kvc.turbo_codebook(int(dim), int(bits))      # host-side table lookup, no device needed
            assert np.array_equal(np.array(c, dtype=np.float32), want)
            assert np.array_equal(np.array(b, dtype=np.float32), ((want[:-1] + want[1:]) / np.float32(2.0)))


@pytest.mark.parametrize("dim,bits", [(32, 4), (512, 3), (1024, 2), (128, 1)])
def test_generated_codebooks_agree_between_library_and_oracle(oracle, kvc, dim, bits):
    """Pairs outside the table come from the generator (:174-233): the library's single-precision k-means
    and the oracle's restatement produce the same floats on the same host."""
    c, _ = kvc.turbo_codebook(dim, bits)
    assert np.array_equal(np.array(c, dtype=np.float32), oracle.generate_centroids(dim, bits))


def test_key_calibration_decision(oracle):
    """computeKeyCalibrationScale (TurboQuantKVCache.swift:867-886): nil for fewer than 32 rows and for keys
    whose rotated coordinates all have the same spread (independent channels, outlier channels included:
    the Walsh-Hadamard rotation spreads every channel evenly); a clamped, mean-normalised scale for keys
    with correlated channels."""
    rng = np.random.default_rng(7)
    D = 128
    signs = oracle.wht_signs(D, 42)
    iid = rng.standard_normal((2, 2, 200, D)).astype(np.float32)
    assert oracle.key_calibration_scale(iid, signs) is None
    out = iid.copy()
    out[..., [3, 90]] *= 20.0
    assert oracle.key_calibration_scale(out, signs) is None
    mix = rng.standard_normal((6, D)).astype(np.float32)
    low = (rng.standard_normal((2, 2, 200, 6)).astype(np.float32) @ mix + 0.25 * iid).astype(np.float32)
    assert oracle.key_calibration_scale(low[:, :1, :7], signs) is None            # 14 rows < 32
    s = oracle.key_calibration_scale(low, signs)
    assert s is not None and s.shape == (D,) and s.dtype == np.float32
    assert s.min() >= 0.25 and s.max() <= 4.0 and abs(float(s.mean()) - 1.0) < 0.05
    assert float(np.max(np.abs(s - 1.0))) >= 0.1
    # the statistic is the population std of the rotated unit rows, up to the fixed-point grid
    unit = low / np.maximum(np.sqrt((low * low).sum(-1, keepdims=True)), 1e-8)
    rot = oracle.MSECodec(D, 3).rotate(unit).reshape(-1, D).astype(np.float64)
    sd = rot.std(axis=0)
    want = np.clip(sd / sd.mean(), 0.25, 4.0)
    assert np.max(np.abs(want - s)) < 1e-5


def test_calibrated_encode_follows_the_scaled_codec(oracle):
    """MSECodec.encode(_:scale:) (TurboQuantKVCache.swift:527-544): indices of rotated / scale, stored norm =
    raw norm / ||codebook[idx] * scale||; decode(scale:) (:573-588) undoes it."""
    rng = np.random.default_rng(8)
    D, bits = 64, 4
    codec = oracle.MSECodec(D, bits, seed=5)
    x = rng.standard_normal((1, 2, 40, D)).astype(np.float32)
    scale = np.clip(1.0 + 0.6 * rng.standard_normal(D), 0.25, 4.0).astype(np.float32)
    packed, norms = codec.encode(x, scale)
    raw = np.sqrt((x * x).sum(-1))
    rot = codec.rotate(x / np.maximum(raw, 1e-8)[..., None])
    idx = oracle.unpack_low_bit(packed, bits, D)
    want = (rot / scale > codec.boundaries[:, None, None, None, None]).sum(0)
    assert (idx != want).mean() < 2e-3          # only values within rounding of a boundary may differ
    recon = codec.codebook[idx] * scale
    assert np.allclose(norms, raw / np.sqrt((recon * recon).sum(-1)), rtol=1e-5)
    # reconstruction quality: decode with the scale folded back in
    approx = oracle.fwht(recon) * np.float32(1.0 / np.sqrt(D)) * codec.signs * norms[..., None]
    cos = (approx * x).sum(-1) / (np.sqrt((approx * approx).sum(-1)) * raw)
    assert cos.min() > 0.85 and cos.mean() > 0.95    # an arbitrary scale on isotropic rows costs some accuracy


def test_group_size_resolution(oracle):
    # KVCacheTests.swift:477-484 (D = 32 falls back 64 -> 32) and KVCache.swift:902-920
    assert oracle.resolved_group_size(64, 32, 32) == 32
    assert oracle.resolved_group_size(64, 128, 128) == 64
    assert oracle.resolved_group_size(96, 128, 128) == 64   # tie between 64 and 128 goes to the smaller
    assert oracle.resolved_group_size(64, 5, 5) is None
    q = oracle.QuantizedKVCache(64, 4)
    ones = oracle.from_f32(np.ones((1, 1, 4, 32), dtype=np.float32), oracle.BF16)
    q.update_quantized(ones, ones)
    assert q.group_size == 32 and q.bits == 4 and q.meta_state == ["256", "4", "32", "4"]


def test_boundary_quantize_equals_argmin(oracle):
    # TurboQuantTests.swift:162-184
    codec = oracle.MSECodec(16, 3, 42)
    rng = np.random.default_rng(0)
    x = rng.standard_normal((4, 16)).astype(np.float32)
    packed, norms = codec.encode(x)
    idx = oracle.unpack_low_bit(packed, 3, 16)
    unit = x / np.maximum(np.linalg.norm(x, axis=-1, keepdims=True), 1e-8)
    rot = codec.rotate(unit)
    argmin = np.argmin(np.abs(rot[..., None] - codec.codebook[None, None]), axis=-1)
    assert np.array_equal(idx, argmin.astype(np.uint32))
    assert np.allclose(norms, np.linalg.norm(x, axis=-1), rtol=1e-6)


def test_fwht_is_an_orthogonal_involution(oracle):
    # TurboQuantTests.swift:186-210: forward then inverse recovers the input to 1e-4
    signs = oracle.wht_signs(128, 42)
    assert set(np.unique(signs)) <= {-1.0, 1.0} and abs(float(signs.sum())) < 64
    rng = np.random.default_rng(1)
    x = rng.standard_normal((8, 128)).astype(np.float32)
    f = np.float32(1 / np.sqrt(128))
    fwd = oracle.fwht(x * signs) * f
    back = oracle.fwht(fwd) * f * signs
    assert float(np.max(np.abs(back - x))) < 1e-4
    H = oracle.fwht(np.eye(128, dtype=np.float32))
    assert np.allclose(H @ H.T, 128 * np.eye(128), atol=1e-3)
    # Sylvester order: H_2n = [[H, H], [H, -H]] (TurboQuantKVCache.swift:263-285)
    assert np.array_equal(H[:64, :64], H[:64, 64:]) and np.array_equal(H[64:, 64:], -H[:64, :64])


@pytest.mark.parametrize("dim,bits,min_cos", [(64, 4, 0.95), (128, 4, 0.90), (32, 3, 0.8)])
def test_codec_quality_bounds(oracle, dim, bits, min_cos):
    # TurboQuantTests.swift:119-160, :212-230
    codec = oracle.MSECodec(dim, bits, 42)
    rng = np.random.default_rng(2)
    x = rng.standard_normal((16, dim)).astype(np.float32)
    dec = codec.decode(*codec.encode(x))
    cos = np.sum(x * dec, -1) / (np.linalg.norm(x, axis=-1) * np.linalg.norm(dec, axis=-1) + 1e-8)
    assert float(cos.mean()) > min_cos


def test_affine_quantizer_properties(oracle):
    """Parity for the quantiser is unpinned (MLX core is not vendored); these are
    the properties MLX documents: w ~ scale*q + bias within half a step, codes in
    range, the extreme of larger magnitude is reproduced exactly."""
    rng = np.random.default_rng(3)
    x = rng.standard_normal((5, 3, 128)).astype(np.float32)
    for bits in (2, 4, 8):
        for g in (32, 64, 128):
            codes, scales, biases = oracle.affine_quantize(x, g, bits)
            assert codes.shape == (5, 3, 128 * bits // 32) and scales.shape == (5, 3, 128 // g)
            deq = oracle.affine_dequantize(codes, scales, biases, g, bits)
            step = np.repeat(np.abs(scales), g, axis=-1)
            idx = np.stack([(codes >> (bits * k)) & ((1 << bits) - 1) for k in range(32 // bits)], axis=-1)
            idx = idx.reshape(5, 3, 128)
            inside = (idx > 0) & (idx < (1 << bits) - 1)
            err = np.abs(deq - x)
            # unclamped codes round to the nearest level; the re-derived scale may clamp the far end
            assert np.all(err[inside] <= 0.5 * step[inside] * (1 + 1e-4) + 1e-6)
            assert np.all(err <= 1.5 * step + 1e-6)
            xg = x.reshape(5, 3, 128 // g, g)
            big = np.where(np.abs(xg.min(-1)) > np.abs(xg.max(-1)), xg.min(-1), xg.max(-1))
            assert np.allclose(biases, big)
    z = np.zeros((1, 64), dtype=np.float32)
    codes, scales, biases = oracle.affine_quantize(z, 64, 8)
    assert not codes.any() and np.all(biases == 0) and np.all(np.abs(scales) == np.float32(1e-7))
    # 8-bit layout pinned by the reference's own kernel (TurboQuantKernels.swift:820-831):
    # element i is byte i%4 of word i/4
    y = np.linspace(-1, 1, 64, dtype=np.float32)[None]
    codes, scales, biases = oracle.affine_quantize(y, 64, 8)
    by = codes.view(np.uint8).reshape(-1)
    assert np.allclose(scales[0, 0] * by.astype(np.float32) + biases[0, 0], y[0], atol=abs(scales[0, 0]) / 2 + 1e-6)


def test_quantized_attention_close_to_full_precision(oracle):
    # KVCacheTests.swift:1185-1217: 8-bit causal quantized attention vs fp, rtol 0.05 atol 0.1, MHA and GQA
    rng = np.random.default_rng(4)
    for hq, hkv in ((4, 4), (8, 2)):
        q = rng.standard_normal((1, hq, 6, 64)).astype(np.float32)
        k = rng.standard_normal((1, hkv, 6, 64)).astype(np.float32)
        v = rng.standard_normal((1, hkv, 6, 64)).astype(np.float32)
        cache = oracle.QuantizedKVCache(64, 8)
        got = oracle.attention_with_cache_update(q, k, v, cache, 0.125, "causal")
        want = oracle.sdpa(q, k, v, 0.125, "causal")
        assert np.allclose(got, want, rtol=0.05, atol=0.1)
        assert np.isfinite(got).all()


def test_rotating_attention_past_wrap_matches_unrotated_history(oracle):
    # KVCacheTests.swift:1451-1491: attention through the ring's own presentation equals a
    # never-rotated history under an explicit causal-and-window mask (1e-5).
    rng = np.random.default_rng(5)
    window, total, D = 8, 21, 16
    K = rng.standard_normal((1, 1, total, D)).astype(np.float32)
    V = rng.standard_normal((1, 1, total, D)).astype(np.float32)
    cache = oracle.RotatingKVCache(window)
    for t in range(total - 1):
        cache.update(K[:, :, t:t + 1], V[:, :, t:t + 1])
    q = rng.standard_normal((1, 2, 1, D)).astype(np.float32)
    got = oracle.attention_with_cache_update(q, K[:, :, -1:], V[:, :, -1:], cache, 0.25, "none")
    mask = np.zeros((1, total), dtype=bool)
    mask[0, total - window:] = True
    want = oracle.sdpa(q, K, V, 0.25, mask)
    assert float(np.max(np.abs(got - want))) < 1e-5


def test_turbo_cache_behaviour(oracle):
    # TurboQuantTests.swift:340-461, :2091-2122, :2242-2264
    rng = np.random.default_rng(6)
    c = oracle.TurboQuantKVCache(bits=4)
    k = rng.standard_normal((1, 2, 250, 64)).astype(np.float32)
    v = rng.standard_normal((1, 2, 250, 64)).astype(np.float32)
    c.update(k, v)
    assert c.offset == 250 and not c.is_compressed and len(c.state) == 2
    for i in range(12):  # growth across the 256-row boundary: 250 + 12 -> 262
        q = rng.standard_normal((1, 4, 1, 64)).astype(np.float32)
        out = c.compressed_attention(q, k[:, :, :1], v[:, :, :1], 0.125)
        assert out.shape == (1, 4, 1, 64) and np.isfinite(out).all()
    assert c.offset == 262 and c.is_compressed and len(c.state) == 4
    assert c.state[0].shape == (1, 2, 262, 8) and c.state[1].shape == (1, 2, 262)
    assert c.meta_state == ["262", "4", "4", "4", "42"]
    assert c.trim(2) == 2 and c.offset == 260
    c.compressed_attention(q, k[:, :, :1], v[:, :, :1], 0.125)
    assert c.offset == 261
    assert c.trim(10_000) == 261 and c.offset == 0 and not c.is_compressed and c.state == []
    asym = oracle.TurboQuantKVCache(bits=4, key_bits=3, value_bits=2)
    asym.update(k[:, :, :8], v[:, :, :8])
    asym.compressed_attention(q, k[:, :, :1], v[:, :, :1], 0.125)
    assert asym.state[0].shape[-1] == oracle.packed_width(64, 3) and asym.state[2].shape[-1] == oracle.packed_width(64, 2)


def test_turbo_attention_tracks_exact_attention(oracle):
    # TurboQuantTests.swift:1872-1960: cosine similarity with exact attention > 0.95 at 4 bits
    rng = np.random.default_rng(7)
    B, Hq, Hkv, T, D = 1, 4, 2, 96, 128
    k = rng.standard_normal((B, Hkv, T, D)).astype(np.float32)
    v = rng.standard_normal((B, Hkv, T, D)).astype(np.float32)
    q = rng.standard_normal((B, Hq, 1, D)).astype(np.float32)
    c = oracle.TurboQuantKVCache(bits=4)
    c.update(k[:, :, :-1], v[:, :, :-1])
    got = c.compressed_attention(q, k[:, :, -1:], v[:, :, -1:], D ** -0.5)
    want = oracle.sdpa(q, k, v, D ** -0.5)
    cos = np.sum(got * want, -1) / (np.linalg.norm(got, axis=-1) * np.linalg.norm(want, axis=-1))
    assert float(cos.min()) > 0.95


def test_turbo_causal_chunk_equals_per_position_decode(oracle):
    # TurboQuantTests.swift:965-1055: an L>1 causal call equals L truncated single-token calls
    rng = np.random.default_rng(8)
    B, Hq, Hkv, T, D, L = 1, 4, 2, 40, 64, 5
    k = rng.standard_normal((B, Hkv, T + L, D)).astype(np.float32)
    v = rng.standard_normal((B, Hkv, T + L, D)).astype(np.float32)
    q = rng.standard_normal((B, Hq, L, D)).astype(np.float32)
    a = oracle.TurboQuantKVCache(bits=4)
    a.update(k[:, :, :T], v[:, :, :T])
    chunk = a.compressed_attention(q, k[:, :, T:], v[:, :, T:], 0.125, "causal")
    b = oracle.TurboQuantKVCache(bits=4)
    b.update(k[:, :, :T], v[:, :, :T])
    for l in range(L):
        one = b.compressed_attention(q[:, :, l:l + 1], k[:, :, T + l:T + l + 1], v[:, :, T + l:T + l + 1], 0.125)
        assert float(np.max(np.abs(one[:, :, 0] - chunk[:, :, l]))) < 1e-5
    assert all(np.array_equal(x, y) for x, y in zip(a.state, b.state))


def test_scheme_tables_and_boundary_protection_host_logic(kvc):
    """resolveTurboScheme / resolveAffineScheme tables (TurboQuantKVCache.swift:1611-1635,
    KVCache.swift:2455-2461) and turboQuantProtectedPaths (KVCacheTree.swift:118-134): host logic of
    the library, no device needed."""
    assert kvc.resolve_turbo_scheme("turbo4") == (4, 4)
    assert kvc.resolve_turbo_scheme("turbo4v2") == (4, 2)
    assert kvc.resolve_turbo_scheme("turbo0v3") == (0, 3)
    assert kvc.resolve_turbo_scheme("turbo8v4") == (8, 4)
    assert kvc.resolve_turbo_scheme("turbo3") == (3, 3) and kvc.resolve_turbo_scheme("turbo2") == (2, 2)
    assert kvc.resolve_turbo_scheme("turbo5") is None and kvc.resolve_turbo_scheme(None) is None
    assert kvc.resolve_affine_scheme("affine4") == (4, 64) and kvc.resolve_affine_scheme("affine8") == (8, 64)
    assert kvc.resolve_affine_scheme("affine2") is None
    S, R, Q, T = kvc.KIND_SIMPLE, kvc.KIND_ROTATING, kvc.KIND_QUANTIZED, kvc.KIND_TURBO
    # fragile scheme, 8 eligible layers: two on each end
    assert kvc.turbo_protected_layers([S] * 8, 4, 4) == [True, True, False, False, False, False, True, True]
    # robust schemes (raw / 8-bit keys with values above 2 bits) protect nothing
    assert kvc.turbo_protected_layers([S] * 8, 0, 4) == [False] * 8
    assert kvc.turbo_protected_layers([S] * 8, 8, 3) == [False] * 8
    # ... but 2-bit values are fragile whatever the keys are
    assert kvc.turbo_protected_layers([S] * 6, 8, 2) == [True, True, False, False, True, True]
    # rotating layers do not count: protection lands on the first / last ELIGIBLE layers
    assert kvc.turbo_protected_layers([R, S, R, S, S, Q, T, R], 3, 3) == [False, True, False, True, False, True, True, False]
    # min(2, eligible / 2): three eligible layers protect one on each end, one protects none
    assert kvc.turbo_protected_layers([S, S, S], 4, 4) == [True, False, True]
    assert kvc.turbo_protected_layers([S], 4, 4) == [False]


def test_prompt_cache_file_format_and_corrupt_rejection(kvc, tmp_path):
    """savePromptCache / loadPromptCache wire format (KVCache.swift:1797-1846, :2031-2138) on empty
    caches (no device needed): key layout of the safetensors header, class names, metaState strings,
    user metadata; corrupt files are rejected the way restoreCacheFromMetaState rejects them."""
    import json
    import struct
    caches = [kvc.KVCacheSimple(), kvc.RotatingKVCache(max_size=32, keep=4), kvc.QuantizedKVCache(32, 4),
              kvc.TurboQuantKVCache(bits=4, key_bits=3, value_bits=4, seed=7)]
    path = str(tmp_path / "prompt.safetensors")
    kvc.save_prompt_cache(path, caches, {"model": "tiny", "note": 'a "quoted"\nline'})
    raw = open(path, "rb").read()
    hlen = struct.unpack("<Q", raw[:8])[0]
    header = json.loads(raw[8:8 + hlen])
    meta = header["__metadata__"]
    assert [meta[f"2.{i}"] for i in range(4)] == ["KVCache", "RotatingKVCache", "QuantizedKVCache", "TurboQuantKVCache"]
    assert meta["0.0.0"] == ""                                      # KVCacheSimple: the single empty placeholder
    assert [meta[f"0.1.{j}"] for j in range(5)] == ["4", "32", "256", "0", "0"]     # keep, maxSize, step, offset, idx
    assert [meta[f"0.2.{j}"] for j in range(4)] == ["256", "0", "32", "4"]          # step, offset, groupSize, bits
    assert meta["1.model"] == "tiny" and meta["1.note"] == 'a "quoted"\nline'
    assert set(header) == {"__metadata__"}                           # empty caches carry no tensors

    loaded, user = kvc.load_prompt_cache(path)
    assert [type(c).__name__ for c in loaded] == ["KVCacheSimple", "RotatingKVCache", "QuantizedKVCache", "TurboQuantKVCache"]
    assert user == {"model": "tiny", "note": 'a "quoted"\nline'}
    assert loaded[1].max_size == 32 and list(loaded[1].meta_state)[:3] == ["4", "32", "256"]
    assert loaded[2].group_size == 32 and loaded[2].bits == 4
    assert list(loaded[3].meta_state) == list(caches[3].meta_state)

    # the oracle's reader accepts the library's file and sees the same triples; the library accepts the oracle's
    import prompt_cache_oracle as pco
    entries, ouser = pco.load(path)
    assert ouser == user
    assert [(e.class_name, e.meta_state, len(e.state)) for e in entries] == \
        [(pco.class_name_of(c), list(c.meta_state), 0) for c in caches]
    opath = str(tmp_path / "oracle.safetensors")
    pco.save(opath, entries, {"k": "v"})
    again, user2 = kvc.load_prompt_cache(opath)
    assert user2 == {"k": "v"}
    assert [list(c.meta_state) for c in again] == [list(c.meta_state) for c in caches]
    with pytest.raises(kvc.KVCError, match="reserved"):
        kvc.save_prompt_cache(path, caches, {"__mlx_lm_state_count": "1"})

    def fixture(class_name, array_count, metadata, shape=(1, 1, 1, 1)):
        """writePromptCacheFixture of the reference's KVCacheTests.swift:30-47: float32 zero arrays "0.j"."""
        p = str(tmp_path / "fixture.safetensors")
        pco.save(p, [pco.Entry(class_name, [np.zeros(shape, np.float32)] * array_count, metadata)])
        return p

    # KVCacheTests.swift:566-588: invalid metadata and invalid state rank are rejected
    for bad in (("KVCacheSimple", 0, ["unexpected"]),
                ("RotatingKVCache", 0, ["0", "32", "invalid", "0", "0", "modelNative"]),
                ("RotatingKVCache", 0, ["0", "32", "256", "0", "0", "invalid-origin"]),
                ("QuantizedKVCache", 0, ["256", "invalid", "64", "4"]),
                ("KVCacheSimple", 2, [""], (1, 1))):
        with pytest.raises(kvc.KVCError):
            kvc.load_prompt_cache(fixture(*bad))
        with pytest.raises(pco.PromptCacheError):
            pco.load(fixture(*bad))

    def write(meta_dict, tensors=None):
        blob = json.dumps({"__metadata__": meta_dict, **(tensors or {})}).encode()
        p = str(tmp_path / "bad.safetensors")
        open(p, "wb").write(struct.pack("<Q", len(blob)) + blob)
        return p

    for bad in ({"2.0": "KVCache", "0.0.0": "x"},                       # placeholder must be empty
                {"2.0": "RotatingKVCache", "0.0.0": "0", "0.0.1": "8"},  # 2 metadata entries instead of 5 / 6
                {"2.0": "QuantizedKVCache", "0.0.0": "256", "0.0.1": "0", "0.0.2": "sixty-four", "0.0.3": "4"},
                {"2.0": "NoSuchCache", "0.0.0": ""},
                {"2.0": "KVCache", "2.1": "KVCache", "0.0.0": ""},             # class count != metaState count
                {"2.0": "KVCache", "0.0.0": "", "1.__mlx_lm_state_version": "1", "1.__mlx_lm_state_count": "1"},
                {"2.0": "__mlx_lm_state_v1__:KVCache", "0.0.0": ""}):
        with pytest.raises(kvc.KVCError):
            kvc.load_prompt_cache(write(bad))
    # an array whose cache index has no class entry (unflattenArrays, KVCache.swift:2166-2185)
    with pytest.raises(kvc.KVCError):
        kvc.load_prompt_cache(write({"2.0": "KVCache", "0.0.0": ""},
                                    {"3.0": {"dtype": "F32", "shape": [1, 1, 1, 1], "data_offsets": [0, 4]}}))
