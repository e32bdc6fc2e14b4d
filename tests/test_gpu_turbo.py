"""GPU parity for the TurboQuant path: packed codebook indices and norms are
bit-identical to the oracle's Walsh-Hadamard encode; compressed attention
(decode and the multi-token causal verify chunk) is within tolerance."""
import numpy as np
import pytest
import torch

from helpers import TOL, bits_equal, max_abs_diff, seeded, to_oracle, worst_excess

pytestmark = pytest.mark.gpu


def test_library_codebook_and_signs_match_the_oracle(kvc, oracle):
    for dim in (64, 128, 256):
        for bits in (2, 3, 4):
            c, b = kvc.turbo_codebook(dim, bits)
            # the shipped table (TurboQuantKVCache.swift:57-94) is the default on both sides ...
            assert np.array_equal(np.array(c, dtype=np.float32), oracle.codebook(dim, bits))
            # ... and the generator lands within the table's own asymmetry of it
            assert np.max(np.abs(np.array(c, dtype=np.float32) - oracle.generate_centroids(dim, bits))) < 2e-4
            assert len(b) == (1 << bits) - 1 and all(b[i] < b[i + 1] for i in range(len(b) - 1))
        assert np.array_equal(np.array(kvc.turbo_signs(dim, 42), dtype=np.float32), oracle.wht_signs(dim, 42))
    assert kvc.turbo_packed_width(128, 3) == 12 and kvc.turbo_packed_width(128, 4) == 16


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("D", [32, 64, 128, 256, 512])
@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("table", ["golden", "generated"])
def test_turbo_encode_bit_exact(kvc, oracle, cuda, dtype, D, bits, table):
    """Boundaries from the reference's shipped centroid table (the fixture under tests/golden, where it has
    the pair) and from the generator; either way the oracle computes its own boundaries, the library is
    only handed the same floats."""
    rows = 517
    x = seeded((rows, D), D + bits, dtype, outlier_frac=0.02)
    x[3] = 0                      # zero row: norm floor
    x[4] = x[4].abs()             # one-sided row
    x[5, 1:] = 0                  # a single spike
    signs = oracle.wht_signs(D, 42)
    if table == "golden":
        if (D, bits) not in oracle.shipped_centroids():
            pytest.skip("the reference ships no table for this pair")
        cb = oracle.shipped_centroids()[(D, bits)]
    else:
        cb = oracle.generate_centroids(D, bits)
    bounds = oracle.boundaries_of(cb)
    packed, norms = kvc.turbo_encode(x.to(cuda), signs, bounds, bits)
    rp, rn = oracle.turbo_encode(to_oracle(x), signs, bounds, bits)
    assert bits_equal(norms, rn), "norms differ"
    assert bits_equal(packed, rp), "packed indices differ"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("D,bits", [(128, 3), (128, 4), (64, 2), (256, 4), (32, 3)])
def test_turbo_encode_bit_exact_many_rows(kvc, oracle, cuda, dtype, D, bits):
    """A prefill-sized row count (the launcher keeps several rows per warp in flight) plus a row count
    that leaves the last warp half empty; unsorted boundaries take the counting path."""
    signs = oracle.wht_signs(D, 7)
    bounds = oracle.boundaries_of(np.array(kvc.turbo_codebook(D, bits)[0], dtype=np.float32))
    for rows, bnd in ((8192 + 5, bounds), (9001, bounds[::-1].copy())):
        x = seeded((rows, D), rows + D + bits, dtype, outlier_frac=0.02)
        packed, norms = kvc.turbo_encode(x.to(cuda), signs, bnd, bits)
        rp, rn = oracle.turbo_encode(to_oracle(x), signs, bnd, bits)
        assert bits_equal(norms, rn), "norms differ"
        assert bits_equal(packed, rp), "packed indices differ"


def _pair(kvc, oracle, **kw):
    g = kvc.TurboQuantKVCache(**kw)
    kb = kw.get("key_bits", kw.get("bits", 4))
    vb = kw.get("value_bits", kw.get("bits", 4))
    return g, kb, vb


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("kw", [dict(bits=4), dict(bits=4, key_bits=3, value_bits=4), dict(bits=3),
                                dict(bits=4, key_bits=0, value_bits=4), dict(bits=4, key_bits=8, value_bits=3),
                                dict(bits=4, key_bits=3, value_bits=4, affine_values=True)],
                         ids=["turbo4", "k3v4", "turbo3", "turbo0v4", "turbo8v3", "k3-affine-v4"])
def test_turbo_cache_decode_and_verify(kvc, oracle, cuda, dtype, kw):
    B, Hq, Hkv, D, P = 2, 8, 2, 128, 250
    g = kvc.TurboQuantKVCache(**kw)
    o = oracle.TurboQuantKVCache(**kw)      # default codecs on both sides: the reference's shipped centroid table
    scale = D ** -0.5
    q, k, v = seeded((B, Hq, P, D), 1, dtype), seeded((B, Hkv, P, D), 2, dtype), seeded((B, Hkv, P, D), 3, dtype)
    out = g.attention(q.to(cuda), k.to(cuda), v.to(cuda), scale, "causal")      # raw prefill + plain SDPA
    ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, scale, "causal")
    assert max_abs_diff(out, ref) <= TOL[dtype]
    assert not g.is_compressed and g.offset == P
    for step in range(12):                                                     # crosses the 256-row boundary
        q, k, v = (seeded((B, Hq, 1, D), 10 + 3 * step, dtype), seeded((B, Hkv, 1, D), 11 + 3 * step, dtype),
                   seeded((B, Hkv, 1, D), 12 + 3 * step, dtype))
        out = g.attention(q.to(cuda), k.to(cuda), v.to(cuda), scale)
        ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, scale)
        assert max_abs_diff(out, ref) <= TOL[dtype], f"decode step {step}"
    assert g.is_compressed and g.offset == o.offset == P + 12
    L = 6                                                                       # 5 draft tokens + bonus
    q, k, v = seeded((B, Hq, L, D), 90, dtype), seeded((B, Hkv, L, D), 91, dtype), seeded((B, Hkv, L, D), 92, dtype)
    out = g.attention(q.to(cuda), k.to(cuda), v.to(cuda), scale, "causal")
    ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, scale, "causal")
    assert max_abs_diff(out, ref) <= TOL[dtype], "verify chunk"
    assert g.trim(L - 2) == o.trim(L - 2)                                       # reject 4 of the 6
    gs, os_ = g.state, o.state
    assert len(gs) == len(os_)
    for a, b in zip(gs, os_):
        assert tuple(a.shape) == tuple(b.shape) and bits_equal(a, np.ascontiguousarray(b))
    assert list(g.meta_state) == list(o.meta_state)
    mask = torch.ones((1, 1, 1, g.offset + 1), dtype=torch.bool)
    mask[..., ::3] = False
    q, k, v = seeded((B, Hq, 1, D), 95, dtype), seeded((B, Hkv, 1, D), 96, dtype), seeded((B, Hkv, 1, D), 97, dtype)
    out = g.attention(q.to(cuda), k.to(cuda), v.to(cuda), scale, mask.to(cuda))
    ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, scale, mask.numpy())
    assert max_abs_diff(out, ref) <= TOL[dtype], "array mask"
    assert g.trim(10_000) == o.trim(10_000) and g.offset == 0 and not g.is_compressed and g.state == []


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("Hq,Hkv,L,P,kw", [
    (16, 2, 6, 1000, dict(bits=4, key_bits=3, value_bits=4)),   # 48 rows per kv head
    (8, 2, 5, 517, dict(bits=4)),                               # 20 rows, 4-bit keys
    (32, 2, 1, 300, dict(bits=4, key_bits=2, value_bits=4)),    # 16 heads per kv head, one position, no mask
    (8, 1, 8, 2049, dict(bits=4, key_bits=3, value_bits=4)),    # 64 rows, the most the kernel takes; ragged last stage
])
def test_short_chunks_run_on_the_tensor_core_verify_kernel(kvc, oracle, cuda, capfd, monkeypatch, dtype, Hq, Hkv, L, P, kw):
    """A verify chunk over a compressed cache (4-bit values, 9 to 64 rows per kv head): the group's rows go
    through the tcgen05 verify kernel."""
    B, D = 2, 128
    monkeypatch.setenv("KVC_TRACE_DISPATCH", "1")
    g, o = kvc.TurboQuantKVCache(**kw), oracle.TurboQuantKVCache(**kw)
    k, v = seeded((B, Hkv, P, D), 1, dtype), seeded((B, Hkv, P, D), 2, dtype)
    g.encode_new_token(k.to(cuda), v.to(cuda))
    o.encode_new_token(to_oracle(k), to_oracle(v))
    mask = "causal" if L > 1 else "none"
    for rnd in range(2):
        q = seeded((B, Hq, L, D), 3 + rnd, dtype)
        k1, v1 = seeded((B, Hkv, L, D), 5 + rnd, dtype), seeded((B, Hkv, L, D), 7 + rnd, dtype)
        capfd.readouterr()
        out = g.attention(q.to(cuda), k1.to(cuda), v1.to(cuda), D ** -0.5, mask)
        torch.cuda.synchronize()
        err = capfd.readouterr().err
        # the tensor-core verify kernel (rows decoded once per group)
        assert "verify_tc" in err
        ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k1), to_oracle(v1), o, D ** -0.5, mask)
        assert max_abs_diff(out, ref) <= TOL[dtype], f"round {rnd}"
        assert g.trim(L - 1) == o.trim(L - 1)
    assert kvc.lib().kvc_device_status() == 0


def test_turbo_starts_compressed_when_first_call_is_decode(kvc, oracle, cuda):
    B, Hq, Hkv, D = 1, 4, 1, 64
    g = kvc.TurboQuantKVCache(bits=4)
    o = oracle.TurboQuantKVCache(bits=4)
    for step in range(5):
        q, k, v = seeded((B, Hq, 1, D), step, torch.float32), seeded((B, Hkv, 1, D), 50 + step, torch.float32), seeded((B, Hkv, 1, D), 70 + step, torch.float32)
        out = g.attention(q.to(cuda), k.to(cuda), v.to(cuda), 0.125)
        ref = o.compressed_attention(to_oracle(q), to_oracle(k), to_oracle(v), 0.125)
        assert max_abs_diff(out, ref) <= 1e-4
    assert g.is_compressed and len(g.state) == 4


def test_simple_to_turbo_conversion(kvc, cuda):
    s = kvc.KVCacheSimple()
    k = seeded((1, 2, 9, 64), 1, torch.bfloat16).to(cuda)
    s.update(k, k)
    t = s.to_turbo(4, 4)
    assert t.offset == 9 and not t.is_compressed and len(t.state) == 2
    assert torch.equal(t.state[0], s.state[0])


@pytest.mark.parametrize("kw", [dict(bits=4), dict(bits=4, key_bits=3, value_bits=4)])
def test_chunked_compressed_append_matches_oracle(kvc, oracle, cuda, kw):
    """encodeNewToken without attention: chunked prefill straight into the compressed
    representation gives the same packed state as the oracle, and decode on top agrees."""
    B, Hq, Hkv, D = 2, 8, 2, 128
    dtype = torch.bfloat16
    g = kvc.TurboQuantKVCache(reserve_tokens=700, **kw)
    o = oracle.TurboQuantKVCache(**kw)
    for i, n in enumerate([256, 100, 1, 243]):
        k, v = seeded((B, Hkv, n, D), 2 * i, dtype), seeded((B, Hkv, n, D), 2 * i + 1, dtype)
        g.encode_new_token(k.to(cuda), v.to(cuda))
        o.encode_new_token(to_oracle(k), to_oracle(v))
    assert g.is_compressed and g.offset == o.offset == 600
    for a, b in zip(g.state, o.state):
        assert tuple(a.shape) == tuple(b.shape) and bits_equal(a, np.ascontiguousarray(b))
    q, k, v = seeded((B, Hq, 1, D), 50, dtype), seeded((B, Hkv, 1, D), 51, dtype), seeded((B, Hkv, 1, D), 52, dtype)
    out = g.attention(q.to(cuda), k.to(cuda), v.to(cuda), D ** -0.5)
    ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, D ** -0.5)
    assert max_abs_diff(out, ref) <= TOL[dtype]


def _correlated_keys(shape, seed, dtype, rank=6, noise=0.25):
    """Keys whose channels are correlated (a low-rank mix plus noise): after the rotation the spread differs
    from one coordinate to the next, which is what makes computeKeyCalibrationScale return a scale."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    D = shape[-1]
    mix = torch.randn((rank, D), generator=torch.Generator(device="cpu").manual_seed(1234), dtype=torch.float32)
    z = torch.randn(shape[:-1] + (rank,), generator=g, dtype=torch.float32)
    return (z @ mix + noise * torch.randn(shape, generator=g, dtype=torch.float32)).to(dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("kw", [dict(bits=4), dict(bits=4, key_bits=3, value_bits=4)], ids=["turbo4", "k3v4"])
def test_key_calibration_matches_oracle(kvc, oracle, cuda, tmp_path, dtype, kw):
    """Raw prefill of correlated keys, then decode: the raw-to-compressed transition derives the per-dimension
    calibration scale (TurboQuantKVCache.swift:867-886, :960-970), keys are encoded through the scaled codec
    (TurboQuantKernels.swift:354-411), the scale is folded into the rotated query (:1348-1352) and becomes the
    fifth state array (:1509-1511). Scale, indices and norms are bit-exact against the oracle, outputs in
    tolerance on the decode kernel, the verify-chunk kernel and the general kernel (array mask)."""
    B, Hq, Hkv, D, P = 2, 8, 2, 128, 300
    scale = D ** -0.5
    g, o = kvc.TurboQuantKVCache(**kw), oracle.TurboQuantKVCache(**kw)
    q, v = seeded((B, Hq, P, D), 1, dtype), seeded((B, Hkv, P, D), 3, dtype)
    k = _correlated_keys((B, Hkv, P, D), 2, dtype)
    out = g.attention(q.to(cuda), k.to(cuda), v.to(cuda), scale, "causal")
    ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, scale, "causal")
    assert max_abs_diff(out, ref) <= TOL[dtype]
    for step in range(8):
        q, v = seeded((B, Hq, 1, D), 10 + 3 * step, dtype), seeded((B, Hkv, 1, D), 12 + 3 * step, dtype)
        k = _correlated_keys((B, Hkv, 1, D), 11 + 3 * step, dtype)
        out = g.attention(q.to(cuda), k.to(cuda), v.to(cuda), scale)
        ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, scale)
        assert max_abs_diff(out, ref) <= TOL[dtype], f"decode step {step}"
    assert o.key_calib_scale is not None, "the oracle did not calibrate: the inputs are not anisotropic enough"
    gs, os_ = g.state, o.state
    assert len(gs) == len(os_) == 5
    for a, b in zip(gs, os_):
        assert tuple(a.shape) == tuple(b.shape) and bits_equal(a, np.ascontiguousarray(b))
    L = 6
    q, v = seeded((B, Hq, L, D), 90, dtype), seeded((B, Hkv, L, D), 92, dtype)
    k = _correlated_keys((B, Hkv, L, D), 91, dtype)
    out = g.attention(q.to(cuda), k.to(cuda), v.to(cuda), scale, "causal")
    ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, scale, "causal")
    assert max_abs_diff(out, ref) <= TOL[dtype], "verify chunk"
    mask = torch.ones((1, 1, 1, g.offset + 1), dtype=torch.bool)
    mask[..., ::3] = False
    q, v = seeded((B, Hq, 1, D), 95, dtype), seeded((B, Hkv, 1, D), 97, dtype)
    k = _correlated_keys((B, Hkv, 1, D), 96, dtype)
    out = g.attention(q.to(cuda), k.to(cuda), v.to(cuda), scale, mask.to(cuda))
    ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, scale, mask.numpy())
    assert max_abs_diff(out, ref) <= TOL[dtype], "array mask"
    # the five-array state survives copy() and a prompt-cache file, and decode continues identically
    c2 = g.copy()
    path = str(tmp_path / "calibrated.safetensors")
    kvc.save_prompt_cache(path, [g])
    loaded, _ = kvc.load_prompt_cache(path)
    q, v = seeded((B, Hq, 1, D), 98, dtype), seeded((B, Hkv, 1, D), 99, dtype)
    k = _correlated_keys((B, Hkv, 1, D), 100, dtype)
    outs = [c.attention(q.to(cuda), k.to(cuda), v.to(cuda), scale) for c in (g, c2, loaded[0])]
    ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, scale)
    assert max_abs_diff(outs[0], ref) <= TOL[dtype]
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    for c in (c2, loaded[0]):
        assert len(c.state) == 5
        for a, b in zip(c.state, o.state):
            assert bits_equal(a, np.ascontiguousarray(b))
    assert g.trim(10_000) == o.trim(10_000) and g.state == [] and not g.is_compressed
    # a fresh sequence of isotropic keys on the same object: the scale is gone and none is derived
    # (enough rows that the sampling noise of the per-dimension spread stays well under the 10 % threshold)
    q, k, v = seeded((B, Hq, 600, D), 101, dtype), seeded((B, Hkv, 600, D), 102, dtype), seeded((B, Hkv, 600, D), 103, dtype)
    g.attention(q.to(cuda), k.to(cuda), v.to(cuda), scale, "causal")
    oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, scale, "causal")
    q, k, v = seeded((B, Hq, 1, D), 104, dtype), seeded((B, Hkv, 1, D), 105, dtype), seeded((B, Hkv, 1, D), 106, dtype)
    out = g.attention(q.to(cuda), k.to(cuda), v.to(cuda), scale)
    ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, scale)
    assert o.key_calib_scale is None and len(g.state) == 4 and max_abs_diff(out, ref) <= TOL[dtype]


def test_outlier_channels_do_not_calibrate(kvc, oracle, cuda):
    """Independent channels, a few of them 20 times larger: the rotation spreads each channel over every
    coordinate, the deviation stays under 10 % and both sides keep the plain four-array state."""
    B, Hq, Hkv, D, P = 1, 8, 2, 128, 200
    dtype = torch.bfloat16
    g, o = kvc.TurboQuantKVCache(bits=4), oracle.TurboQuantKVCache(bits=4)
    q, k, v = seeded((B, Hq, P, D), 1, dtype), seeded((B, Hkv, P, D), 2, dtype, outlier_frac=0.02), seeded((B, Hkv, P, D), 3, dtype)
    g.attention(q.to(cuda), k.to(cuda), v.to(cuda), D ** -0.5, "causal")
    oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, D ** -0.5, "causal")
    q, k, v = seeded((B, Hq, 1, D), 4, dtype), seeded((B, Hkv, 1, D), 5, dtype, outlier_frac=0.02), seeded((B, Hkv, 1, D), 6, dtype)
    out = g.attention(q.to(cuda), k.to(cuda), v.to(cuda), D ** -0.5)
    ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, D ** -0.5)
    assert o.key_calib_scale is None and len(g.state) == len(o.state) == 4
    for a, b in zip(g.state, o.state):
        assert bits_equal(a, np.ascontiguousarray(b))
    assert max_abs_diff(out, ref) <= TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("D,kw", [(80, dict(bits=4)), (96, dict(bits=4, key_bits=3, value_bits=4)), (80, dict(bits=3)),
                                  (96, dict(bits=4, key_bits=0, value_bits=4))],
                         ids=["d80-turbo4", "d96-k3v4", "d80-turbo3", "d96-rawk-v4"])
def test_dense_rotation_codec_for_other_head_dims(kvc, oracle, cuda, tmp_path, dtype, D, kw):
    """Head dims that are not powers of two (the reference pre-populates 80 and 96 for real models,
    TurboQuantKVCache.swift:98-110) take the dense random rotation and the norm-corrected encode
    (fusedEncodeSource, TurboQuantKernels.swift:103-204). Both sides are handed the same rotation matrices
    (the oracle's QR; the library's own generator is checked against it below): packed indices and
    corrected norms bit-exact, raw prefill -> compress -> decode -> verify chunk -> array mask in tolerance."""
    B, Hq, Hkv, P = 2, 8, 2, 150
    scale = D ** -0.5
    g, o = kvc.TurboQuantKVCache(**kw), oracle.TurboQuantKVCache(**kw)
    kr, vr = oracle.rotation_matrix(D, 42), oracle.rotation_matrix(D, 43)
    g.set_rotation(kr, vr, D)
    q, k, v = seeded((B, Hq, P, D), 1, dtype), seeded((B, Hkv, P, D), 2, dtype), seeded((B, Hkv, P, D), 3, dtype)
    out = g.attention(q.to(cuda), k.to(cuda), v.to(cuda), scale, "causal")
    ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, scale, "causal")
    assert max_abs_diff(out, ref) <= TOL[dtype]
    for step in range(6):
        q, k, v = (seeded((B, Hq, 1, D), 10 + 3 * step, dtype), seeded((B, Hkv, 1, D), 11 + 3 * step, dtype),
                   seeded((B, Hkv, 1, D), 12 + 3 * step, dtype))
        out = g.attention(q.to(cuda), k.to(cuda), v.to(cuda), scale)
        ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, scale)
        assert max_abs_diff(out, ref) <= TOL[dtype], f"decode step {step}"
    assert g.is_compressed and g.offset == o.offset == P + 6
    gs, os_ = g.state, o.state
    assert len(gs) == len(os_)
    for a, b in zip(gs, os_):
        assert tuple(a.shape) == tuple(b.shape) and bits_equal(a, np.ascontiguousarray(b))
    q, k, v = seeded((B, Hq, 6, D), 90, dtype), seeded((B, Hkv, 6, D), 91, dtype), seeded((B, Hkv, 6, D), 92, dtype)
    out = g.attention(q.to(cuda), k.to(cuda), v.to(cuda), scale, "causal")
    ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, scale, "causal")
    assert max_abs_diff(out, ref) <= TOL[dtype], "verify chunk"
    mask = torch.ones((1, 1, 1, g.offset + 1), dtype=torch.bool)
    mask[..., ::3] = False
    q, k, v = seeded((B, Hq, 1, D), 95, dtype), seeded((B, Hkv, 1, D), 96, dtype), seeded((B, Hkv, 1, D), 97, dtype)
    out = g.attention(q.to(cuda), k.to(cuda), v.to(cuda), scale, mask.to(cuda))
    ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, scale, mask.numpy())
    assert max_abs_diff(out, ref) <= TOL[dtype], "array mask"
    for a, b in zip(g.state, o.state):
        assert bits_equal(a, np.ascontiguousarray(b))
    assert kvc.device_status() == 0


def test_library_rotation_generator(kvc, oracle):
    """The library's own dense rotation (splitmix64 + Box-Muller + Householder QR in double precision) is
    orthogonal and equals the oracle's restatement of the same recipe up to float32 rounding."""
    for D, seed in ((80, 42), (96, 43), (24, 7), (160, 9)):
        r = kvc.turbo_rotation(D, seed)
        assert np.abs(r.astype(np.float64) @ r.astype(np.float64).T - np.eye(D)).max() < 1e-6
        assert np.abs(r - oracle.rotation_matrix(D, seed)).max() < 1e-6


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,Hq,Hkv,L,P,kb,mask", [
    (1, 9, 1, 1, 50, 3, "none"),        # nine rows, one key tile, one CTA
    (1, 8, 1, 8, 120, 3, "causal"),     # 64 rows; the chunk itself crosses the first tile boundary
    (3, 6, 2, 3, 128 * 5, 2, "causal"), # 2-bit keys; stored rows a multiple of the tile; several splits per unit
    (2, 16, 2, 7, 1531, 3, "causal"),   # 56 rows, ragged last tile, splits with a shorter last one
    (16, 64, 8, 6, 700, 3, "causal"),   # the 70B layout: 128 units, one CTA each, no split
    (2, 16, 2, 5, 900, 4, "causal"),    # 4-bit keys (turbo4): the keys read the value pair table
    (40, 12, 4, 3, 300, 3, "causal"),   # 160 units of three tiles on fewer SMs: CTAs that walk two or three units, whole and cut
    (37, 25, 5, 2, 530, 2, "causal"),   # 185 units of five tiles: ranges of seven tiles, every unit cut somewhere else
])
def test_tensor_core_verify_kernel_shapes(kvc, oracle, cuda, capfd, monkeypatch, dtype, B, Hq, Hkv, L, P, kb, mask):
    """Edge shapes of the tcgen05 verify kernel (9 .. 64 rows per kv head, 2- / 3-bit keys, 4-bit values): row
    counts, tile boundaries, split counts; two rounds in a row with a rejection in between."""
    D = 128
    monkeypatch.setenv("KVC_TRACE_DISPATCH", "1")
    kw = dict(bits=4, key_bits=kb, value_bits=4)
    g, o = kvc.TurboQuantKVCache(**kw), oracle.TurboQuantKVCache(**kw)
    k, v = seeded((B, Hkv, P, D), 1, dtype), seeded((B, Hkv, P, D), 2, dtype)
    g.encode_new_token(k.to(cuda), v.to(cuda))
    o.encode_new_token(to_oracle(k), to_oracle(v))
    for rnd in range(2):
        q = seeded((B, Hq, L, D), 3 + rnd, dtype)
        k1, v1 = seeded((B, Hkv, L, D), 5 + rnd, dtype), seeded((B, Hkv, L, D), 7 + rnd, dtype)
        capfd.readouterr()
        out = g.attention(q.to(cuda), k1.to(cuda), v1.to(cuda), D ** -0.5, mask)
        torch.cuda.synchronize()
        assert "verify_tc" in capfd.readouterr().err
        ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k1), to_oracle(v1), o, D ** -0.5, mask)
        assert max_abs_diff(out, ref) <= TOL[dtype], f"round {rnd}"
        assert g.trim(max(L - 1, 0)) == o.trim(max(L - 1, 0))
    assert kvc.lib().kvc_device_status() == 0


def test_tensor_core_verify_kernel_with_calibrated_keys(kvc, oracle, cuda, capfd, monkeypatch):
    """Correlated keys: the cache calibrates at compression; the verify kernel's rotated queries carry the scale."""
    monkeypatch.setenv("KVC_TRACE_DISPATCH", "1")
    B, Hq, Hkv, D, P, L = 2, 8, 2, 128, 600, 6
    dtype = torch.bfloat16
    kw = dict(bits=4, key_bits=3, value_bits=4)
    g, o = kvc.TurboQuantKVCache(**kw), oracle.TurboQuantKVCache(**kw)
    q, v = seeded((B, Hq, P, D), 1, dtype), seeded((B, Hkv, P, D), 3, dtype)
    k = _correlated_keys((B, Hkv, P, D), 2, dtype)
    g.attention(q.to(cuda), k.to(cuda), v.to(cuda), D ** -0.5, "causal")
    oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, D ** -0.5, "causal")
    q1, k1, v1 = seeded((B, Hq, 1, D), 4, dtype), _correlated_keys((B, Hkv, 1, D), 5, dtype), seeded((B, Hkv, 1, D), 6, dtype)
    g.attention(q1.to(cuda), k1.to(cuda), v1.to(cuda), D ** -0.5)
    oracle.attention_with_cache_update(to_oracle(q1), to_oracle(k1), to_oracle(v1), o, D ** -0.5)
    assert g.is_compressed and len(g.state) == 5
    q2 = seeded((B, Hq, L, D), 7, dtype)
    k2, v2 = _correlated_keys((B, Hkv, L, D), 8, dtype), seeded((B, Hkv, L, D), 9, dtype)
    capfd.readouterr()
    out = g.attention(q2.to(cuda), k2.to(cuda), v2.to(cuda), D ** -0.5, "causal")
    torch.cuda.synchronize()
    assert "verify_tc" in capfd.readouterr().err
    ref = oracle.attention_with_cache_update(to_oracle(q2), to_oracle(k2), to_oracle(v2), o, D ** -0.5, "causal")
    assert worst_excess(out, ref, dtype) <= 0
    assert kvc.lib().kvc_device_status() == 0
