"""The TMA-staged tensor-core decode kernels over packed caches (affine codes,
TurboQuant indices) against the oracle, driven through the cache objects the
way attentionWithCacheUpdate drives them."""
import numpy as np
import pytest
import torch

from helpers import TOL, bits_equal, max_abs_diff, oracle_f32, seeded, to_oracle, worst_excess

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,Hq,Hkv,D,bits,group,P", [
    (2, 28, 4, 128, 4, 64, 3000),    # Qwen2-7B shape, 4-bit (7 query heads per KV head)
    (2, 32, 8, 128, 8, 64, 1000),
    (1, 32, 8, 64, 8, 64, 1024),     # Llama-3.2-1B shape
    (2, 8, 2, 128, 4, 32, 200),
    (2, 8, 2, 128, 4, 128, 77),
    (1, 64, 8, 128, 8, 128, 129),
    (2, 16, 4, 64, 4, 64, 63),
])
def test_affine_decode_kernel_matches_oracle(kvc, oracle, cuda, dtype, B, Hq, Hkv, D, bits, group, P):
    g, o = kvc.QuantizedKVCache(group, bits), oracle.QuantizedKVCache(group, bits)
    k = seeded((B, Hkv, P, D), 1, dtype, outlier_frac=0.01)
    v = seeded((B, Hkv, P, D), 2, dtype, outlier_frac=0.01)
    g.update_quantized(k.to(cuda), v.to(cuda))
    o.update_quantized(to_oracle(k), to_oracle(v))
    scale = D ** -0.5
    for step in range(3):
        q = seeded((B, Hq, 1, D), 10 + step, dtype)
        k1, v1 = seeded((B, Hkv, 1, D), 20 + step, dtype), seeded((B, Hkv, 1, D), 30 + step, dtype)
        out = g.attention(q.to(cuda), k1.to(cuda), v1.to(cuda), scale)
        ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k1), to_oracle(v1), o, scale)
        # the x20 outlier channels of V make some outputs larger than 1: the stated absolute
        # tolerance on the arithmetic plus one spacing of the 16-bit store (helpers.worst_excess)
        assert worst_excess(out, ref, dtype) <= 0, f"step {step}"
    assert kvc.lib().kvc_device_status() == 0
    for a, b in zip(g.state, o.state):
        assert bits_equal(a, np.ascontiguousarray(b))


def test_affine_small_causal_chunk(kvc, oracle, cuda):
    B, Hq, Hkv, D, L = 2, 4, 2, 128, 6
    g, o = kvc.QuantizedKVCache(64, 4), oracle.QuantizedKVCache(64, 4)
    k, v = seeded((B, Hkv, 500, D), 1, torch.bfloat16), seeded((B, Hkv, 500, D), 2, torch.bfloat16)
    g.update_quantized(k.to(cuda), v.to(cuda))
    o.update_quantized(to_oracle(k), to_oracle(v))
    q = seeded((B, Hq, L, D), 3, torch.bfloat16)
    k1, v1 = seeded((B, Hkv, L, D), 4, torch.bfloat16), seeded((B, Hkv, L, D), 5, torch.bfloat16)
    out = g.attention(q.to(cuda), k1.to(cuda), v1.to(cuda), 0.09, "causal")
    ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k1), to_oracle(v1), o, 0.09, "causal")
    assert max_abs_diff(out, ref) <= 2e-2


def test_affine_kernel_with_large_queries_and_scales(kvc, oracle, cuda):
    """Outlier channels x20 in K/V and queries of magnitude ~10: the f16 operand
    path must stay within tolerance."""
    B, Hq, Hkv, D = 1, 8, 2, 128
    g, o = kvc.QuantizedKVCache(64, 4), oracle.QuantizedKVCache(64, 4)
    k = seeded((B, Hkv, 700, D), 1, torch.bfloat16, outlier_frac=0.05)
    v = seeded((B, Hkv, 700, D), 2, torch.bfloat16, outlier_frac=0.05)
    g.update_quantized(k.to(cuda), v.to(cuda))
    o.update_quantized(to_oracle(k), to_oracle(v))
    q = (seeded((B, Hq, 1, D), 3, torch.float32) * 4).to(torch.bfloat16)
    k1, v1 = seeded((B, Hkv, 1, D), 4, torch.bfloat16), seeded((B, Hkv, 1, D), 5, torch.bfloat16)
    out = g.attention(q.to(cuda), k1.to(cuda), v1.to(cuda), D ** -0.5)
    ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k1), to_oracle(v1), o, D ** -0.5)
    # outlier channels make outputs larger than 1: stated tolerance plus one spacing of the bf16 store
    assert worst_excess(out, ref, torch.bfloat16) <= 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,Hq,Hkv,P,kb,vb", [
    (1, 64, 8, 3000, 3, 4),     # Llama-3-70B head layout, 3-bit keys / 4-bit values
    (2, 8, 2, 700, 4, 4),
    (2, 8, 2, 130, 4, 2),
    (1, 16, 4, 257, 3, 3),
    (2, 4, 4, 64, 2, 2),
])
def test_turbo_decode_kernel_matches_oracle(kvc, oracle, cuda, dtype, B, Hq, Hkv, P, kb, vb):
    """The lookup-table tensor-core decode kernel over packed TurboQuant rows (D = 128)."""
    D = 128
    kw = dict(bits=max(kb, vb), key_bits=kb, value_bits=vb)
    g = kvc.TurboQuantKVCache(**kw)
    o = oracle.TurboQuantKVCache(**kw)
    k, v = seeded((B, Hkv, P, D), 1, dtype), seeded((B, Hkv, P, D), 2, dtype)
    g.encode_new_token(k.to(cuda), v.to(cuda))
    o.encode_new_token(to_oracle(k), to_oracle(v))
    scale = D ** -0.5
    n0 = kvc.launch_count(reset=True)
    for step in range(3):
        q = seeded((B, Hq, 1, D), 10 + step, dtype)
        k1, v1 = seeded((B, Hkv, 1, D), 20 + step, dtype), seeded((B, Hkv, 1, D), 30 + step, dtype)
        out = g.attention(q.to(cuda), k1.to(cuda), v1.to(cuda), scale)
        ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k1), to_oracle(v1), o, scale)
        assert max_abs_diff(out, ref) <= TOL[dtype], f"step {step}"
    # one encode launch and ONE attention launch per step: the merge is folded into the kernel
    assert kvc.launch_count(reset=True) <= 6
    assert kvc.lib().kvc_device_status() == 0
    for a, b in zip(g.state, o.state):
        assert bits_equal(a, np.ascontiguousarray(b))


def test_turbo_kernel_small_causal_chunk(kvc, oracle, cuda):
    B, Hq, Hkv, D, L = 2, 4, 2, 128, 4     # 2 query heads per KV head x 4 positions = 8 rows
    kw = dict(bits=4, key_bits=3, value_bits=4)
    g = kvc.TurboQuantKVCache(**kw)
    o = oracle.TurboQuantKVCache(**kw)
    k, v = seeded((B, Hkv, 500, D), 1, torch.bfloat16), seeded((B, Hkv, 500, D), 2, torch.bfloat16)
    g.encode_new_token(k.to(cuda), v.to(cuda))
    o.encode_new_token(to_oracle(k), to_oracle(v))
    q = seeded((B, Hq, L, D), 3, torch.bfloat16)
    k1, v1 = seeded((B, Hkv, L, D), 4, torch.bfloat16), seeded((B, Hkv, L, D), 5, torch.bfloat16)
    out = g.attention(q.to(cuda), k1.to(cuda), v1.to(cuda), 0.09, "causal")
    ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k1), to_oracle(v1), o, 0.09, "causal")
    assert max_abs_diff(out, ref) <= 2e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,Hq,Hkv,bits,group,P,L", [
    (2, 8, 2, 4, 64, 300, 64),       # prefill chunk over a quantised prefix: 256 rows per KV head
    (1, 28, 4, 4, 64, 2100, 6),      # verify round, Qwen2-7B layout: 7 heads x 6 positions = 42 rows
    (1, 8, 2, 8, 64, 500, 40),       # 8-bit, 160 rows: three row blocks, the last one partial
    (1, 4, 1, 4, 32, 4000, 5),       # group 32; one unit, long prefix: several splits + merge
    (2, 8, 2, 8, 128, 77, 33),       # group 128
    (1, 2, 1, 4, 128, 0, 130),       # chunk into an empty cache
])
def test_affine_chunk_kernel_matches_oracle(kvc, oracle, cuda, dtype, B, Hq, Hkv, bits, group, P, L):
    """Multi-token chunks over the affine cache: dequantise-to-shared-memory tensor-core kernel; the verify round
    of the Qwen2-7B layout (groups of 64, 42 rows per kv head) goes to the tcgen05 verify kernel."""
    D = 128
    g, o = kvc.QuantizedKVCache(group, bits, reserve_tokens=P + L), oracle.QuantizedKVCache(group, bits)
    if P:
        k, v = seeded((B, Hkv, P, D), 1, dtype), seeded((B, Hkv, P, D), 2, dtype)
        g.update_quantized(k.to(cuda), v.to(cuda))
        o.update_quantized(to_oracle(k), to_oracle(v))
    q = seeded((B, Hq, L, D), 3, dtype)
    k1, v1 = seeded((B, Hkv, L, D), 4, dtype), seeded((B, Hkv, L, D), 5, dtype)
    kvc.launch_count(reset=True)
    out = g.attention(q.to(cuda), k1.to(cuda), v1.to(cuda), D ** -0.5, "causal")
    launches = kvc.launch_count(reset=True)
    if group == 64 and 16 < (Hq // Hkv) * L <= 64:
        assert 3 <= launches <= 4       # quantise-append + the tcgen05 verify kernel behind its query kernel (+ merge)
    else:
        assert launches == 2            # quantise-append + one attention launch
    ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k1), to_oracle(v1), o, D ** -0.5, "causal")
    assert max_abs_diff(out, ref) <= TOL[dtype]
    assert kvc.lib().kvc_device_status() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,Hq,Hkv,kb,vb,P,L", [
    (1, 64, 8, 3, 4, 2100, 6),       # verify round, Llama-3-70B layout: 8 heads x 6 positions = 48 rows
    (2, 8, 2, 4, 4, 300, 40),        # 160 rows per KV head
    (1, 4, 1, 3, 3, 3000, 5),        # one unit, long prefix: several splits + merge + rotation
    (1, 8, 2, 4, 2, 130, 17),
    (1, 4, 2, 2, 2, 64, 9),
])
def test_turbo_chunk_kernel_matches_oracle(kvc, oracle, cuda, dtype, B, Hq, Hkv, kb, vb, P, L):
    """Verify rounds / chunks over the TurboQuant cache (compressed phase)."""
    D = 128
    kw = dict(bits=max(kb, vb), key_bits=kb, value_bits=vb)
    g = kvc.TurboQuantKVCache(reserve_tokens=P + L, **kw)
    o = oracle.TurboQuantKVCache(**kw)
    k, v = seeded((B, Hkv, P, D), 1, dtype), seeded((B, Hkv, P, D), 2, dtype)
    g.encode_new_token(k.to(cuda), v.to(cuda))
    o.encode_new_token(to_oracle(k), to_oracle(v))
    q = seeded((B, Hq, L, D), 3, dtype)
    k1, v1 = seeded((B, Hkv, L, D), 4, dtype), seeded((B, Hkv, L, D), 5, dtype)
    kvc.launch_count(reset=True)
    out = g.attention(q.to(cuda), k1.to(cuda), v1.to(cuda), D ** -0.5, "causal")
    # encode-append + one attention launch; the tensor-core verify kernel (2- / 3-bit keys, 4-bit values, 9..128
    # rows per kv head) adds the query rotation in front, the output rotation behind and a merge when it splits
    assert kvc.launch_count(reset=True) <= 5
    ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k1), to_oracle(v1), o, D ** -0.5, "causal")
    assert max_abs_diff(out, ref) <= TOL[dtype]
    assert kvc.lib().kvc_device_status() == 0


@pytest.mark.parametrize("bits", [4, 8])
def test_varlen_decode_over_independent_caches(kvc, oracle, cuda, bits):
    """A ragged decode batch held the reference's way (one cache per sequence): the var-len call
    appends and attends all of them in two launches; per-sequence results equal the oracle's and
    the per-cache calls', and the caches hold identical codes afterwards."""
    Hq, Hkv, D, dtype = 28, 4, 128, torch.bfloat16
    lengths = [37, 64, 1, 300, 2049, 511, 130, 65, 1000, 5]
    n = len(lengths)
    var = [kvc.QuantizedKVCache(64, bits, reserve_tokens=t + 8) for t in lengths]
    one = [kvc.QuantizedKVCache(64, bits, reserve_tokens=t + 8) for t in lengths]
    orc = [oracle.QuantizedKVCache(64, bits) for _ in lengths]
    for i, t in enumerate(lengths):
        k, v = seeded((1, Hkv, t, D), 10 * i, dtype), seeded((1, Hkv, t, D), 10 * i + 1, dtype)
        for c in (var[i], one[i]):
            c.update_quantized(k.to(cuda), v.to(cuda))
        orc[i].update_quantized(to_oracle(k), to_oracle(v))
    scale = D ** -0.5
    for step in range(3):
        q = [seeded((1, Hq, 1, D), 1000 + 100 * step + i, dtype) for i in range(n)]
        k = [seeded((1, Hkv, 1, D), 2000 + 100 * step + i, dtype) for i in range(n)]
        v = [seeded((1, Hkv, 1, D), 3000 + 100 * step + i, dtype) for i in range(n)]
        dq, dk, dv = [t.to(cuda) for t in q], [t.to(cuda) for t in k], [t.to(cuda) for t in v]
        outs = [torch.empty((1, Hq, 1, D), dtype=dtype, device=cuda) for _ in range(n)]
        kvc.launch_count(reset=True)
        kvc.DecodeStep(var, dq, dk, dv, outs, scale).run_varlen()
        assert kvc.launch_count(reset=True) == 2
        for i in range(n):
            ref = oracle.attention_with_cache_update(to_oracle(q[i]), to_oracle(k[i]), to_oracle(v[i]), orc[i], scale)
            assert max_abs_diff(outs[i], ref) <= TOL[dtype], f"step {step} sequence {i}"
            single = one[i].attention(dq[i], dk[i], dv[i], scale)
            assert max_abs_diff(outs[i], to_oracle(single)) <= 1e-2
    assert kvc.lib().kvc_device_status() == 0
    for a, b, o in zip(var, one, orc):
        assert a.offset == b.offset == o.offset
        for x, y in zip(a.state, b.state):
            assert torch.equal(x, y)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,Hq,Hkv,D,bits,group,P,L,mask", [
    (2, 8, 2, 128, 4, 64, 260, 640, "causal"),     # 80 blocks of 128 rows on a quantised prefix
    (1, 16, 4, 128, 8, 32, 0, 600, "causal"),      # chunk into an empty cache, last block partial
    (5, 16, 2, 128, 2, 128, 1000, 128, "none"),    # 2-bit codes, no mask, ragged last key tile
    (2, 32, 8, 64, 4, 64, 777, 300, "causal"),     # head dim 64
])
def test_affine_prefill_chunk_on_the_tensor_core_kernel(kvc, oracle, cuda, capfd, monkeypatch, dtype, B, Hq, Hkv, D, bits,
                                                        group, P, L, mask):
    """Long chunks over the affine cache: the rows are written out once as f16 / bf16 and the
    contraction runs on the tcgen05 kernel."""
    monkeypatch.setenv("KVC_TRACE_DISPATCH", "1")
    g, o = kvc.QuantizedKVCache(group, bits), oracle.QuantizedKVCache(group, bits)
    if P:
        k, v = seeded((B, Hkv, P, D), 1, dtype), seeded((B, Hkv, P, D), 2, dtype)
        g.update_quantized(k.to(cuda), v.to(cuda))
        o.update_quantized(to_oracle(k), to_oracle(v))
    q = seeded((B, Hq, L, D), 3, dtype)
    k1, v1 = seeded((B, Hkv, L, D), 4, dtype), seeded((B, Hkv, L, D), 5, dtype)
    capfd.readouterr()
    out = g.attention(q.to(cuda), k1.to(cuda), v1.to(cuda), D ** -0.5, mask)
    torch.cuda.synchronize()
    err = capfd.readouterr().err
    assert "chunk_mat" in err and "chunk_tc" in err
    ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k1), to_oracle(v1), o, D ** -0.5, mask)
    assert max_abs_diff(out, ref) <= TOL[dtype]
    assert kvc.lib().kvc_device_status() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,Hq,Hkv,D,kb,vb,P,L,mask", [
    (2, 8, 2, 128, 3, 4, 260, 640, "causal"),
    (1, 16, 4, 128, 4, 4, 1, 600, "causal"),
    (5, 16, 2, 128, 2, 2, 1000, 128, "none"),
    (3, 8, 8, 128, 4, 2, 500, 512, "causal"),
    (2, 32, 8, 64, 3, 3, 777, 300, "causal"),      # head dim 64
])
def test_turbo_prefill_chunk_on_the_tensor_core_kernel(kvc, oracle, cuda, capfd, monkeypatch, dtype, B, Hq, Hkv, D, kb, vb,
                                                       P, L, mask):
    """Long chunks over the compressed TurboQuant cache: rows written out in the rotated basis,
    queries rotated in, outputs rotated back, contraction on the tcgen05 kernel."""
    monkeypatch.setenv("KVC_TRACE_DISPATCH", "1")
    kw = dict(bits=max(kb, vb), key_bits=kb, value_bits=vb)
    g, o = kvc.TurboQuantKVCache(**kw), oracle.TurboQuantKVCache(**kw)
    k, v = seeded((B, Hkv, P, D), 1, dtype), seeded((B, Hkv, P, D), 2, dtype)
    g.encode_new_token(k.to(cuda), v.to(cuda))
    o.encode_new_token(to_oracle(k), to_oracle(v))
    q = seeded((B, Hq, L, D), 3, dtype)
    k1, v1 = seeded((B, Hkv, L, D), 4, dtype), seeded((B, Hkv, L, D), 5, dtype)
    capfd.readouterr()
    out = g.attention(q.to(cuda), k1.to(cuda), v1.to(cuda), D ** -0.5, mask)
    torch.cuda.synchronize()
    err = capfd.readouterr().err
    assert "chunk_mat" in err and "chunk_tc" in err
    ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k1), to_oracle(v1), o, D ** -0.5, mask)
    assert max_abs_diff(out, ref) <= TOL[dtype]
    assert kvc.lib().kvc_device_status() == 0


def test_calibrated_turbo_prefill_chunk_on_the_tensor_core_kernel(kvc, oracle, cuda, capfd, monkeypatch):
    """Correlated keys: the cache calibrates at compression, and the chunk's rotated queries carry the
    calibration scale."""
    monkeypatch.setenv("KVC_TRACE_DISPATCH", "1")
    B, Hq, Hkv, D, P, L = 2, 8, 2, 128, 600, 640
    dtype = torch.bfloat16
    kw = dict(bits=4, key_bits=3, value_bits=4)
    g, o = kvc.TurboQuantKVCache(**kw), oracle.TurboQuantKVCache(**kw)
    q = seeded((B, Hq, P, D), 1, dtype)
    from test_gpu_turbo import _correlated_keys
    k, v = _correlated_keys((B, Hkv, P, D), 2, dtype), seeded((B, Hkv, P, D), 3, dtype)
    g.attention(q.to(cuda), k.to(cuda), v.to(cuda), D ** -0.5, "causal")          # raw prefill
    oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, D ** -0.5, "causal")
    q1, k1, v1 = seeded((B, Hq, 1, D), 4, dtype), _correlated_keys((B, Hkv, 1, D), 5, dtype), seeded((B, Hkv, 1, D), 6, dtype)
    g.attention(q1.to(cuda), k1.to(cuda), v1.to(cuda), D ** -0.5)                  # compresses and calibrates
    oracle.attention_with_cache_update(to_oracle(q1), to_oracle(k1), to_oracle(v1), o, D ** -0.5)
    assert g.is_compressed and len(g.state) == 5 and len(o.state) == 5
    q2 = seeded((B, Hq, L, D), 7, dtype)
    k2, v2 = _correlated_keys((B, Hkv, L, D), 8, dtype), seeded((B, Hkv, L, D), 9, dtype)
    capfd.readouterr()
    out = g.attention(q2.to(cuda), k2.to(cuda), v2.to(cuda), D ** -0.5, "causal")
    torch.cuda.synchronize()
    assert "chunk_mat" in capfd.readouterr().err
    ref = oracle.attention_with_cache_update(to_oracle(q2), to_oracle(k2), to_oracle(v2), o, D ** -0.5, "causal")
    from helpers import worst_excess
    assert worst_excess(out, ref, dtype) <= 0
    assert kvc.lib().kvc_device_status() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,Hq,Hkv,bits,group,P,L", [
    (2, 28, 4, 4, 64, 1000, 6),      # Qwen2-7B layout, verify round: 42 rows per kv head; tensor-core kernel, split keys
    (1, 32, 4, 8, 64, 517, 5),       # 8-bit codes, 40 rows: tensor-core kernel
    (2, 16, 2, 8, 64, 1300, 6),      # 8-bit codes, 48 rows, bigger
    (2, 8, 1, 4, 128, 2049, 8),      # 64 rows; group 128: units of eight rows on the decode kernel
    (1, 17, 1, 4, 64, 300, 1),       # 17 heads on one kv head, one position, no causal limit to speak of
    (16, 56, 8, 4, 64, 700, 6),      # 128 units: one CTA each, six tiles in a row, no split
    (1, 8, 1, 4, 64, 120, 8),        # 64 rows; the chunk itself crosses the first tile boundary
    (40, 20, 4, 4, 64, 300, 4),      # 160 units of three tiles on fewer SMs: CTAs that walk two or three units
])
def test_affine_verify_rounds(kvc, oracle, cuda, capfd, monkeypatch, dtype, B, Hq, Hkv, bits, group, P, L):
    """17 to 64 query rows per kv head over the affine cache. 4- or 8-bit codes in groups of 64: the tcgen05 verify
    kernel (rows decoded once per kv head). Otherwise the group is cut into units of eight rows, each streamed
    through the 8-row decode kernel with its own causal limits (one attention launch)."""
    D = 128
    monkeypatch.setenv("KVC_TRACE_DISPATCH", "1")
    g, o = kvc.QuantizedKVCache(group, bits), oracle.QuantizedKVCache(group, bits)
    k, v = seeded((B, Hkv, P, D), 1, dtype), seeded((B, Hkv, P, D), 2, dtype)
    g.update_quantized(k.to(cuda), v.to(cuda))
    o.update_quantized(to_oracle(k), to_oracle(v))
    mask = "causal" if L > 1 else "none"
    for rnd in range(2):
        q = seeded((B, Hq, L, D), 3 + rnd, dtype)
        k1, v1 = seeded((B, Hkv, L, D), 5 + rnd, dtype), seeded((B, Hkv, L, D), 7 + rnd, dtype)
        kvc.launch_count(reset=True)
        capfd.readouterr()
        out = g.attention(q.to(cuda), k1.to(cuda), v1.to(cuda), D ** -0.5, mask)
        torch.cuda.synchronize()
        launches, err = kvc.launch_count(reset=True), capfd.readouterr().err
        if group == 64:
            assert "verify_tc affine" in err
        else:
            assert launches == 2            # quantise-append + one attention launch
        ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k1), to_oracle(v1), o, D ** -0.5, mask)
        assert max_abs_diff(out, ref) <= TOL[dtype], f"round {rnd}"
        assert g.trim(max(L - 1, 0)) == o.trim(max(L - 1, 0))
    assert kvc.lib().kvc_device_status() == 0


@pytest.mark.parametrize("kind", ["turbo_k3v4", "turbo_k4v4", "affine4"])
def test_decode_at_every_context_length_around_the_stage_boundaries(kvc, oracle, cuda, kind):
    """The 15-warp decode kernels stream 240-token stages and cut the last one short at the stored rows
    rounded up to 256: every context length around multiples of 240 and of 256 (and the first tokens of
    an empty cache) against the oracle, in one growing cache."""
    B, Hq, Hkv, D = 1, 8, 1, 128
    dtype = torch.bfloat16
    if kind == "affine4":
        g, o = kvc.QuantizedKVCache(64, 4), oracle.QuantizedKVCache(64, 4)
    else:
        kw = dict(bits=4, key_bits=3 if kind == "turbo_k3v4" else 4, value_bits=4)
        g, o = kvc.TurboQuantKVCache(**kw), oracle.TurboQuantKVCache(**kw)
    scale = D ** -0.5
    check_at = set(range(1, 6)) | {t + d for t in (240, 256, 480, 512, 720, 768, 960, 1024) for d in (-2, -1, 0, 1, 2)}
    T = 0
    for target in sorted(check_at):
        fill = target - 1 - T               # rows to add before the decode step that makes the context `target`
        if fill > 0:
            k, v = seeded((B, Hkv, fill, D), 1000 + target, dtype), seeded((B, Hkv, fill, D), 2000 + target, dtype)
            if kind == "affine4":
                g.update_quantized(k.to(cuda), v.to(cuda))
                o.update_quantized(to_oracle(k), to_oracle(v))
            else:
                g.encode_new_token(k.to(cuda), v.to(cuda))
                o.encode_new_token(to_oracle(k), to_oracle(v))
            T += fill
        q = seeded((B, Hq, 1, D), 3000 + target, dtype)
        k1, v1 = seeded((B, Hkv, 1, D), 4000 + target, dtype), seeded((B, Hkv, 1, D), 5000 + target, dtype)
        out = g.attention(q.to(cuda), k1.to(cuda), v1.to(cuda), scale)
        ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k1), to_oracle(v1), o, scale)
        T += 1
        assert g.offset == o.offset == T == target
        assert max_abs_diff(out, ref) <= TOL[dtype], f"context {target}"
    assert kvc.lib().kvc_device_status() == 0
