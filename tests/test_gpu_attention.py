"""GPU parity: attention outputs of the CUDA library vs the CPU oracle on the
same seeded inputs. Tolerance: max-abs 1e-4 for fp32, 2e-2 for bf16/f16."""
import numpy as np
import pytest
import torch

from helpers import TOL, bits_equal, max_abs_diff, seeded, to_oracle

pytestmark = pytest.mark.gpu


def _check(gpu_out, ref, dtype, what=""):
    err = max_abs_diff(gpu_out, ref)
    assert err <= TOL[dtype], f"{what}: max-abs {err} > {TOL[dtype]}"
    assert torch.isfinite(gpu_out.float()).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("T", [1, 2, 63, 64, 65, 257, 1000])
def test_sdpa_decode_matches_oracle(kvc, oracle, cuda, dtype, T):
    B, Hq, Hkv, D = 2, 8, 2, 128
    q = seeded((B, Hq, 1, D), 1, dtype)
    k, v = seeded((B, Hkv, T, D), 2, dtype), seeded((B, Hkv, T, D), 3, dtype)
    out = kvc.scaled_dot_product_attention(q.to(cuda), k.to(cuda), v.to(cuda), D ** -0.5)
    ref = oracle.sdpa(to_oracle(q), to_oracle(k), to_oracle(v), D ** -0.5)
    _check(out, ref, dtype, f"T={T}")


@pytest.mark.parametrize("D,Hq,Hkv", [(64, 32, 8), (128, 32, 8), (256, 4, 1), (128, 28, 4), (128, 64, 8), (80, 4, 4)])
def test_sdpa_shapes_of_the_configs(kvc, oracle, cuda, D, Hq, Hkv):
    B, T = 2, 300
    q = seeded((B, Hq, 1, D), 4, torch.bfloat16)
    k, v = seeded((B, Hkv, T, D), 5, torch.bfloat16), seeded((B, Hkv, T, D), 6, torch.bfloat16)
    out = kvc.scaled_dot_product_attention(q.to(cuda), k.to(cuda), v.to(cuda), D ** -0.5)
    _check(out, oracle.sdpa(to_oracle(q), to_oracle(k), to_oracle(v), D ** -0.5), torch.bfloat16)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("L,T", [(6, 6), (6, 200), (17, 64), (64, 130)])
def test_sdpa_masks(kvc, oracle, cuda, dtype, L, T):
    B, Hq, Hkv, D = 2, 4, 2, 64
    q = seeded((B, Hq, L, D), 7, dtype)
    k, v = seeded((B, Hkv, T, D), 8, dtype), seeded((B, Hkv, T, D), 9, dtype)
    qo, ko, vo = to_oracle(q), to_oracle(k), to_oracle(v)
    qd, kd, vd = q.to(cuda), k.to(cuda), v.to(cuda)
    _check(kvc.scaled_dot_product_attention(qd, kd, vd, 0.125, "causal"), oracle.sdpa(qo, ko, vo, 0.125, "causal"), dtype, "causal")
    _check(kvc.scaled_dot_product_attention(qd, kd, vd, 0.125, "none"), oracle.sdpa(qo, ko, vo, 0.125, "none"), dtype, "none")
    win = oracle.create_causal_mask(L, T - L, 5)
    _check(kvc.scaled_dot_product_attention(qd, kd, vd, 0.125, torch.from_numpy(win).to(cuda)),
           oracle.sdpa(qo, ko, vo, 0.125, win), dtype, "bool window mask")
    g = torch.Generator().manual_seed(3)
    add = torch.randn((B, 1, L, T), generator=g)
    add[:, :, :, ::7] = float("-inf")
    add[:, :, :, 0] = 0.0
    _check(kvc.scaled_dot_product_attention(qd, kd, vd, 0.125, add.to(cuda)),
           oracle.sdpa(qo, ko, vo, 0.125, add.numpy()), dtype, "additive mask")
    per_batch = torch.from_numpy(win)[None, None].expand(B, 1, L, T).contiguous()
    _check(kvc.scaled_dot_product_attention(qd, kd, vd, 0.125, per_batch.to(cuda)),
           oracle.sdpa(qo, ko, vo, 0.125, win), dtype, "4-d bool mask")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("bits,group", [(8, 64), (4, 64), (4, 32), (8, 128), (2, 64)])
def test_quantized_sdpa_matches_oracle(kvc, oracle, cuda, dtype, bits, group):
    B, Hq, Hkv, T, D = 2, 8, 2, 333, 128
    q = seeded((B, Hq, 1, D), 10, dtype)
    k = seeded((B, Hkv, T, D), 11, dtype, outlier_frac=0.01)
    v = seeded((B, Hkv, T, D), 12, dtype, outlier_frac=0.01)
    qk, qv = oracle.affine_quantize(to_oracle(k), group, bits), oracle.affine_quantize(to_oracle(v), group, bits)

    def dev(t3):
        import helpers
        return (torch.from_numpy(t3[0].view(np.int32)).to(cuda), helpers.from_oracle(t3[1], dtype).to(cuda),
                helpers.from_oracle(t3[2], dtype).to(cuda))
    out = kvc.quantized_scaled_dot_product_attention(q.to(cuda), dev(qk), dev(qv), D ** -0.5, "none", group, bits)
    ref = oracle.quantized_sdpa(to_oracle(q), qk, qv, D ** -0.5, "none", group, bits)
    _check(out, ref, dtype)
    q6 = seeded((B, Hq, 6, D), 13, dtype)
    out = kvc.quantized_scaled_dot_product_attention(q6.to(cuda), dev(qk), dev(qv), D ** -0.5, "causal", group, bits)
    ref = oracle.quantized_sdpa(to_oracle(q6), qk, qv, D ** -0.5, "causal", group, bits)
    _check(out, ref, dtype, "causal verify chunk")


@pytest.mark.parametrize("kind", ["simple", "rotating", "quantized8", "quantized4"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_with_cache_update_decode_loop(kvc, oracle, cuda, kind, dtype):
    """Prefill then a decode loop through the fused call; outputs in tolerance and
    cache state bit-exact at every step."""
    B, Hq, Hkv, D = 1, 8, 2, 64
    make = {"simple": (lambda: kvc.KVCacheSimple(), lambda: oracle.KVCacheSimple()),
            "rotating": (lambda: kvc.RotatingKVCache(48), lambda: oracle.RotatingKVCache(48)),
            "quantized8": (lambda: kvc.QuantizedKVCache(64, 8), lambda: oracle.QuantizedKVCache(64, 8)),
            "quantized4": (lambda: kvc.QuantizedKVCache(64, 4), lambda: oracle.QuantizedKVCache(64, 4))}[kind]
    g, o = make[0](), make[1]()
    P = 40
    q, k, v = seeded((B, Hq, P, D), 20, dtype), seeded((B, Hkv, P, D), 21, dtype), seeded((B, Hkv, P, D), 22, dtype)
    out = kvc.attention_with_cache_update(q.to(cuda), k.to(cuda), v.to(cuda), g, 0.125, "causal")
    ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, 0.125, "causal")
    _check(out, ref, dtype, "prefill")
    for step in range(24):
        q, k, v = (seeded((B, Hq, 1, D), 100 + 3 * step, dtype), seeded((B, Hkv, 1, D), 101 + 3 * step, dtype),
                   seeded((B, Hkv, 1, D), 102 + 3 * step, dtype))
        out = kvc.attention_with_cache_update(q.to(cuda), k.to(cuda), v.to(cuda), g, 0.125, "none")
        ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, 0.125, "none")
        _check(out, ref, dtype, f"step {step}")
        assert g.offset == o.offset and list(g.meta_state) == list(o.meta_state)
    for gs, os_ in zip(g.state, o.state):
        assert bits_equal(gs, np.ascontiguousarray(os_))


def test_rotating_attention_past_wrap_matches_unrotated_history(kvc, oracle, cuda):
    # KVCacheTests.swift:1451-1491 on the device, tolerance 1e-5 as in the reference test
    window, total, D = 8, 21, 16
    K, V = seeded((1, 1, total, D), 30, torch.float32), seeded((1, 1, total, D), 31, torch.float32)
    cache = kvc.RotatingKVCache(window)
    for t in range(total - 1):
        cache.update(K[:, :, t:t + 1].to(cuda), V[:, :, t:t + 1].to(cuda))
    q = seeded((1, 2, 1, D), 32, torch.float32)
    got = cache.attention(q.to(cuda), K[:, :, -1:].to(cuda), V[:, :, -1:].to(cuda), 0.25)
    mask = np.zeros((1, total), dtype=bool)
    mask[0, total - window:] = True
    want = oracle.sdpa(to_oracle(q), to_oracle(K), to_oracle(V), 0.25, mask)
    assert max_abs_diff(got, want) < 1e-5


def test_staged_round_attention(kvc, oracle, cuda):
    """Verify chunk over a wrapped ring: presentation + array mask from the live cache."""
    B, Hq, Hkv, D, W, L = 1, 4, 1, 64, 16, 4
    g, o = kvc.RotatingKVCache(W), oracle.RotatingKVCache(W)
    for t in range(30):
        k, v = seeded((B, Hkv, 1, D), 2 * t, torch.float32), seeded((B, Hkv, 1, D), 2 * t + 1, torch.float32)
        g.update(k.to(cuda), v.to(cuda))
        o.update(to_oracle(k), to_oracle(v))
    q, k, v = seeded((B, Hq, L, D), 200, torch.float32), seeded((B, Hkv, L, D), 201, torch.float32), seeded((B, Hkv, L, D), 202, torch.float32)
    gm, om = g.make_mask(L, W), o.make_mask(L, W)
    assert np.array_equal(gm.cpu().numpy(), om)
    rnd = kvc.StagedRound(g, L)
    out = rnd.attention(q.to(cuda), k.to(cuda), v.to(cuda), 0.125, gm)
    orr = oracle.StagedRound(o, L)
    pk, pv = orr.update(to_oracle(k), to_oracle(v))
    ref = oracle.sdpa(to_oracle(q), np.ascontiguousarray(pk), np.ascontiguousarray(pv), 0.125, om)
    assert max_abs_diff(out, ref) < 1e-4
    assert rnd.offset == o.offset + L
    rnd.commit(2)
    orr.commit(2)
    assert g.offset == o.offset and list(g.meta_state) == list(o.meta_state)


def test_host_entry_point_matches_device_entry_point(kvc, cuda):
    B, Hq, Hkv, D = 2, 8, 2, 128
    a, b = kvc.KVCacheSimple(), kvc.KVCacheSimple()
    for step in range(5):
        S = 33 if step == 0 else 1
        q, k, v = seeded((B, Hq, S, D), 3 * step, torch.bfloat16), seeded((B, Hkv, S, D), 3 * step + 1, torch.bfloat16), seeded((B, Hkv, S, D), 3 * step + 2, torch.bfloat16)
        mode = "causal" if S > 1 else "none"
        dev = a.attention(q.to(cuda), k.to(cuda), v.to(cuda), 0.1, mode)
        host = b.attention_host(q.pin_memory(), k.pin_memory(), v.pin_memory(), 0.1, mode)
        assert torch.equal(dev.cpu(), host)


def test_batched_host_call_matches_per_layer_device_calls(kvc, cuda):
    """kvc_attention_batch with host buffers: copies run ahead on side streams; the results and
    the cache contents are those of the per-layer device calls, step after step."""
    B, Hq, Hkv, D, layers = 2, 8, 2, 128, 5
    dev_caches = [kvc.KVCacheSimple() for _ in range(layers)]
    host_caches = [kvc.KVCacheSimple() for _ in range(layers)]
    for i in range(layers):
        k, v = seeded((B, Hkv, 40 + i, D), 100 + i, torch.bfloat16), seeded((B, Hkv, 40 + i, D), 200 + i, torch.bfloat16)
        dev_caches[i].update(k.to(cuda), v.to(cuda))
        host_caches[i].update(k.to(cuda), v.to(cuda))
    hq = [torch.empty((B, Hq, 1, D), dtype=torch.bfloat16).pin_memory() for _ in range(layers)]
    hk = [torch.empty((B, Hkv, 1, D), dtype=torch.bfloat16).pin_memory() for _ in range(layers)]
    hv = [torch.empty((B, Hkv, 1, D), dtype=torch.bfloat16).pin_memory() for _ in range(layers)]
    ho = [torch.zeros((B, Hq, 1, D), dtype=torch.bfloat16).pin_memory() for _ in range(layers)]
    step = kvc.DecodeStep(host_caches, hq, hk, hv, ho, 0.1, host=True)
    for it in range(4):
        for i in range(layers):
            hq[i].copy_(seeded((B, Hq, 1, D), 1000 + 10 * it + i, torch.bfloat16))
            hk[i].copy_(seeded((B, Hkv, 1, D), 2000 + 10 * it + i, torch.bfloat16))
            hv[i].copy_(seeded((B, Hkv, 1, D), 3000 + 10 * it + i, torch.bfloat16))
        step.run(synchronize=True)
        for i in range(layers):
            ref = dev_caches[i].attention(hq[i].to(cuda), hk[i].to(cuda), hv[i].to(cuda), 0.1)
            assert torch.equal(ref.cpu(), ho[i]), f"step {it} layer {i}"
    for a, b in zip(dev_caches, host_caches):
        assert a.offset == b.offset
        for x, y in zip(a.state, b.state):
            assert torch.equal(x, y)
