"""The specialised decode kernel (TMA-staged, tensor-core) against the oracle and
against the general kernel, on the shapes the benchmark configurations use."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import TOL, bits_equal, max_abs_diff, seeded, to_oracle

pytestmark = pytest.mark.gpu

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,Hq,Hkv,D,T", [
    (8, 32, 8, 128, 777),      # Llama-3-8B attention shape
    (4, 4, 1, 256, 512),       # Gemma-3-1B local layer, full window
    (4, 4, 1, 256, 37),
    (1, 32, 8, 64, 1280),      # Llama-3.2-1B
    (2, 28, 4, 128, 3000),     # Qwen2-7B: 7 query heads per KV head
    (2, 64, 8, 128, 4097),     # Llama-3-70B: 8 query heads per KV head
    (1, 16, 1, 128, 200),      # 16 rows: the full MMA tile
    (3, 8, 2, 128, 1), (3, 8, 2, 128, 63), (3, 8, 2, 128, 64), (3, 8, 2, 128, 65),
])
def test_decode_kernel_matches_oracle(kvc, oracle, cuda, dtype, B, Hq, Hkv, D, T):
    q = seeded((B, Hq, 1, D), 1, dtype)
    k, v = seeded((B, Hkv, T, D), 2, dtype), seeded((B, Hkv, T, D), 3, dtype)
    out = kvc.scaled_dot_product_attention(q.to(cuda), k.to(cuda), v.to(cuda), D ** -0.5)
    ref = oracle.sdpa(to_oracle(q), to_oracle(k), to_oracle(v), D ** -0.5)
    assert max_abs_diff(out, ref) <= TOL[dtype]
    assert kvc.lib().kvc_device_status() == 0


def test_decode_kernel_reads_strided_cache_views(kvc, oracle, cuda):
    """The cache hands the kernel views whose head stride is the capacity, not the length."""
    B, Hq, Hkv, D = 2, 8, 2, 128
    cache = kvc.KVCacheSimple(reserve_tokens=4096)
    o = oracle.KVCacheSimple()
    for step, S in enumerate((700, 1, 1, 1)):
        q, k, v = (seeded((B, Hq, 1, D), 3 * step, torch.bfloat16), seeded((B, Hkv, S, D), 3 * step + 1, torch.bfloat16),
                   seeded((B, Hkv, S, D), 3 * step + 2, torch.bfloat16))
        if S > 1:
            cache.update(k.to(cuda), v.to(cuda))
            o.update(to_oracle(k), to_oracle(v))
            continue
        out = cache.attention(q.to(cuda), k.to(cuda), v.to(cuda), 0.09)
        ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, 0.09)
        assert max_abs_diff(out, ref) <= 2e-2
    assert kvc.lib().kvc_device_status() == 0


def test_small_causal_chunk_on_the_decode_kernel(kvc, oracle, cuda):
    # 2 query heads per KV head x 6 positions = 12 rows: still one MMA tile
    B, Hq, Hkv, D, L, T = 2, 4, 2, 128, 6, 333
    q = seeded((B, Hq, L, D), 5, torch.bfloat16)
    k, v = seeded((B, Hkv, T, D), 6, torch.bfloat16), seeded((B, Hkv, T, D), 7, torch.bfloat16)
    out = kvc.scaled_dot_product_attention(q.to(cuda), k.to(cuda), v.to(cuda), 0.1, "causal")
    ref = oracle.sdpa(to_oracle(q), to_oracle(k), to_oracle(v), 0.1, "causal")
    assert max_abs_diff(out, ref) <= 2e-2


def test_general_and_decode_kernels_agree():
    """Same inputs through both device paths (the general one forced by the
    environment switch in a child process)."""
    code = r"""
import os, sys, torch
sys.path.insert(0, os.path.join(%r, "mlx-swift-lm_b200", "python"))
sys.path.insert(0, os.path.join(%r, "tests"))
import kvcache_b200 as kvc
from helpers import seeded
dev = torch.device("cuda:0")
q = seeded((2, 32, 1, 128), 1, torch.bfloat16).to(dev)
k = seeded((2, 8, 2049, 128), 2, torch.bfloat16).to(dev)
v = seeded((2, 8, 2049, 128), 3, torch.bfloat16).to(dev)
out = kvc.scaled_dot_product_attention(q, k, v, 0.088)
torch.save(out.float().cpu(), sys.argv[1])
print(kvc.launch_count())
""" % (ROOT, ROOT)
    outs = []
    for path in ("decode", "general"):
        env = dict(os.environ)
        env["KVC_ATTENTION_PATH"] = path
        f = f"/tmp/kvc_path_{path}.pt"
        subprocess.run([sys.executable, "-c", code, f], check=True, env=env, timeout=300)
        outs.append(torch.load(f))
    assert float((outs[0] - outs[1]).abs().max()) <= 2e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,Hq,Hkv,D,L,T,mask", [
    (2, 8, 2, 128, 64, 300, "causal"),      # prefill chunk on top of a 236-token prefix
    (1, 64, 8, 128, 6, 2100, "causal"),     # verify round: 8 heads x 6 positions = 48 rows
    (1, 8, 2, 128, 200, 200, "causal"),     # 800 rows per KV head: 13 row blocks, the last one partial
    (2, 4, 1, 256, 40, 552, "causal"),      # head dim 256
    (2, 8, 2, 64, 96, 130, "causal"),       # head dim 64
    (1, 4, 1, 128, 17, 5000, "none"),       # few units, long context: several splits + merge
    (1, 32, 8, 128, 5, 999, "none"),        # token count not a multiple of the tile
    (1, 2, 1, 128, 512, 512, "causal"),     # one 512-token chunk from an empty cache
])
def test_chunk_kernel_matches_oracle(kvc, oracle, cuda, dtype, B, Hq, Hkv, D, L, T, mask):
    """Multi-token chunks (more than 16 rows per KV head): rows split across the warps of the mma.sync chunk
    kernel; 17 to 64 rows per KV head at head dim 128 go to the tcgen05 verify kernel."""
    q = seeded((B, Hq, L, D), 1, dtype)
    k, v = seeded((B, Hkv, T, D), 2, dtype), seeded((B, Hkv, T, D), 3, dtype)
    n0 = kvc.launch_count(reset=True)
    out = kvc.scaled_dot_product_attention(q.to(cuda), k.to(cuda), v.to(cuda), D ** -0.5, mask)
    launches = kvc.launch_count(reset=True)
    if D == 128 and 16 < (Hq // Hkv) * L <= 64:
        assert 2 <= launches <= 3       # the tcgen05 verify kernel behind its query kernel (+ merge)
    else:
        assert launches == 1            # one kernel: partial + merge in one launch
    ref = oracle.sdpa(to_oracle(q), to_oracle(k), to_oracle(v), D ** -0.5, mask)
    assert max_abs_diff(out, ref) <= TOL[dtype]
    assert kvc.lib().kvc_device_status() == 0


def test_chunked_prefill_through_the_cache(kvc, oracle, cuda):
    """attentionWithCacheUpdate with 128-token chunks, then decode: chunk and decode kernels on one cache."""
    B, Hq, Hkv, D = 2, 8, 2, 128
    cache, o = kvc.KVCacheSimple(), oracle.KVCacheSimple()
    for step, S in enumerate((128, 128, 128, 1, 1)):
        q, k, v = (seeded((B, Hq, S, D), 3 * step, torch.bfloat16), seeded((B, Hkv, S, D), 3 * step + 1, torch.bfloat16),
                   seeded((B, Hkv, S, D), 3 * step + 2, torch.bfloat16))
        mask = "causal" if S > 1 else "none"
        out = cache.attention(q.to(cuda), k.to(cuda), v.to(cuda), 0.09, mask)
        ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, 0.09, mask)
        assert max_abs_diff(out, ref) <= 2e-2, f"step {step}"
    assert kvc.lib().kvc_device_status() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_fused_append_decode_is_one_launch_and_bit_exact_cache(kvc, oracle, cuda, dtype):
    """Decode on a KVCacheSimple: the attention kernel scores the new row from its source and writes
    it into the cache itself (one launch per call); outputs match the oracle and the cache rows are
    bit-identical, across a tile boundary (63 -> 66 tokens) and a growth step."""
    B, Hq, Hkv, D = 2, 8, 2, 128
    g, o = kvc.KVCacheSimple(step=64), oracle.KVCacheSimple(step=64)
    k, v = seeded((B, Hkv, 61, D), 1, dtype), seeded((B, Hkv, 61, D), 2, dtype)
    g.update(k.to(cuda), v.to(cuda))
    o.update(to_oracle(k), to_oracle(v))
    for step in range(6):
        q, k1, v1 = (seeded((B, Hq, 1, D), 10 + step, dtype), seeded((B, Hkv, 1, D), 20 + step, dtype),
                     seeded((B, Hkv, 1, D), 30 + step, dtype))
        kvc.launch_count(reset=True)
        out = g.attention(q.to(cuda), k1.to(cuda), v1.to(cuda), D ** -0.5)
        n = kvc.launch_count(reset=True)
        assert n == 1 or g.offset in (65,), f"step {step}: {n} launches"     # 64 -> 65 grows the buffer (copies)
        ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k1), to_oracle(v1), o, D ** -0.5)
        assert max_abs_diff(out, ref) <= TOL[dtype], f"step {step}"
        for a, b in zip(g.state, o.state):
            assert bits_equal(a, np.ascontiguousarray(b)), f"step {step}"
    # an empty cache: the new token is the only one
    e, eo = kvc.KVCacheSimple(), oracle.KVCacheSimple()
    q, k1, v1 = seeded((B, Hq, 1, D), 90, dtype), seeded((B, Hkv, 1, D), 91, dtype), seeded((B, Hkv, 1, D), 92, dtype)
    out = e.attention(q.to(cuda), k1.to(cuda), v1.to(cuda), D ** -0.5)
    ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k1), to_oracle(v1), eo, D ** -0.5)
    assert max_abs_diff(out, ref) <= TOL[dtype]
    assert kvc.lib().kvc_device_status() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_batched_decode_steps_over_layers(kvc, oracle, cuda, dtype):
    """Several decode steps of a 5-layer stack through one batched call per step (the layers' kernels
    follow one another on the stream, each appending its own new row): outputs match the oracle layer
    by layer and the caches hold the oracle's bytes. Layer 3 shares its cache object with nothing but
    starts one step late from a shorter prefix, and the prefix of layer 2 ends exactly on its capacity
    so that its first step re-allocates."""
    B, Hq, Hkv, D, Lyr = 2, 8, 2, 128, 5
    scale = D ** -0.5
    prefix = [700, 1300, 512, 65, 2049]
    g, o = [], []
    for i in range(Lyr):
        gc = kvc.KVCacheSimple(step=256)
        oc = oracle.KVCacheSimple(step=256)
        k, v = seeded((B, Hkv, prefix[i], D), 10 + i, dtype), seeded((B, Hkv, prefix[i], D), 20 + i, dtype)
        gc.update(k.to(cuda), v.to(cuda))
        oc.update(to_oracle(k), to_oracle(v))
        g.append(gc)
        o.append(oc)
    for step in range(6):
        qs = [seeded((B, Hq, 1, D), 100 + 10 * step + i, dtype) for i in range(Lyr)]
        ks = [seeded((B, Hkv, 1, D), 200 + 10 * step + i, dtype) for i in range(Lyr)]
        vs = [seeded((B, Hkv, 1, D), 300 + 10 * step + i, dtype) for i in range(Lyr)]
        dq, dk, dv = [t.to(cuda) for t in qs], [t.to(cuda) for t in ks], [t.to(cuda) for t in vs]
        outs = [torch.empty_like(t) for t in dq]
        n0 = kvc.launch_count(reset=True)
        kvc.DecodeStep(g, dq, dk, dv, outs, scale).run(synchronize=True)
        launches = kvc.launch_count(reset=True)
        assert Lyr <= launches <= Lyr + 4, launches         # one kernel per layer (append fused in) + growth copies
        for i in range(Lyr):
            ref = oracle.attention_with_cache_update(to_oracle(qs[i]), to_oracle(ks[i]), to_oracle(vs[i]), o[i], scale, "none")
            assert max_abs_diff(outs[i], ref) <= TOL[dtype], (step, i)
    for gc, oc in zip(g, o):
        assert gc.offset == oc.offset
        for a, b in zip(gc.state, oc.state):
            assert bits_equal(a, np.ascontiguousarray(b))
    assert kvc.lib().kvc_device_status() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,Hq,Hkv,L,T,mask", [
    (2, 8, 2, 640, 900, "causal"),       # 5 full row blocks per head on a 260-token prefix
    (1, 16, 4, 600, 600, "causal"),      # chunk from an empty cache, last row block partial, T not a tile multiple
    (1, 8, 8, 1300, 1300, "none"),       # no mask: only the ragged last key tile is masked
    (4, 8, 1, 384, 3000, "causal"),      # long prefix: 24 key tiles per block, multi-query
    (4, 32, 8, 100, 100, "causal"),      # one partial row block and one partial key tile per CTA
    (2, 64, 8, 64, 5001, "none"),        # the shortest chunk the kernel takes, ragged last key tile
    (5, 16, 16, 129, 257, "causal"),     # one row past a block, one key past a tile
])
def test_tensor_core_chunk_kernel_matches_oracle(kvc, oracle, cuda, capfd, monkeypatch, dtype, B, Hq, Hkv, L, T, mask):
    """Long chunks over raw K/V at head dim 128 run on the tcgen05 kernel (128 query rows per CTA)."""
    D = 128
    monkeypatch.setenv("KVC_TRACE_DISPATCH", "1")
    q = seeded((B, Hq, L, D), 1, dtype)
    k, v = seeded((B, Hkv, T, D), 2, dtype), seeded((B, Hkv, T, D), 3, dtype)
    kvc.launch_count(reset=True)
    out = kvc.scaled_dot_product_attention(q.to(cuda), k.to(cuda), v.to(cuda), D ** -0.5, mask)
    torch.cuda.synchronize()
    assert kvc.launch_count(reset=True) == 1
    assert "chunk_tc" in capfd.readouterr().err
    ref = oracle.sdpa(to_oracle(q), to_oracle(k), to_oracle(v), D ** -0.5, mask)
    assert max_abs_diff(out, ref) <= TOL[dtype]
    assert kvc.lib().kvc_device_status() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,Hq,Hkv,L,T,mask", [
    (2, 32, 8, 300, 777, "causal"),
    (1, 32, 8, 512, 512, "causal"),
    (5, 16, 2, 128, 1000, "none"),
])
def test_tensor_core_chunk_kernel_head_dim_64(kvc, oracle, cuda, capfd, monkeypatch, dtype, B, Hq, Hkv, L, T, mask):
    """The same kernel at head dim 64 (one 64-element box per Q / K / V tile, 64 output columns)."""
    D = 64
    monkeypatch.setenv("KVC_TRACE_DISPATCH", "1")
    q = seeded((B, Hq, L, D), 4, dtype)
    k, v = seeded((B, Hkv, T, D), 5, dtype), seeded((B, Hkv, T, D), 6, dtype)
    out = kvc.scaled_dot_product_attention(q.to(cuda), k.to(cuda), v.to(cuda), D ** -0.5, mask)
    torch.cuda.synchronize()
    assert "chunk_tc" in capfd.readouterr().err
    ref = oracle.sdpa(to_oracle(q), to_oracle(k), to_oracle(v), D ** -0.5, mask)
    assert max_abs_diff(out, ref) <= TOL[dtype]
    assert kvc.lib().kvc_device_status() == 0


def test_tensor_core_chunk_through_the_cache(kvc, oracle, cuda):
    """A 512-token prefill chunk on top of a stored prefix through attentionWithCacheUpdate, strided
    (transposed-projection) queries included; the same call with the kernel switched off agrees."""
    B, Hq, Hkv, D = 2, 16, 4, 128
    g, o = kvc.KVCacheSimple(), oracle.KVCacheSimple()
    for i, S in enumerate((333, 512)):
        k, v = seeded((B, Hkv, S, D), 10 + i, torch.bfloat16), seeded((B, Hkv, S, D), 20 + i, torch.bfloat16)
        q = seeded((B, Hq, S, D), 30 + i, torch.bfloat16)
        dq = q.to(cuda).transpose(1, 2).contiguous().transpose(1, 2)     # [B, S, Hq, D] storage
        out = kvc.attention_with_cache_update(dq, k.to(cuda), v.to(cuda), g, D ** -0.5, "causal")
        ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, D ** -0.5, "causal")
        assert max_abs_diff(out, ref) <= TOL[torch.bfloat16]
    assert kvc.lib().kvc_device_status() == 0


@pytest.mark.parametrize("D,keep,max_size,prefill", [(128, 0, 96, 70), (128, 4, 80, 200), (256, 0, 64, 10), (64, 3, 130, 129)])
def test_rotating_ring_decode_appends_inside_the_attention_kernel(kvc, oracle, cuda, D, keep, max_size, prefill):
    """Single-token steps on a RotatingKVCache (updateInPlace, KVCache.swift:684-740) through
    attentionWithCacheUpdate: while the buffer grows the row lands at the end, once the ring has
    wrapped it replaces the oldest row in the middle of the buffer. One launch per step; outputs and
    the physical ring match the oracle at every step."""
    B, Hq, Hkv = 2, 4, 2
    dtype = torch.bfloat16
    scale = D ** -0.5
    g, o = kvc.RotatingKVCache(max_size, keep=keep, step=32), oracle.RotatingKVCache(max_size, keep=keep, step=32)
    k, v = seeded((B, Hkv, prefill, D), 1, dtype), seeded((B, Hkv, prefill, D), 2, dtype)
    q = seeded((B, Hq, prefill, D), 3, dtype)
    kvc.attention_with_cache_update(q.to(cuda), k.to(cuda), v.to(cuda), g, scale, "causal")
    oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, scale, "causal")
    fused_steps = 0
    for step in range(150):
        k, v = seeded((B, Hkv, 1, D), 10 + 3 * step, dtype), seeded((B, Hkv, 1, D), 11 + 3 * step, dtype)
        q = seeded((B, Hq, 1, D), 12 + 3 * step, dtype)
        kvc.launch_count(reset=True)
        out = kvc.attention_with_cache_update(q.to(cuda), k.to(cuda), v.to(cuda), g, scale, "none")
        fused_steps += kvc.launch_count(reset=True) == 1
        ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k), to_oracle(v), o, scale, "none")
        assert max_abs_diff(out, ref) <= TOL[dtype], step
        assert g.offset == o.offset and list(g.meta_state) == list(o.meta_state), step
        if step % 37 == 0 or step == 149:
            for a, b in zip(g.state, o.state):
                assert bits_equal(a, np.ascontiguousarray(b)), step
    assert fused_steps >= 140        # growth and the one ring rebuild after the prefill cost extra launches
    assert kvc.lib().kvc_device_status() == 0


def test_bounded_wait_reports_through_the_status_word(kvc, cuda):
    """Every device-side wait in the library is bounded; one that runs out stores a code in the
    per-device status word and the kernel returns. The probe kernel waits on a word nothing ever
    sets: the status reads 40 afterwards, the context stays usable, and a reset clears the word."""
    assert kvc.device_status() == 0
    kvc.device_wait_probe(1 << 10)
    torch.cuda.synchronize()
    assert kvc.device_status() == 40
    kvc.device_status_reset()
    assert kvc.device_status() == 0
    q = seeded((1, 8, 1, 128), 1, torch.bfloat16).to(cuda)
    k = seeded((1, 2, 300, 128), 2, torch.bfloat16).to(cuda)
    out = kvc.scaled_dot_product_attention(q, k, k, 0.09)       # the device still answers
    assert torch.isfinite(out.float()).all() and kvc.device_status() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,Hq,Hkv,L,P,mask", [
    (2, 32, 8, 6, 1000, "causal"),     # Llama-3-8B layout, verify round: 24 rows per kv head; split keys
    (8, 32, 8, 6, 2100, "causal"),     # 64 units of 17 tiles on 148 SMs: CTAs that walk a cut unit and a whole one
    (1, 17, 1, 1, 300, "none"),        # 17 heads on one kv head, one position
    (1, 8, 1, 8, 120, "causal"),       # 64 rows; the chunk itself crosses the first tile boundary
    (40, 12, 4, 6, 300, "causal"),     # 160 units of three tiles: more units than SMs
])
def test_raw_cache_verify_rounds_run_on_the_tensor_core_verify_kernel(kvc, oracle, cuda, capfd, monkeypatch, dtype, B, Hq, Hkv, L, P, mask):
    """17 to 64 query rows per kv head over a KVCacheSimple at head dim 128: the tcgen05 verify kernel with
    TMA-loaded K / V tiles; two rounds in a row with a rejection in between."""
    D = 128
    monkeypatch.setenv("KVC_TRACE_DISPATCH", "1")
    g, o = kvc.KVCacheSimple(), oracle.KVCacheSimple()
    k, v = seeded((B, Hkv, P, D), 1, dtype), seeded((B, Hkv, P, D), 2, dtype)
    g.update(k.to(cuda), v.to(cuda))
    o.update(to_oracle(k), to_oracle(v))
    for rnd in range(2):
        q = seeded((B, Hq, L, D), 3 + rnd, dtype)
        k1, v1 = seeded((B, Hkv, L, D), 5 + rnd, dtype), seeded((B, Hkv, L, D), 7 + rnd, dtype)
        capfd.readouterr()
        out = g.attention(q.to(cuda), k1.to(cuda), v1.to(cuda), D ** -0.5, mask)
        torch.cuda.synchronize()
        assert "verify_tc raw" in capfd.readouterr().err
        ref = oracle.attention_with_cache_update(to_oracle(q), to_oracle(k1), to_oracle(v1), o, D ** -0.5, mask)
        assert max_abs_diff(out, ref) <= TOL[dtype], f"round {rnd}"
        assert g.trim(max(L - 1, 0)) == o.trim(max(L - 1, 0))
    assert kvc.lib().kvc_device_status() == 0


def test_verify_rounds_agree_with_the_tensor_core_verify_kernel_switched_off(tmp_path):
    """The same verify rounds (TurboQuant K4/V4 and K3/V4, affine 4-bit, raw bf16) with the tcgen05 verify
    kernel and, in a child process with KVC_VERIFY_TC=0, on the kernels behind it (eight-row units on the
    decode kernels, the mma.sync chunk kernel): outputs agree within the attention tolerance and the
    trace names the path that ran."""
    code = r"""
import os, sys, torch
sys.path.insert(0, os.path.join(%r, "mlx-swift-lm_b200", "python"))
sys.path.insert(0, os.path.join(%r, "tests"))
import kvcache_b200 as kvc
from helpers import seeded
dev = torch.device("cuda:0")
B, Hq, Hkv, D, P, L = 2, 16, 2, 128, 700, 6
dt = torch.bfloat16
outs = []
for kind in ("k4v4", "k3v4", "affine4", "raw"):
    if kind == "affine4": c = kvc.QuantizedKVCache(64, 4)
    elif kind == "raw": c = kvc.KVCacheSimple()
    else: c = kvc.TurboQuantKVCache(bits=4, key_bits=4 if kind == "k4v4" else 3, value_bits=4)
    k, v = seeded((B, Hkv, P, D), 1, dt).to(dev), seeded((B, Hkv, P, D), 2, dt).to(dev)
    if kind == "affine4": c.update_quantized(k, v)
    elif kind == "raw": c.update(k, v)
    else: c.encode_new_token(k, v)
    q = seeded((B, Hq, L, D), 3, dt).to(dev)
    k1, v1 = seeded((B, Hkv, L, D), 4, dt).to(dev), seeded((B, Hkv, L, D), 5, dt).to(dev)
    outs.append(c.attention(q, k1, v1, D ** -0.5, "causal").float().cpu())
torch.cuda.synchronize()
assert kvc.lib().kvc_device_status() == 0
torch.save(outs, sys.argv[1])
""" % (ROOT, ROOT)
    results, traces = [], []
    for switch in ("1", "0"):
        env = dict(os.environ)
        env["KVC_VERIFY_TC"] = switch
        env["KVC_TRACE_DISPATCH"] = "1"
        f = str(tmp_path / f"verify_{switch}.pt")
        r = subprocess.run([sys.executable, "-c", code, f], check=True, env=env, timeout=300, capture_output=True, text=True)
        results.append(torch.load(f))
        traces.append(r.stderr)
    assert traces[0].count("verify_tc") >= 4 and "verify_tc" not in traces[1]
    for a, b in zip(*results):
        assert float((a - b).abs().max()) <= 2e-2
