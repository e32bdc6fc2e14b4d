#!/usr/bin/env python
"""KV-cache decode benchmark.

One "step" is one decode step of the workload: every layer appends one new
token per sequence to its cache and attends over the whole cache
(attentionWithCacheUpdate per layer). The headline metric is decode tokens/s
(batch tokens per step / step time) together with the achieved HBM bandwidth
of the dominant attention kernel against the measured copy peak.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

The default workload is the TurboQuant cache at the Llama-3-70B attention shape
(80 layers, 64 query heads, 8 KV heads, head dim 128, batch 16, context 32768,
3-bit keys / 4-bit values): the largest configuration that fits one GPU. The
same line also carries a speculative verify leg (6 query rows per sequence:
5 draft tokens + the bonus token, causal, trimmed off again after the round).

Under torchrun (N > 1) the default partition shards the KV heads of ONE batch
across the ranks (the batch where the heads do not divide) and ends every layer
with an exchange of the attention outputs: total work is fixed ("strong"
scaling). `--parallel sequences` instead gives every rank its own batch of B
sequences with no data-path collective ("weak" scaling).
Inputs are synthetic (seeded N(0,1)); no dataset is involved.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (os.path.join(ROOT, "mlx-swift-lm_b200", "python"), os.path.join(ROOT, "oracle")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

METRIC = "kv_cache_decode_tokens_per_s"
UNIT = "tokens/s"

# Shapes are BASELINE.json's configs; `context` is the cache length when the
# timed decode starts.
WORKLOADS = {
    "cfg2_simple_bf16_llama3_8b": dict(kind="simple", layers=32, Hq=32, Hkv=8, D=128, B=8, dtype="bf16",
                                       context=8192, chunk=512),
    "cfg1_quant8_f32_llama32_1b": dict(kind="quantized", bits=8, group=64, layers=16, Hq=32, Hkv=8, D=64, B=1,
                                       dtype="f32", context=1024, chunk=1024),
    # Gemma-3-1B: every sixth layer global (KVCacheSimple, step 1024), the others sliding-window
    # RotatingKVCache(maxSize 512, keep 0); the rings have wrapped before the first timed step
    "cfg3_rotating_bf16_gemma3_1b": dict(kind="gemma3", layers=26, Hq=4, Hkv=1, D=256, B=4, dtype="bf16",
                                         context=2048, chunk=512, window=512),
    "cfg4_quant4_bf16_qwen2_7b": dict(kind="quantized", bits=4, group=64, layers=28, Hq=28, Hkv=4, D=128, B=32,
                                      dtype="bf16", context=17408, chunk=512),
    # the same shape held the reference's way: 32 independent sequences (one cache per sequence and
    # layer), lengths ~U[2048, 32768] from a seed, one var-len call per layer
    "cfg4_ragged_quant4_bf16_qwen2_7b": dict(kind="quantized", ragged=True, bits=4, group=64, layers=28, Hq=28, Hkv=4,
                                             D=128, B=32, dtype="bf16", context=17408, chunk=512,
                                             min_len=2048, max_len=32768, seed=4),
    "cfg5_turbo_k3v4_llama3_70b": dict(kind="turbo", key_bits=3, value_bits=4, layers=80, Hq=64, Hkv=8, D=128,
                                       B=16, dtype="bf16", context=32768, chunk=512),
}
# Two layers of the default workload: the small case for multi-pass ncu captures
# (per-layer working set 269 MB > L2, 0.6 GB on the device).
WORKLOADS["cfg2_profile_2layers"] = dict(WORKLOADS["cfg2_simple_bf16_llama3_8b"], layers=2)
WORKLOADS["cfg4_profile_2layers"] = dict(WORKLOADS["cfg4_quant4_bf16_qwen2_7b"], layers=2)
WORKLOADS["cfg4_ragged_profile_2layers"] = dict(WORKLOADS["cfg4_ragged_quant4_bf16_qwen2_7b"], layers=2)
WORKLOADS["cfg5_profile_2layers"] = dict(WORKLOADS["cfg5_turbo_k3v4_llama3_70b"], layers=2)
# Prefill of the default model shape: one 512-token chunk per layer on top of the 8192-token prefix
# (attentionWithCacheUpdate with a causal mask), 4 layers so that a capture stays small. A side
# workload: its metric is prefill tokens/s and its roofline is the tensor-core one.
WORKLOADS["cfg2_prefill512_4layers"] = dict(WORKLOADS["cfg2_simple_bf16_llama3_8b"], layers=4, prefill=512)
DEFAULT_WORKLOAD = "cfg5_turbo_k3v4_llama3_70b"
VERIFY_ROWS = 6   # 5 draft tokens + 1 bonus token per speculative round (Evaluate.swift:1205-1208)
MIN_TIMED_S = 0.5  # the timed region is repeated (whole passes of K steps) until it covers this much
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, from the ncu
# captures summarised under profiles/ (taken on the 2-layer variants: a launch is the same size)
NCU_TRAFFIC_BYTES = {
    "cfg2_simple_bf16_llama3_8b": (268.8e6 + 5.0e6, "profiles/attn_decode_flat_bf16_cfg2_llama3_8b.md"),
    "cfg4_quant4_bf16_qwen2_7b": (323.8e6 + 4.4e6, "profiles/attn_affine_decode8_cfg4_qwen2_7b.md"),
    "cfg5_turbo_k3v4_llama3_70b": (506.2e6 + 4.1e6, "profiles/attn_turbo_v4_cfg5_llama3_70b.md"),
}
for _k in ("cfg2", "cfg4", "cfg5"):
    _full = [n for n in NCU_TRAFFIC_BYTES if n.startswith(_k)][0]
    NCU_TRAFFIC_BYTES[_k + "_profile_2layers"] = NCU_TRAFFIC_BYTES[_full]


def bytes_per_token_head(w) -> float:
    """Algorithmic bytes of K plus V for one cached token of one KV head."""
    D = w["D"]
    es = 4 if w["dtype"] == "f32" else 2
    if w["kind"] in ("simple", "rotating", "gemma3"):
        return 2 * D * es
    if w["kind"] == "quantized":
        per = D * w["bits"] / 8 + 2 * (D // w["group"]) * es
        return 2 * per
    kpw = (D * w["key_bits"] + 31) // 32 * 4 + 4
    vpw = (D * w["value_bits"] + 31) // 32 * 4 + 4
    return kpw + vpw


def partition(w, world: int, mode: str):
    """Per-rank shape of the workload on `world` ranks.

    Returns dict(shard_axis, B_local, Hkv_local, Hq_local, B_global, scaling,
    parallelism, collective). mode "sequences": each rank holds B whole sequences
    (independent caches; nothing crosses ranks). mode "heads": one batch of B,
    KV heads split across ranks (batch split when heads do not divide), outputs
    all-gathered per layer."""
    B, Hq, Hkv = w["B"], w["Hq"], w["Hkv"]
    if world == 1:
        return dict(shard_axis=1, B_local=B, Hkv_local=Hkv, Hq_local=Hq, B_global=B, scaling="weak",
                    parallelism="single", collective=False)
    if mode == "sequences":
        return dict(shard_axis=0, B_local=B, Hkv_local=Hkv, Hq_local=Hq, B_global=B * world, scaling="weak",
                    parallelism=f"sequences x{world} (B={B} per rank, no collective)", collective=False)
    if mode != "heads":
        raise ValueError(f"unknown partition mode {mode!r}")
    if Hkv % world == 0:
        return dict(shard_axis=1, B_local=B, Hkv_local=Hkv // world, Hq_local=Hq // world, B_global=B,
                    scaling="strong", parallelism=f"kv-head x{world} + all-gather", collective=True)
    if B % world:
        # neither axis divides: independent sequences per rank
        return partition(w, world, "sequences")
    return dict(shard_axis=0, B_local=B // world, Hkv_local=Hkv, Hq_local=Hq, B_global=B, scaling="strong",
                parallelism=f"batch x{world} + all-gather", collective=True)


def job_config(args, w, world):
    """The `config` object of the JSON line: the workload and how it is laid over the ranks. Both arms
    (this library and the CPU reference) print the same object for the same command line."""
    part = partition(w, world, args.parallel)
    ctx0 = w["context"] + max(args.warmup, 3)
    per_layer = part["B_local"] * part["Hkv_local"] * ctx0 * bytes_per_token_head(w)
    cfg = {"workload": args.workload, **{k: w[k] for k in ("layers", "Hq", "Hkv", "D")}, "B": part["B_global"],
           "context_start": ctx0, "parallelism": part["parallelism"], "verify_rows": VERIFY_ROWS,
           "l2": "inputs larger than L2 (per-layer K+V working set per GPU "
                 f"{per_layer / 1e6:.0f} MB; all layers {w['layers'] * per_layer / 1e9:.2f} GB per step)"}
    return cfg, part


def torch_dtype(name):
    import torch
    return {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[name]


# ---------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------

class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "25"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return

        def pump():
            for line in self.proc.stdout:
                self.rows.append((time.perf_counter(), [c.strip() for c in line.split(",")]))
        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                pass

    def summary(self, t0: float, t1: float):
        sel = [r for ts, r in self.rows if t0 <= ts <= t1 and len(r) >= 9] or [r for _, r in self.rows if len(r) >= 9]
        if not sel:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm = [float(r[1]) for r in sel if r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in sel if r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in sel:
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sel)}


# ---------------------------------------------------------------------------
# CPU arm (the oracle, timed): reference implementation of the path on host cores
# ---------------------------------------------------------------------------

def cpu_decode_step_time(w, budget_s: float, steps: int = 1, warmup: int = 0):
    """Times the oracle's decode step (append + attention per layer) on a bounded
    sample: `layers_sample` layer calls per step over one layer's cache arrays,
    scaled to the workload's layer count. Returns (seconds per full step, info)."""
    import numpy as np
    import kvcache_oracle as orc

    orc.build()
    orc.use_all_host_threads()   # torch.distributed.run hands its workers OMP_NUM_THREADS=1
    B, Hq, Hkv, D, T0 = w["B"], w["Hq"], w["Hkv"], w["D"], w["context"]
    if w["kind"] == "gemma3":
        # per-layer average of what a step reads: 22 wrapped 512-token rings and 4 full-context layers
        n_glob = len([i for i in range(w["layers"]) if i % 6 == 5])
        T0 = (n_glob * w["context"] + (w["layers"] - n_glob) * min(w["window"], w["context"])) // w["layers"]
        w = dict(w, kind="simple")
    rng = np.random.default_rng(0)
    es_dtype = np.float32 if w["dtype"] == "f32" else np.uint16

    def rnd(shape):
        x = rng.standard_normal(shape, dtype=np.float32)
        return x if w["dtype"] == "f32" else orc.f32_to_bf16_bits(x)

    cap = T0 + 64
    q = rnd((B, Hq, 1, D))
    nk, nv = rnd((B, Hkv, 1, D)), rnd((B, Hkv, 1, D))
    scale = D ** -0.5
    if w["kind"] == "simple":
        K = np.empty((B, Hkv, cap, D), dtype=es_dtype)
        V = np.empty((B, Hkv, cap, D), dtype=es_dtype)
        blk = rnd((B, Hkv, 1024, D))
        for t in range(0, cap, 1024):
            n = min(1024, cap - t)
            K[:, :, t:t + n] = blk[:, :, :n]
            V[:, :, t:t + n] = blk[:, :, :n]

        def layer_call(T):
            orc.append_rows(nk, K, T)
            orc.append_rows(nv, V, T)
            return orc.attention(q, orc.RawSource(K[:, :, :T + 1]), orc.RawSource(V[:, :, :T + 1]), scale, precise=False)
    elif w["kind"] == "quantized":
        blk = rnd((B, Hkv, 1024, D))
        qk = orc.affine_quantize(blk, w["group"], w["bits"])
        reps = (cap + 1023) // 1024
        ck = [np.ascontiguousarray(np.concatenate([a] * reps, axis=2)[:, :, :cap]) for a in qk]
        cv = [a.copy() for a in ck]

        def layer_call(T):
            nq = orc.affine_quantize(nk, w["group"], w["bits"])
            nq2 = orc.affine_quantize(nv, w["group"], w["bits"])
            for i in range(3):
                ck[i][:, :, T:T + 1] = nq[i]
                cv[i][:, :, T:T + 1] = nq2[i]
            return orc.attention(q, orc.AffineSource(*(a[:, :, :T + 1] for a in ck), w["group"], w["bits"]),
                                 orc.AffineSource(*(a[:, :, :T + 1] for a in cv), w["group"], w["bits"]), scale,
                                 precise=False)
    else:
        kc = orc.MSECodec(D, w["key_bits"], 42)
        vc = orc.MSECodec(D, w["value_bits"], 43)
        blk = rnd((B, Hkv, 1024, D))
        kp, kn = kc.encode(blk)
        vp, vn = vc.encode(blk)
        reps = (cap + 1023) // 1024
        KP = np.ascontiguousarray(np.concatenate([kp] * reps, axis=2)[:, :, :cap])
        KN = np.ascontiguousarray(np.concatenate([kn] * reps, axis=2)[:, :, :cap])
        VP = np.ascontiguousarray(np.concatenate([vp] * reps, axis=2)[:, :, :cap])
        VN = np.ascontiguousarray(np.concatenate([vn] * reps, axis=2)[:, :, :cap])

        def layer_call(T):
            a, b = kc.encode(nk)
            c, d = vc.encode(nv)
            KP[:, :, T:T + 1], KN[:, :, T:T + 1], VP[:, :, T:T + 1], VN[:, :, T:T + 1] = a, b, c, d
            return orc.attention(q, orc.TurboSource(KP[:, :, :T + 1], KN[:, :, :T + 1], kc.codebook, w["key_bits"]),
                                 orc.TurboSource(VP[:, :, :T + 1], VN[:, :, :T + 1], vc.codebook, w["value_bits"]),
                                 scale, q_signs=kc.signs, o_signs=vc.signs, precise=False)

    t0 = time.perf_counter()
    layer_call(T0)
    t_layer = time.perf_counter() - t0
    total_calls = max(1, int(budget_s / max(t_layer, 1e-6)))
    per_step = max(1, min(w["layers"], total_calls // max(1, steps + warmup)))
    times = []
    T = T0
    for s in range(warmup + steps):
        t0 = time.perf_counter()
        for _ in range(per_step):
            layer_call(T)
        dt = time.perf_counter() - t0
        T = min(T + 1, cap - 2)
        if s >= warmup:
            times.append(dt * w["layers"] / per_step)
    info = {"cores": orc.num_threads(),
            "sample": f"{per_step} of {w['layers']} layer calls per step (append + attention over one layer's "
                      f"cache at context {T0}), scaled to {w['layers']} layers; {steps} timed steps"}
    return sum(times) / len(times), info


def run_reference(args, w, rank, world):
    """The reference arm: the CPU restatement of the reference path (MLX itself cannot run on this box) on
    all host cores, rank 0 only, on the same job (same global batch at every N) and the same `config`."""
    if rank != 0:
        return
    cfg, part = job_config(args, w, world)
    wj = dict(w, B=part["B_global"])
    sec, info = cpu_decode_step_time(wj, budget_s=90.0, steps=max(1, args.steps), warmup=min(args.warmup, 1))
    value = part["B_global"] / sec
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": part["scaling"],
            "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic", "impl": "reference",
            "config": cfg,
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": info["cores"], "kind": "port", "sample": info["sample"]},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------

def make_cache(kvc, w, reserve, layer=0):
    if w["kind"] == "gemma3":
        if layer % 6 == 5:
            return kvc.KVCacheSimple(step=1024, reserve_tokens=reserve)
        return kvc.RotatingKVCache(max_size=w["window"], keep=0)
    if w["kind"] == "simple":
        return kvc.KVCacheSimple(step=256, reserve_tokens=reserve)
    if w["kind"] == "quantized":
        return kvc.QuantizedKVCache(w["group"], w["bits"], reserve_tokens=reserve)
    if w["kind"] == "turbo":
        return kvc.TurboQuantKVCache(bits=max(w["key_bits"], w["value_bits"]), key_bits=w["key_bits"],
                                     value_bits=w["value_bits"], reserve_tokens=reserve)
    raise ValueError(w["kind"])


def fill_cache(kvc, cache, w, Bl, Hl, chunk_k, chunk_v):
    remaining = w["context"]
    while remaining > 0:
        n = min(remaining, chunk_k.shape[2])
        k, v = chunk_k[:, :, :n], chunk_v[:, :, :n]
        if w["kind"] in ("simple", "gemma3"):
            cache.update(k, v)
        elif w["kind"] == "quantized":
            cache.update_quantized(k, v)
        else:
            cache.encode_new_token(k, v)
        remaining -= n


def run_ragged(args, w, rank, world, local_rank):
    """cfg4 the reference's way: every sequence has its own cache per layer (its own offset); one
    kvc_attention_varlen call per layer appends and attends all sequences (two launches)."""
    import numpy as np
    import torch
    import kvcache_b200 as kvc

    assert world == 1, "the ragged workload is a single-GPU parity / measurement case"
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    dtype = torch_dtype(w["dtype"])
    n, Hq, Hkv, D, Lyr = w["B"], w["Hq"], w["Hkv"], w["D"], w["layers"]
    rng = np.random.default_rng(w["seed"])
    lengths = [int(x) for x in rng.integers(w["min_len"], w["max_len"] + 1, size=n)]
    steps, warmup = args.steps, args.warmup
    total_steps = warmup + steps * 3 + 64
    g = torch.Generator(device="cpu").manual_seed(99)
    chunk_k = torch.randn((1, Hkv, w["chunk"], D), generator=g).to(dtype).to(dev)
    chunk_v = torch.randn((1, Hkv, w["chunk"], D), generator=g).to(dtype).to(dev)
    layers = []
    for _ in range(Lyr):
        caches = []
        for t in lengths:
            c = kvc.QuantizedKVCache(w["group"], w["bits"], reserve_tokens=t + total_steps + 8)
            left = t
            while left > 0:
                m = min(left, w["chunk"])
                c.update_quantized(chunk_k[:, :, :m], chunk_v[:, :, :m])
                left -= m
            caches.append(c)
        layers.append(caches)
    torch.cuda.synchronize()
    scale = D ** -0.5
    # per layer: stacked device tensors, sequence i uses row i
    q_all = [torch.randn((n, Hq, 1, D), generator=g).to(dtype).to(dev) for _ in range(Lyr)]
    k_all = [torch.randn((n, Hkv, 1, D), generator=g).to(dtype).to(dev) for _ in range(Lyr)]
    v_all = [torch.randn((n, Hkv, 1, D), generator=g).to(dtype).to(dev) for _ in range(Lyr)]
    o_all = [torch.empty((n, Hq, 1, D), dtype=dtype, device=dev) for _ in range(Lyr)]
    plans = [kvc.DecodeStep(layers[l], [q_all[l][i:i + 1] for i in range(n)], [k_all[l][i:i + 1] for i in range(n)],
                            [v_all[l][i:i + 1] for i in range(n)], [o_all[l][i:i + 1] for i in range(n)], scale)
             for l in range(Lyr)]

    def one_step():
        for pl in plans:
            pl.run_varlen()

    for _ in range(warmup):
        one_step()
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.25)
    torch.cuda.synchronize()
    sum_t0 = sum(c.offset for c in layers[0])
    kvc.launch_count(reset=True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0 = time.perf_counter()
    e0.record()
    for _ in range(steps):
        one_step()
    e1.record()
    torch.cuda.synchronize()
    w1 = time.perf_counter()
    launches = kvc.launch_count()
    ms_total = e0.elapsed_time(e1)
    time.sleep(0.15)
    sampler.stop()
    clocks = sampler.summary(w0, w1)

    kvc.timing_enable(True)
    kvc.timing_read(reset=True)
    rsteps = min(steps, 8)
    sum_r0 = sum(c.offset for c in layers[0])
    for _ in range(rsteps):
        one_step()
    torch.cuda.synchronize()
    k_ms, k_n = kvc.timing_read(reset=True)
    kvc.timing_enable(False)
    alg_bytes = Hkv * (sum_r0 + n * (rsteps + 1) / 2) * bytes_per_token_head(w) + 2 * n * Hq * D * 2
    k_avg_ms = k_ms / max(k_n, 1)
    peak, peak_src = 6545.0, "fallback 6545 GB/s (MEASURED_PEAKS.json absent)"
    mp = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(mp):
        try:
            peak = float(json.load(open(mp))["hbm_gbs"])
            peak_src = "MEASURED_PEAKS.json hbm_gbs (measured copy)"
        except Exception:
            pass
    achieved = alg_bytes / (k_avg_ms * 1e-3) / 1e9 if k_n else None
    traffic = NCU_TRAFFIC_BYTES.get(args.workload) if world == 1 else None
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": (achieved / peak) if achieved else None, "traffic": traffic[0] if traffic else None,
                "traffic_source": ("ncu dram__bytes_read.sum + dram__bytes_write.sum per launch, " + traffic[1]) if traffic else None,
                "kernel": "var-len attention (dominant)", "launch_ms": k_avg_ms, "launches_timed": k_n,
                "algorithmic_bytes_per_launch": alg_bytes, "peak_source": peak_src}

    # end to end: pinned host q/k/v per layer -> device, var-len call, outputs back to the host
    hq = [t.cpu().pin_memory() for t in q_all]
    hk = [t.cpu().pin_memory() for t in k_all]
    hv = [t.cpu().pin_memory() for t in v_all]
    ho = [torch.empty((n, Hq, 1, D), dtype=dtype).pin_memory() for _ in range(Lyr)]

    def e2e_step():
        for l in range(Lyr):
            q_all[l].copy_(hq[l], non_blocking=True)
            k_all[l].copy_(hk[l], non_blocking=True)
            v_all[l].copy_(hv[l], non_blocking=True)
            plans[l].run_varlen()
            ho[l].copy_(o_all[l], non_blocking=True)
        torch.cuda.synchronize()
        return float(ho[-1][0, 0, 0, 0])

    for _ in range(min(warmup, 3)):
        e2e_step()
    t0 = time.perf_counter()
    for _ in range(steps):
        e2e_step()
    e2e_s = time.perf_counter() - t0
    es = 2
    e2e = {"value": n * steps / e2e_s, "unit": UNIT, "h2d_bytes_per_step": Lyr * n * (Hq + 2 * Hkv) * D * es,
           "d2h_bytes_per_step": Lyr * n * Hq * D * es,
           "note": "per layer: pinned host q/k/v -> device, kvc_attention_varlen, outputs -> host; one sync per step"}
    line = {"metric": METRIC, "value": n * steps / (ms_total * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": steps,
            "warmup": warmup, "ms_per_step": ms_total / steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
            "config": {"workload": args.workload, "layers": Lyr, "Hq": Hq, "Hkv": Hkv, "D": D, "B": n,
                       "sequence_lengths": {"min": min(lengths), "max": max(lengths), "sum": sum_t0},
                       "parallelism": "single; 32 independent caches per layer, one var-len call per layer",
                       "l2": f"inputs larger than L2 (per-layer working set {Hkv * sum_t0 * bytes_per_token_head(w) / 1e6:.0f} MB)"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "roofline": roofline, "cpu_baseline": None}
    print(json.dumps(line), flush=True)


def run_prefill(args, w, rank, world, local_rank):
    """One step = a chunk of w["prefill"] new tokens through every layer (append + causal attention over
    prefix + chunk), then the chunk is trimmed off again so that every step does the same work. Each
    rank runs its own sequences (no collective)."""
    import torch
    import kvcache_b200 as kvc

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (the library has no CPU fallback)"
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)
    dtype = torch_dtype(w["dtype"])
    B, Hq, Hkv, D, Lyr, L, ctx = w["B"], w["Hq"], w["Hkv"], w["D"], w["layers"], w["prefill"], w["context"]
    g = torch.Generator(device="cpu").manual_seed(99 + rank)
    chunk_k = torch.randn((B, Hkv, w["chunk"], D), generator=g).to(dtype).to(dev)
    chunk_v = torch.randn((B, Hkv, w["chunk"], D), generator=g).to(dtype).to(dev)
    caches = [make_cache(kvc, w, ctx + L + 8, i) for i in range(Lyr)]
    for c in caches:
        fill_cache(kvc, c, w, B, Hkv, chunk_k, chunk_v)
    qs = [torch.randn((B, Hq, L, D), generator=g).to(dtype).to(dev) for _ in range(Lyr)]
    ks = [torch.randn((B, Hkv, L, D), generator=g).to(dtype).to(dev) for _ in range(Lyr)]
    vs = [torch.randn((B, Hkv, L, D), generator=g).to(dtype).to(dev) for _ in range(Lyr)]
    outs = [torch.empty_like(q) for q in qs]
    scale = D ** -0.5

    def one_step():
        for i, c in enumerate(caches):
            c.attention(qs[i], ks[i], vs[i], scale, "causal", out=outs[i])
            c.trim(L)

    for _ in range(args.warmup):
        one_step()
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.25)
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    kvc.launch_count(reset=True)
    kvc.timing_enable(True)
    kvc.timing_read(reset=True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0 = time.perf_counter()
    e0.record()
    for _ in range(args.steps):
        one_step()
    e1.record()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    w1 = time.perf_counter()
    k_ms, k_n = kvc.timing_read(reset=True)
    kvc.timing_enable(False)
    launches = kvc.launch_count()
    ms_total = e0.elapsed_time(e1)
    if dist is not None:
        t = torch.tensor([ms_total], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    time.sleep(0.15)
    sampler.stop()
    # visible (query, key) pairs of one layer call: row l of the chunk sees ctx + l + 1 keys
    pairs = sum(ctx + l + 1 for l in range(L))
    flops = 4.0 * B * Hq * pairs * D
    k_avg_ms = k_ms / max(k_n, 1)
    achieved = flops / (k_avg_ms * 1e-3) / 1e12 if k_n else None
    peak, peak_src = 1590.0, "fallback 1590 TFLOP/s (MEASURED_PEAKS.json absent)"
    mp = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(mp):
        try:
            peak = float(json.load(open(mp))["bf16_tflops"])
            peak_src = "MEASURED_PEAKS.json bf16_tflops (cuBLAS burst)"
        except Exception:
            pass
    if rank == 0:
        print(json.dumps({
            "metric": "kv_cache_prefill_tokens_per_s", "value": world * B * L * args.steps / (ms_total * 1e-3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": w["dtype"], "data": "synthetic",
            "config": {"workload": args.workload, "layers": Lyr, "Hq": Hq, "Hkv": Hkv, "D": D, "B": B, "context": ctx,
                       "chunk": L, "parallelism": "single" if world == 1 else f"sequences x{world}",
                       "l2": f"per-layer K+V working set {B * Hkv * (ctx + L) * 2 * D * 2 / 1e6:.0f} MB"},
            "clocks": sampler.summary(w0, w1), "e2e": None, "gpu_launches": launches,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": (achieved / peak) if achieved else None, "traffic": None,
                         "kernel": "attention over the chunk (dominant)", "launch_ms": k_avg_ms, "launches_timed": k_n,
                         "timing": "CUDA events around each attention launch (kvc_timing)",
                         "flops_per_launch": flops, "peak_source": peak_src},
            "cpu_baseline": None}), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def run_ours(args, w, rank, world, local_rank):
    import torch
    import kvcache_b200 as kvc

    if w.get("ragged"):
        return run_ragged(args, w, rank, world, local_rank)
    if w.get("prefill"):
        return run_prefill(args, w, rank, world, local_rank)

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (the library has no CPU fallback)"
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)

    dtype = torch_dtype(w["dtype"])
    Hq, D, Lyr = w["Hq"], w["D"], w["layers"]
    cfg, part = job_config(args, w, world)
    shard_axis, Bl, Hkvl, Hql = part["shard_axis"], part["B_local"], part["Hkv_local"], part["Hq_local"]
    B, parallelism = part["B_global"], part["parallelism"]
    steps, warmup = args.steps, args.warmup
    total_steps = warmup + steps * 21 + 64 + VERIFY_ROWS   # timed passes, roofline pass, end-to-end passes
    reserve = w["context"] + total_steps + 8

    g = torch.Generator(device="cpu").manual_seed(1234 + rank)
    chunk = min(w["chunk"], w["context"])
    chunk_k = torch.randn((Bl, Hkvl, chunk, D), generator=g).to(dtype).to(dev)
    chunk_v = torch.randn((Bl, Hkvl, chunk, D), generator=g).to(dtype).to(dev)
    caches = [make_cache(kvc, w, reserve, i) for i in range(Lyr)]
    for c in caches:
        fill_cache(kvc, c, w, Bl, Hkvl, chunk_k, chunk_v)
    torch.cuda.synchronize()

    # per-layer step inputs, resident in HBM
    qs = [torch.randn((Bl, Hql, 1, D), generator=g).to(dtype).to(dev) for _ in range(Lyr)]
    ks = [torch.randn((Bl, Hkvl, 1, D), generator=g).to(dtype).to(dev) for _ in range(Lyr)]
    vs = [torch.randn((Bl, Hkvl, 1, D), generator=g).to(dtype).to(dev) for _ in range(Lyr)]
    scale = D ** -0.5
    comm = None
    if part["collective"]:
        uid = [kvc.Comm.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)
        comm = kvc.Comm(rank, world, uid[0])
        # gathered outputs in symmetric memory: the per-layer exchange runs as peer stores over NVLink
        # (--exchange nccl keeps them in ordinary memory: ncclAllGather + re-ordering kernel)
        if args.exchange == "peer":
            all_outs = comm.symm_empty((Lyr, B, Hq, 1, D), dtype, dev)
            outs = [all_outs[i] for i in range(Lyr)]
        else:
            outs = [torch.empty((B, Hq, 1, D), dtype=dtype, device=dev) for _ in range(Lyr)]
    else:
        outs = [torch.empty((Bl, Hql, 1, D), dtype=dtype, device=dev) for _ in range(Lyr)]
    step = kvc.DecodeStep(caches, qs, ks, vs, outs, scale)

    def one_step():
        if comm is not None:
            step.run_sharded(comm, shard_axis)
        else:
            step.run()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if dist is None:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed_pass(fn, n):
        """Exactly n calls of fn between two events, a barrier and a device sync on both sides; the
        time is the maximum over the ranks."""
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1))

    for _ in range(warmup):
        one_step()
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.25)
    barrier()
    ctx0 = caches[0].offset
    kvc.launch_count(reset=True)
    w0 = time.perf_counter()
    # The timed region is whole passes of exactly `steps` steps, repeated until it covers MIN_TIMED_S
    # (at most 10 passes); the reported time is the median pass. Every rank takes the same count.
    pass_ms = [timed_pass(one_step, steps)]
    launches = kvc.launch_count()
    while sum(pass_ms) < MIN_TIMED_S * 1e3 and len(pass_ms) < 10:
        pass_ms.append(timed_pass(one_step, steps))
    w1 = time.perf_counter()
    ms_total = statistics.median(pass_ms)
    ms_per_step = ms_total / steps
    value = B * steps / (ms_total * 1e-3)
    time.sleep(0.15)
    sampler.stop()
    clocks = sampler.summary(w0, w1)

    # speculative verify leg: every layer appends VERIFY_ROWS rows and attends with a causal mask, then
    # the rows are trimmed off again (all rejected), so that every round does the same work
    verify = None
    if VERIFY_ROWS and w["kind"] in ("simple", "quantized", "turbo"):
        Lv = VERIFY_ROWS
        vq = [torch.randn((Bl, Hql, Lv, D), generator=g).to(dtype).to(dev) for _ in range(Lyr)]
        vk = [torch.randn((Bl, Hkvl, Lv, D), generator=g).to(dtype).to(dev) for _ in range(Lyr)]
        vv = [torch.randn((Bl, Hkvl, Lv, D), generator=g).to(dtype).to(dev) for _ in range(Lyr)]
        if comm is not None and args.exchange == "peer":
            all_vo = comm.symm_empty((Lyr, B, Hq, Lv, D), dtype, dev)
            vo = [all_vo[i] for i in range(Lyr)]
        elif comm is not None:
            vo = [torch.empty((B, Hq, Lv, D), dtype=dtype, device=dev) for _ in range(Lyr)]
        else:
            vo = [torch.empty((Bl, Hql, Lv, D), dtype=dtype, device=dev) for _ in range(Lyr)]
        vstep = kvc.DecodeStep(caches, vq, vk, vv, vo, scale, mask="causal")

        def one_round():
            if comm is not None:
                vstep.run_sharded(comm, shard_axis)
            else:
                vstep.run()
            kvc.trim_prompt_cache(caches, Lv)

        for _ in range(3):
            one_round()
        rounds = max(2, min(steps, 16))
        v_ms = timed_pass(one_round, rounds) / rounds
        verify = {"rows": Lv, "ms_per_round": v_ms, "tokens_per_s_if_all_accepted": B * Lv / (v_ms * 1e-3),
                  "vs_decode_step": v_ms / ms_per_step,
                  "note": "one round = append 6 rows + causal attention in every layer, then trim(6)"}
        del vq, vk, vv, vo, vstep

    # roofline pass: bracket the dominant attention kernel with events
    # The dominant kernel's launch duration. When a step is nothing but that kernel (one launch per
    # layer: the attention kernel appends the new row itself), CUDA events around a run of steps give
    # it directly; otherwise the library brackets each attention launch with its own events.
    rsteps = min(steps, 16)
    ctx_r0 = caches[0].offset
    only_attention = launches == steps * Lyr and comm is None
    if only_attention:
        r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        r0.record()
        for _ in range(rsteps):
            one_step()
        r1.record()
        torch.cuda.synchronize()
        k_ms, k_n = r0.elapsed_time(r1), rsteps * Lyr
    else:
        kvc.timing_enable(True)
        kvc.timing_read(reset=True)
        for _ in range(rsteps):
            one_step()
        torch.cuda.synchronize()
        k_ms, k_n = kvc.timing_read(reset=True)
        kvc.timing_enable(False)
    ctx_mid = ctx_r0 + (rsteps + 1) / 2
    es = 4 if w["dtype"] == "f32" else 2
    if w["kind"] == "gemma3":
        n_glob = len([i for i in range(Lyr) if i % 6 == 5])
        ctx_mid = (n_glob * ctx_mid + (Lyr - n_glob) * min(w["window"], ctx_mid)) / Lyr   # average over the layers
    alg_bytes = Bl * Hkvl * ctx_mid * bytes_per_token_head(w) + 2 * Bl * Hql * D * es
    k_avg_ms = k_ms / max(k_n, 1)
    achieved = alg_bytes / (k_avg_ms * 1e-3) / 1e9 if k_n else None
    peak, peak_src = 6545.0, "fallback 6545 GB/s (MEASURED_PEAKS.json absent)"
    mp = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(mp):
        try:
            peak = float(json.load(open(mp))["hbm_gbs"])
            peak_src = "MEASURED_PEAKS.json hbm_gbs (measured copy)"
        except Exception:
            pass
    traffic = NCU_TRAFFIC_BYTES.get(args.workload) if world == 1 else None
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": (achieved / peak) if achieved else None, "traffic": traffic[0] if traffic else None,
                "traffic_source": ("ncu dram__bytes_read.sum + dram__bytes_write.sum per launch, " + traffic[1]) if traffic else None,
                "kernel": "attention (dominant)", "launch_ms": k_avg_ms, "launches_timed": k_n,
                "timing": ("CUDA events around %d back-to-back steps of one launch per layer" % rsteps) if only_attention
                          else "CUDA events around each attention launch (kvc_timing)",
                "algorithmic_bytes_per_launch": alg_bytes, "peak_source": peak_src}

    # end to end through the host-buffer entry point
    hq = [torch.randn((Bl, Hql, 1, D), generator=g).to(dtype).pin_memory() for _ in range(Lyr)]
    hk = [torch.randn((Bl, Hkvl, 1, D), generator=g).to(dtype).pin_memory() for _ in range(Lyr)]
    hv = [torch.randn((Bl, Hkvl, 1, D), generator=g).to(dtype).pin_memory() for _ in range(Lyr)]
    ho = [torch.empty((Bl, Hql, 1, D), dtype=dtype).pin_memory() for _ in range(Lyr)]
    if comm is None:
        hstep = kvc.DecodeStep(caches, hq, hk, hv, ho, scale, host=True)

        def e2e_step():
            hstep.run(synchronize=True)
            return float(ho[-1][0, 0, 0, 0])  # the step's result is read on the host
    else:
        # sharded: this rank's inputs travel host -> device, the sharded step (attention + exchange per
        # layer) runs, and the GATHERED outputs of every layer travel back to this rank's host
        hfull = [torch.empty((B, Hq, 1, D), dtype=dtype).pin_memory() for _ in range(Lyr)]

        def e2e_step():
            for i in range(Lyr):
                qs[i].copy_(hq[i], non_blocking=True)
                ks[i].copy_(hk[i], non_blocking=True)
                vs[i].copy_(hv[i], non_blocking=True)
            step.run_sharded(comm, shard_axis)
            for i in range(Lyr):
                hfull[i].copy_(outs[i], non_blocking=True)
            torch.cuda.synchronize()
            return float(hfull[-1][0, 0, 0, 0])

    for _ in range(min(warmup, 3)):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        e2e_step()
    barrier()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    e2e_repeats = 1
    while e2e_s * e2e_repeats < MIN_TIMED_S and e2e_repeats < 10:
        # same rule as the device-timed region: whole passes of `steps` steps, the last pass is reported
        barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            e2e_step()
        barrier()
        e2e_s = max_over_ranks(time.perf_counter() - t0)
        e2e_repeats += 1
    h2d = world * Lyr * (Bl * Hql * D + 2 * Bl * Hkvl * D) * es  # summed over ranks
    d2h = world * Lyr * (B * Hq if comm is not None else Bl * Hql) * D * es
    e2e = {"value": B * steps / e2e_s, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
           "note": ("kvc_attention_batch with pinned host q/k/v in and outputs out for every layer (copies run on side "
                    "streams ahead of / behind the layer kernels), one stream sync per step, result read on the host"
                    if comm is None else
                    "per rank: pinned host q/k/v of its shard -> device, the sharded step (attention + output exchange per "
                    "layer), the gathered outputs of every layer -> pinned host, one sync per step")
                   + ("; bytes summed over ranks, time is the max over ranks" if world > 1 else "")}

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        sec, info = cpu_decode_step_time(w, budget_s=20.0, steps=3, warmup=0)
        cpu_baseline = {"value": B / sec, "unit": UNIT, "cores": info["cores"], "kind": "port", "sample": info["sample"]}

    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
                "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": part["scaling"], "vs_baseline": None,
                "dtype": w["dtype"], "data": "synthetic", "config": cfg,
                "timed_passes": {"count": len(pass_ms), "ms": pass_ms, "reported": "median",
                                 "context_at_first_timed_step": ctx0},
                "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "roofline": roofline,
                "verify": verify, "cpu_baseline": cpu_baseline}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="per-layer output exchange of the sharded partition: peer stores into symmetric memory "
                         "(default) or ncclAllGather")
    ap.add_argument("--parallel", default="heads", choices=["sequences", "heads"],
                    help="N>1 partition: KV heads of one batch + per-layer output exchange (strong, default) or "
                         "independent sequences per rank (weak)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    w = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, w, rank, world)
        return
    run_ours(args, w, rank, world, local_rank)


if __name__ == "__main__":
    main()
