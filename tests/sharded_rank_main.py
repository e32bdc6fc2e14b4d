"""One rank of the multi-GPU sharded-attention parity check (launched by
test_gpu_sharded.py through torch.distributed.run, one process per GPU).

Every rank draws the same full problem, keeps its shard of the KV heads (or of
the batch) in its own cache, runs kvc_attention_sharded, and compares the
gathered output with the oracle's attention over the full problem. Every case
runs twice: with the gathered buffer in ordinary device memory (ncclAllGather)
and in symmetric memory (peer stores + arrival counters), a decode step and a
6-row causal verify chunk each.

A last step makes the bounded arrival wait run out from the HOST side: the last
rank withholds one exchange, the other ranks' wait gives up after its (shortened)
limit, stores its code in the status word and the kernel returns; the withheld
exchange is then issued, so the counters are level again. Nothing on a device
faults, traps or spins without a limit."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
for p in (os.path.join(ROOT, "mlx-swift-lm_b200", "python"), os.path.join(ROOT, "oracle"), os.path.dirname(__file__)):
    if p not in sys.path:
        sys.path.insert(0, p)

from helpers import TOL, max_abs_diff, seeded, to_oracle  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    import kvcache_b200 as kvc
    import kvcache_oracle as orc
    orc.build()

    uid = [kvc.Comm.unique_id() if rank == 0 else None]
    dist.broadcast_object_list(uid, src=0)
    comm = kvc.Comm(rank, world, uid[0])
    failures = []
    cases = [
        # (kind, dtype, B, Hq, Hkv, D, P, shard_axis)
        ("simple", torch.bfloat16, 2, 8 * world, 2 * world, 128, 700, 1),
        ("simple", torch.float32, 2 * world, 4, 2, 64, 130, 0),
        ("quantized", torch.bfloat16, 2, 4 * world, 2 * world, 128, 300, 1),
        ("turbo", torch.bfloat16, 2, 8 * world, world, 128, 600, 1),
    ]
    for kind, dtype, B, Hq, Hkv, D, P, axis in cases:
        for mode in ("nccl", "peer"):
            k = seeded((B, Hkv, P, D), 1, dtype)
            v = seeded((B, Hkv, P, D), 2, dtype)
            scale = D ** -0.5
            if kind == "simple":
                g, o = kvc.KVCacheSimple(), orc.KVCacheSimple()
                o.update(to_oracle(k), to_oracle(v))
            elif kind == "quantized":
                g, o = kvc.QuantizedKVCache(64, 4), orc.QuantizedKVCache(64, 4)
                o.update_quantized(to_oracle(k), to_oracle(v))
            else:
                g = kvc.TurboQuantKVCache(bits=4, key_bits=3, value_bits=4)
                o = orc.TurboQuantKVCache(bits=4, key_bits=3, value_bits=4)
                o.encode_new_token(to_oracle(k), to_oracle(v))

            def shard(t, heads):
                if axis == 1:
                    n = heads // world
                    return t[:, rank * n:(rank + 1) * n].contiguous().to(dev)
                n = B // world
                return t[rank * n:(rank + 1) * n].contiguous().to(dev)

            if kind == "simple":
                g.update(shard(k, Hkv), shard(v, Hkv))
            elif kind == "quantized":
                g.update_quantized(shard(k, Hkv), shard(v, Hkv))
            else:
                g.encode_new_token(shard(k, Hkv), shard(v, Hkv))
            for L, mask in ((1, "none"), (6, "causal")):
                q = seeded((B, Hq, L, D), 3 + L, dtype)
                k1, v1 = seeded((B, Hkv, L, D), 4 + L, dtype), seeded((B, Hkv, L, D), 5 + L, dtype)
                ref = orc.attention_with_cache_update(to_oracle(q), to_oracle(k1), to_oracle(v1), o, scale, mask)
                if mode == "peer":
                    out = comm.symm_empty((B, Hq, L, D), dtype, dev)
                else:
                    out = torch.empty((B, Hq, L, D), dtype=dtype, device=dev)
                out.zero_()
                torch.cuda.synchronize()
                dist.barrier()      # every rank has cleared its buffer before anyone pushes into it
                n0 = kvc.launch_count(reset=True)
                comm.attention_sharded(g, shard(q, Hq), shard(k1, Hkv), shard(v1, Hkv), scale, out, mask=mask,
                                       shard_axis=axis)
                torch.cuda.synchronize()
                diff = max_abs_diff(out, ref)
                if not diff <= TOL[dtype]:
                    failures.append(f"{kind} {dtype} axis {axis} {mode} L {L}: max abs diff {diff}")
    status = kvc.lib().kvc_device_status()
    if status != 0:
        failures.append(f"device status {status}")

    # ---- the arrival wait runs out: the last rank withholds one exchange ----
    B, Hq, Hkv, D = 2, 4 * world, world, 64
    g = kvc.KVCacheSimple()
    kk = seeded((B, Hkv, 40, D), 50, torch.bfloat16)
    g.update(kk[:, rank:rank + 1].contiguous().to(dev), kk[:, rank:rank + 1].contiguous().to(dev))
    out = comm.symm_empty((B, Hq, 1, D), torch.bfloat16, dev)
    q = seeded((B, Hq, 1, D), 51, torch.bfloat16)[:, rank * 4:(rank + 1) * 4].contiguous().to(dev)
    k1 = seeded((B, Hkv, 1, D), 52, torch.bfloat16)[:, rank:rank + 1].contiguous().to(dev)
    comm.set_wait_limit(1 << 14)                 # about a millisecond
    torch.cuda.synchronize()
    dist.barrier()
    withheld = rank == world - 1
    if not withheld:
        comm.attention_sharded(g, q, k1, k1, D ** -0.5, out, shard_axis=1)
        torch.cuda.synchronize()
        if kvc.lib().kvc_device_status() != 41:
            failures.append(f"expected status 41 after a withheld exchange, got {kvc.lib().kvc_device_status()}")
    dist.barrier()
    if withheld:
        comm.attention_sharded(g, q, k1, k1, D ** -0.5, out, shard_axis=1)   # the late exchange: everyone else has pushed
        torch.cuda.synchronize()
        if kvc.lib().kvc_device_status() != 0:
            failures.append(f"the late rank should not time out, status {kvc.lib().kvc_device_status()}")
    kvc.device_status_reset()
    comm.set_wait_limit(1 << 26)
    dist.barrier()
    # counters are level again: one more exchange works on every rank
    comm.attention_sharded(g, q, k1, k1, D ** -0.5, out, shard_axis=1)
    torch.cuda.synchronize()
    if kvc.lib().kvc_device_status() != 0:
        failures.append(f"status {kvc.lib().kvc_device_status()} after the counters were levelled")

    flag = torch.tensor([len(failures)], device=dev)
    dist.all_reduce(flag)
    dist.barrier()
    del comm
    dist.destroy_process_group()
    for f in failures:
        print(f"rank {rank}: {f}", flush=True)
    if rank == 0:
        print("SHARDED_PARITY_OK" if int(flag.item()) == 0 else "SHARDED_PARITY_FAILED", flush=True)
    sys.exit(0 if int(flag.item()) == 0 else 1)


if __name__ == "__main__":
    main()
