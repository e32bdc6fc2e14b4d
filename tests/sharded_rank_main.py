"""One rank of the multi-GPU sharded-attention parity check (launched by
test_gpu_sharded.py through torch.distributed.run, one process per GPU).

Every rank draws the same full problem, keeps its shard of the KV heads (or of
the batch) in its own cache, runs kvc_attention_sharded, and compares the
gathered output with the oracle's attention over the full problem."""
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
    ]
    for kind, dtype, B, Hq, Hkv, D, P, axis in cases:
        k = seeded((B, Hkv, P, D), 1, dtype)
        v = seeded((B, Hkv, P, D), 2, dtype)
        q = seeded((B, Hq, 1, D), 3, dtype)
        k1, v1 = seeded((B, Hkv, 1, D), 4, dtype), seeded((B, Hkv, 1, D), 5, dtype)
        scale = D ** -0.5
        if kind == "simple":
            g, o = kvc.KVCacheSimple(), orc.KVCacheSimple()
            o.update(to_oracle(k), to_oracle(v))
        else:
            g, o = kvc.QuantizedKVCache(64, 4), orc.QuantizedKVCache(64, 4)
            o.update_quantized(to_oracle(k), to_oracle(v))
        ref = orc.attention_with_cache_update(to_oracle(q), to_oracle(k1), to_oracle(v1), o, scale)

        def shard(t, heads):
            if axis == 1:
                n = heads // world
                return t[:, rank * n:(rank + 1) * n].contiguous().to(dev)
            n = B // world
            return t[rank * n:(rank + 1) * n].contiguous().to(dev)

        if kind == "simple":
            g.update(shard(k, Hkv), shard(v, Hkv))
        else:
            g.update_quantized(shard(k, Hkv), shard(v, Hkv))
        out = torch.empty((B, Hq, 1, D), dtype=dtype, device=dev)
        comm.attention_sharded(g, shard(q, Hq), shard(k1, Hkv), shard(v1, Hkv), scale, out, shard_axis=axis)
        torch.cuda.synchronize()
        diff = max_abs_diff(out, ref)
        if not diff <= TOL[dtype]:
            failures.append(f"{kind} {dtype} axis {axis}: max abs diff {diff}")
    status = kvc.lib().kvc_device_status()
    if status != 0:
        failures.append(f"device status {status}")
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
