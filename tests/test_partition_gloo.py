"""Host logic of the N>1 bench path on CPU: two gloo ranks partition a workload,
run the oracle on their shard, and reassemble / reduce the way bench.py does."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))

import bench  # noqa: E402

W = dict(kind="simple", layers=2, Hq=8, Hkv=4, D=64, B=2, dtype="f32", context=37, chunk=16)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def test_partition_covers_every_unit_once():
    for world in (1, 2, 4):
        for mode in ("sequences", "heads"):
            p = bench.partition(W, world, mode)
            units_local = p["B_local"] * p["Hkv_local"]
            if world == 1 or mode == "sequences":
                assert p["B_global"] == W["B"] * world and not p["collective"] and p["scaling"] == "weak"
                assert units_local == W["B"] * W["Hkv"]
            else:
                assert p["collective"] and p["scaling"] == "strong" and p["B_global"] == W["B"]
                assert units_local * world == W["B"] * W["Hkv"]
            assert p["Hq_local"] * W["Hkv"] == p["Hkv_local"] * W["Hq"]
    odd = dict(W, Hkv=3, Hq=6)
    assert bench.partition(odd, 2, "heads")["shard_axis"] == 0      # falls back to the batch
    # neither the heads nor the batch divide: every rank keeps whole sequences, nothing is exchanged
    none = bench.partition(dict(odd, B=3), 2, "heads")
    assert not none["collective"] and none["scaling"] == "weak" and none["B_global"] == 6


def _rank_main(rank, world, port, mode, q_out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import kvcache_oracle as orc
    orc.build()
    B, Hq, Hkv, D, T = W["B"], W["Hq"], W["Hkv"], W["D"], W["context"]
    p = bench.partition(W, world, mode)
    scale = D ** -0.5
    if mode == "heads":
        rng = np.random.default_rng(7)          # every rank draws the same full problem
        q = rng.standard_normal((B, Hq, 1, D), dtype=np.float32)
        k = rng.standard_normal((B, Hkv, T, D), dtype=np.float32)
        v = rng.standard_normal((B, Hkv, T, D), dtype=np.float32)
        full = orc.attention(q, orc.RawSource(k), orc.RawSource(v), scale)
        h0, hq0 = rank * p["Hkv_local"], rank * p["Hq_local"]
        part = orc.attention(np.ascontiguousarray(q[:, hq0:hq0 + p["Hq_local"]]),
                             orc.RawSource(np.ascontiguousarray(k[:, h0:h0 + p["Hkv_local"]])),
                             orc.RawSource(np.ascontiguousarray(v[:, h0:h0 + p["Hkv_local"]])), scale)
        mine = torch.from_numpy(np.ascontiguousarray(part))
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        gathered = torch.cat(parts, dim=p["shard_axis"]).numpy()
        ok = bool(np.array_equal(gathered, np.asarray(full)))
    else:
        rng = np.random.default_rng(100 + rank)  # every rank serves its own sequences
        q = rng.standard_normal((p["B_local"], Hq, 1, D), dtype=np.float32)
        k = rng.standard_normal((p["B_local"], Hkv, T, D), dtype=np.float32)
        v = rng.standard_normal((p["B_local"], Hkv, T, D), dtype=np.float32)
        out = orc.attention(q, orc.RawSource(k), orc.RawSource(v), scale)
        ok = bool(np.isfinite(np.asarray(out)).all()) and p["B_global"] == B * world
    # the timing reduction bench.py uses: max over ranks
    t = torch.tensor([1.0 + rank], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ok = ok and float(t.item()) == float(world)
    dist.barrier()
    dist.destroy_process_group()
    q_out.put((rank, ok))


@pytest.mark.parametrize("mode", ["sequences", "heads"])
def test_two_gloo_ranks(mode):
    world = 2
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, mode, q_out)) for r in range(world)]
    for pr in procs:
        pr.start()
    results = [q_out.get(timeout=120) for _ in range(world)]
    for pr in procs:
        pr.join(timeout=60)
        assert pr.exitcode == 0
    assert sorted(results) == [(0, True), (1, True)]
