"""kvc_sdpa_noalloc, the entry point for hosts that cannot let a library allocate
device memory on their request path (their own pool owns the GPU's budget, or
the device-wide stall of cudaMalloc/cudaFree is unacceptable mid-decode).

It must give the same attention output as kvc_sdpa while taking its split-K
scratch from a fixed array inside the library instead of a grown arena. The
array is shared by all calls and keeps whatever the previous call left in it,
so the check runs two different calls back to back: the second one would go
wrong if stale partials leaked. This file sorts last on purpose, so a run that
stops at the first failure has already executed every other test; it also
passes when run alone in a fresh process.
"""
import pytest
import torch

from helpers import TOL, max_abs_diff, seeded, to_oracle

pytestmark = pytest.mark.gpu


def _pair(kvc, cuda, dtype, B, Hq, Hkv, L, T, D, seed, mask):
    q = seeded((B, Hq, L, D), seed, dtype).to(cuda)
    k = seeded((B, Hkv, T, D), seed + 1, dtype).to(cuda)
    v = seeded((B, Hkv, T, D), seed + 2, dtype).to(cuda)
    out = torch.empty_like(q)  # the caller brings inputs and outputs
    got = kvc.scaled_dot_product_attention_noalloc(q, k, v, D ** -0.5, mask, out=out)
    want = kvc.scaled_dot_product_attention(q, k, v, D ** -0.5, mask)
    return got, want


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_no_alloc_entry_point_matches_the_regular_one_twice_in_a_row(kvc, cuda, dtype):
    # first call: decode shape, many splits -> fills a large part of the array
    got, want = _pair(kvc, cuda, dtype, B=2, Hq=8, Hkv=2, L=1, T=3000, D=128, seed=1, mask="none")
    assert float((got.float() - want.float()).abs().max()) <= TOL[dtype]
    # second call straight after: other shape, fewer and shorter splits, causal chunk
    got, want = _pair(kvc, cuda, dtype, B=1, Hq=4, Hkv=4, L=6, T=70, D=64, seed=7, mask="causal")
    assert float((got.float() - want.float()).abs().max()) <= TOL[dtype]
    # and the first shape again, with new data
    got, want = _pair(kvc, cuda, dtype, B=2, Hq=8, Hkv=2, L=1, T=2999, D=128, seed=11, mask="none")
    assert float((got.float() - want.float()).abs().max()) <= TOL[dtype]
    torch.cuda.synchronize()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_no_alloc_entry_point_matches_the_oracle(kvc, oracle, cuda, dtype):
    """The same two-calls-in-a-row pattern against the CPU oracle (not only against the library's
    other entry point, which shares its authors)."""
    for B, Hq, Hkv, L, T, D, seed, mask in ((2, 8, 2, 1, 1500, 128, 21, "none"), (1, 4, 2, 5, 90, 64, 27, "causal")):
        q, k, v = seeded((B, Hq, L, D), seed, dtype), seeded((B, Hkv, T, D), seed + 1, dtype), seeded((B, Hkv, T, D), seed + 2, dtype)
        dq, dk, dv = q.to(cuda), k.to(cuda), v.to(cuda)
        got = kvc.scaled_dot_product_attention_noalloc(dq, dk, dv, D ** -0.5, mask, out=torch.empty_like(dq))
        ref = oracle.sdpa(to_oracle(q), to_oracle(k), to_oracle(v), D ** -0.5, mask)
        assert max_abs_diff(got, ref) <= TOL[dtype]


def test_no_alloc_entry_point_allocates_nothing(kvc, cuda):
    """What the name promises: with inputs and output already on the device and one warm-up call
    behind it (the first call on a device looks up the address of the fixed array), further calls
    change neither the driver's free-memory figure nor the memory PyTorch's allocator holds."""
    q = seeded((2, 8, 1, 128), 31, torch.bfloat16).to(cuda)
    k = seeded((2, 2, 2500, 128), 32, torch.bfloat16).to(cuda)
    v = seeded((2, 2, 2500, 128), 33, torch.bfloat16).to(cuda)
    out = torch.empty_like(q)
    kvc.scaled_dot_product_attention_noalloc(q, k, v, 0.09, out=out)     # warm-up: symbol lookup
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    held0, reserved0 = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    for _ in range(5):
        kvc.scaled_dot_product_attention_noalloc(q, k, v, 0.09, out=out)
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, "the driver's free memory moved during no-alloc calls"
    assert torch.cuda.memory_allocated() == held0 and torch.cuda.memory_reserved() == reserved0


def test_no_alloc_entry_point_rejects_what_does_not_fit(kvc, cuda):
    # B*Hq*L*(4*D+8) bytes of partials for a single split already exceed the 4 MiB array
    q = torch.zeros((16, 64, 8, 256), dtype=torch.bfloat16, device=cuda)
    k = torch.zeros((16, 8, 4, 256), dtype=torch.bfloat16, device=cuda)
    with pytest.raises(kvc.KVCError) as e:
        kvc.scaled_dot_product_attention_noalloc(q, k, k, 1.0, out=torch.empty_like(q))
    assert e.value.status == kvc.ERR_INVALID_ARG and "static scratch" in e.value.message
    # an array mask is not offered by this variant
    small = torch.zeros((1, 2, 1, 64), dtype=torch.bfloat16, device=cuda)
    with pytest.raises(kvc.KVCError):
        kvc.scaled_dot_product_attention_noalloc(small, small, small, 1.0, torch.ones((1, 1), dtype=torch.bool, device=cuda),
                                                 out=torch.empty_like(small))
