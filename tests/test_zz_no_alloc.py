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

from helpers import TOL, seeded

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
