"""Shared helpers for the parity tests: seeded inputs and torch<->oracle storage."""
import numpy as np
import torch


def seeded(shape, seed, dtype=torch.float32, outlier_frac=0.0, outlier_scale=20.0):
    """~N(0,1) from a fixed-seed Philox stream on the host, cast to `dtype`."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    x = torch.randn(shape, generator=g, dtype=torch.float32)
    if outlier_frac > 0:
        D = shape[-1]
        n = max(1, int(round(D * outlier_frac)))
        idx = torch.randperm(D, generator=g)[:n]
        x[..., idx] *= outlier_scale
    return x.to(dtype)


def to_oracle(t: torch.Tensor) -> np.ndarray:
    """torch tensor -> oracle storage (float32 / float16 arrays, uint16 bit patterns for bf16)."""
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16).copy()
    if t.dtype in (torch.int32,):
        return t.numpy().view(np.uint32).copy()
    if t.dtype == torch.bool:
        return t.numpy().copy()
    return t.numpy().copy()


def from_oracle(a: np.ndarray, dtype) -> torch.Tensor:
    if dtype == torch.bfloat16:
        return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)
    return torch.from_numpy(np.ascontiguousarray(a))


def oracle_f32(a: np.ndarray) -> np.ndarray:
    if a.dtype == np.uint16:
        return (a.astype(np.uint32) << 16).view(np.float32)
    return a.astype(np.float32)


def max_abs_diff(gpu: torch.Tensor, ref: np.ndarray) -> float:
    g = gpu.detach().float().cpu().numpy()
    return float(np.max(np.abs(g - oracle_f32(ref)))) if g.size else 0.0


def bits_equal(gpu: torch.Tensor, ref: np.ndarray) -> bool:
    """Bit-exact comparison of a device tensor with oracle storage."""
    g = to_oracle(gpu)
    if g.dtype != ref.dtype:
        ref = ref.view(g.dtype) if ref.itemsize == g.itemsize else ref.astype(g.dtype)
    return g.shape == ref.shape and bool(np.array_equal(g.view(np.uint8) if g.dtype.kind == "f" else g,
                                                         np.ascontiguousarray(ref).view(np.uint8) if ref.dtype.kind == "f" else ref))


TOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2, torch.float16: 2e-2}
