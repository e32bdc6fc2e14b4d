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


def store_ulp(x: np.ndarray, dtype) -> np.ndarray:
    """Spacing of `dtype` (bf16: 8 significand bits, f16: 11) at the magnitude of x; 0 for float32."""
    if dtype == torch.float32:
        return np.zeros_like(x, dtype=np.float32)
    sig = 8 if dtype == torch.bfloat16 else 11
    mag = np.maximum(np.abs(x.astype(np.float32)), np.float32(2.0 ** -14))
    return np.exp2(np.floor(np.log2(mag)) - (sig - 1)).astype(np.float32)


def worst_excess(gpu: torch.Tensor, ref: np.ndarray, dtype) -> float:
    """Largest amount by which |gpu - ref| exceeds the stated absolute tolerance plus the store rounding.

    The tolerance (2e-2 for bf16 / f16, 1e-4 for f32) bounds the error of the arithmetic. Both results are
    then rounded to `dtype`, which moves each of them by up to half a spacing: two results whose unrounded
    values differ by less than the tolerance may land one spacing further apart. Below magnitude 1 a bf16
    spacing (<= 2^-8) is well inside 2e-2 and was always absorbed by it; with x20 outlier channels outputs
    reach ~10, where one spacing is 2^-4, so the bound is stated per element: TOL + spacing(max(|gpu|, |ref|)).
    Returns <= 0 when every element is inside."""
    g = gpu.detach().float().cpu().numpy()
    r = oracle_f32(ref)
    bound = np.float32(TOL[dtype]) + store_ulp(np.maximum(np.abs(g), np.abs(r)), dtype)
    return float(np.max(np.abs(g - r) - bound)) if g.size else 0.0
