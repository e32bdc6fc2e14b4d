"""CPU oracle for the KV-cache hot path of mlx-swift-lm.

TEST INFRASTRUCTURE ONLY. This module restates, with numpy arrays, the cache
classes of Libraries/MLXLMCommon (KVCache.swift, TurboQuantKVCache.swift,
RotatingStagedKVCache.swift, KVCacheRound.swift) operation by operation --
slices, concatenations and index bookkeeping exactly as the Swift code performs
them -- and wraps the C arithmetic in kvc_oracle.c (affine quantiser,
Walsh-Hadamard encode, attention). Tests compare the CUDA library with it; the
benchmark times it as the CPU baseline. Nothing in the shipped package imports
it.

Element storage: float32 arrays hold f32 data, float16 arrays hold f16 data and
uint16 arrays hold the raw bit patterns of bf16 data (numpy has no bfloat16).
Cache bookkeeping is pure data movement, so the storage type never matters to
it.

Parity status: state machines / packing / WHT encode / attention follow code in
the reference tree and are pinned by the reference's own test expectations
(tests/test_oracle_pins.py). The affine quantiser follows MLX's published
algorithm (un-vendored dependency mlx-swift 0.31.x): parity unpinned. The sign
vector generator is this project's own.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libkvc_oracle.so")

F32, F16, BF16 = 0, 1, 2


def build(force: bool = False) -> str:
    """Compile kvc_oracle.c with the Makefile beside it."""
    src = os.path.join(_HERE, "kvc_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.orc_packed_width.restype = ctypes.c_int
        _lib.orc_num_threads.restype = ctypes.c_int
    return _lib


def _p(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


# ---------------------------------------------------------------------------
# dtype helpers
# ---------------------------------------------------------------------------

def dtype_code(a: np.ndarray) -> int:
    if a.dtype == np.float32:
        return F32
    if a.dtype == np.float16:
        return F16
    if a.dtype == np.uint16:
        return BF16
    raise TypeError(f"unsupported storage dtype {a.dtype}")


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bfloat16 bit patterns (uint16)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = u + 0x7FFF + ((u >> 16) & 1)
    return (u >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def to_f32(a: np.ndarray) -> np.ndarray:
    if a.dtype == np.uint16:
        return bf16_bits_to_f32(a)
    return a.astype(np.float32)


def from_f32(x: np.ndarray, code: int) -> np.ndarray:
    if code == F32:
        return np.ascontiguousarray(x, dtype=np.float32)
    if code == F16:
        return np.ascontiguousarray(x, dtype=np.float32).astype(np.float16)
    return f32_to_bf16_bits(x)


# ---------------------------------------------------------------------------
# arithmetic (C)
# ---------------------------------------------------------------------------

def affine_quantize(x: np.ndarray, group_size: int, bits: int):
    """MLX `quantized(x, groupSize:, bits:)`, affine mode, over the last axis.

    Returns (codes uint32 [..., D*bits/32], scales [..., D/g], biases [..., D/g])
    with scales/biases in x's storage dtype.
    """
    x = np.ascontiguousarray(x)
    D = x.shape[-1]
    rows = int(np.prod(x.shape[:-1], dtype=np.int64))
    codes = np.zeros(x.shape[:-1] + (D * bits // 32,), dtype=np.uint32)
    scales = np.zeros(x.shape[:-1] + (D // group_size,), dtype=x.dtype)
    biases = np.zeros_like(scales)
    if rows:
        lib().orc_affine_quantize(_p(x), dtype_code(x), ctypes.c_int64(rows), D, group_size, bits,
                                  _p(codes), _p(scales), _p(biases))
    return codes, scales, biases


def affine_dequantize(codes, scales, biases, group_size: int, bits: int) -> np.ndarray:
    codes = np.ascontiguousarray(codes)
    scales = np.ascontiguousarray(scales)
    biases = np.ascontiguousarray(biases)
    D = codes.shape[-1] * 32 // bits
    rows = int(np.prod(codes.shape[:-1], dtype=np.int64))
    out = np.zeros(codes.shape[:-1] + (D,), dtype=scales.dtype)
    if rows:
        lib().orc_affine_dequantize(_p(codes), _p(scales), _p(biases), dtype_code(scales),
                                    ctypes.c_int64(rows), D, group_size, bits, _p(out))
    return out


def packed_width(count: int, bits: int) -> int:
    return int(lib().orc_packed_width(count, bits))


def pack_low_bit(idx: np.ndarray, bits: int) -> np.ndarray:
    idx = np.ascontiguousarray(idx, dtype=np.uint32)
    count = idx.shape[-1]
    rows = int(np.prod(idx.shape[:-1], dtype=np.int64))
    out = np.zeros(idx.shape[:-1] + (packed_width(count, bits),), dtype=np.uint32)
    lib().orc_pack(_p(idx), ctypes.c_int64(rows), count, bits, _p(out))
    return out


def unpack_low_bit(packed: np.ndarray, bits: int, count: int) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint32)
    rows = int(np.prod(packed.shape[:-1], dtype=np.int64))
    out = np.zeros(packed.shape[:-1] + (count,), dtype=np.uint32)
    lib().orc_unpack(_p(packed), ctypes.c_int64(rows), count, bits, _p(out))
    return out


def fwht(x: np.ndarray) -> np.ndarray:
    """Unnormalised Walsh-Hadamard transform over the last axis (float32)."""
    y = np.ascontiguousarray(x, dtype=np.float32).copy()
    D = y.shape[-1]
    lib().orc_fwht(_p(y), ctypes.c_int64(y.size // D), D)
    return y


def generate_centroids(dim: int, bits: int) -> np.ndarray:
    """TurboQuantCodebook.generateCentroids (TurboQuantKVCache.swift:174-233)."""
    out = np.zeros(1 << bits, dtype=np.float32)
    lib().orc_codebook(dim, bits, _p(out))
    return out


_SHIPPED_CENTROIDS = None


def shipped_centroids() -> dict:
    """The centroid table the reference ships as data (TurboQuantKVCache.swift:57-94), read from the
    fixture that tests/golden/make_golden.py parsed out of the Swift source."""
    global _SHIPPED_CENTROIDS
    if _SHIPPED_CENTROIDS is None:
        import json
        path = os.path.join(_HERE, "..", "tests", "golden", "turbo_codebooks.json")
        raw = json.load(open(path))["centroids"]
        _SHIPPED_CENTROIDS = {(int(d), int(b)): np.array(v, dtype=np.float32)
                              for d, per in raw.items() for b, v in per.items()}
    return _SHIPPED_CENTROIDS


def codebook(dim: int, bits: int) -> np.ndarray:
    """TurboQuantCodebook.codebook(dim:bits:) (:130-147): the shipped table first, else the generator."""
    table = shipped_centroids()
    if (dim, bits) in table:
        return table[(dim, bits)].copy()
    return generate_centroids(dim, bits)


def boundaries_of(centroids: np.ndarray) -> np.ndarray:
    c = np.asarray(centroids, dtype=np.float32)
    return ((c[:-1] + c[1:]) / np.float32(2.0)).astype(np.float32)


def wht_signs(dim: int, seed: int) -> np.ndarray:
    """Seeded +-1 vector: splitmix64 stream, one draw per dimension, top bit -> +1."""
    mask = (1 << 64) - 1
    x = seed & mask
    out = np.zeros(dim, dtype=np.float32)
    for i in range(dim):
        x = (x + 0x9E3779B97F4A7C15) & mask
        z = x
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
        z = z ^ (z >> 31)
        out[i] = 1.0 if (z >> 63) else -1.0
    return out


def turbo_encode(x: np.ndarray, signs: np.ndarray, boundaries: np.ndarray, bits: int):
    """Fused WHT encode of rows [..., D] -> (packed uint32 [..., PW], raw norms float32 [...])."""
    x = np.ascontiguousarray(x)
    D = x.shape[-1]
    rows = int(np.prod(x.shape[:-1], dtype=np.int64))
    packed = np.zeros(x.shape[:-1] + (packed_width(D, bits),), dtype=np.uint32)
    norms = np.zeros(x.shape[:-1], dtype=np.float32)
    signs = np.ascontiguousarray(signs, dtype=np.float32)
    boundaries = np.ascontiguousarray(boundaries, dtype=np.float32)
    if rows:
        lib().orc_turbo_encode(_p(x), dtype_code(x), ctypes.c_int64(rows), D, _p(signs), _p(boundaries), bits,
                               _p(packed), _p(norms))
    return packed, norms


def turbo_encode_scaled(x: np.ndarray, signs: np.ndarray, boundaries: np.ndarray, centroids: np.ndarray,
                        scale: np.ndarray, bits: int):
    """Calibrated encode (fusedEncodeDispatchScaled, TurboQuantKVCache.swift:787-796): rotated / scale is
    quantised and the stored norm is corrected by the norm of the scaled reconstruction."""
    x = np.ascontiguousarray(x)
    D = x.shape[-1]
    rows = int(np.prod(x.shape[:-1], dtype=np.int64))
    packed = np.zeros(x.shape[:-1] + (packed_width(D, bits),), dtype=np.uint32)
    norms = np.zeros(x.shape[:-1], dtype=np.float32)
    signs = np.ascontiguousarray(signs, dtype=np.float32)
    boundaries = np.ascontiguousarray(boundaries, dtype=np.float32)
    centroids = np.ascontiguousarray(centroids, dtype=np.float32)
    scale = np.ascontiguousarray(scale, dtype=np.float32)
    if rows:
        lib().orc_turbo_encode_scaled(_p(x), dtype_code(x), ctypes.c_int64(rows), D, _p(signs), _p(boundaries),
                                      _p(centroids), _p(scale), bits, _p(packed), _p(norms))
    return packed, norms


def rotation_matrix(dim: int, seed: int) -> np.ndarray:
    """Seeded dense rotation for head dims that are not powers of two (TurboQuantRotation.rotationMatrix,
    TurboQuantKVCache.swift:246-259: QR of a Gaussian matrix, columns flipped by the signs of R's diagonal).
    The reference's draw comes from MLXRandom and MLX's QR (not reproducible here: parity unpinned); this
    project's own recipe is Box-Muller normals from the splitmix64 stream, row-major, and a double-precision QR."""
    mask = (1 << 64) - 1
    x = seed & mask
    n = dim * dim
    vals = np.zeros(n + 1, dtype=np.float64)

    def nxt():
        nonlocal x
        x = (x + 0x9E3779B97F4A7C15) & mask
        z = x
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
        z = z ^ (z >> 31)
        return ((z >> 11) + 0.5) / 9007199254740992.0

    for i in range(0, n, 2):
        u1, u2 = nxt(), nxt()
        r, t = np.sqrt(-2.0 * np.log(u1)), 6.283185307179586476925286766559 * u2
        vals[i], vals[i + 1] = r * np.cos(t), r * np.sin(t)
    a = vals[:n].reshape(dim, dim)
    qm, rm = np.linalg.qr(a)
    return (qm * np.sign(np.diag(rm))[None, :]).astype(np.float32)


def turbo_encode_dense(x: np.ndarray, rotation: np.ndarray, boundaries: np.ndarray, centroids: np.ndarray, bits: int,
                       scale: Optional[np.ndarray] = None):
    """Dense-rotation encode (fusedEncodeSource, TurboQuantKernels.swift:103-204): norm-corrected norms."""
    x = np.ascontiguousarray(x)
    D = x.shape[-1]
    rows = int(np.prod(x.shape[:-1], dtype=np.int64))
    packed = np.zeros(x.shape[:-1] + (packed_width(D, bits),), dtype=np.uint32)
    norms = np.zeros(x.shape[:-1], dtype=np.float32)
    rotation = np.ascontiguousarray(rotation, dtype=np.float32)
    boundaries = np.ascontiguousarray(boundaries, dtype=np.float32)
    centroids = np.ascontiguousarray(centroids, dtype=np.float32)
    sc = None if scale is None else np.ascontiguousarray(scale, dtype=np.float32)
    if rows:
        lib().orc_turbo_encode_dense(_p(x), dtype_code(x), ctypes.c_int64(rows), D, _p(rotation), _p(boundaries),
                                     _p(centroids), _p(sc), bits, _p(packed), _p(norms))
    return packed, norms


def key_calibration_scale(all_keys: np.ndarray, signs: Optional[np.ndarray], rotation: Optional[np.ndarray] = None) -> Optional[np.ndarray]:
    """computeKeyCalibrationScale (TurboQuantKVCache.swift:867-886): per-dimension standard deviation of the
    rotated unit keys pooled over (batch, head, token), divided by its mean over the dimensions, clamped to
    [0.25, 4]; None with fewer than 32 rows or when every dimension is within 10 % of 1.

    MLX's `std` reduction order is not available here, so the two moments are accumulated as fixed-point
    integers (exact, order-free) and turned into the population standard deviation in float64; the clamp
    and the deviation test follow the Swift lines in float32."""
    x = np.ascontiguousarray(all_keys)
    D = x.shape[-1]
    rows = int(np.prod(x.shape[:-1], dtype=np.int64))
    if rows < 32:
        return None
    sums = np.zeros(2 * D, dtype=np.int64)
    if rotation is not None:
        lib().orc_turbo_calib_sums_dense(_p(x), dtype_code(x), ctypes.c_int64(rows), D,
                                         _p(np.ascontiguousarray(rotation, dtype=np.float32)), _p(sums))
    else:
        lib().orc_turbo_calib_sums(_p(x), dtype_code(x), ctypes.c_int64(rows), D,
                                   _p(np.ascontiguousarray(signs, dtype=np.float32)), _p(sums))
    mean = sums[:D].astype(np.float64) / 1073741824.0 / float(rows)
    ex2 = sums[D:].astype(np.float64) / 68719476736.0 / float(rows)
    sd = np.sqrt(np.maximum(ex2 - mean * mean, 0.0)).astype(np.float32)
    mean_sd = np.float32(max(np.float32(np.sum(sd.astype(np.float64)) / float(D)), np.float32(1e-8)))
    clamped = np.minimum(np.maximum(sd / mean_sd, np.float32(0.25)), np.float32(4.0)).astype(np.float32)
    if not float(np.max(np.abs(clamped - np.float32(1.0)))) >= 0.1:
        return None
    return clamped


class _Source(ctypes.Structure):
    _fields_ = [("kind", ctypes.c_int32), ("dtype", ctypes.c_int32), ("data", ctypes.c_void_p),
                ("scales", ctypes.c_void_p), ("biases", ctypes.c_void_p), ("norms", ctypes.c_void_p),
                ("sb", ctypes.c_int64), ("sh", ctypes.c_int64), ("st", ctypes.c_int64),
                ("gsb", ctypes.c_int64), ("gsh", ctypes.c_int64), ("gst", ctypes.c_int64),
                ("bits", ctypes.c_int32), ("group", ctypes.c_int32), ("codebook", ctypes.c_float * 16)]


class _Attn(ctypes.Structure):
    _fields_ = [("q", ctypes.c_void_p), ("out", ctypes.c_void_p), ("q_dtype", ctypes.c_int32),
                ("B", ctypes.c_int32), ("Hq", ctypes.c_int32), ("Hkv", ctypes.c_int32),
                ("L", ctypes.c_int32), ("D", ctypes.c_int32), ("T", ctypes.c_int64),
                ("scale", ctypes.c_float), ("k", _Source), ("v", _Source),
                ("mask_mode", ctypes.c_int32), ("mask_dtype", ctypes.c_int32), ("mask", ctypes.c_void_p),
                ("msb", ctypes.c_int64), ("msh", ctypes.c_int64), ("msl", ctypes.c_int64), ("mst", ctypes.c_int64),
                ("causal_offset", ctypes.c_int64), ("q_signs", ctypes.c_void_p), ("q_calib", ctypes.c_void_p),
                ("o_signs", ctypes.c_void_p), ("precise", ctypes.c_int32),
                ("q_rot", ctypes.c_void_p), ("o_rot", ctypes.c_void_p)]


def _estrides(a: np.ndarray):
    return [s // a.itemsize for s in a.strides]


@dataclass
class RawSource:
    data: np.ndarray  # [B, H, T, D], last axis contiguous


@dataclass
class AffineSource:
    codes: np.ndarray   # [B, H, T, W] uint32
    scales: np.ndarray  # [B, H, T, D/g]
    biases: np.ndarray
    group_size: int
    bits: int


@dataclass
class TurboSource:
    packed: np.ndarray  # [B, H, T, PW] uint32
    norms: np.ndarray   # [B, H, T] float32
    codebook: np.ndarray
    bits: int


def _fill_source(dst: _Source, src, keep: list):
    if isinstance(src, RawSource):
        a = src.data
        assert a.strides[-1] == a.itemsize
        keep.append(a)
        dst.kind, dst.dtype, dst.data = 0, dtype_code(a), a.ctypes.data
        dst.sb, dst.sh, dst.st = _estrides(a)[:3]
    elif isinstance(src, AffineSource):
        c, s, b = src.codes, src.scales, src.biases
        assert c.strides[-1] == 4 and s.strides[-1] == s.itemsize and b.strides == s.strides
        keep.extend([c, s, b])
        dst.kind, dst.dtype, dst.data = 1, dtype_code(s), c.ctypes.data
        dst.scales, dst.biases = s.ctypes.data, b.ctypes.data
        dst.sb, dst.sh, dst.st = _estrides(c)[:3]
        dst.gsb, dst.gsh, dst.gst = _estrides(s)[:3]
        dst.bits, dst.group = src.bits, src.group_size
    else:
        p, n = src.packed, src.norms
        assert p.strides[-1] == 4 and n.dtype == np.float32
        keep.extend([p, n])
        dst.kind, dst.dtype, dst.data, dst.norms = 2, 0, p.ctypes.data, n.ctypes.data
        dst.sb, dst.sh, dst.st = _estrides(p)[:3]
        dst.gsb, dst.gsh, dst.gst = _estrides(n)[:3]
        dst.bits = src.bits
        for i, c in enumerate(np.asarray(src.codebook, dtype=np.float32)):
            dst.codebook[i] = float(c)


def attention(q: np.ndarray, k_src, v_src, scale: float, mask="none", *, q_signs=None, q_calib=None,
              o_signs=None, q_rot=None, o_rot=None, precise: bool = True) -> np.ndarray:
    """softmax(scale * q k^T + mask) v over any cache representation.

    q [B, Hq, L, D] in storage dtype; returns the same shape and dtype.
    mask: "none", "causal", or an array (bool keep-mask or additive floats)
    broadcastable to [B, Hq, L, T].
    """
    q = np.ascontiguousarray(q)
    B, Hq, L, D = q.shape
    a = _Attn()
    keep: list = [q]
    _fill_source(a.k, k_src, keep)
    _fill_source(a.v, v_src, keep)
    first = k_src.data if isinstance(k_src, RawSource) else (k_src.codes if isinstance(k_src, AffineSource) else k_src.packed)
    Hkv, T = first.shape[1], first.shape[2]
    out = np.zeros_like(q)
    a.q, a.out, a.q_dtype = q.ctypes.data, out.ctypes.data, dtype_code(q)
    a.B, a.Hq, a.Hkv, a.L, a.D, a.T = B, Hq, Hkv, L, D, T
    a.scale = scale
    a.precise = 1 if precise else 0
    if isinstance(mask, str):
        if mask == "causal":
            a.mask_mode, a.causal_offset = 1, T - L
        else:
            a.mask_mode = 0
    else:
        m = np.asarray(mask)
        if m.dtype == np.bool_:
            m = np.ascontiguousarray(np.broadcast_to(m, (B, Hq, L, T))).astype(np.uint8)
            a.mask_dtype = 4
        else:
            m = np.ascontiguousarray(np.broadcast_to(m.astype(np.float32), (B, Hq, L, T)))
            a.mask_dtype = 0
        keep.append(m)
        a.mask_mode, a.mask = 2, m.ctypes.data
        a.msb, a.msh, a.msl, a.mst = _estrides(m)
    for name, arr in (("q_signs", q_signs), ("q_calib", q_calib), ("o_signs", o_signs), ("q_rot", q_rot), ("o_rot", o_rot)):
        if arr is not None:
            arr = np.ascontiguousarray(arr, dtype=np.float32)
            keep.append(arr)
            setattr(a, name, arr.ctypes.data)
    lib().orc_attention(ctypes.byref(a))
    return out


def append_rows(src: np.ndarray, dst: np.ndarray, pos: int) -> None:
    """dst[:, :, pos:pos+S, :] = src with OpenMP (timed CPU baseline helper)."""
    B, H, S, W = src.shape
    lib().orc_append(_p(np.ascontiguousarray(src)), _p(dst), src.itemsize, B, H, S, W,
                     ctypes.c_int64(dst.shape[2]), ctypes.c_int64(pos))


def num_threads() -> int:
    return int(lib().orc_num_threads())


def use_all_host_threads() -> int:
    """Run the C kernels on every hardware thread this process may use, whatever OMP_NUM_THREADS says
    (torch.distributed.run exports OMP_NUM_THREADS=1 to its workers)."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().orc_set_num_threads(ctypes.c_int(n))
    return num_threads()


# ---------------------------------------------------------------------------
# masks (KVCache.swift:253-275)
# ---------------------------------------------------------------------------

def create_causal_mask(n: int, offset: int, window_size: Optional[int] = None, lengths=None) -> np.ndarray:
    """createCausalMask (KVCache.swift:253-275): [n, offset + n] bool, or [B, 1, n, offset + n] with `lengths`."""
    rinds = np.arange(offset + n, dtype=np.int32)
    linds = np.arange(offset, offset + n, dtype=np.int32) if offset != 0 else rinds
    linds = linds[:, None]
    rinds = rinds[None]
    mask = linds >= rinds
    if window_size is not None:
        mask = mask & (linds < rinds + window_size)
    if lengths is not None:
        ln = np.asarray(lengths, dtype=np.int32)[:, None, None, None]
        mask = mask & (rinds < ln)
    return mask


# ---------------------------------------------------------------------------
# cache state machines
# ---------------------------------------------------------------------------

def _zeros(shape, like: np.ndarray) -> np.ndarray:
    return np.zeros(shape, dtype=like.dtype)


class BaseKVCache:
    """BaseKVCache defaults (KVCache.swift:184-251)."""

    def __init__(self):
        self.offset = 0

    max_size: Optional[int] = None

    @property
    def is_trimmable(self) -> bool:
        return False

    def is_trimmable_after(self, positions: int) -> bool:
        return self.is_trimmable

    def trim(self, n: int) -> int:
        return 0

    @property
    def meta_state(self) -> List[str]:
        return [""]

    def make_mask(self, n: int, window_size: Optional[int] = None, return_array: bool = False):
        if n == 1:
            return "none"
        if return_array or (window_size is not None and n > window_size):
            return create_causal_mask(n, self.offset, window_size)
        return "causal"


class KVCacheSimple(BaseKVCache):
    """KVCacheSimple (KVCache.swift:391-538)."""

    def __init__(self, step: int = 256):
        super().__init__()
        self.keys: Optional[np.ndarray] = None
        self.values: Optional[np.ndarray] = None
        self.step = step

    def update(self, keys: np.ndarray, values: np.ndarray):
        previous = self.offset
        S = keys.shape[2]
        reset = (self.keys is None) or (previous + S > self.keys.shape[2])
        if reset:
            B, H, _, kd = keys.shape
            vd = values.shape[3]
            n_steps = (self.step + S - 1) // self.step
            new_k = _zeros((B, H, n_steps * self.step, kd), keys)
            new_v = _zeros((B, H, n_steps * self.step, vd), values)
            if self.keys is not None:
                ck, cv = self.keys, self.values
                if previous % self.step != 0:
                    ck, cv = ck[:, :, :previous], cv[:, :, :previous]
                self.keys = np.concatenate([ck, new_k], axis=2)
                self.values = np.concatenate([cv, new_v], axis=2)
            else:
                self.keys, self.values = new_k, new_v
        self.offset += S
        self.keys[:, :, previous:self.offset] = keys
        self.values[:, :, previous:self.offset] = values
        return self.keys[:, :, :self.offset], self.values[:, :, :self.offset]

    @property
    def state(self) -> List[np.ndarray]:
        if self.keys is None:
            return []
        return [self.keys[:, :, :self.offset], self.values[:, :, :self.offset]]

    @state.setter
    def state(self, arrays: Sequence[np.ndarray]):
        assert len(arrays) == 2
        self.keys, self.values = np.array(arrays[0]), np.array(arrays[1])
        self.offset = self.keys.shape[2]

    @property
    def is_trimmable(self) -> bool:
        return True

    def trim(self, n: int) -> int:
        t = min(self.offset, n)
        self.offset -= t
        return t

    def copy(self) -> "KVCacheSimple":
        new = KVCacheSimple(self.step)
        s = self.state
        if s:
            new.state = [a.copy() for a in s]
        return new

    def to_quantized(self, group_size: int = 64, bits: int = 4) -> "QuantizedKVCache":
        if self.keys is not None:
            ck, cv = self.keys[:, :, :self.offset], self.values[:, :, :self.offset]
            eff = resolved_group_size(group_size, ck.shape[3], cv.shape[3])
            if eff is None:
                raise ValueError("KV cache quantization requires head dimensions divisible by 32, 64 or 128")
            q = QuantizedKVCache(group_size=eff, bits=bits)
            q.offset = self.offset
            q.keys = affine_quantize(ck, eff, bits)
            q.values = affine_quantize(cv, eff, bits)
            return q
        q = QuantizedKVCache(group_size=group_size, bits=bits)
        q.offset = self.offset
        return q


class ChunkedKVCache(KVCacheSimple):
    """ChunkedKVCache (KVCache.swift:1213-1304): a KVCacheSimple whose front can be dropped."""

    def __init__(self, chunk_size: Optional[int] = None, step: int = 256):
        super().__init__(step)
        self.chunk_size = chunk_size
        self.start_position = 0

    def maybe_trim_front(self):
        if self.keys is None or self.chunk_size is None or self.keys.shape[2] < self.chunk_size:
            return
        self.start_position += self.keys.shape[2] - self.chunk_size
        self.keys = self.keys[:, :, -self.chunk_size:]
        self.values = self.values[:, :, -self.chunk_size:]

    def update(self, keys, values):
        prev = self.offset - self.start_position
        S = keys.shape[2]
        if self.keys is None or prev + S > self.keys.shape[2]:
            B, H, _, kd = keys.shape
            n_steps = (self.step + S - 1) // self.step
            new_k = _zeros((B, H, n_steps * self.step, kd), keys)
            new_v = _zeros((B, H, n_steps * self.step, values.shape[3]), values)
            if self.keys is not None:
                ck, cv = self.keys, self.values
                if prev % self.step != 0:
                    ck, cv = ck[:, :, :prev], cv[:, :, :prev]
                self.keys = np.concatenate([ck, new_k], axis=2)
                self.values = np.concatenate([cv, new_v], axis=2)
            else:
                self.keys, self.values = new_k, new_v
        self.offset += S
        end = self.offset - self.start_position
        self.keys[:, :, prev:end] = keys
        self.values[:, :, prev:end] = values
        return self.keys[:, :, :end], self.values[:, :, :end]

    def trim(self, n: int) -> int:
        t = min(self.offset - self.start_position, n)
        self.offset -= t
        return t

    @property
    def meta_state(self) -> List[str]:
        return ["None" if self.chunk_size is None else str(self.chunk_size), str(self.start_position)]

    @meta_state.setter
    def meta_state(self, m: Sequence[str]):
        assert len(m) == 2, "ChunkedKVCache metaState must have exactly 2 values"
        self.chunk_size = None if m[0] == "None" else int(m[0])
        self.start_position = int(m[1])

    def copy(self) -> "ChunkedKVCache":
        new = ChunkedKVCache(self.chunk_size, self.step)
        s = self.state
        if s:
            new.state = [a.copy() for a in s]
        new.meta_state = self.meta_state
        return new


class CacheList(BaseKVCache):
    """CacheList (KVCache.swift:1556-1726): a composite of child caches."""

    def __init__(self, *caches):
        super().__init__()
        self.caches = list(caches)

    def __getitem__(self, i):
        return self.caches[i]

    def update(self, keys, values):
        raise RuntimeError("CacheList should not use update(keys:values:) - use subscript access instead")

    @property
    def state(self) -> List[np.ndarray]:
        return [a for c in self.caches for a in c.state]

    @state.setter
    def state(self, arrays):
        lengths = [len(c.state) for c in self.caches]
        start = 0
        for c, n in zip(self.caches, lengths):
            c.state = list(arrays[start:start + n])
            start += n

    def copy(self) -> "CacheList":
        return CacheList(*[c.copy() for c in self.caches])

    @property
    def is_trimmable(self) -> bool:
        return self.is_trimmable_after(0)

    def is_trimmable_after(self, positions: int) -> bool:
        return all(c.is_trimmable_after(positions) for c in self.caches)

    def trim(self, n: int) -> int:
        result = 0
        for c in self.caches:
            result = c.trim(n)
        return result

    @property
    def meta_state(self) -> List[str]:
        out = [str(len(self.caches))]
        for c in self.caches:
            meta = list(c.meta_state)
            out += [class_name(c), str(len(c.state)), str(len(meta))] + meta
        return out


def class_name(cache) -> str:
    """cacheClassName (KVCache.swift:1739-1751)."""
    for cls, name in ((ChunkedKVCache, "ChunkedKVCache"), (RotatingKVCache, "RotatingKVCache"),
                      (QuantizedKVCache, "QuantizedKVCache"), (TurboQuantKVCache, "TurboQuantKVCache"),
                      (KVCacheSimple, "KVCache"), (CacheList, "CacheList")):
        if isinstance(cache, cls):
            return name
    return "KVCache"


class RotatingKVCache(BaseKVCache):
    """RotatingKVCache (KVCache.swift:541-900)."""

    def __init__(self, max_size: int, keep: int = 0, step: int = 256):
        super().__init__()
        self.keep = keep
        self.keys: Optional[np.ndarray] = None
        self.values: Optional[np.ndarray] = None
        self.max_cache_size = max_size
        self.step = step
        self.idx = 0
        self.origin = "modelNative"

    @property
    def max_size(self) -> int:  # type: ignore[override]
        return self.max_cache_size

    def _trim(self, trim_size: int, a: np.ndarray, append: Optional[np.ndarray] = None) -> np.ndarray:
        if trim_size > 0:
            parts = [a[:, :, :self.keep], a[:, :, trim_size + self.keep:]]
        else:
            parts = [a]
        if append is not None:
            parts.append(append)
        return np.concatenate(parts, axis=2)

    def _temporal_order(self, a: np.ndarray) -> np.ndarray:
        if self.idx == a.shape[2]:
            return a
        if self.idx < self.offset:
            return np.concatenate([a[:, :, :self.keep], a[:, :, self.idx:], a[:, :, self.keep:self.idx]], axis=2)
        return a[:, :, :self.idx]

    def logical_view(self, tail: int) -> Optional[Tuple[np.ndarray, np.ndarray]]:
        if self.keys is None:
            return None
        ok, ov = self._temporal_order(self.keys), self._temporal_order(self.values)
        available = ok.shape[2]
        requested = min(max(tail, 0), available)
        bound = max(requested, min(self.keep, available))
        trim_size = available - bound
        if trim_size <= 0:
            return ok, ov
        if self.keep == 0:
            return ok[:, :, trim_size:], ov[:, :, trim_size:]
        return self._trim(trim_size, ok), self._trim(trim_size, ov)

    def _update_concat(self, keys, values):
        if self.keys is None:
            self.keys, self.values = np.array(keys), np.array(values)
        else:
            self.keys = self._temporal_order(self.keys)
            self.values = self._temporal_order(self.values)
            self.idx = self.keys.shape[2]
            trim_size = self.idx - self.max_cache_size + 1
            self.keys = self._trim(trim_size, self.keys, keys)
            self.values = self._trim(trim_size, self.values, values)
        self.offset += keys.shape[2]
        self.idx = self.keys.shape[2]
        return self.keys, self.values

    def _update_in_place(self, keys, values):
        B, H, S, kd = keys.shape
        vd = values.shape[3]
        prev = self.offset
        if self.keys is None or (prev >= self.keys.shape[2] and self.keys.shape[2] < self.max_cache_size):
            new_size = min(self.step, self.max_cache_size - prev)
            new_k = _zeros((B, H, new_size, kd), keys)
            new_v = _zeros((B, H, new_size, vd), values)
            if self.keys is not None:
                self.keys = np.concatenate([self.keys, new_k], axis=2)
                self.values = np.concatenate([self.values, new_v], axis=2)
            else:
                self.keys, self.values = new_k, new_v
            self.idx = prev
        trim_size = self.keys.shape[2] - self.max_cache_size
        if trim_size > 0:
            self.keys = self._trim(trim_size, self.keys)
            self.values = self._trim(trim_size, self.values)
            self.idx = self.max_cache_size
        if self.idx == self.max_cache_size:
            self.idx = self.keep
        self.keys[:, :, self.idx:self.idx + S] = keys
        self.values[:, :, self.idx:self.idx + S] = values
        self.offset += S
        self.idx += S
        if self.offset < self.max_cache_size:
            return self.keys[:, :, :self.offset], self.values[:, :, :self.offset]
        return self.keys, self.values

    def update(self, keys, values):
        if keys.shape[2] == 1:
            return self._update_in_place(keys, values)
        return self._update_concat(keys, values)

    @property
    def state(self) -> List[np.ndarray]:
        if self.keys is None:
            return []
        if self.offset < self.keys.shape[2]:
            return [self.keys[:, :, :self.offset], self.values[:, :, :self.offset]]
        return [self.keys, self.values]

    @state.setter
    def state(self, arrays):
        assert len(arrays) == 2
        self.keys, self.values = np.array(arrays[0]), np.array(arrays[1])

    @property
    def meta_state(self) -> List[str]:
        return [str(self.keep), str(self.max_cache_size), str(self.step), str(self.offset), str(self.idx), self.origin]

    @meta_state.setter
    def meta_state(self, m: Sequence[str]):
        assert len(m) in (5, 6)
        self.keep, self.max_cache_size, self.step = int(m[0]), int(m[1]), int(m[2])
        self.offset, self.idx = int(m[3]), int(m[4])
        self.origin = m[5] if len(m) == 6 else "modelNative"

    @property
    def is_trimmable(self) -> bool:
        return self.is_trimmable_after(0)

    def is_trimmable_after(self, positions: int) -> bool:
        return self.offset + positions < self.max_cache_size

    def trim(self, n: int) -> int:
        t = min(self.offset, n)
        self.offset -= t
        self.idx -= t
        return t

    def make_mask(self, n: int, window_size: Optional[int] = None, return_array: bool = False):
        if n > 1:
            actual = window_size if window_size is not None else self.max_cache_size
            capped = min(self.max_cache_size - 1, self.offset)
            if capped + n > actual or return_array:
                return create_causal_mask(n, capped, actual)
            return "causal"
        if window_size is None:
            return "none"
        if self.offset >= window_size and self.max_cache_size > window_size:
            cur = self.idx
            if cur >= self.max_cache_size:
                cur = 0
            size = self.offset + 1 if self.offset < self.max_cache_size else self.max_cache_size
            mask = np.arange(size) >= (size - window_size)
            return np.roll(mask, cur + 1)
        return "none"

    def copy(self) -> "RotatingKVCache":
        new = RotatingKVCache(self.max_cache_size, self.keep, self.step)
        s = self.state
        if s:
            new.state = [a.copy() for a in s]
        new.meta_state = self.meta_state
        return new


def resolved_group_size(requested: int, key_head_dim: int, value_head_dim: int) -> Optional[int]:
    """resolvedKVQuantizationGroupSize (KVCache.swift:902-920)."""
    requested = max(1, requested)
    compatible = [g for g in (32, 64, 128) if key_head_dim % g == 0 and value_head_dim % g == 0]
    if not compatible:
        return None
    return min(compatible, key=lambda g: (abs(g - requested), g))


class QuantizedKVCache(BaseKVCache):
    """QuantizedKVCache (KVCache.swift:923-1210)."""

    def __init__(self, group_size: int = 64, bits: int = 8):
        super().__init__()
        self.keys: Optional[Tuple[np.ndarray, np.ndarray, np.ndarray]] = None
        self.values: Optional[Tuple[np.ndarray, np.ndarray, np.ndarray]] = None
        self.step = 256
        self.group_size = group_size
        self.bits = bits

    def update_quantized(self, keys: np.ndarray, values: np.ndarray):
        B, H, S, kd = keys.shape
        vd = values.shape[3]
        prev = self.offset
        eff = resolved_group_size(self.group_size, kd, vd)
        if eff is not None and eff != self.group_size and self.keys is None and self.values is None and self.offset == 0:
            self.group_size = eff
        if eff is None:
            raise ValueError("KV cache quantization requires head dimensions divisible by 32, 64 or 128")
        if self.keys is None or (prev + S) > self.keys[0].shape[-2]:
            new_steps = ((self.step + S - 1) // self.step) * self.step
            if self.keys is not None:
                if prev % self.step != 0:
                    self.keys = tuple(a[:, :, :prev] for a in self.keys)
                    self.values = tuple(a[:, :, :prev] for a in self.values)

                def expand(t):
                    return tuple(np.concatenate([a, np.zeros((B, H, new_steps, a.shape[-1]), dtype=a.dtype)], axis=2)
                                 for a in t)
                self.keys, self.values = expand(self.keys), expand(self.values)
            else:
                def init(dim):
                    return affine_quantize(_zeros((B, H, new_steps, dim), keys), self.group_size, self.bits)
                self.keys, self.values = init(kd), init(vd)
        self.offset += S
        qk = affine_quantize(keys, self.group_size, self.bits)
        qv = affine_quantize(values, self.group_size, self.bits)
        for i in range(3):
            self.keys[i][:, :, prev:self.offset] = qk[i]
            self.values[i][:, :, prev:self.offset] = qv[i]
        return (tuple(a[:, :, :self.offset] for a in self.keys), tuple(a[:, :, :self.offset] for a in self.values))

    @property
    def state(self) -> List[np.ndarray]:
        if self.keys is None:
            return []
        return [a[:, :, :self.offset] for a in (*self.keys, *self.values)]

    @state.setter
    def state(self, arrays):
        assert len(arrays) == 6
        self.keys = tuple(np.array(a) for a in arrays[:3])
        self.values = tuple(np.array(a) for a in arrays[3:])

    @property
    def meta_state(self) -> List[str]:
        return [str(self.step), str(self.offset), str(self.group_size), str(self.bits)]

    @meta_state.setter
    def meta_state(self, m):
        assert len(m) == 4
        self.offset, self.group_size, self.bits = int(m[1]), int(m[2]), int(m[3])

    @property
    def is_trimmable(self) -> bool:
        return True

    def trim(self, n: int) -> int:
        t = min(self.offset, n)
        self.offset -= t
        return t

    def copy(self) -> "QuantizedKVCache":
        new = QuantizedKVCache(self.group_size, self.bits)
        s = self.state
        if s:
            new.state = [a.copy() for a in s]
        new.meta_state = self.meta_state
        return new

    def to_unquantized(self) -> KVCacheSimple:
        simple = KVCacheSimple()
        simple.offset = self.offset
        if self.keys is not None:
            k = tuple(a[:, :, :self.offset] for a in self.keys)
            v = tuple(a[:, :, :self.offset] for a in self.values)
            simple.state = [affine_dequantize(*k, self.group_size, self.bits),
                            affine_dequantize(*v, self.group_size, self.bits)]
        return simple


def quantized_sdpa(q, qkeys, qvalues, scale, mask="none", group_size=64, bits=8, precise=True):
    """quantizedScaledDotProductAttention (KVCache.swift:2351-2447)."""
    return attention(q, AffineSource(*qkeys, group_size, bits), AffineSource(*qvalues, group_size, bits),
                     scale, mask, precise=precise)


def sdpa(q, keys, values, scale, mask="none", precise=True):
    """MLXFast.scaledDotProductAttention as called from AttentionUtils.swift:86-93."""
    return attention(q, RawSource(keys), RawSource(values), scale, mask, precise=precise)


@dataclass
class MSECodec:
    """MSECodec, Walsh-Hadamard path (TurboQuantKVCache.swift:441-621)."""
    dim: int
    bits: int
    seed: int = 42
    codebook: np.ndarray = field(default=None)  # type: ignore[assignment]
    signs: np.ndarray = field(default=None)     # type: ignore[assignment]
    rotation: np.ndarray = field(default=None)  # type: ignore[assignment]  dense Pi [D, D], non-power-of-two dims

    def __post_init__(self):
        if self.codebook is None:
            self.codebook = codebook(self.dim, self.bits)
        # MSECodec.init (:459-486): Walsh-Hadamard for power-of-two dims up to 1024, dense otherwise
        self.use_wht = self.dim > 0 and (self.dim & (self.dim - 1)) == 0 and self.dim <= 1024
        if self.use_wht:
            if self.signs is None:
                self.signs = wht_signs(self.dim, self.seed)
            self.rotation = None
        else:
            if self.rotation is None:
                self.rotation = rotation_matrix(self.dim, self.seed)
            self.signs = None
        self.boundaries = boundaries_of(self.codebook)

    def encode(self, x: np.ndarray, scale: Optional[np.ndarray] = None):
        if not self.use_wht:
            return turbo_encode_dense(x, self.rotation, self.boundaries, self.codebook, self.bits, scale)
        if scale is not None:
            return turbo_encode_scaled(x, self.signs, self.boundaries, self.codebook, scale, self.bits)
        return turbo_encode(x, self.signs, self.boundaries, self.bits)

    def rotate(self, x_f32: np.ndarray) -> np.ndarray:
        """x . Pi^T = H(signs * x) / sqrt(D), or the dense product."""
        if not self.use_wht:
            return (x_f32.astype(np.float64) @ self.rotation.astype(np.float64).T).astype(np.float32)
        return fwht(x_f32 * self.signs) * np.float32(1.0 / np.sqrt(np.float32(self.dim)))

    def decode(self, packed: np.ndarray, norms: np.ndarray) -> np.ndarray:
        """MSECodec.decode (:573-588): codebook lookup, inverse rotation, norm rescale."""
        idx = unpack_low_bit(packed, self.bits, self.dim)
        approx = self.codebook[idx]
        if not self.use_wht:
            un = (approx.astype(np.float64) @ self.rotation.astype(np.float64)).astype(np.float32)
        else:
            un = fwht(approx) * np.float32(1.0 / np.sqrt(np.float32(self.dim))) * self.signs
        return norms[..., None] * un


class TurboQuantKVCache(BaseKVCache):
    """TurboQuantKVCache (TurboQuantKVCache.swift:633-1604), Walsh-Hadamard codecs.

    affine_values=True stores values as group-wise affine codes instead of
    codebook indices (the "values 4-bit affine" benchmark layout; not a mode of
    the reference class).
    """

    def __init__(self, bits: int = 4, key_bits: Optional[int] = None, value_bits: Optional[int] = None,
                 seed: int = 42, key_group_size: int = 64, affine_values: bool = False,
                 key_codebook=None, value_codebook=None):
        super().__init__()
        self.bits = bits
        self.key_bits = bits if key_bits is None else key_bits
        self.value_bits = bits if value_bits is None else value_bits
        self.raw_key_mode = self.key_bits == 0
        self.affine_key_mode = self.key_bits == 8
        self.affine_values = affine_values
        self.seed = seed
        self.key_group_size = key_group_size
        self.step = 256
        self.raw_keys = self.raw_values = None
        self.key_packed = self.key_norms = self.val_packed = self.val_norms = None
        self.aff_key = None
        self.aff_val = None
        self.is_compressed = False
        self.key_codec: Optional[MSECodec] = None
        self.value_codec: Optional[MSECodec] = None
        self.key_calib_scale: Optional[np.ndarray] = None
        self._kcb, self._vcb = key_codebook, value_codebook

    def _ensure_codecs(self, head_dim: int):
        if self.value_codec is not None or (self.affine_values and self.key_codec is not None):
            return
        if not self.raw_key_mode and not self.affine_key_mode and self.key_codec is None:
            self.key_codec = MSECodec(head_dim, self.key_bits, self.seed, codebook=self._kcb)
        if not self.affine_values:
            self.value_codec = MSECodec(head_dim, self.value_bits, self.seed + 1, codebook=self._vcb)

    # raw prefill phase (:802-846): identical to KVCacheSimple.update
    def update(self, keys, values):
        previous = self.offset
        S = keys.shape[2]
        reset = self.raw_keys is None or (previous + S > self.raw_keys.shape[2])
        if reset:
            B, H, _, kd = keys.shape
            n_steps = (self.step + S - 1) // self.step
            new_k = _zeros((B, H, n_steps * self.step, kd), keys)
            new_v = _zeros((B, H, n_steps * self.step, values.shape[3]), values)
            if self.raw_keys is not None:
                ck, cv = self.raw_keys, self.raw_values
                if previous % self.step != 0:
                    ck, cv = ck[:, :, :previous], cv[:, :, :previous]
                self.raw_keys = np.concatenate([ck, new_k], axis=2)
                self.raw_values = np.concatenate([cv, new_v], axis=2)
            else:
                self.raw_keys, self.raw_values = new_k, new_v
        self.offset += S
        self.raw_keys[:, :, previous:self.offset] = keys
        self.raw_values[:, :, previous:self.offset] = values
        return self.raw_keys[:, :, :self.offset], self.raw_values[:, :, :self.offset]

    def _grow(self, a: Optional[np.ndarray], need: int, shape_tail, dtype):
        B, H = shape_tail[0], shape_tail[1]
        rest = tuple(shape_tail[2:])
        if a is not None and a.shape[2] >= need:
            return a
        new_alloc = ((need + self.step - 1) // self.step) * self.step
        n = np.zeros((B, H, new_alloc) + rest, dtype=dtype)
        if a is not None:
            n[:, :, :a.shape[2]] = a
        return n

    def _encode_rows(self, keys, values, prev: int):
        B, H, S, D = keys.shape
        end = prev + S
        if self.affine_values:
            q = affine_quantize(values, self.key_group_size, self.value_bits)
            if self.aff_val is None:
                self.aff_val = [None, None, None]
            for i in range(3):
                self.aff_val[i] = self._grow(self.aff_val[i], end, (B, H, q[i].shape[-1]), q[i].dtype)
                self.aff_val[i][:, :, prev:end] = q[i]
        else:
            vp, vn = self.value_codec.encode(values)
            self.val_packed = self._grow(self.val_packed, end, (B, H, vp.shape[-1]), np.uint32)
            self.val_norms = self._grow(self.val_norms, end, (B, H), np.float32)
            self.val_packed[:, :, prev:end] = vp
            self.val_norms[:, :, prev:end] = vn
        if self.affine_key_mode:
            q = affine_quantize(keys, self.key_group_size, 8)
            if self.aff_key is None:
                self.aff_key = [None, None, None]
            for i in range(3):
                self.aff_key[i] = self._grow(self.aff_key[i], end, (B, H, q[i].shape[-1]), q[i].dtype)
                self.aff_key[i][:, :, prev:end] = q[i]
        elif self.raw_key_mode:
            self.raw_keys = self._grow(self.raw_keys, end, (B, H, D), keys.dtype)
            self.raw_keys[:, :, prev:end] = keys
        else:
            kp, kn = self.key_codec.encode(keys, self.key_calib_scale)
            self.key_packed = self._grow(self.key_packed, end, (B, H, kp.shape[-1]), np.uint32)
            self.key_norms = self._grow(self.key_norms, end, (B, H), np.float32)
            self.key_packed[:, :, prev:end] = kp
            self.key_norms[:, :, prev:end] = kn

    def _compress_raw(self):
        if self.is_compressed or self.raw_keys is None or self.offset <= 0:
            return
        ak, av = self.raw_keys[:, :, :self.offset], self.raw_values[:, :, :self.offset]
        self._ensure_codecs(ak.shape[-1])
        if self.affine_key_mode:
            self.key_group_size = resolved_group_size(self.key_group_size, ak.shape[-1], ak.shape[-1])
        keep_raw = self.raw_keys if self.raw_key_mode else None
        self.raw_keys = None if not self.raw_key_mode else keep_raw
        if not self.raw_key_mode and not self.affine_key_mode:
            # computed once from the whole raw key cache, reused by every later encode (:960-962)
            self.key_calib_scale = key_calibration_scale(ak, self.key_codec.signs, self.key_codec.rotation)
        self._encode_rows(ak, av, 0)
        self.raw_values = None
        self.is_compressed = True

    def encode_new_token(self, keys, values):
        """The cache-side half of compressedAttention (:1176-1200): compress a raw prefix if
        there is one (compressRawCache :895), then encode and append the new rows
        (encodeNewToken :1010-1147)."""
        D = keys.shape[-1]
        if not self.is_compressed:
            self._compress_raw()
        self._ensure_codecs(D)
        prev = self.offset
        self._encode_rows(keys, values, prev)
        self.offset = prev + keys.shape[2]
        self.is_compressed = True

    def compressed_attention(self, q, keys, values, scale, mask="none", precise=True):
        """compressedAttention (:1164-1446)."""
        L = q.shape[2]
        self.encode_new_token(keys, values)
        T = self.offset
        if isinstance(mask, str) and L == 1:
            mask = "none"
        kw = {}
        if self.raw_key_mode:
            ks = RawSource(self.raw_keys[:, :, :T])
        elif self.affine_key_mode:
            ks = AffineSource(*(a[:, :, :T] for a in self.aff_key), self.key_group_size, 8)
        else:
            ks = TurboSource(self.key_packed[:, :, :T], self.key_norms[:, :, :T], self.key_codec.codebook, self.key_bits)
            if self.key_codec.use_wht:
                kw["q_signs"] = self.key_codec.signs
            else:
                kw["q_rot"] = self.key_codec.rotation
            if self.key_calib_scale is not None:
                kw["q_calib"] = self.key_calib_scale    # folded into the rotated query (:1348-1352)
        if self.affine_values:
            vs = AffineSource(*(a[:, :, :T] for a in self.aff_val), self.key_group_size, self.value_bits)
        else:
            vs = TurboSource(self.val_packed[:, :, :T], self.val_norms[:, :, :T], self.value_codec.codebook, self.value_bits)
            if self.value_codec.use_wht:
                kw["o_signs"] = self.value_codec.signs
            else:
                kw["o_rot"] = self.value_codec.rotation
        return attention(q, ks, vs, scale, mask, precise=precise, **kw)

    @property
    def state(self) -> List[np.ndarray]:
        o = self.offset
        if self.is_compressed:
            if o <= 0:
                return []
            out = []
            if self.affine_key_mode:
                out += [a[:, :, :o] for a in self.aff_key]
            elif self.raw_key_mode:
                out += [self.raw_keys[:, :, :o]]
            else:
                out += [self.key_packed[:, :, :o], self.key_norms[:, :, :o]]
            if self.affine_values:
                out += [a[:, :, :o] for a in self.aff_val]
            else:
                out += [self.val_packed[:, :, :o], self.val_norms[:, :, :o]]
            if (self.key_calib_scale is not None and not self.affine_key_mode and not self.raw_key_mode
                    and not self.affine_values):
                out.append(self.key_calib_scale)        # fifth array of the standard state (:1509-1511)
            return out
        if self.raw_keys is None or o <= 0:
            return []
        return [self.raw_keys[:, :, :o], self.raw_values[:, :, :o]]

    @property
    def meta_state(self) -> List[str]:
        return [str(self.offset), str(self.bits), str(self.key_bits), str(self.value_bits), str(self.seed)]

    @property
    def is_trimmable(self) -> bool:
        return True

    def trim(self, n: int) -> int:
        if n <= 0 or self.offset <= 0:
            return 0
        t = min(n, self.offset)
        self.offset -= t
        if self.offset == 0:
            self.raw_keys = self.raw_values = None
            self.key_packed = self.key_norms = self.val_packed = self.val_norms = None
            self.aff_key = self.aff_val = None
            self.key_calib_scale = None
            self.is_compressed = False
        return t


def attention_with_cache_update(q, keys, values, cache, scale, mask="none", precise=True):
    """attentionWithCacheUpdate (AttentionUtils.swift:37-95)."""
    if isinstance(cache, TurboQuantKVCache):
        if q.shape[2] > 1 and not cache.is_compressed:
            ck, cv = cache.update(keys, values)
            return sdpa(q, ck, cv, scale, mask, precise)
        return cache.compressed_attention(q, keys, values, scale, mask, precise)
    if isinstance(cache, QuantizedKVCache):
        qk, qv = cache.update_quantized(keys, values)
        return quantized_sdpa(q, qk, qv, scale, mask, cache.group_size, cache.bits, precise)
    ck, cv = cache.update(keys, values)
    return sdpa(q, ck, cv, scale, mask, precise)


# ---------------------------------------------------------------------------
# staged rounds (RotatingStagedKVCache.swift, KVCacheRound.swift, KVCachePlan.swift:219-347)
# ---------------------------------------------------------------------------

def rope(x: np.ndarray, offset: int, dims: int, traditional: bool = False, base: float = 10000.0,
         scale: float = 1.0) -> np.ndarray:
    """applyRotaryPosition(rope, to: x, offset:) (MLXLMCommon/RoPEApplication.swift:58-69) for x [B, H, L, D] in
    storage dtype. The rotation is MLX's published RoPE (un-vendored mlx-swift: parity unpinned): pair i of a
    head at position p = offset + l turns by p * scale * base^(-2i/dims); pairs are (i, i + dims/2), or
    (2i, 2i+1) when `traditional`; features past `dims` pass through. Float32 arithmetic."""
    code = dtype_code(x)
    xf = to_f32(x).copy()
    B, H, L, D = xf.shape
    half = dims // 2
    inv_freq = np.exp2(-np.arange(half, dtype=np.float64) * (np.log2(np.float64(np.float32(base))) / half)).astype(np.float32)
    pos = (np.arange(L, dtype=np.float32) + np.float32(offset)) * np.float32(scale)
    theta = (pos[:, None] * inv_freq[None, :]).astype(np.float32)
    cs, sn = np.cos(theta).astype(np.float32), np.sin(theta).astype(np.float32)
    if traditional:
        x0, x1 = xf[..., 0:dims:2].copy(), xf[..., 1:dims:2].copy()
        xf[..., 0:dims:2] = x0 * cs - x1 * sn
        xf[..., 1:dims:2] = x0 * sn + x1 * cs
    else:
        x0, x1 = xf[..., :half].copy(), xf[..., half:dims].copy()
        xf[..., :half] = x0 * cs - x1 * sn
        xf[..., half:dims] = x0 * sn + x1 * cs
    return from_f32(xf, code)


def attention_rope(q, keys, values, cache, rope_cfg: dict, scale, mask="none", precise=True):
    """The attention block's cache step (MLXLLM/Models/Llama.swift:58-69): rotate q and k at the cache's
    ropeOffset (its offset; 0 without a cache), then attentionWithCacheUpdate."""
    offset = cache.offset if cache is not None else 0
    rq = rope(q, offset, **rope_cfg)
    rk = rope(keys, offset, **rope_cfg)
    if cache is None:
        return sdpa(rq, rk, values, scale, mask, precise=precise)
    return attention_with_cache_update(rq, rk, values, cache, scale, mask, precise=precise)


class StagedRound:
    """One cache's share of a speculative round."""

    def __init__(self, cache, max_positions: int):
        self.cache = cache
        self.rotating = isinstance(cache, RotatingKVCache)
        if not self.rotating and not cache.is_trimmable_after(max_positions):
            raise RuntimeError("round refused: cache could not be rewound")
        self.start_offset = cache.offset
        self.staged_k = self.staged_v = None
        self.restore = None

    @property
    def staged_count(self) -> int:
        return 0 if self.staged_k is None else self.staged_k.shape[2]

    @property
    def offset(self) -> int:
        return self.cache.offset + (self.staged_count if self.rotating else 0)

    def update(self, keys, values):
        if not self.rotating:
            return self.cache.update(keys, values)
        self.staged_k = keys if self.staged_k is None else np.concatenate([self.staged_k, keys], axis=2)
        self.staged_v = values if self.staged_v is None else np.concatenate([self.staged_v, values], axis=2)
        bound = min(self.cache.offset, self.cache.max_cache_size - 1)
        view = self.cache.logical_view(bound) if bound > 0 else None
        if view is None:
            return self.staged_k, self.staged_v
        return (np.concatenate([view[0], self.staged_k], axis=2), np.concatenate([view[1], self.staged_v], axis=2))

    def commit(self, retaining: int):
        c = self.cache
        if not self.rotating:
            written = c.offset - self.start_offset
            keep = min(max(retaining, 0), written)
            if written > keep:
                c.trim(written - keep)
            return None
        restore = None
        if not c.is_trimmable_after(retaining) and len(c.state) == 2:
            restore = {"state": [a.copy() for a in c.state], "meta": list(c.meta_state),
                       "replay": None if self.staged_k is None else (self.staged_k.copy(), self.staged_v.copy()),
                       "committed": retaining}
        if self.staged_k is not None:
            keep = min(max(retaining, 0), self.staged_k.shape[2])
            if keep > 0:
                c.update(self.staged_k[:, :, :keep], self.staged_v[:, :, :keep])
        self.staged_k = self.staged_v = None
        return restore


def rewind_last_round(cache, restore, count: int) -> int:
    """KVCacheStorage.rewindLastRound for one leaf."""
    if count <= 0:
        return 0
    if restore is None:
        if not cache.is_trimmable:
            return 0
        return cache.trim(count)
    rewound = min(count, restore["committed"])
    if rewound <= 0:
        return 0
    cache.state = restore["state"]
    cache.meta_state = restore["meta"]
    retaining = restore["committed"] - rewound
    if retaining > 0 and restore["replay"] is not None:
        cache.update(restore["replay"][0][:, :, :retaining], restore["replay"][1][:, :, :retaining])
    return rewound
