"""ctypes binding of libkvcache_b200.so with the reference's names.

The classes mirror the cache classes of mlx-swift-lm's MLXLMCommon
(KVCacheSimple, RotatingKVCache, QuantizedKVCache, TurboQuantKVCache) and the
free functions attentionWithCacheUpdate / quantizedScaledDotProductAttention,
so that tests read like the reference's own. Every call goes through the C ABI
declared in include/kvcache_b200.h; torch only supplies device memory and
streams. There is no fallback: if the shared library is missing, importing this
package raises.
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional, Sequence, Tuple

_HERE = os.path.dirname(os.path.abspath(__file__))
_PKG = os.path.abspath(os.path.join(_HERE, "..", ".."))
LIB_PATH = os.path.join(_PKG, "lib", "libkvcache_b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python mlx-swift-lm_b200/build.py` "
        "(there is no CPU or PyTorch fallback for this library)")

_lib = ctypes.CDLL(LIB_PATH)

KVC_MAX_DIMS = 5
F32, F16, BF16, U32, BOOL = 0, 1, 2, 3, 4
KIND_SIMPLE, KIND_ROTATING, KIND_QUANTIZED, KIND_TURBO, KIND_CHUNKED, KIND_LIST = 0, 1, 2, 3, 4, 5
MASK_NONE, MASK_CAUSAL, MASK_ARRAY = 0, 1, 2

OK = 0
ERR_INTERNAL, ERR_INVALID_ARG, ERR_INVALID_STATE, ERR_UNSUPPORTED = -1, -2, -3, -4
ERR_CUDA, ERR_OOM, ERR_NOT_TRIMMABLE, ERR_TIMEOUT, ERR_COMM = -5, -6, -7, -8, -9


class KVCError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"[kvc {status}] {message}")
        self.status = status
        self.message = message


class Tensor(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("dtype", ctypes.c_int32), ("ndim", ctypes.c_int32),
                ("shape", ctypes.c_int64 * KVC_MAX_DIMS), ("stride", ctypes.c_int64 * KVC_MAX_DIMS)]


class Config(ctypes.Structure):
    _fields_ = [("kind", ctypes.c_int32), ("device", ctypes.c_int32), ("step", ctypes.c_int32),
                ("max_size", ctypes.c_int32), ("keep", ctypes.c_int32), ("group_size", ctypes.c_int32),
                ("bits", ctypes.c_int32), ("key_bits", ctypes.c_int32), ("value_bits", ctypes.c_int32),
                ("key_group_size", ctypes.c_int32), ("seed", ctypes.c_uint64),
                ("reserve_tokens", ctypes.c_int64), ("turbo_affine_values", ctypes.c_int32)]


_vp = ctypes.c_void_p
_TP = ctypes.POINTER(Tensor)

_lib.kvc_version.restype = ctypes.c_char_p
_lib.kvc_last_error_message.restype = ctypes.c_char_p
_lib.kvc_offset.restype = ctypes.c_int64
_lib.kvc_offset.argtypes = [_vp]
_lib.kvc_max_size.restype = ctypes.c_int64
_lib.kvc_max_size.argtypes = [_vp]
_lib.kvc_ring_index.restype = ctypes.c_int64
_lib.kvc_ring_index.argtypes = [_vp]
_lib.kvc_memory_bytes.restype = ctypes.c_int64
_lib.kvc_memory_bytes.argtypes = [_vp]
_lib.kvc_round_offset.restype = ctypes.c_int64
_lib.kvc_round_offset.argtypes = [_vp]
_lib.kvc_launch_count.restype = ctypes.c_int64
_lib.kvc_free.argtypes = [_vp]
_lib.kvc_free.restype = None
_lib.kvc_round_free.argtypes = [_vp]
_lib.kvc_round_free.restype = None
_lib.kvc_comm_free.argtypes = [_vp]
_lib.kvc_comm_free.restype = None
for _name in ("kvc_kind_of", "kvc_group_size", "kvc_bits", "kvc_is_compressed", "kvc_is_trimmable",
              "kvc_state_count"):
    getattr(_lib, _name).argtypes = [_vp]
_lib.kvc_is_trimmable_after.argtypes = [_vp, ctypes.c_int64]
_lib.kvc_set_offset.argtypes = [_vp, ctypes.c_int64]
_lib.kvc_attention.argtypes = [_vp, _TP, _TP, _TP, ctypes.c_float, ctypes.c_int32, _TP, _TP, _vp]
_lib.kvc_attention_host.argtypes = [_vp, _TP, _TP, _TP, ctypes.c_float, ctypes.c_int32, _TP, _TP, _vp,
                                    ctypes.c_int32]
_lib.kvc_round_attention.argtypes = [_vp, _TP, _TP, _TP, ctypes.c_float, ctypes.c_int32, _TP, _TP, _vp]
_lib.kvc_sdpa.argtypes = [_TP, _TP, _TP, ctypes.c_float, ctypes.c_int32, _TP, _TP, _vp]
_lib.kvc_sdpa_noalloc.argtypes = [_TP, _TP, _TP, ctypes.c_float, ctypes.c_int32, _TP, _vp]
_lib.kvc_quantized_sdpa.argtypes = [_TP, _TP, _TP, ctypes.c_float, ctypes.c_int32, _TP, ctypes.c_int32,
                                    ctypes.c_int32, _TP, _vp]
_lib.kvc_attention_sharded.argtypes = [_vp, _vp, _TP, _TP, _TP, ctypes.c_float, ctypes.c_int32, _TP, _TP,
                                       ctypes.c_int32, _vp]
_lib.kvc_update.argtypes = [_vp, _TP, _TP, _vp, _TP, _TP]
_lib.kvc_update_quantized.argtypes = [_vp, _TP, _TP, _vp, _TP, _TP]
_lib.kvc_round_update.argtypes = [_vp, _TP, _TP, _vp, _TP, _TP]
_lib.kvc_logical_view.argtypes = [_vp, ctypes.c_int64, _vp, _TP, _TP]
_lib.kvc_state_get.argtypes = [_vp, ctypes.c_int32, _TP]
_lib.kvc_state_set.argtypes = [_vp, _TP, ctypes.c_int32, _vp]
_lib.kvc_state_export.argtypes = [_vp, ctypes.c_int32, _vp, ctypes.c_size_t, _TP, _vp]
_lib.kvc_trim.argtypes = [_vp, ctypes.c_int64, ctypes.POINTER(ctypes.c_int64)]
_lib.kvc_reserve.argtypes = [_vp, ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                             ctypes.c_int32, _vp]
_lib.kvc_copy.argtypes = [_vp, _vp, ctypes.POINTER(_vp)]
_lib.kvc_to_quantized.argtypes = [_vp, ctypes.c_int32, ctypes.c_int32, _vp, ctypes.POINTER(_vp)]
_lib.kvc_to_unquantized.argtypes = [_vp, _vp, ctypes.POINTER(_vp)]
_lib.kvc_to_turbo.argtypes = [_vp, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, _vp, ctypes.POINTER(_vp)]
_lib.kvc_round_begin.argtypes = [_vp, ctypes.c_int32, ctypes.POINTER(_vp)]
_lib.kvc_round_commit.argtypes = [_vp, ctypes.c_int32, _vp]
_lib.kvc_round_rollback.argtypes = [_vp, _vp]
_lib.kvc_rewind_last_round.argtypes = [_vp, ctypes.c_int64, _vp, ctypes.POINTER(ctypes.c_int64)]
_lib.kvc_meta_state.argtypes = [_vp, ctypes.c_char_p, ctypes.c_size_t, ctypes.POINTER(ctypes.c_size_t)]
_lib.kvc_set_meta_state.argtypes = [_vp, ctypes.c_char_p]
_lib.kvc_make_mask.argtypes = [_vp, ctypes.c_int32, ctypes.c_int64, ctypes.c_int32,
                               ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int64),
                               ctypes.POINTER(ctypes.c_int64), _vp, _vp]
_lib.kvc_affine_quantize.argtypes = [_TP, ctypes.c_int32, ctypes.c_int32, _TP, _TP, _TP, _vp]
_lib.kvc_affine_dequantize.argtypes = [_TP, _TP, _TP, ctypes.c_int32, ctypes.c_int32, _TP, _vp]
_lib.kvc_save_prompt_cache.argtypes = [ctypes.c_char_p, ctypes.POINTER(_vp), ctypes.c_int32, ctypes.POINTER(ctypes.c_char_p),
                                       ctypes.POINTER(ctypes.c_char_p), ctypes.c_int32, _vp]
_lib.kvc_save_prompt_cache.restype = ctypes.c_int32
_lib.kvc_load_prompt_cache.argtypes = [ctypes.c_char_p, ctypes.c_int32, ctypes.POINTER(_vp), ctypes.c_int32,
                                       ctypes.POINTER(ctypes.c_int32), ctypes.c_char_p, ctypes.c_size_t,
                                       ctypes.POINTER(ctypes.c_size_t), _vp]
_lib.kvc_load_prompt_cache.restype = ctypes.c_int32
_lib.kvc_resolve_turbo_scheme.argtypes = [ctypes.c_char_p, ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int32)]
_lib.kvc_resolve_turbo_scheme.restype = ctypes.c_int32
_lib.kvc_resolve_affine_scheme.argtypes = [ctypes.c_char_p, ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int32)]
_lib.kvc_resolve_affine_scheme.restype = ctypes.c_int32
_lib.kvc_turbo_protected_layers.argtypes = [ctypes.POINTER(ctypes.c_int32), ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                                            ctypes.POINTER(ctypes.c_int32)]
_lib.kvc_turbo_protected_layers.restype = ctypes.c_int32
_lib.kvc_maybe_affine_quantize.argtypes = [ctypes.POINTER(_vp), ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_int64,
                                           _vp, ctypes.POINTER(ctypes.c_int32)]
_lib.kvc_maybe_affine_quantize.restype = ctypes.c_int32
_lib.kvc_maybe_turbo_quantize.argtypes = [ctypes.POINTER(_vp), ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_int64,
                                          _vp, ctypes.POINTER(ctypes.c_int32)]
_lib.kvc_maybe_turbo_quantize.restype = ctypes.c_int32
_lib.kvc_attention_varlen.argtypes = [ctypes.POINTER(_vp), ctypes.c_int32, _TP, _TP, _TP, ctypes.c_float, _TP, _vp]
_lib.kvc_attention_varlen.restype = ctypes.c_int32
_lib.kvc_turbo_encode_new_token.argtypes = [_vp, _TP, _TP, _vp]
_lib.kvc_turbo_encode_new_token.restype = ctypes.c_int32
_lib.kvc_turbo_encode.argtypes = [_TP, _vp, ctypes.POINTER(ctypes.c_float), ctypes.c_int32, _TP, _TP, _vp]
_lib.kvc_turbo_codebook.argtypes = [ctypes.c_int32, ctypes.c_int32, ctypes.POINTER(ctypes.c_float),
                                    ctypes.POINTER(ctypes.c_float)]
_lib.kvc_turbo_signs.argtypes = [ctypes.c_int32, ctypes.c_uint64, ctypes.POINTER(ctypes.c_float)]
_lib.kvc_turbo_set_codec.argtypes = [_vp] + [ctypes.POINTER(ctypes.c_float)] * 4 + [ctypes.c_int32]
_lib.kvc_trim_prompt_cache.argtypes = [ctypes.POINTER(_vp), ctypes.c_int32, ctypes.c_int64,
                                       ctypes.POINTER(ctypes.c_int64)]
_lib.kvc_can_trim_prompt_cache.argtypes = [ctypes.POINTER(_vp), ctypes.c_int32]
_lib.kvc_list_create.argtypes = [ctypes.POINTER(_vp), ctypes.c_int32, ctypes.POINTER(_vp)]
_lib.kvc_list_count.argtypes = [_vp]
_lib.kvc_list_child.argtypes = [_vp, ctypes.c_int32]
_lib.kvc_list_child.restype = _vp
_lib.kvc_maybe_trim_front.argtypes = [_vp, _vp]
_lib.kvc_start_position.argtypes = [_vp]
_lib.kvc_start_position.restype = ctypes.c_int64
_lib.kvc_prepare.argtypes = [_vp, ctypes.POINTER(ctypes.c_int32), ctypes.c_int32]
_lib.kvc_finalize.argtypes = [_vp]
_lib.kvc_create_causal_mask.argtypes = [ctypes.c_int32, ctypes.c_int64, ctypes.c_int64, _vp, ctypes.c_int32, _vp, _vp]
class RopeConfig(ctypes.Structure):
    _fields_ = [("dims", ctypes.c_int32), ("traditional", ctypes.c_int32), ("base", ctypes.c_float),
                ("scale", ctypes.c_float)]


_lib.kvc_rope.argtypes = [_TP, ctypes.c_int64, ctypes.POINTER(RopeConfig), _TP, _vp]
_lib.kvc_attention_rope.argtypes = [_vp, _TP, _TP, _TP, ctypes.POINTER(RopeConfig), ctypes.c_float, ctypes.c_int32,
                                    _TP, _TP, _vp]
_lib.kvc_storage_begin_round.argtypes = [ctypes.POINTER(_vp), ctypes.c_int32, ctypes.c_int32, ctypes.POINTER(_vp)]
_lib.kvc_storage_round_attention.argtypes = [ctypes.POINTER(_vp), ctypes.c_int32, _TP, _TP, _TP, ctypes.c_float,
                                             ctypes.c_int32, _TP, _vp]
_lib.kvc_storage_commit.argtypes = [ctypes.POINTER(_vp), ctypes.c_int32, ctypes.c_int32, _vp]
_lib.kvc_speculate_rewind.argtypes = [ctypes.POINTER(_vp), ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                                      ctypes.c_int32, ctypes.POINTER(ctypes.c_int64)]
_lib.kvc_turbo_rotation.argtypes = [ctypes.c_int32, ctypes.c_uint64, ctypes.POINTER(ctypes.c_float)]
_lib.kvc_turbo_set_rotation.argtypes = [_vp, ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_float), ctypes.c_int32]
_lib.kvc_comm_init.argtypes = [ctypes.c_int32, ctypes.c_int32, ctypes.c_char_p, ctypes.POINTER(_vp)]
_lib.kvc_comm_unique_id.argtypes = [ctypes.c_char_p]
_lib.kvc_comm_symm_alloc.argtypes = [_vp, ctypes.c_size_t, _vp, ctypes.POINTER(_vp)]
_lib.kvc_comm_set_wait_limit.argtypes = [_vp, ctypes.c_uint32]
_lib.kvc_attention_batch.argtypes = [ctypes.POINTER(_vp), ctypes.c_int32, _TP, _TP, _TP, ctypes.c_float,
                                     ctypes.c_int32, _TP, _vp, ctypes.c_int32, ctypes.c_int32]
_lib.kvc_attention_sharded_batch.argtypes = [_vp, ctypes.POINTER(_vp), ctypes.c_int32, _TP, _TP, _TP,
                                             ctypes.c_float, ctypes.c_int32, _TP, ctypes.c_int32, _vp]
_lib.kvc_device_wait_probe.argtypes = [ctypes.c_uint32, _vp]
_lib.kvc_timing_enable.argtypes = [ctypes.c_int32]
_lib.kvc_timing_enable.restype = None
_lib.kvc_timing_read.argtypes = [ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_int64), ctypes.c_int32]


def lib() -> ctypes.CDLL:
    return _lib


def version() -> str:
    return _lib.kvc_version().decode()


def device_available() -> bool:
    return bool(_lib.kvc_device_available())


def launch_count(reset: bool = False) -> int:
    return int(_lib.kvc_launch_count(1 if reset else 0))


def check(status: int) -> None:
    if status != OK:
        msg = _lib.kvc_last_error_message()
        raise KVCError(status, msg.decode() if msg else "unknown error")


# ---------------------------------------------------------------------------
# torch <-> kvc_tensor
# ---------------------------------------------------------------------------

def _torch():
    import torch
    return torch


def _dtype_code(t) -> int:
    torch = _torch()
    return {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16, torch.int32: U32,
            torch.uint32: U32, torch.bool: BOOL, torch.uint8: BOOL}[t.dtype]


def _torch_dtype(code: int):
    torch = _torch()
    return {F32: torch.float32, F16: torch.float16, BF16: torch.bfloat16, U32: torch.int32, BOOL: torch.uint8}[code]


def as_tensor(t) -> Tensor:
    """Describe a torch tensor (device or host) as a kvc_tensor."""
    out = Tensor()
    out.data = t.data_ptr()
    out.dtype = _dtype_code(t)
    out.ndim = t.dim()
    for i in range(t.dim()):
        out.shape[i] = t.shape[i]
        out.stride[i] = t.stride(i)
    return out


def view_to_torch(v: Tensor, device):
    """Wrap a kvc_tensor view of library memory as a torch tensor (no copy)."""
    torch = _torch()
    nd = v.ndim
    shape = [int(v.shape[i]) for i in range(nd)]
    stride = [int(v.stride[i]) for i in range(nd)]
    dt = _torch_dtype(v.dtype)
    esize = torch.empty((), dtype=dt).element_size()
    if any(s == 0 for s in shape) or not v.data:
        return torch.empty(shape, dtype=dt, device=device)
    extent = 1 + sum((shape[i] - 1) * stride[i] for i in range(nd))
    return _from_pointer(int(v.data), extent * esize, dt, device).as_strided(shape, stride)


class _CudaArray:
    """Minimal __cuda_array_interface__ carrier for a raw device pointer."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 3, "strides": None}


def _from_pointer(ptr: int, nbytes: int, dtype, device):
    torch = _torch()
    base = torch.as_tensor(_CudaArray(ptr, nbytes), device=device)
    return base.view(dtype)


def _stream_ptr(stream=None) -> int:
    torch = _torch()
    if stream is None:
        if not torch.cuda.is_available():
            return 0   # host-only calls (file headers, empty caches) on a machine without a device
        stream = torch.cuda.current_stream()
    return int(stream.cuda_stream)


def _mask_args(mask):
    if mask is None or (isinstance(mask, str) and mask == "none"):
        return MASK_NONE, None, None
    if isinstance(mask, str):
        if mask == "causal":
            return MASK_CAUSAL, None, None
        raise ValueError(f"unknown mask mode {mask!r}")
    torch = _torch()
    m = mask
    if m.dtype == torch.bool:
        m = m.to(torch.uint8)
    t = as_tensor(m)
    return MASK_ARRAY, ctypes.byref(t), (m, t)


# ---------------------------------------------------------------------------
# cache classes
# ---------------------------------------------------------------------------

class KVCache:
    """Base of the four cache classes; owns one kvc_cache handle."""

    def __init__(self, handle: int, device=None):
        self._h = ctypes.c_void_p(handle)
        self._device = device

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            _lib.kvc_free(h)
            self._h = None

    @classmethod
    def _create(cls, cfg: Config):
        h = ctypes.c_void_p()
        check(_lib.kvc_create(ctypes.byref(cfg), ctypes.byref(h)))
        return h.value

    @staticmethod
    def _config(kind: int, **kw) -> Config:
        cfg = Config()
        _lib.kvc_config_default(ctypes.byref(cfg), kind)
        for k, v in kw.items():
            if v is not None:
                setattr(cfg, k, v)
        return cfg

    def _dev(self, like=None):
        if like is not None:
            self._device = like.device
        return self._device

    # --- protocol surface -------------------------------------------------
    @property
    def offset(self) -> int:
        return int(_lib.kvc_offset(self._h))

    @offset.setter
    def offset(self, n: int):
        check(_lib.kvc_set_offset(self._h, n))

    @property
    def max_size(self) -> Optional[int]:
        m = int(_lib.kvc_max_size(self._h))
        return None if m < 0 else m

    def prepare(self, lengths=None) -> None:
        """prepare(lengths:): the reference's empty default for these cache kinds (KVCache.swift:229-231)."""
        n = 0 if lengths is None else len(lengths)
        arr = (ctypes.c_int32 * max(n, 1))(*(list(lengths) if lengths is not None else []))
        check(_lib.kvc_prepare(self._h, arr, n))

    def finalize(self) -> None:
        check(_lib.kvc_finalize(self._h))

    def update(self, keys, values, stream=None):
        ok, ov = Tensor(), Tensor()
        tk, tv = as_tensor(keys), as_tensor(values)
        check(_lib.kvc_update(self._h, ctypes.byref(tk), ctypes.byref(tv), _stream_ptr(stream),
                              ctypes.byref(ok), ctypes.byref(ov)))
        dev = self._dev(keys)
        return view_to_torch(ok, dev), view_to_torch(ov, dev)

    @property
    def state(self) -> List:
        n = int(_lib.kvc_state_count(self._h))
        out = []
        for i in range(n):
            t = Tensor()
            check(_lib.kvc_state_get(self._h, i, ctypes.byref(t)))
            out.append(view_to_torch(t, self._device))
        return out

    @state.setter
    def state(self, arrays: Sequence):
        arr = (Tensor * max(len(arrays), 1))()
        for i, a in enumerate(arrays):
            arr[i] = as_tensor(a)
            self._device = a.device
        check(_lib.kvc_state_set(self._h, arr, len(arrays), _stream_ptr()))

    def export_state(self, index: int):
        """Device -> host copy of state array `index` as a contiguous torch tensor."""
        torch = _torch()
        desc = Tensor()
        check(_lib.kvc_state_export(self._h, index, None, 0, ctypes.byref(desc), _stream_ptr()))
        shape = [int(desc.shape[i]) for i in range(desc.ndim)]
        out = torch.empty(shape, dtype=_torch_dtype(desc.dtype))
        check(_lib.kvc_state_export(self._h, index, out.data_ptr(), out.numel() * out.element_size(),
                                    ctypes.byref(desc), _stream_ptr()))
        return out

    @property
    def meta_state(self) -> List[str]:
        n = ctypes.c_size_t()
        check(_lib.kvc_meta_state(self._h, None, 0, ctypes.byref(n)))
        buf = ctypes.create_string_buffer(n.value)
        check(_lib.kvc_meta_state(self._h, buf, n.value, ctypes.byref(n)))
        return buf.value.decode().split("\n")

    @meta_state.setter
    def meta_state(self, values: Sequence[str]):
        check(_lib.kvc_set_meta_state(self._h, "\n".join(values).encode()))

    @property
    def is_trimmable(self) -> bool:
        return bool(_lib.kvc_is_trimmable(self._h))

    def is_trimmable_after(self, positions: int) -> bool:
        return bool(_lib.kvc_is_trimmable_after(self._h, positions))

    def trim(self, n: int) -> int:
        out = ctypes.c_int64()
        check(_lib.kvc_trim(self._h, n, ctypes.byref(out)))
        return int(out.value)

    def make_mask(self, n: int, window_size: Optional[int] = None, return_array: bool = False):
        """Returns "none", "causal" or a bool tensor, like makeMask(n:windowSize:returnArray:)."""
        torch = _torch()
        mode, rows, cols = ctypes.c_int32(), ctypes.c_int64(), ctypes.c_int64()
        ws = -1 if window_size is None else window_size
        check(_lib.kvc_make_mask(self._h, n, ws, int(return_array), ctypes.byref(mode), ctypes.byref(rows),
                                 ctypes.byref(cols), None, None))
        if mode.value == MASK_NONE:
            return "none"
        if mode.value == MASK_CAUSAL:
            return "causal"
        dev = self._device if self._device is not None else torch.device("cuda")
        out = torch.empty((rows.value, cols.value), dtype=torch.uint8, device=dev)
        check(_lib.kvc_make_mask(self._h, n, ws, int(return_array), ctypes.byref(mode), ctypes.byref(rows),
                                 ctypes.byref(cols), out.data_ptr(), _stream_ptr()))
        out = out.bool()
        return out[0] if n == 1 else out

    def copy(self):
        h = ctypes.c_void_p()
        check(_lib.kvc_copy(self._h, _stream_ptr(), ctypes.byref(h)))
        new = object.__new__(type(self))
        KVCache.__init__(new, h.value, self._device)
        return new

    def reserve(self, tokens: int, batch: int, kv_heads: int, head_dim: int, dtype, stream=None):
        torch = _torch()
        code = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}[dtype]
        check(_lib.kvc_reserve(self._h, tokens, batch, kv_heads, head_dim, code, _stream_ptr(stream)))

    @property
    def memory_bytes(self) -> int:
        return int(_lib.kvc_memory_bytes(self._h))

    def attention(self, queries, keys, values, scale: float, mask="none", out=None, stream=None):
        """attentionWithCacheUpdate for this cache; returns [B, Hq, L, D] in the query dtype."""
        torch = _torch()
        self._dev(queries)
        if out is None:
            out = torch.empty(queries.shape, dtype=queries.dtype, device=queries.device)
        mode, mptr, _keep = _mask_args(mask)
        tq, tk, tv, to = as_tensor(queries), as_tensor(keys), as_tensor(values), as_tensor(out)
        check(_lib.kvc_attention(self._h, ctypes.byref(tq), ctypes.byref(tk), ctypes.byref(tv),
                                 ctypes.c_float(scale), mode, mptr, ctypes.byref(to), _stream_ptr(stream)))
        return out

    def attention_host(self, queries, keys, values, scale: float, mask="none", out=None, stream=None,
                       synchronize: bool = True):
        """Same, with every tensor in host memory (the end-to-end entry point)."""
        torch = _torch()
        if out is None:
            out = torch.empty(queries.shape, dtype=queries.dtype)
        mode, mptr, _keep = _mask_args(mask)
        tq, tk, tv, to = as_tensor(queries), as_tensor(keys), as_tensor(values), as_tensor(out)
        check(_lib.kvc_attention_host(self._h, ctypes.byref(tq), ctypes.byref(tk), ctypes.byref(tv),
                                      ctypes.c_float(scale), mode, mptr, ctypes.byref(to),
                                      _stream_ptr(stream), 1 if synchronize else 0))
        return out


class KVCacheSimple(KVCache):
    def __init__(self, step: int = 256, reserve_tokens: int = 0):
        super().__init__(self._create(self._config(KIND_SIMPLE, step=step, reserve_tokens=reserve_tokens)))

    def to_quantized(self, group_size: int = 64, bits: int = 4) -> "QuantizedKVCache":
        h = ctypes.c_void_p()
        check(_lib.kvc_to_quantized(self._h, group_size, bits, _stream_ptr(), ctypes.byref(h)))
        new = object.__new__(QuantizedKVCache)
        KVCache.__init__(new, h.value, self._device)
        return new

    def to_turbo(self, key_bits: int, value_bits: int, key_group_size: int = 64) -> "TurboQuantKVCache":
        h = ctypes.c_void_p()
        check(_lib.kvc_to_turbo(self._h, key_bits, value_bits, key_group_size, _stream_ptr(), ctypes.byref(h)))
        new = object.__new__(TurboQuantKVCache)
        KVCache.__init__(new, h.value, self._device)
        return new


class ChunkedKVCache(KVCache):
    """ChunkedKVCache(chunkSize:) (KVCache.swift:1213-1304)."""

    def __init__(self, chunk_size: Optional[int] = None, step: int = 256):
        super().__init__(self._create(self._config(KIND_CHUNKED, max_size=-1 if chunk_size is None else chunk_size,
                                                   step=step)))

    def maybe_trim_front(self, stream=None) -> None:
        check(_lib.kvc_maybe_trim_front(self._h, _stream_ptr(stream)))

    @property
    def start_position(self) -> int:
        return int(_lib.kvc_start_position(self._h))


class CacheList(KVCache):
    """CacheList(caches...) (KVCache.swift:1556-1726). The list owns its children: the Python objects
    passed in give their handles up and must not be used afterwards; use list[i]."""

    def __init__(self, *caches: "KVCache"):
        n = len(caches)
        arr = (_vp * max(n, 1))(*[c._h for c in caches])
        h = ctypes.c_void_p()
        check(_lib.kvc_list_create(arr, n, ctypes.byref(h)))
        dev = None
        for c in caches:
            dev = dev or c._device
            c._h = None                      # ownership moved into the list
        super().__init__(h.value, dev)
        self._kinds = [type(c) for c in caches]

    def __len__(self) -> int:
        return int(_lib.kvc_list_count(self._h))

    def __getitem__(self, i: int) -> "KVCache":
        h = _lib.kvc_list_child(self._h, i)
        if not h:
            raise IndexError(i)
        return _borrowed(h, self._device, self)


class RotatingKVCache(KVCache):
    def __init__(self, max_size: int, keep: int = 0, step: int = 256):
        super().__init__(self._create(self._config(KIND_ROTATING, max_size=max_size, keep=keep, step=step)))

    @property
    def idx(self) -> int:
        return int(_lib.kvc_ring_index(self._h))

    def logical_view(self, tail: int, stream=None):
        ok, ov = Tensor(), Tensor()
        st = _lib.kvc_logical_view(self._h, tail, _stream_ptr(stream), ctypes.byref(ok), ctypes.byref(ov))
        if st == ERR_INVALID_STATE:
            return None
        check(st)
        return view_to_torch(ok, self._device), view_to_torch(ov, self._device)

    def to_quantized(self, group_size: int = 64, bits: int = 4):
        h = ctypes.c_void_p()
        check(_lib.kvc_to_quantized(self._h, group_size, bits, _stream_ptr(), ctypes.byref(h)))

    def rewind_last_round(self, count: int, stream=None) -> int:
        out = ctypes.c_int64()
        check(_lib.kvc_rewind_last_round(self._h, count, _stream_ptr(stream), ctypes.byref(out)))
        return int(out.value)


class QuantizedKVCache(KVCache):
    def __init__(self, group_size: int = 64, bits: int = 8, reserve_tokens: int = 0):
        super().__init__(self._create(self._config(KIND_QUANTIZED, group_size=group_size, bits=bits,
                                                   reserve_tokens=reserve_tokens)))

    @property
    def group_size(self) -> int:
        return int(_lib.kvc_group_size(self._h))

    @property
    def bits(self) -> int:
        return int(_lib.kvc_bits(self._h))

    def update_quantized(self, keys, values, stream=None):
        ok, ov = (Tensor * 3)(), (Tensor * 3)()
        tk, tv = as_tensor(keys), as_tensor(values)
        check(_lib.kvc_update_quantized(self._h, ctypes.byref(tk), ctypes.byref(tv), _stream_ptr(stream), ok, ov))
        dev = self._dev(keys)
        return (tuple(view_to_torch(ok[i], dev) for i in range(3)),
                tuple(view_to_torch(ov[i], dev) for i in range(3)))

    def to_unquantized(self) -> KVCacheSimple:
        h = ctypes.c_void_p()
        check(_lib.kvc_to_unquantized(self._h, _stream_ptr(), ctypes.byref(h)))
        new = object.__new__(KVCacheSimple)
        KVCache.__init__(new, h.value, self._device)
        return new


class TurboQuantKVCache(KVCache):
    def __init__(self, bits: int = 4, key_bits: Optional[int] = None, value_bits: Optional[int] = None,
                 seed: int = 42, key_group_size: int = 64, affine_values: bool = False, reserve_tokens: int = 0):
        super().__init__(self._create(self._config(
            KIND_TURBO, bits=bits, key_bits=-1 if key_bits is None else key_bits,
            value_bits=-1 if value_bits is None else value_bits, seed=seed, key_group_size=key_group_size,
            turbo_affine_values=1 if affine_values else 0, reserve_tokens=reserve_tokens)))

    @property
    def is_compressed(self) -> bool:
        return bool(_lib.kvc_is_compressed(self._h))

    def set_codec(self, key_centroids=None, value_centroids=None, key_signs=None, value_signs=None, dim=0):
        def arr(x):
            if x is None:
                return None
            return (ctypes.c_float * len(x))(*[float(v) for v in x])
        check(_lib.kvc_turbo_set_codec(self._h, arr(key_centroids), arr(value_centroids), arr(key_signs),
                                       arr(value_signs), dim))

    def set_rotation(self, key_rotation=None, value_rotation=None, dim=0):
        """Hand the cache the dense rotations a host already holds (row-major [dim, dim]); None keeps the default."""
        import numpy as _np

        def arr(x):
            if x is None:
                return None
            a = _np.ascontiguousarray(x, dtype=_np.float32).reshape(-1)
            return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), a
        k, v = arr(key_rotation), arr(value_rotation)
        check(_lib.kvc_turbo_set_rotation(self._h, k[0] if k else None, v[0] if v else None, dim))

    def encode_new_token(self, keys, values, stream=None):
        """Compressed-domain append of keys/values [B, H, S, D] (encodeNewToken); no attention."""
        tk, tv = as_tensor(keys), as_tensor(values)
        check(_lib.kvc_turbo_encode_new_token(self._h, ctypes.byref(tk), ctypes.byref(tv), _stream_ptr(stream)))

    def compressed_attention(self, queries, keys, values, scale, mask="none", out=None, stream=None):
        return self.attention(queries, keys, values, scale, mask, out, stream)


class StagedRound:
    """kvc_round: one cache's share of a speculative verify round."""

    def __init__(self, cache: KVCache, max_positions: int):
        h = ctypes.c_void_p()
        check(_lib.kvc_round_begin(cache._h, max_positions, ctypes.byref(h)))
        self._h = h
        self.cache = cache

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            _lib.kvc_round_free(h)
            self._h = None

    @property
    def offset(self) -> int:
        return int(_lib.kvc_round_offset(self._h))

    def update(self, keys, values, stream=None):
        ok, ov = Tensor(), Tensor()
        tk, tv = as_tensor(keys), as_tensor(values)
        check(_lib.kvc_round_update(self._h, ctypes.byref(tk), ctypes.byref(tv), _stream_ptr(stream),
                                    ctypes.byref(ok), ctypes.byref(ov)))
        return view_to_torch(ok, keys.device), view_to_torch(ov, keys.device)

    def attention(self, queries, keys, values, scale, mask="none", out=None, stream=None):
        torch = _torch()
        if out is None:
            out = torch.empty(queries.shape, dtype=queries.dtype, device=queries.device)
        mode, mptr, _keep = _mask_args(mask)
        tq, tk, tv, to = as_tensor(queries), as_tensor(keys), as_tensor(values), as_tensor(out)
        check(_lib.kvc_round_attention(self._h, ctypes.byref(tq), ctypes.byref(tk), ctypes.byref(tv),
                                       ctypes.c_float(scale), mode, mptr, ctypes.byref(to), _stream_ptr(stream)))
        return out

    def commit(self, retaining: int, stream=None):
        check(_lib.kvc_round_commit(self._h, retaining, _stream_ptr(stream)))

    def rollback(self, stream=None):
        check(_lib.kvc_round_rollback(self._h, _stream_ptr(stream)))


# ---------------------------------------------------------------------------
# free functions
# ---------------------------------------------------------------------------

def _borrowed(handle: int, device, owner) -> "KVCache":
    """A view object on a handle owned by something else (a CacheList child): never frees it."""
    kind = int(_lib.kvc_kind_of(ctypes.c_void_p(handle)))
    cls = {KIND_SIMPLE: KVCacheSimple, KIND_ROTATING: RotatingKVCache, KIND_QUANTIZED: QuantizedKVCache,
           KIND_TURBO: TurboQuantKVCache, KIND_CHUNKED: ChunkedKVCache, KIND_LIST: CacheList}.get(kind, KVCache)
    obj = object.__new__(cls)
    KVCache.__init__(obj, handle, device)
    obj._owner = owner          # keeps the owning list alive
    obj.__class__ = type("Borrowed" + cls.__name__, (cls,), {"__del__": lambda self: None})
    return obj


def create_causal_mask(n: int, offset: int, window_size: Optional[int] = None, lengths=None, device=None, stream=None):
    """createCausalMask(n:offset:windowSize:lengths:) (KVCache.swift:253-275) as a bool tensor on the device:
    [n, offset + n], or [B, 1, n, offset + n] when `lengths` (a sequence of B ints or an int32 device tensor) is given."""
    torch = _torch()
    dev = device if device is not None else torch.device("cuda")
    ws = -1 if window_size is None else window_size
    if lengths is None:
        out = torch.empty((n, offset + n), dtype=torch.uint8, device=dev)
        check(_lib.kvc_create_causal_mask(n, offset, ws, None, 0, out.data_ptr(), _stream_ptr(stream)))
        return out.bool()
    ln = lengths if hasattr(lengths, "data_ptr") else torch.tensor(list(lengths), dtype=torch.int32, device=dev)
    ln = ln.to(dtype=torch.int32, device=dev).contiguous()
    B = int(ln.numel())
    out = torch.empty((B, 1, n, offset + n), dtype=torch.uint8, device=dev)
    check(_lib.kvc_create_causal_mask(n, offset, ws, ln.data_ptr(), B, out.data_ptr(), _stream_ptr(stream)))
    return out.bool()


def attention_with_cache_update(queries, keys, values, cache: Optional[KVCache], scale: float, mask="none"):
    """attentionWithCacheUpdate(queries:keys:values:cache:scale:mask:)."""
    if cache is None:
        return scaled_dot_product_attention(queries, keys, values, scale, mask)
    return cache.attention(queries, keys, values, scale, mask)


def scaled_dot_product_attention(queries, keys, values, scale: float, mask="none", out=None, stream=None):
    torch = _torch()
    if out is None:
        out = torch.empty(queries.shape, dtype=queries.dtype, device=queries.device)
    mode, mptr, _keep = _mask_args(mask)
    tq, tk, tv, to = as_tensor(queries), as_tensor(keys), as_tensor(values), as_tensor(out)
    check(_lib.kvc_sdpa(ctypes.byref(tq), ctypes.byref(tk), ctypes.byref(tv), ctypes.c_float(scale), mode, mptr,
                        ctypes.byref(to), _stream_ptr(stream)))
    return out


def scaled_dot_product_attention_noalloc(queries, keys, values, scale: float, mask="none", out=None,
                                         stream=None):
    """kvc_sdpa_noalloc: same result as scaled_dot_product_attention, but the library
    allocates nothing (split partials live in a fixed array of the device image).
    `out` should be supplied by callers that must not allocate themselves."""
    torch = _torch()
    if out is None:
        out = torch.empty(queries.shape, dtype=queries.dtype, device=queries.device)
    mode, _mptr, _keep = _mask_args(mask)
    tq, tk, tv, to = as_tensor(queries), as_tensor(keys), as_tensor(values), as_tensor(out)
    check(_lib.kvc_sdpa_noalloc(ctypes.byref(tq), ctypes.byref(tk), ctypes.byref(tv), ctypes.c_float(scale), mode,
                                ctypes.byref(to), _stream_ptr(stream)))
    return out


def quantized_scaled_dot_product_attention(queries, quantized_keys, quantized_values, scale: float,
                                           mask="none", group_size: int = 64, bits: int = 8, out=None,
                                           stream=None):
    torch = _torch()
    if out is None:
        out = torch.empty(queries.shape, dtype=queries.dtype, device=queries.device)
    mode, mptr, _keep = _mask_args(mask)
    qk, qv = (Tensor * 3)(), (Tensor * 3)()
    for i in range(3):
        qk[i] = as_tensor(quantized_keys[i])
        qv[i] = as_tensor(quantized_values[i])
    tq, to = as_tensor(queries), as_tensor(out)
    check(_lib.kvc_quantized_sdpa(ctypes.byref(tq), qk, qv, ctypes.c_float(scale), mode, mptr, group_size, bits,
                                  ctypes.byref(to), _stream_ptr(stream)))
    return out


def quantized(x, group_size: int = 64, bits: int = 4, stream=None):
    """MLX quantized(_:groupSize:bits:) -> (wq int32-viewed uint32, scales, biases)."""
    torch = _torch()
    D = x.shape[-1]
    x = x.contiguous()
    codes = torch.empty(x.shape[:-1] + (D * bits // 32,), dtype=torch.int32, device=x.device)
    scales = torch.empty(x.shape[:-1] + (D // group_size,), dtype=x.dtype, device=x.device)
    biases = torch.empty_like(scales)
    tx, tc, ts, tb = as_tensor(x), as_tensor(codes), as_tensor(scales), as_tensor(biases)
    check(_lib.kvc_affine_quantize(ctypes.byref(tx), group_size, bits, ctypes.byref(tc), ctypes.byref(ts),
                                   ctypes.byref(tb), _stream_ptr(stream)))
    return codes, scales, biases


def dequantized(codes, scales, biases, group_size: int = 64, bits: int = 4, stream=None):
    torch = _torch()
    D = codes.shape[-1] * 32 // bits
    out = torch.empty(codes.shape[:-1] + (D,), dtype=scales.dtype, device=codes.device)
    tc, ts, tb, to = (as_tensor(codes.contiguous()), as_tensor(scales.contiguous()),
                      as_tensor(biases.contiguous()), as_tensor(out))
    check(_lib.kvc_affine_dequantize(ctypes.byref(tc), ctypes.byref(ts), ctypes.byref(tb), group_size, bits,
                                     ctypes.byref(to), _stream_ptr(stream)))
    return out


def turbo_codebook(dim: int, bits: int) -> Tuple[List[float], List[float]]:
    c = (ctypes.c_float * (1 << bits))()
    b = (ctypes.c_float * ((1 << bits) - 1))()
    check(_lib.kvc_turbo_codebook(dim, bits, c, b))
    return list(c), list(b)


def turbo_signs(dim: int, seed: int) -> List[float]:
    s = (ctypes.c_float * dim)()
    check(_lib.kvc_turbo_signs(dim, seed, s))
    return list(s)


def turbo_rotation(dim: int, seed: int):
    """The library's seeded dense rotation for head dims that are not powers of two, as a numpy [dim, dim] array."""
    import numpy as _np
    out = _np.zeros((dim, dim), dtype=_np.float32)
    check(_lib.kvc_turbo_rotation(dim, seed, out.ctypes.data_as(ctypes.POINTER(ctypes.c_float))))
    return out


def turbo_packed_width(count: int, bits: int) -> int:
    return int(_lib.kvc_turbo_packed_width(count, bits))


def turbo_encode(rows, signs, boundaries, bits: int, stream=None):
    """fusedEncodeWHT: rows [N, D] -> (packed int32-viewed uint32 [N, PW], norms f32 [N])."""
    torch = _torch()
    rows = rows.contiguous()
    n, D = rows.shape
    pw = turbo_packed_width(D, bits)
    packed = torch.empty((n, pw), dtype=torch.int32, device=rows.device)
    norms = torch.empty((n,), dtype=torch.float32, device=rows.device)
    signs_dev = torch.as_tensor(signs, dtype=torch.float32, device=rows.device).contiguous()
    b = (ctypes.c_float * len(boundaries))(*[float(v) for v in boundaries])
    tr, tp, tn = as_tensor(rows), as_tensor(packed), as_tensor(norms)
    check(_lib.kvc_turbo_encode(ctypes.byref(tr), signs_dev.data_ptr(), b, bits, ctypes.byref(tp),
                                ctypes.byref(tn), _stream_ptr(stream)))
    return packed, norms


class DecodeStep:
    """Pre-marshalled arguments of one decode step over a list of caches.

    The tensors of every layer are described once; `run()` then issues the
    whole step with a single C call (kvc_attention_batch), which is how a native
    caller would drive the per-layer calls without interpreter overhead.
    """

    def __init__(self, caches: Sequence[KVCache], queries, keys, values, outs, scale: float,
                 mask: str = "none", host: bool = False):
        n = len(caches)
        assert len(queries) == len(keys) == len(values) == len(outs) == n
        self._keep = (list(caches), list(queries), list(keys), list(values), list(outs))
        self.n = n
        self.handles = (_vp * n)(*[c._h for c in caches])
        self.q = (Tensor * n)(*[as_tensor(t) for t in queries])
        self.k = (Tensor * n)(*[as_tensor(t) for t in keys])
        self.v = (Tensor * n)(*[as_tensor(t) for t in values])
        self.o = (Tensor * n)(*[as_tensor(t) for t in outs])
        self.scale = ctypes.c_float(scale)
        self.mode = {"none": MASK_NONE, "causal": MASK_CAUSAL}[mask]
        self.host = 1 if host else 0

    def run(self, stream=None, synchronize: bool = False):
        check(_lib.kvc_attention_batch(self.handles, self.n, self.q, self.k, self.v, self.scale, self.mode,
                                       self.o, _stream_ptr(stream), self.host, 1 if synchronize else 0))

    def run_varlen(self, stream=None):
        """The caches are independent sequences of one layer (one new token each): kvc_attention_varlen."""
        check(_lib.kvc_attention_varlen(self.handles, self.n, self.q, self.k, self.v, self.scale, self.o,
                                        _stream_ptr(stream)))

    def run_sharded(self, comm: "Comm", shard_axis: int = 1, stream=None):
        check(_lib.kvc_attention_sharded_batch(comm._h, self.handles, self.n, self.q, self.k, self.v, self.scale,
                                               self.mode, self.o, shard_axis, _stream_ptr(stream)))


def device_status() -> int:
    """0 unless a bounded device-side wait has run out since the last reset (kvc_device_status)."""
    return int(_lib.kvc_device_status())


def device_status_reset() -> None:
    check(_lib.kvc_device_status_reset())


def device_wait_probe(iterations: int = 1 << 12, stream=None) -> None:
    """A kernel whose bounded wait runs out on purpose (kvc_device_wait_probe)."""
    check(_lib.kvc_device_wait_probe(iterations, _stream_ptr(stream)))


def rope(x, offset: int, dims: int, traditional: bool = False, base: float = 10000.0, scale: float = 1.0, out=None,
         stream=None):
    """applyRotaryPosition(rope, to: x, offset:) for x [B, H, L, D] on the device."""
    torch = _torch()
    if out is None:
        out = torch.empty_like(x)
    cfg = RopeConfig(dims, int(traditional), base, scale)
    tx, to = as_tensor(x), as_tensor(out)
    check(_lib.kvc_rope(ctypes.byref(tx), offset, ctypes.byref(cfg), ctypes.byref(to), _stream_ptr(stream)))
    return out


def attention_rope(queries, keys, values, cache: Optional["KVCache"], rope_cfg: dict, scale: float, mask="none", out=None,
                   stream=None):
    """The attention block's cache step (Llama.swift:58-69): rotary positions at cache.ropeOffset for queries
    and keys, then attentionWithCacheUpdate."""
    torch = _torch()
    if out is None:
        out = torch.empty(queries.shape, dtype=queries.dtype, device=queries.device)
    cfg = RopeConfig(rope_cfg["dims"], int(rope_cfg.get("traditional", False)), rope_cfg.get("base", 10000.0),
                     rope_cfg.get("scale", 1.0))
    mode, mptr, _keep = _mask_args(mask)
    tq, tk, tv, to = as_tensor(queries), as_tensor(keys), as_tensor(values), as_tensor(out)
    check(_lib.kvc_attention_rope(cache._h if cache is not None else None, ctypes.byref(tq), ctypes.byref(tk),
                                  ctypes.byref(tv), ctypes.byref(cfg), ctypes.c_float(scale), mode, mptr, ctypes.byref(to),
                                  _stream_ptr(stream)))
    return out


class StorageRound:
    """A staged speculative round over the layer list of a model (KVCacheStorage.beginRound / commit,
    KVCachePlan.swift:219-300). Opening is all or nothing; `attention` runs the verify pass of every layer;
    `commit(retaining)` keeps that many of the written positions in every cache (0 = rollback)."""

    def __init__(self, caches: Sequence["KVCache"], max_positions: int):
        self.caches = list(caches)
        n = len(self.caches)
        arr = (_vp * n)(*[c._h for c in self.caches])
        self._rounds = (_vp * n)()
        self._n = n
        check(_lib.kvc_storage_begin_round(arr, n, max_positions, self._rounds))
        self._open = True

    def attention(self, queries, keys, values, scale: float, outs, mask: str = "causal", stream=None):
        n = self._n
        q = (Tensor * n)(*[as_tensor(t) for t in queries])
        k = (Tensor * n)(*[as_tensor(t) for t in keys])
        v = (Tensor * n)(*[as_tensor(t) for t in values])
        o = (Tensor * n)(*[as_tensor(t) for t in outs])
        mode = {"none": MASK_NONE, "causal": MASK_CAUSAL}[mask]
        check(_lib.kvc_storage_round_attention(self._rounds, n, q, k, v, ctypes.c_float(scale), mode, o, _stream_ptr(stream)))
        return outs

    def commit(self, retaining: int, stream=None) -> None:
        if self._open:
            self._open = False
            check(_lib.kvc_storage_commit(self._rounds, self._n, retaining, _stream_ptr(stream)))

    def rollback(self, stream=None) -> None:
        self.commit(0, stream)

    def __del__(self):
        try:
            self.commit(0)
        except Exception:
            pass


def speculate_rewind(caches: Sequence["KVCache"], num_draft: int, accepted: int, is_draft: bool = False) -> int:
    """The rewind at the end of speculateRound (Evaluate.swift:1262-1264)."""
    arr = (_vp * len(caches))(*[c._h for c in caches])
    out = ctypes.c_int64()
    check(_lib.kvc_speculate_rewind(arr, len(caches), num_draft, accepted, int(is_draft), ctypes.byref(out)))
    return int(out.value)


def timing_enable(on: bool) -> None:
    _lib.kvc_timing_enable(1 if on else 0)


def timing_read(reset: bool = True) -> Tuple[float, int]:
    ms, n = ctypes.c_double(), ctypes.c_int64()
    check(_lib.kvc_timing_read(ctypes.byref(ms), ctypes.byref(n), 1 if reset else 0))
    return float(ms.value), int(n.value)


def trim_prompt_cache(caches: Sequence[KVCache], num_tokens: int) -> int:
    arr = (_vp * len(caches))(*[c._h for c in caches])
    out = ctypes.c_int64()
    check(_lib.kvc_trim_prompt_cache(arr, len(caches), num_tokens, ctypes.byref(out)))
    return int(out.value)


def can_trim_prompt_cache(caches: Sequence[KVCache]) -> bool:
    arr = (_vp * len(caches))(*[c._h for c in caches])
    return bool(_lib.kvc_can_trim_prompt_cache(arr, len(caches)))


class Comm:
    """kvc_comm: NCCL communicator for KV-head / batch sharded attention."""

    def __init__(self, rank: int, world: int, unique_id: bytes):
        h = ctypes.c_void_p()
        check(_lib.kvc_comm_init(rank, world, unique_id, ctypes.byref(h)))
        self._h = h
        self.rank, self.world = rank, world

    @staticmethod
    def unique_id() -> bytes:
        buf = ctypes.create_string_buffer(128)
        check(_lib.kvc_comm_unique_id(buf))
        return buf.raw

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            _lib.kvc_comm_free(h)
            self._h = None

    def symm_empty(self, shape, dtype, device, stream=None):
        """A tensor of `shape` in symmetric memory (kvc_comm_symm_alloc; collective: every rank makes the
        same call). Gathered outputs placed in such tensors are exchanged with peer stores over NVLink
        instead of ncclAllGather. The memory belongs to the communicator and lives as long as it does."""
        torch = _torch()
        n = 1
        for d in shape:
            n *= int(d)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        ptr = ctypes.c_void_p()
        check(_lib.kvc_comm_symm_alloc(self._h, nbytes, _stream_ptr(stream), ctypes.byref(ptr)))
        return _from_pointer(int(ptr.value), nbytes, dtype, device).view(*shape)

    def set_wait_limit(self, iterations: int) -> None:
        check(_lib.kvc_comm_set_wait_limit(self._h, iterations))

    def attention_sharded(self, cache: KVCache, queries, keys, values, scale, out_full, mask="none",
                          shard_axis: int = 1, stream=None):
        mode, mptr, _keep = _mask_args(mask)
        tq, tk, tv, to = as_tensor(queries), as_tensor(keys), as_tensor(values), as_tensor(out_full)
        check(_lib.kvc_attention_sharded(self._h, cache._h, ctypes.byref(tq), ctypes.byref(tk), ctypes.byref(tv),
                                         ctypes.c_float(scale), mode, mptr, ctypes.byref(to), shard_axis,
                                         _stream_ptr(stream)))
        return out_full


# ---------------------------------------------------------------------------
# list-level dynamic conversion (maybeQuantizeKVCache)
# ---------------------------------------------------------------------------

def resolve_turbo_scheme(scheme: Optional[str]):
    """resolveTurboScheme: (key_bits, value_bits) or None."""
    if scheme is None:
        return None
    kb, vb = ctypes.c_int32(), ctypes.c_int32()
    if not _lib.kvc_resolve_turbo_scheme(scheme.encode(), ctypes.byref(kb), ctypes.byref(vb)):
        return None
    return int(kb.value), int(vb.value)


def resolve_affine_scheme(scheme: Optional[str]):
    """resolveAffineScheme: (bits, group_size) or None."""
    if scheme is None:
        return None
    b, g = ctypes.c_int32(), ctypes.c_int32()
    if not _lib.kvc_resolve_affine_scheme(scheme.encode(), ctypes.byref(b), ctypes.byref(g)):
        return None
    return int(b.value), int(g.value)


def turbo_protected_layers(kinds: Sequence[int], key_bits: int, value_bits: int) -> List[bool]:
    n = len(kinds)
    arr = (ctypes.c_int32 * n)(*kinds)
    out = (ctypes.c_int32 * n)()
    check(_lib.kvc_turbo_protected_layers(arr, n, key_bits, value_bits, out))
    return [bool(x) for x in out]


def _wrap_handle(handle, like: "KVCache") -> "KVCache":
    kind = int(_lib.kvc_kind_of(ctypes.c_void_p(handle)))
    cls = {KIND_SIMPLE: KVCacheSimple, KIND_ROTATING: RotatingKVCache, KIND_QUANTIZED: QuantizedKVCache,
           KIND_TURBO: TurboQuantKVCache}[kind]
    obj = cls.__new__(cls)
    KVCache.__init__(obj, handle, like._device)
    return obj


def _rewrite_list(caches: List["KVCache"], fn) -> bool:
    n = len(caches)
    arr = (_vp * n)(*[c._h for c in caches])
    before = [int(ctypes.cast(arr[i], ctypes.c_void_p).value or 0) for i in range(n)]
    done = ctypes.c_int32()
    check(fn(arr, n, ctypes.byref(done)))
    for i in range(n):
        now = int(ctypes.cast(arr[i], ctypes.c_void_p).value or 0)
        if now != before[i]:
            caches[i]._h = None          # the library freed the old handle
            caches[i] = _wrap_handle(now, caches[i])
    return bool(done.value)


def maybe_affine_quantize_kv_cache(caches: List["KVCache"], bits: int, group_size: int = 64,
                                   compression_start: int = 0, stream=None) -> bool:
    """maybeAffineQuantizeKVCache: rewrites the list in place; False while a layer still waits."""
    return _rewrite_list(caches, lambda arr, n, done: _lib.kvc_maybe_affine_quantize(
        arr, n, bits, group_size, compression_start, _stream_ptr(stream), done))


def maybe_turbo_quantize_kv_cache(caches: List["KVCache"], key_bits: int, value_bits: int,
                                  quantized_kv_start: int = 0, stream=None) -> bool:
    """maybeTurboQuantizeKVCache: rewrites the list in place; False while a layer still waits."""
    return _rewrite_list(caches, lambda arr, n, done: _lib.kvc_maybe_turbo_quantize(
        arr, n, key_bits, value_bits, quantized_kv_start, _stream_ptr(stream), done))


# ---------------------------------------------------------------------------
# prompt-cache files (savePromptCache / loadPromptCache)
# ---------------------------------------------------------------------------

def save_prompt_cache(path: str, caches: Sequence["KVCache"], metadata: Optional[dict] = None, stream=None) -> None:
    """savePromptCache(url:cache:metadata:): a safetensors file in the mlx-lm prompt-cache layout."""
    metadata = metadata or {}
    n = len(caches)
    arr = (_vp * n)(*[c._h for c in caches])
    keys = (ctypes.c_char_p * len(metadata))(*[str(k).encode() for k in metadata])
    vals = (ctypes.c_char_p * len(metadata))(*[str(v).encode() for v in metadata.values()])
    check(_lib.kvc_save_prompt_cache(os.fsencode(path), arr, n, keys, vals, len(metadata), _stream_ptr(stream)))


def load_prompt_cache(path: str, device: int = -1, stream=None):
    """loadPromptCache(url:) -> (caches, metadata)."""
    count, need = ctypes.c_int32(), ctypes.c_size_t()
    # first pass: how many caches, how much metadata
    check(_lib.kvc_load_prompt_cache(os.fsencode(path), device, None, 0, ctypes.byref(count), None, 0,
                                     ctypes.byref(need), _stream_ptr(stream)))
    n = int(count.value)
    arr = (_vp * max(n, 1))()
    buf = ctypes.create_string_buffer(max(int(need.value), 1))
    check(_lib.kvc_load_prompt_cache(os.fsencode(path), device, arr, n, ctypes.byref(count), buf, len(buf),
                                     ctypes.byref(need), _stream_ptr(stream)))
    torch_dev = None
    try:
        import torch
        if torch.cuda.is_available():
            torch_dev = torch.device("cuda", torch.cuda.current_device() if device < 0 else device)
    except Exception:
        pass
    caches = []
    for i in range(int(count.value)):
        h = int(ctypes.cast(arr[i], ctypes.c_void_p).value)
        kind = int(_lib.kvc_kind_of(ctypes.c_void_p(h)))
        cls = {KIND_SIMPLE: KVCacheSimple, KIND_ROTATING: RotatingKVCache, KIND_QUANTIZED: QuantizedKVCache,
               KIND_TURBO: TurboQuantKVCache, KIND_CHUNKED: ChunkedKVCache, KIND_LIST: CacheList}[kind]
        obj = cls.__new__(cls)
        KVCache.__init__(obj, h, torch_dev)
        caches.append(obj)
    parts = buf.raw[:max(int(need.value) - 2, 0)].decode().split("\0") if int(need.value) > 1 else []
    meta = {parts[i]: parts[i + 1] for i in range(0, len(parts) - 1, 2)}
    return caches, meta
