"""CPU oracle for the prompt-cache file format of mlx-swift-lm.

TEST INFRASTRUCTURE ONLY: nothing in the shipped package imports this module.

Restates savePromptCache / loadPromptCacheSnapshot / restoreCacheFromMetaState of
Libraries/MLXLMCommon/KVCache.swift (:1797-1846, :1873-1913, :2031-2138, :2140-2210)
over numpy arrays. A file is a safetensors container (published format: an 8-byte
little-endian header length, a JSON header {name: {dtype, shape, data_offsets}} with
the string map "__metadata__", then the raw little-endian tensor bytes) holding

    tensors    "i.j"     array j of cache i's `state`
    metadata   "0.i.j"   string j of cache i's `metaState`
               "1.key"   the caller's metadata
               "2.i"     the class name of cache i

The container itself is written by the un-vendored mlx-swift (`save(arrays:metadata:url:)`);
its byte layout here follows the published safetensors specification: parity of the container
bytes is unpinned, the key layout and the validation rules follow the reference tree.

bf16 arrays travel as uint16 bit patterns tagged "BF16" (numpy has no bfloat16), the same
convention as kvcache_oracle.
"""
from __future__ import annotations

import json
import struct
from typing import Dict, List, Sequence, Tuple

import numpy as np

STATE_PREFIX = "__mlx_lm_state_"          # reserved namespace of model-state entries (KVCache.swift:2016-2025)

_ST_OF = {np.dtype(np.float32): "F32", np.dtype(np.float16): "F16", np.dtype(np.uint32): "U32",
          np.dtype(np.uint8): "U8", np.dtype(np.int32): "I32", np.dtype(np.bool_): "BOOL"}
_NP_OF = {"F32": np.float32, "F16": np.float16, "U32": np.uint32, "U8": np.uint8, "I32": np.int32,
          "BOOL": np.bool_, "BF16": np.uint16}


class PromptCacheError(ValueError):
    """KVCacheError raised by the reference's loader."""


class Entry:
    """One cache of a file: class name, `state` arrays, `metaState` strings. `bf16[j]` says that
    array j (uint16) holds bf16 bit patterns."""

    def __init__(self, class_name: str, state: Sequence[np.ndarray], meta_state: Sequence[str],
                 bf16: Sequence[bool] = ()):
        self.class_name = class_name
        self.state = [np.ascontiguousarray(a) for a in state]
        self.meta_state = [str(m) for m in meta_state]
        self.bf16 = list(bf16) if bf16 else [False] * len(self.state)


def class_name_of(cache) -> str:
    """cacheClassName (KVCache.swift:1989-2010): the simple cache is stored under Python's name."""
    n = type(cache).__name__
    return "KVCache" if n == "KVCacheSimple" else n


def entry_of(cache, bf16: bool = False) -> Entry:
    """The (class, state, metaState) triple savePromptCache stores for an oracle cache. `bf16`
    marks uint16 state arrays as bf16 bit patterns."""
    st = list(cache.state)
    return Entry(class_name_of(cache), st, list(cache.meta_state),
                 [bf16 and a.dtype == np.uint16 for a in st])


def save(path: str, entries: Sequence[Entry], metadata: Dict[str, str] | None = None) -> None:
    """savePromptCache(url:cache:metadata:) without model state (KVCache.swift:1797-1846)."""
    metadata = dict(metadata or {})
    if any(k.startswith(STATE_PREFIX) for k in metadata):
        raise PromptCacheError("User metadata uses the reserved prompt cache state namespace")
    meta: Dict[str, str] = {}
    tensors: List[Tuple[str, np.ndarray, str]] = []
    for i, e in enumerate(entries):
        for j, a in enumerate(e.state):
            tag = "BF16" if e.bf16[j] else _ST_OF[a.dtype]
            tensors.append((f"{i}.{j}", a, tag))
        for j, m in enumerate(e.meta_state):
            meta[f"0.{i}.{j}"] = m
        meta[f"2.{i}"] = e.class_name
    for k, v in metadata.items():
        meta[f"1.{k}"] = v
    header: Dict[str, object] = {"__metadata__": meta}
    pos = 0
    for name, a, tag in tensors:
        header[name] = {"dtype": tag, "shape": list(a.shape), "data_offsets": [pos, pos + a.nbytes]}
        pos += a.nbytes
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for _, a, _ in tensors:
            f.write(a.tobytes())


def _read_container(path: str):
    raw = open(path, "rb").read()
    if len(raw) < 8:
        raise PromptCacheError("not a safetensors file")
    (hlen,) = struct.unpack("<Q", raw[:8])
    if 8 + hlen > len(raw):
        raise PromptCacheError("safetensors header exceeds the file")
    header = json.loads(raw[8:8 + hlen])
    meta = header.pop("__metadata__", {}) or {}
    body = raw[8 + hlen:]
    arrays: Dict[str, Tuple[np.ndarray, bool]] = {}
    for name, d in header.items():
        lo, hi = d["data_offsets"]
        dt = np.dtype(_NP_OF[d["dtype"]])
        n = int(np.prod(d["shape"], dtype=np.int64)) if d["shape"] else 1
        if hi - lo != n * dt.itemsize or hi > len(body):
            raise PromptCacheError(f"tensor '{name}' does not match its shape")
        arrays[name] = (np.frombuffer(body[lo:hi], dtype=dt).reshape(d["shape"]).copy(), d["dtype"] == "BF16")
    return arrays, meta


def _integers(values: Sequence[str], cls: str) -> List[int]:
    out = []
    for v in values:
        try:
            out.append(int(v))
        except ValueError:
            raise PromptCacheError(f"Corrupt prompt cache: {cls} metadata must contain integers.")
    return out


def _validate(cls: str, state, state_counts, meta, meta_counts) -> None:
    """validatePromptCache (KVCache.swift:2140-2154)."""
    if len(state) not in state_counts or len(meta) not in meta_counts or any(a.ndim != 4 for a in state):
        raise PromptCacheError(f"Corrupt prompt cache: invalid {cls} state or metadata shape.")


def check_entry(e: Entry) -> None:
    """The acceptance rules of restoreCacheFromMetaState (KVCache.swift:2031-2138) for the cache
    classes of the hot path; every other class name is outside it and reported as unknown."""
    c, st, ms = e.class_name, e.state, e.meta_state
    if c in ("KVCache", "KVCacheSimple"):
        _validate("KVCacheSimple", st, {0, 2}, ms, {1})
        if ms != [""]:
            raise PromptCacheError("Corrupt prompt cache: KVCacheSimple metadata must contain its single empty placeholder.")
    elif c == "RotatingKVCache":
        _validate(c, st, {0, 2}, ms, {5, 6})
        _integers(ms[:5], c)
        if len(ms) == 6 and ms[5] not in ("modelNative", "requested"):     # RotatingKVCache.CapacityOrigin
            raise PromptCacheError(f"Corrupt prompt cache: invalid RotatingKVCache capacity origin '{ms[5]}'.")
    elif c == "QuantizedKVCache":
        _validate(c, st, {0, 4, 6}, ms, {4})
        _integers(ms, c)
    elif c == "TurboQuantKVCache":
        if len(ms) < 5:
            raise PromptCacheError("Invalid TurboQuantKVCache metaState")
        try:
            [int(v) for v in ms[1:5]]
        except ValueError:
            raise PromptCacheError("Invalid TurboQuantKVCache metaState")
    else:
        raise PromptCacheError(f"Unknown cache class: {c}")


def load(path: str) -> Tuple[List[Entry], Dict[str, str]]:
    """loadPromptCache(url:) (KVCache.swift:1859-1913, unflatten helpers :2166-2260)."""
    arrays, meta = _read_container(path)
    info: Dict[int, Dict[int, str]] = {}
    classes: Dict[int, str] = {}
    user: Dict[str, str] = {}
    for k, v in meta.items():
        head, _, rest = k.partition(".")
        if head == "0":
            i, _, j = rest.partition(".")
            info.setdefault(int(i), {})[int(j)] = v
        elif head == "1":
            user[rest] = v
        elif head == "2":
            classes[int(rest)] = v
    if any(k.startswith(STATE_PREFIX) for k in user) or any(k.startswith(STATE_PREFIX) for k in arrays):
        raise PromptCacheError("Prompt cache contains model state; use loadPromptCacheSnapshot(url:) to restore it")
    n = len(classes)
    if sorted(classes) != list(range(n)) or len(info) != n:
        raise PromptCacheError("Mismatch in cache counts")
    per: Dict[int, Dict[int, Tuple[np.ndarray, bool]]] = {}
    for k, a in arrays.items():
        parts = k.split(".")
        if len(parts) != 2 or not all(p.isdigit() for p in parts) or int(parts[0]) >= n:
            raise PromptCacheError(f"Corrupt prompt cache: invalid array key '{k}'.")
        per.setdefault(int(parts[0]), {})[int(parts[1])] = a
    entries = []
    for i in range(n):
        got = per.get(i, {})
        if sorted(got) != list(range(len(got))):
            raise PromptCacheError(f"Corrupt prompt cache: missing array for cache {i}.")
        ms = info.get(i, {})
        if sorted(ms) != list(range(len(ms))):
            raise PromptCacheError("Invalid cache metadata format")
        e = Entry(classes[i], [got[j][0] for j in range(len(got))], [ms[j] for j in range(len(ms))],
                  [got[j][1] for j in range(len(got))])
        check_entry(e)
        entries.append(e)
    return entries, user
