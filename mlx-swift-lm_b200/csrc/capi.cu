// extern "C" surface of the library (include/kvcache_b200.h). Each entry point
// validates its arguments, runs the C++ implementation and converts exceptions
// into a status code plus a thread-local message, so nothing propagates across
// the C boundary.
#include "cache.h"

#include <string>
#include <utility>
#include <vector>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <memory>
#include <sstream>

namespace kvc {
int launch_attention(const AttnArgs &a, cudaStream_t stream);
void round_begin(kvc_cache *c, int max_positions, kvc_round **out);
void round_update(kvc_round *r, const kvc_tensor &k, const kvc_tensor &v, cudaStream_t s,
                  kvc_tensor *ok, kvc_tensor *ov);
void round_commit(kvc_round *r, int retain, cudaStream_t s);
int64_t rewind_last_round(kvc_cache *c, int64_t count, cudaStream_t s);
}  // namespace kvc

namespace {

thread_local std::string g_last_error;
thread_local bool g_has_error = false;

kvc_status set_error(kvc_status code, const std::string &msg) {
    g_last_error = msg;
    g_has_error = true;
    return code;
}

}  // namespace

extern "C" kvc_status kvc_internal_set_error(kvc_status code, const char *msg) {
    return set_error(code, msg ? msg : "");
}

namespace {

template <typename F>
kvc_status guarded(F &&f) {
    try {
        f();
        return KVC_OK;
    } catch (const kvc::Error &e) {
        return set_error(e.code, e.what());
    } catch (const std::bad_alloc &) {
        return set_error(KVC_ERR_OUT_OF_MEMORY, "host allocation failed");
    } catch (const std::exception &e) {
        return set_error(KVC_ERR_INTERNAL, e.what());
    } catch (...) {
        return set_error(KVC_ERR_INTERNAL, "unknown error");
    }
}

#define KVC_CHECK_HANDLE(h)                                                    \
    if (!(h)) return set_error(KVC_ERR_INVALID_ARG, "null handle: " #h)

cudaStream_t as_stream(void *s) { return (cudaStream_t)s; }

// Bind the handle's device for the duration of a call.
struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int device) {
        if (cudaGetDevice(&prev) != cudaSuccess) {
            // No device: pure bookkeeping calls still work; the first call that
            // needs device memory fails with KVC_ERR_CUDA (there is no CPU fallback).
            (void)cudaGetLastError();
            prev = -1;
            return;
        }
        if (device >= 0 && device != prev) KVC_CUDA(cudaSetDevice(device));
        else prev = -1;
    }
    ~DeviceGuard() {
        if (prev >= 0) (void)cudaSetDevice(prev);
    }
};

size_t tensor_bytes_contiguous(const kvc_tensor &t) {
    size_t n = 1;
    for (int i = 0; i < t.ndim; ++i) n *= (size_t)t.shape[i];
    return n * kvc::dtype_size(t.dtype);
}

bool is_contiguous(const kvc_tensor &t) {
    int64_t expect = 1;
    for (int i = t.ndim - 1; i >= 0; --i) {
        if (t.shape[i] != 1 && t.stride[i] != expect) return false;
        expect *= t.shape[i];
    }
    return true;
}

void *stage_get(kvc_cache *c, int slot, size_t bytes, cudaStream_t s) {
    if (c->stage_bytes[slot] >= bytes && c->stage[slot]) return c->stage[slot];
    if (c->stage[slot]) kvc::dev_free(c->stage[slot], s);
    size_t want = std::max<size_t>(bytes, 4096);
    c->stage[slot] = kvc::dev_alloc(want, s);
    c->stage_bytes[slot] = want;
    return c->stage[slot];
}

}  // namespace

extern "C" {

const char *kvc_version(void) { return "kvcache_b200 0.1.0 (sm_100a)"; }

const char *kvc_last_error_message(void) { return g_has_error ? g_last_error.c_str() : nullptr; }

int32_t kvc_device_available(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    if (n <= 0) return 0;
    int dev = 0, major = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) { (void)cudaGetLastError(); return 0; }
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    return major == 10 ? 1 : 0;
}

void kvc_config_default(kvc_config *cfg, int32_t kind) {
    if (!cfg) return;
    std::memset(cfg, 0, sizeof(*cfg));
    cfg->kind = kind;
    cfg->device = -1;
    cfg->step = 256;
    cfg->max_size = 0;
    cfg->keep = 0;
    cfg->group_size = 64;
    cfg->bits = kind == KVC_KIND_TURBO ? 4 : 8;
    cfg->key_bits = -1;
    cfg->value_bits = -1;
    cfg->key_group_size = 64;
    cfg->seed = 42;
    cfg->reserve_tokens = 0;
    cfg->turbo_affine_values = 0;
}

kvc_status kvc_create(const kvc_config *cfg, kvc_cache **out) {
    if (!cfg || !out) return set_error(KVC_ERR_INVALID_ARG, "kvc_create: null argument");
    *out = nullptr;
    return guarded([&] {
        KVC_REQUIRE(cfg->kind >= KVC_KIND_SIMPLE && cfg->kind <= KVC_KIND_CHUNKED,
                    "kvc_create: unknown kind (a CacheList is made by kvc_list_create)");
        KVC_REQUIRE(cfg->step > 0, "kvc_create: step must be positive");
        std::unique_ptr<kvc_cache> c(new kvc_cache());
        c->cfg = *cfg;
        c->device = cfg->device;
        if (cfg->kind == KVC_KIND_ROTATING) {
            KVC_REQUIRE(cfg->max_size > 0, "RotatingKVCache requires a positive maxSize");
            KVC_REQUIRE(cfg->keep >= 0 && cfg->keep < cfg->max_size, "RotatingKVCache: keep must be in [0, maxSize)");
        }
        if (cfg->kind == KVC_KIND_QUANTIZED) {
            KVC_REQUIRE(cfg->bits == 2 || cfg->bits == 4 || cfg->bits == 8,
                        "QuantizedKVCache: this build packs 2, 4 or 8 bits");
            c->group_size = cfg->group_size;
            c->bits = cfg->bits;
            c->cfg.step = 256;  // QuantizedKVCache.step is a constant (KVCache.swift:934)
        }
        if (cfg->kind == KVC_KIND_TURBO) {
            const int kb = cfg->key_bits < 0 ? cfg->bits : cfg->key_bits;
            const int vb = cfg->value_bits < 0 ? cfg->bits : cfg->value_bits;
            c->key_bits = kb;
            c->value_bits = vb;
            c->raw_key = kb == 0;
            c->affine_key = kb == 8;
            c->affine_value = cfg->turbo_affine_values != 0;
            c->key_group = cfg->key_group_size > 0 ? cfg->key_group_size : 64;
            KVC_REQUIRE(c->raw_key || c->affine_key || (kb >= 1 && kb <= 4), "TurboQuant: key bits must be 0, 1..4 or 8");
            if (c->affine_value) KVC_REQUIRE(vb == 2 || vb == 4 || vb == 8, "affine values need 2, 4 or 8 bits");
            else KVC_REQUIRE(vb >= 1 && vb <= 4, "TurboQuant: value bits must be 1..4");
            c->cfg.step = 256;  // TurboQuantKVCache.step is a constant (TurboQuantKVCache.swift:693)
        }
        *out = c.release();
    });
}

void kvc_free(kvc_cache *cache) {
    if (!cache) return;
    try {
        if (cache->open_round) cache->open_round->cache = nullptr;
        delete cache;   // frees in the order of the handle's last stream, on the handle's device
    } catch (...) {
    }
}

kvc_status kvc_list_create(kvc_cache *const *children, int32_t count, kvc_cache **out) {
    if (!out || (count > 0 && !children)) return set_error(KVC_ERR_INVALID_ARG, "kvc_list_create: null argument");
    *out = nullptr;
    return guarded([&] {
        KVC_REQUIRE(count >= 0, "kvc_list_create: negative count");
        for (int i = 0; i < count; ++i) {
            KVC_REQUIRE(children[i] != nullptr, "kvc_list_create: null child");
            for (int j = 0; j < i; ++j) KVC_REQUIRE(children[i] != children[j], "kvc_list_create: a child appears twice");
        }
        std::unique_ptr<kvc_cache> c(new kvc_cache());
        kvc_config_default(&c->cfg, KVC_KIND_LIST);
        c->device = count > 0 ? children[0]->device : -1;
        c->children.assign(children, children + count);
        *out = c.release();
    });
}

int32_t kvc_list_count(const kvc_cache *list) {
    return (list && list->cfg.kind == KVC_KIND_LIST) ? (int32_t)list->children.size() : -1;
}

kvc_cache *kvc_list_child(const kvc_cache *list, int32_t index) {
    if (!list || list->cfg.kind != KVC_KIND_LIST || index < 0 || index >= (int32_t)list->children.size()) return nullptr;
    return list->children[(size_t)index];
}

kvc_status kvc_maybe_trim_front(kvc_cache *c, void *stream) {
    KVC_CHECK_HANDLE(c);
    return guarded([&] {
        DeviceGuard dg(c->device);
        kvc::cache_maybe_trim_front(c, as_stream(stream));
    });
}

int64_t kvc_start_position(const kvc_cache *c) { return (c && c->cfg.kind == KVC_KIND_CHUNKED) ? c->start_position : 0; }

kvc_status kvc_prepare(kvc_cache *c, const int32_t *lengths, int32_t count) {
    KVC_CHECK_HANDLE(c);
    (void)lengths; (void)count;   // BaseKVCache.prepare(lengths:) is empty for these cache kinds (KVCache.swift:229-231)
    if (c->cfg.kind == KVC_KIND_LIST)
        for (kvc_cache *child : c->children) (void)kvc_prepare(child, lengths, count);
    return KVC_OK;
}

kvc_status kvc_finalize(kvc_cache *c) {
    KVC_CHECK_HANDLE(c);
    if (c->cfg.kind == KVC_KIND_LIST)
        for (kvc_cache *child : c->children) (void)kvc_finalize(child);
    return KVC_OK;
}

kvc_status kvc_create_causal_mask(int32_t n, int64_t offset, int64_t window_size, const int32_t *lengths_dev, int32_t batch,
                                  void *out_mask, void *stream) {
    if (!out_mask) return set_error(KVC_ERR_INVALID_ARG, "kvc_create_causal_mask: null output");
    return guarded([&] {
        KVC_REQUIRE(n >= 0 && offset >= 0, "kvc_create_causal_mask: negative size");
        if (lengths_dev) {
            KVC_REQUIRE(batch > 0, "kvc_create_causal_mask: lengths need a batch size");
            kvc::launch_causal_mask_lengths((uint8_t *)out_mask, n, offset, window_size, lengths_dev, batch, as_stream(stream));
        } else {
            kvc::launch_causal_mask((uint8_t *)out_mask, n, offset, window_size, as_stream(stream));
        }
    });
}

int64_t kvc_offset(const kvc_cache *c) { return c ? c->offset : -1; }
kvc_status kvc_set_offset(kvc_cache *c, int64_t offset) {
    KVC_CHECK_HANDLE(c);
    c->offset = offset;
    c->restore.valid = false;
    return KVC_OK;
}
int64_t kvc_max_size(const kvc_cache *c) {
    if (!c) return -1;
    return c->cfg.kind == KVC_KIND_ROTATING ? c->cfg.max_size : -1;
}
int32_t kvc_kind_of(const kvc_cache *c) { return c ? c->cfg.kind : -1; }
int64_t kvc_ring_index(const kvc_cache *c) {
    if (!c || c->cfg.kind != KVC_KIND_ROTATING) return -1;
    return c->idx;
}
int32_t kvc_group_size(const kvc_cache *c) {
    if (!c) return -1;
    return c->cfg.kind == KVC_KIND_TURBO ? c->key_group : c->group_size;
}
int32_t kvc_bits(const kvc_cache *c) {
    if (!c) return -1;
    return c->cfg.kind == KVC_KIND_TURBO ? c->cfg.bits : c->bits;
}
int32_t kvc_is_compressed(const kvc_cache *c) { return (c && c->compressed) ? 1 : 0; }

int64_t kvc_memory_bytes(const kvc_cache *c) {
    if (!c) return 0;
    int64_t total = 0;
    const kvc::Array4 *arrays[] = {&c->k, &c->v, &c->k_alt, &c->v_alt, &c->k_view, &c->v_view,
                                   &c->kq, &c->ks, &c->kb, &c->vq, &c->vs, &c->vb,
                                   &c->kp, &c->kn, &c->vp, &c->vn};
    for (auto *a : arrays)
        if (a->allocated()) total += (int64_t)a->bytes();
    return total;
}

kvc_status kvc_reserve(kvc_cache *c, int64_t tokens, int32_t batch, int32_t kv_heads,
                       int32_t head_dim, int32_t dtype, void *stream) {
    KVC_CHECK_HANDLE(c);
    return guarded([&] {
        DeviceGuard dg(c->device);
        cudaStream_t s = as_stream(stream);
        KVC_REQUIRE(tokens >= 0 && batch > 0 && kv_heads > 0 && head_dim > 0, "kvc_reserve: bad shape");
        c->cfg.reserve_tokens = std::max<int64_t>(c->cfg.reserve_tokens, tokens);
        const int64_t step = std::max<int32_t>(c->cfg.step, 1);
        switch (c->cfg.kind) {
            case KVC_KIND_SIMPLE:
            case KVC_KIND_TURBO:
                if (c->cfg.kind == KVC_KIND_TURBO && c->compressed) return;
                if (!c->k.allocated()) {
                    if (c->offset != 0) return;
                    // only pre-allocate the raw arrays of a turbo cache when asked
                    // through kvc_update; a compressed-from-start turbo cache uses
                    // reserve_tokens when it first allocates.
                    if (c->cfg.kind == KVC_KIND_TURBO) return;
                    KVC_REQUIRE(kvc::is_float_dtype(dtype), "kvc_reserve: dtype must be floating");
                    c->k.alloc(batch, kv_heads, std::max<int64_t>(tokens, 1), head_dim, dtype, s);
                    c->v.alloc(batch, kv_heads, std::max<int64_t>(tokens, 1), head_dim, dtype, s);
                } else {
                    c->k.ensure(tokens, c->offset, step, s);
                    c->v.ensure(tokens, c->offset, step, s);
                }
                return;
            case KVC_KIND_QUANTIZED:
                if (c->kq.allocated())
                    for (kvc::Array4 *a : {&c->kq, &c->ks, &c->kb, &c->vq, &c->vs, &c->vb})
                        a->ensure(tokens, c->offset, step, s);
                return;
            default: return;  // a rotating cache is bounded by maxSize
        }
    });
}

kvc_status kvc_update(kvc_cache *c, const kvc_tensor *keys, const kvc_tensor *values, void *stream,
                      kvc_tensor *out_k, kvc_tensor *out_v) {
    KVC_CHECK_HANDLE(c);
    if (!keys || !values) return set_error(KVC_ERR_INVALID_ARG, "kvc_update: null tensor");
    return guarded([&] {
        DeviceGuard dg(c->device);
        kvc::cache_update(c, *keys, *values, as_stream(stream), out_k, out_v);
    });
}

kvc_status kvc_update_quantized(kvc_cache *c, const kvc_tensor *keys, const kvc_tensor *values,
                                void *stream, kvc_tensor out_k[3], kvc_tensor out_v[3]) {
    KVC_CHECK_HANDLE(c);
    if (!keys || !values) return set_error(KVC_ERR_INVALID_ARG, "kvc_update_quantized: null tensor");
    return guarded([&] {
        DeviceGuard dg(c->device);
        kvc::cache_update_quantized(c, *keys, *values, as_stream(stream), out_k, out_v);
    });
}

kvc_status kvc_quantized_state(kvc_cache *c, kvc_tensor out_k[3], kvc_tensor out_v[3]) {
    KVC_CHECK_HANDLE(c);
    return guarded([&] {
        KVC_REQUIRE(c->cfg.kind == KVC_KIND_QUANTIZED, "getQuantizedState needs a QuantizedKVCache");
        if (!c->kq.allocated()) kvc::fail(KVC_ERR_INVALID_STATE, "getQuantizedState: the cache is empty");
        if (out_k) { out_k[0] = c->kq.view(c->offset); out_k[1] = c->ks.view(c->offset); out_k[2] = c->kb.view(c->offset); }
        if (out_v) { out_v[0] = c->vq.view(c->offset); out_v[1] = c->vs.view(c->offset); out_v[2] = c->vb.view(c->offset); }
    });
}

kvc_status kvc_attention(kvc_cache *c, const kvc_tensor *q, const kvc_tensor *k, const kvc_tensor *v,
                         float scale, int32_t mask_mode, const kvc_tensor *mask,
                         const kvc_tensor *out, void *stream) {
    KVC_CHECK_HANDLE(c);
    if (!q || !k || !v || !out) return set_error(KVC_ERR_INVALID_ARG, "kvc_attention: null tensor");
    return guarded([&] {
        DeviceGuard dg(c->device);
        kvc::cache_attention(c, *q, *k, *v, scale, mask_mode, mask, *out, as_stream(stream));
    });
}

namespace {
// Copy streams and a growing set of reusable events per device for the host-buffer batch call.
struct SidePipe {
    cudaStream_t h2d = nullptr, d2h = nullptr;
    std::vector<cudaEvent_t> events;
};

SidePipe &side_pipe(int device, size_t need_events) {
    static thread_local SidePipe pipes[64];
    KVC_REQUIRE(device >= 0 && device < 64, "device index out of range");
    SidePipe &p = pipes[device];
    if (!p.h2d) {
        KVC_CUDA(cudaStreamCreateWithFlags(&p.h2d, cudaStreamNonBlocking));
        KVC_CUDA(cudaStreamCreateWithFlags(&p.d2h, cudaStreamNonBlocking));
    }
    while (p.events.size() < need_events) {
        cudaEvent_t e;
        KVC_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        p.events.push_back(e);
    }
    return p;
}
}  // namespace

kvc_status kvc_attention_host(kvc_cache *c, const kvc_tensor *q, const kvc_tensor *k,
                              const kvc_tensor *v, float scale, int32_t mask_mode,
                              const kvc_tensor *mask, const kvc_tensor *out, void *stream,
                              int32_t synchronize) {
    KVC_CHECK_HANDLE(c);
    if (!q || !k || !v || !out) return set_error(KVC_ERR_INVALID_ARG, "kvc_attention_host: null tensor");
    return guarded([&] {
        DeviceGuard dg(c->device);
        cudaStream_t s = as_stream(stream);
        KVC_REQUIRE(is_contiguous(*q) && is_contiguous(*k) && is_contiguous(*v) && is_contiguous(*out),
                    "kvc_attention_host: host tensors must be contiguous");
        const size_t qb = tensor_bytes_contiguous(*q), kb = tensor_bytes_contiguous(*k),
                     vb = tensor_bytes_contiguous(*v), ob = tensor_bytes_contiguous(*out);
        auto al = [](size_t x) { return (x + 255) / 256 * 256; };
        // one staging slab: q | k | v | out
        char *slab = (char *)stage_get(c, 0, al(qb) + al(kb) + al(vb) + al(ob), s);
        char *dq = slab, *dk = dq + al(qb), *dv = dk + al(kb), *dout = dv + al(vb);
        KVC_CUDA(cudaMemcpyAsync(dq, q->data, qb, cudaMemcpyHostToDevice, s));
        KVC_CUDA(cudaMemcpyAsync(dk, k->data, kb, cudaMemcpyHostToDevice, s));
        KVC_CUDA(cudaMemcpyAsync(dv, v->data, vb, cudaMemcpyHostToDevice, s));
        kvc_tensor tq = *q, tk = *k, tv = *v, to = *out, tm;
        tq.data = dq; tk.data = dk; tv.data = dv; to.data = dout;
        const kvc_tensor *pm = nullptr;
        if (mask_mode == KVC_MASK_ARRAY) {
            KVC_REQUIRE(mask && is_contiguous(*mask), "kvc_attention_host: array mask must be contiguous");
            const size_t mb = tensor_bytes_contiguous(*mask);
            void *dm = stage_get(c, 1, mb, s);
            KVC_CUDA(cudaMemcpyAsync(dm, mask->data, mb, cudaMemcpyHostToDevice, s));
            tm = *mask;
            tm.data = dm;
            pm = &tm;
        }
        kvc::cache_attention(c, tq, tk, tv, scale, mask_mode, pm, to, s);
        KVC_CUDA(cudaMemcpyAsync(out->data, dout, ob, cudaMemcpyDeviceToHost, s));
        if (synchronize) KVC_CUDA(cudaStreamSynchronize(s));
    });
}

kvc_status kvc_sdpa(const kvc_tensor *q, const kvc_tensor *k, const kvc_tensor *v, float scale,
                    int32_t mask_mode, const kvc_tensor *mask, const kvc_tensor *out, void *stream) {
    if (!q || !k || !v || !out) return set_error(KVC_ERR_INVALID_ARG, "kvc_sdpa: null tensor");
    return guarded([&] {
        DeviceGuard dg(-1);
        KVC_REQUIRE(k->ndim == 4 && v->ndim == 4, "kvc_sdpa: keys/values must be [B, Hkv, T, D]");
        KVC_REQUIRE(k->dtype == v->dtype && k->dtype == q->dtype, "kvc_sdpa: dtypes must match");
        KVC_REQUIRE(k->stride[3] == 1 && v->stride[3] == 1, "kvc_sdpa: keys/values must be contiguous along the head dim");
        KVC_REQUIRE(k->shape[2] == v->shape[2] && k->shape[1] == v->shape[1], "kvc_sdpa: keys and values disagree");
        KVC_REQUIRE(k->shape[3] == q->shape[3] && v->shape[3] == q->shape[3], "kvc_sdpa: head dims must match");
        kvc::AttnArgs a = kvc::make_attn_args(*q, *out, scale, mask_mode, mask, k->shape[2], (int)k->shape[1]);
        a.k = kvc::raw_source(*k);
        a.v = kvc::raw_source(*v);
        kvc::launch_attention(a, as_stream(stream));
    });
}

kvc_status kvc_quantized_sdpa(const kvc_tensor *q, const kvc_tensor qk[3], const kvc_tensor qv[3],
                              float scale, int32_t mask_mode, const kvc_tensor *mask,
                              int32_t group_size, int32_t bits, const kvc_tensor *out, void *stream) {
    if (!q || !qk || !qv || !out) return set_error(KVC_ERR_INVALID_ARG, "kvc_quantized_sdpa: null tensor");
    return guarded([&] {
        DeviceGuard dg(-1);
        KVC_REQUIRE(bits == 2 || bits == 4 || bits == 8, "quantized SDPA: bits must be 2, 4 or 8");
        for (int i = 0; i < 3; ++i)
            KVC_REQUIRE(qk[i].ndim == 4 && qv[i].ndim == 4 && qk[i].stride[3] == 1 && qv[i].stride[3] == 1,
                        "quantized SDPA: quantized tuples must be 4-d and contiguous along the last dim");
        KVC_REQUIRE(qk[0].dtype == KVC_U32 && qv[0].dtype == KVC_U32, "quantized SDPA: codes must be uint32");
        KVC_REQUIRE(qk[0].shape[3] * 32 / bits == q->shape[3], "quantized SDPA: key codes do not match the head dim");
        KVC_REQUIRE(qv[0].shape[3] * 32 / bits == q->shape[3], "quantized SDPA: value head dim must equal the query head dim");
        kvc::AttnArgs a = kvc::make_attn_args(*q, *out, scale, mask_mode, mask, qk[0].shape[2], (int)qk[0].shape[1]);
        auto src = [&](const kvc_tensor t[3]) {
            kvc::KVSource s;
            s.kind = kvc::SRC_AFFINE;
            s.dtype = t[1].dtype;
            s.data = t[0].data; s.scales = t[1].data; s.biases = t[2].data;
            s.sb = t[0].stride[0]; s.sh = t[0].stride[1]; s.st = t[0].stride[2];
            s.gsb = t[1].stride[0]; s.gsh = t[1].stride[1]; s.gst = t[1].stride[2];
            s.bits = bits; s.group = group_size; s.words = (int)t[0].shape[3];
            return s;
        };
        a.k = src(qk);
        a.v = src(qv);
        kvc::launch_attention(a, as_stream(stream));
    });
}

static kvc_tensor flatten_rows(const kvc_tensor &t) {
    // [..., W] contiguous -> [1, 1, rows, W]
    kvc_tensor o{};
    int64_t rows = 1;
    for (int i = 0; i + 1 < t.ndim; ++i) rows *= t.shape[i];
    o.data = t.data; o.dtype = t.dtype; o.ndim = 4;
    o.shape[0] = 1; o.shape[1] = 1; o.shape[2] = rows; o.shape[3] = t.shape[t.ndim - 1];
    o.stride[3] = 1; o.stride[2] = o.shape[3]; o.stride[1] = rows * o.shape[3]; o.stride[0] = o.stride[1];
    return o;
}

kvc_status kvc_affine_quantize(const kvc_tensor *x, int32_t group_size, int32_t bits,
                               const kvc_tensor *codes, const kvc_tensor *scales,
                               const kvc_tensor *biases, void *stream) {
    if (!x || !codes || !scales || !biases) return set_error(KVC_ERR_INVALID_ARG, "kvc_affine_quantize: null tensor");
    return guarded([&] {
        DeviceGuard dg(-1);
        KVC_REQUIRE(is_contiguous(*x) && is_contiguous(*codes) && is_contiguous(*scales) && is_contiguous(*biases),
                    "kvc_affine_quantize: tensors must be contiguous");
        KVC_REQUIRE(x->ndim >= 1 && x->ndim <= KVC_MAX_DIMS, "kvc_affine_quantize: bad rank");
        kvc_tensor fx = flatten_rows(*x), fc = flatten_rows(*codes), fs = flatten_rows(*scales);
        const int D = (int)fx.shape[3];
        KVC_REQUIRE(group_size > 0 && D % group_size == 0, "kvc_affine_quantize: last dim must be a multiple of the group size");
        KVC_REQUIRE(fc.shape[2] == fx.shape[2] && fc.shape[3] == (int64_t)D * bits / 32 && codes->dtype == KVC_U32,
                    "kvc_affine_quantize: codes must be uint32 [..., D*bits/32]");
        KVC_REQUIRE(fs.shape[2] == fx.shape[2] && fs.shape[3] == D / group_size && scales->dtype == x->dtype &&
                        biases->dtype == x->dtype,
                    "kvc_affine_quantize: scales/biases must be [..., D/group] in the input dtype");
        kvc::QuantAppendArgs a;
        a.src = fx.data; a.dtype = fx.dtype;
        a.s_sb = 0; a.s_sh = 0; a.s_ss = D; a.s_sd = 1;
        a.codes = (uint32_t *)fc.data; a.scales = scales->data; a.biases = biases->data;
        a.c_sb = 0; a.c_sh = 0; a.c_st = fc.shape[3];
        a.g_sb = 0; a.g_sh = 0; a.g_st = fs.shape[3];
        a.B = 1; a.H = 1; a.S = (int)fx.shape[2]; a.D = D;
        a.group = group_size; a.bits = bits; a.pos = 0;
        kvc::launch_affine_quantize(a, as_stream(stream));
    });
}

kvc_status kvc_affine_dequantize(const kvc_tensor *codes, const kvc_tensor *scales,
                                 const kvc_tensor *biases, int32_t group_size, int32_t bits,
                                 const kvc_tensor *out, void *stream) {
    if (!codes || !scales || !biases || !out) return set_error(KVC_ERR_INVALID_ARG, "kvc_affine_dequantize: null tensor");
    return guarded([&] {
        DeviceGuard dg(-1);
        KVC_REQUIRE(is_contiguous(*codes) && is_contiguous(*scales) && is_contiguous(*biases) && is_contiguous(*out),
                    "kvc_affine_dequantize: tensors must be contiguous");
        kvc_tensor fo = flatten_rows(*out), fc = flatten_rows(*codes), fs = flatten_rows(*scales);
        const int D = (int)fo.shape[3];
        KVC_REQUIRE(fc.shape[3] == (int64_t)D * bits / 32 && fs.shape[3] == D / group_size, "kvc_affine_dequantize: shape mismatch");
        kvc::DequantArgs d;
        d.codes = (const uint32_t *)codes->data; d.scales = scales->data; d.biases = biases->data;
        d.out = out->data; d.dtype = out->dtype; d.rows = fo.shape[2];
        d.c_srow = fc.shape[3]; d.g_srow = fs.shape[3]; d.o_srow = D;
        d.D = D; d.group = group_size; d.bits = bits;
        kvc::launch_affine_dequantize(d, as_stream(stream));
    });
}

kvc_status kvc_trim(kvc_cache *c, int64_t n, int64_t *out_trimmed) {
    KVC_CHECK_HANDLE(c);
    return guarded([&] {
        const int64_t t = kvc::cache_trim(c, n);
        if (out_trimmed) *out_trimmed = t;
    });
}

int32_t kvc_is_trimmable(const kvc_cache *c) { return c ? (kvc::cache_is_trimmable_after(c, 0) ? 1 : 0) : 0; }
int32_t kvc_is_trimmable_after(const kvc_cache *c, int64_t positions) {
    return c ? (kvc::cache_is_trimmable_after(c, positions) ? 1 : 0) : 0;
}

int32_t kvc_can_trim_prompt_cache(kvc_cache *const *caches, int32_t count) {
    // canTrimPromptCache (KVCache.swift:2293-2295)
    if (!caches) return 0;
    for (int i = 0; i < count; ++i)
        if (!caches[i] || !kvc_is_trimmable(caches[i])) return 0;
    return 1;
}

kvc_status kvc_trim_prompt_cache(kvc_cache *const *caches, int32_t count, int64_t n, int64_t *out_trimmed) {
    // trimPromptCache (KVCache.swift:2302-2306): all-or-nothing, returns the first cache's count
    if (out_trimmed) *out_trimmed = 0;
    if (!caches || count <= 0) return KVC_OK;
    if (!kvc_can_trim_prompt_cache(caches, count)) return KVC_OK;
    return guarded([&] {
        int64_t first = 0;
        for (int i = 0; i < count; ++i) {
            const int64_t t = kvc::cache_trim(caches[i], n);
            if (i == 0) first = t;
        }
        if (out_trimmed) *out_trimmed = first;
    });
}

kvc_status kvc_make_mask(const kvc_cache *c, int32_t n, int64_t window_size, int32_t return_array,
                         int32_t *out_mode, int64_t *out_rows, int64_t *out_cols, void *out_mask,
                         void *stream) {
    KVC_CHECK_HANDLE(c);
    if (!out_mode || !out_rows || !out_cols) return set_error(KVC_ERR_INVALID_ARG, "kvc_make_mask: null output");
    return guarded([&] {
        if (out_mask) {
            DeviceGuard dg(c->device);
            kvc::cache_make_mask(c, n, window_size, return_array != 0, out_mode, out_rows, out_cols, out_mask,
                                 as_stream(stream));
        } else {
            kvc::cache_make_mask(c, n, window_size, return_array != 0, out_mode, out_rows, out_cols, nullptr,
                                 nullptr);
        }
    });
}

int32_t kvc_state_count(const kvc_cache *c) { return c ? kvc::cache_state_count(c) : 0; }

kvc_status kvc_state_get(kvc_cache *c, int32_t index, kvc_tensor *out) {
    KVC_CHECK_HANDLE(c);
    if (!out) return set_error(KVC_ERR_INVALID_ARG, "kvc_state_get: null output");
    return guarded([&] { *out = kvc::cache_state_get(c, index); });
}

kvc_status kvc_state_set(kvc_cache *c, const kvc_tensor *arrays, int32_t count, void *stream) {
    KVC_CHECK_HANDLE(c);
    if (!arrays && count > 0) return set_error(KVC_ERR_INVALID_ARG, "kvc_state_set: null arrays");
    return guarded([&] {
        DeviceGuard dg(c->device);
        kvc::cache_state_set(c, arrays, count, as_stream(stream));
    });
}

kvc_status kvc_state_export(kvc_cache *c, int32_t index, void *host_dst, size_t host_bytes,
                            kvc_tensor *out_desc, void *stream) {
    KVC_CHECK_HANDLE(c);
    return guarded([&] {
        DeviceGuard dg(c->device);
        cudaStream_t s = as_stream(stream);
        kvc_tensor t = kvc::cache_state_get(c, index);
        const int nd = t.ndim;
        if (nd < 3) {
            // a plain vector (the TurboQuant key-calibration scale): one contiguous copy
            int64_t count = 1;
            for (int i = 0; i < nd; ++i) count *= t.shape[i];
            const size_t bytes = (size_t)count * kvc::dtype_size(t.dtype);
            if (out_desc) {
                *out_desc = t;
                out_desc->data = host_dst;
            }
            if (!host_dst) return;
            KVC_REQUIRE(host_bytes >= bytes, "kvc_state_export: destination too small");
            KVC_CUDA(cudaMemcpyAsync(host_dst, t.data, bytes, cudaMemcpyDeviceToHost, s));
            KVC_CUDA(cudaStreamSynchronize(s));
            return;
        }
        const int64_t W = nd == 4 ? t.shape[3] : 1;
        const size_t es = kvc::dtype_size(t.dtype);
        const size_t need = (size_t)(t.shape[0] * t.shape[1] * t.shape[2] * W) * es;
        if (out_desc) {
            *out_desc = t;
            out_desc->data = host_dst;
            // contiguous strides of the exported copy
            int64_t st = 1;
            for (int i = nd - 1; i >= 0; --i) { out_desc->stride[i] = st; st *= t.shape[i]; }
        }
        if (!host_dst) return;
        KVC_REQUIRE(host_bytes >= need, "kvc_state_export: destination too small");
        if (need == 0) return;
        // rows of one (batch, head) plane are contiguous: a pitched 2-D copy packs the planes
        const size_t width = (size_t)(t.shape[2] * W) * es;
        const size_t spitch = (size_t)t.stride[1] * es;
        KVC_CUDA(cudaMemcpy2DAsync(host_dst, width, t.data, spitch, width,
                                   (size_t)(t.shape[0] * t.shape[1]), cudaMemcpyDeviceToHost, s));
        KVC_CUDA(cudaStreamSynchronize(s));
    });
}

kvc_status kvc_meta_state(const kvc_cache *c, char *buf, size_t buf_len, size_t *out_len) {
    KVC_CHECK_HANDLE(c);
    return guarded([&] {
        auto m = kvc::cache_meta_state(c);
        std::string joined;
        for (size_t i = 0; i < m.size(); ++i) {
            if (i) joined += '\n';
            joined += m[i];
        }
        if (out_len) *out_len = joined.size() + 1;
        if (buf && buf_len > 0) {
            const size_t n = std::min(buf_len - 1, joined.size());
            std::memcpy(buf, joined.data(), n);
            buf[n] = '\0';
            if (n < joined.size()) kvc::fail(KVC_ERR_INVALID_ARG, "kvc_meta_state: buffer too small");
        }
    });
}

kvc_status kvc_set_meta_state(kvc_cache *c, const char *joined) {
    KVC_CHECK_HANDLE(c);
    if (!joined) return set_error(KVC_ERR_INVALID_ARG, "kvc_set_meta_state: null string");
    return guarded([&] {
        std::vector<std::string> m;
        std::string cur;
        for (const char *p = joined;; ++p) {
            if (*p == '\n' || *p == '\0') {
                m.push_back(cur);
                cur.clear();
                if (*p == '\0') break;
            } else {
                cur += *p;
            }
        }
        kvc::cache_set_meta_state(c, m);
    });
}

kvc_status kvc_copy(const kvc_cache *c, void *stream, kvc_cache **out) {
    KVC_CHECK_HANDLE(c);
    if (!out) return set_error(KVC_ERR_INVALID_ARG, "kvc_copy: null output");
    *out = nullptr;
    return guarded([&] {
        DeviceGuard dg(c->device);
        *out = kvc::cache_copy(c, as_stream(stream));
    });
}

kvc_status kvc_to_quantized(const kvc_cache *c, int32_t group_size, int32_t bits, void *stream, kvc_cache **out) {
    KVC_CHECK_HANDLE(c);
    if (!out) return set_error(KVC_ERR_INVALID_ARG, "kvc_to_quantized: null output");
    *out = nullptr;
    return guarded([&] {
        DeviceGuard dg(c->device);
        KVC_REQUIRE(bits == 2 || bits == 4 || bits == 8, "toQuantized: this build packs 2, 4 or 8 bits");
        *out = kvc::cache_to_quantized(c, group_size, bits, as_stream(stream));
    });
}

kvc_status kvc_to_unquantized(const kvc_cache *c, void *stream, kvc_cache **out) {
    KVC_CHECK_HANDLE(c);
    if (!out) return set_error(KVC_ERR_INVALID_ARG, "kvc_to_unquantized: null output");
    *out = nullptr;
    return guarded([&] {
        DeviceGuard dg(c->device);
        *out = kvc::cache_to_unquantized(c, as_stream(stream));
    });
}

kvc_status kvc_to_turbo(const kvc_cache *c, int32_t key_bits, int32_t value_bits, int32_t key_group_size,
                        void *stream, kvc_cache **out) {
    KVC_CHECK_HANDLE(c);
    if (!out) return set_error(KVC_ERR_INVALID_ARG, "kvc_to_turbo: null output");
    *out = nullptr;
    return guarded([&] {
        DeviceGuard dg(c->device);
        *out = kvc::cache_to_turbo(c, key_bits, value_bits, key_group_size, as_stream(stream));
    });
}

// ---------------------------------------------------------------------
// prompt-cache files
// ---------------------------------------------------------------------
kvc_status kvc_save_prompt_cache(const char *path, kvc_cache *const *caches, int32_t count,
                                 const char *const *meta_keys, const char *const *meta_values, int32_t meta_count,
                                 void *stream) {
    if (!path || (!caches && count > 0) || ((!meta_keys || !meta_values) && meta_count > 0))
        return set_error(KVC_ERR_INVALID_ARG, "kvc_save_prompt_cache: null argument");
    for (int i = 0; i < count; ++i) KVC_CHECK_HANDLE(caches[i]);
    return guarded([&] {
        DeviceGuard dg(count > 0 ? caches[0]->device : -1);
        kvc::save_prompt_cache(path, caches, count, meta_keys, meta_values, meta_count, as_stream(stream));
    });
}

kvc_status kvc_load_prompt_cache(const char *path, int32_t device, kvc_cache **out_caches, int32_t capacity,
                                 int32_t *out_count, char *meta_buf, size_t meta_len, size_t *meta_needed,
                                 void *stream) {
    if (!path || !out_count) return set_error(KVC_ERR_INVALID_ARG, "kvc_load_prompt_cache: null argument");
    *out_count = 0;
    return guarded([&] {
        DeviceGuard dg(device);
        std::vector<kvc_cache *> caches;
        std::vector<std::pair<std::string, std::string>> meta;
        kvc::load_prompt_cache(path, device, caches, meta, as_stream(stream));
        // NUL-terminated strings, key then value, closed by an empty key: values may hold any text
        std::string joined;
        for (size_t i = 0; i < meta.size(); ++i) {
            joined += meta[i].first;
            joined += '\0';
            joined += meta[i].second;
            joined += '\0';
        }
        joined += '\0';
        if (meta_needed) *meta_needed = joined.size();
        if (meta_buf && meta_len) {
            if (meta_len >= joined.size()) std::memcpy(meta_buf, joined.data(), joined.size());
            else std::memset(meta_buf, 0, meta_len);   // too small: reads as "no entries"
        }
        if ((int)caches.size() > capacity || !out_caches) {
            for (kvc_cache *c : caches) kvc_free(c);
            *out_count = (int32_t)caches.size();
            if (out_caches) kvc::fail(KVC_ERR_INVALID_ARG, "kvc_load_prompt_cache: the file holds more caches than `capacity`");
            return;
        }
        for (size_t i = 0; i < caches.size(); ++i) out_caches[i] = caches[i];
        *out_count = (int32_t)caches.size();
    });
}

// ---------------------------------------------------------------------
// list-level dynamic conversion
// ---------------------------------------------------------------------
int32_t kvc_resolve_turbo_scheme(const char *scheme, int32_t *key_bits, int32_t *value_bits) {
    if (!scheme) return 0;
    static const struct { const char *name; int kb, vb; } table[] = {
        {"turbo0v4", 0, 4}, {"turbo0v3", 0, 3}, {"turbo0v2", 0, 2}, {"turbo8v4", 8, 4}, {"turbo8v3", 8, 3},
        {"turbo8v2", 8, 2}, {"turbo4", 4, 4},   {"turbo4v2", 4, 2}, {"turbo3", 3, 3},   {"turbo2", 2, 2}};
    for (const auto &e : table)
        if (std::strcmp(scheme, e.name) == 0) {
            if (key_bits) *key_bits = e.kb;
            if (value_bits) *value_bits = e.vb;
            return 1;
        }
    return 0;
}

int32_t kvc_resolve_affine_scheme(const char *scheme, int32_t *bits, int32_t *group_size) {
    if (!scheme) return 0;
    int b = 0;
    if (std::strcmp(scheme, "affine4") == 0) b = 4;
    else if (std::strcmp(scheme, "affine8") == 0) b = 8;
    else return 0;
    if (bits) *bits = b;
    if (group_size) *group_size = 64;
    return 1;
}

kvc_status kvc_turbo_protected_layers(const int32_t *kinds, int32_t count, int32_t key_bits, int32_t value_bits,
                                      int32_t *flags) {
    if ((!kinds || !flags) && count > 0) return set_error(KVC_ERR_INVALID_ARG, "kvc_turbo_protected_layers: null argument");
    for (int i = 0; i < count; ++i) flags[i] = 0;
    const bool fragile = (key_bits > 0 && key_bits < 8) || value_bits <= 2;
    if (!fragile) return KVC_OK;
    std::vector<int> eligible;
    for (int i = 0; i < count; ++i)
        if (kinds[i] == KVC_KIND_SIMPLE || kinds[i] == KVC_KIND_QUANTIZED || kinds[i] == KVC_KIND_TURBO) eligible.push_back(i);
    const int boundary = std::min<int>(2, (int)eligible.size() / 2);
    for (int j = 0; j < boundary; ++j) {
        flags[eligible[(size_t)j]] = 1;
        flags[eligible[eligible.size() - 1 - (size_t)j]] = 1;
    }
    return KVC_OK;
}

kvc_status kvc_maybe_affine_quantize(kvc_cache **caches, int32_t count, int32_t bits, int32_t group_size,
                                     int64_t compression_start, void *stream, int32_t *complete) {
    if (!caches && count > 0) return set_error(KVC_ERR_INVALID_ARG, "kvc_maybe_affine_quantize: null argument");
    return guarded([&] {
        bool waiting = false;
        for (int i = 0; i < count; ++i) {
            kvc_cache *c = caches[i];
            if (!c || c->cfg.kind != KVC_KIND_SIMPLE) continue;
            if (c->offset <= compression_start) {
                waiting = true;
                continue;
            }
            DeviceGuard dg(c->device);
            kvc_cache *q = nullptr;
            try {
                q = kvc::cache_to_quantized(c, group_size, bits, as_stream(stream));
            } catch (const kvc::Error &) {
                q = nullptr;  // `try? simple.toQuantized`: the layer stays in full precision
            }
            if (q) {
                kvc_free(c);
                caches[i] = q;
            }
        }
        if (complete) *complete = waiting ? 0 : 1;
    });
}

kvc_status kvc_maybe_turbo_quantize(kvc_cache **caches, int32_t count, int32_t key_bits, int32_t value_bits,
                                    int64_t quantized_kv_start, void *stream, int32_t *complete) {
    if (!caches && count > 0) return set_error(KVC_ERR_INVALID_ARG, "kvc_maybe_turbo_quantize: null argument");
    return guarded([&] {
        std::vector<int32_t> kinds((size_t)count), prot((size_t)count);
        for (int i = 0; i < count; ++i) kinds[(size_t)i] = caches[i] ? caches[i]->cfg.kind : -1;
        kvc_turbo_protected_layers(kinds.data(), count, key_bits, value_bits, prot.data());
        bool waiting = false;
        for (int i = 0; i < count; ++i) {
            kvc_cache *c = caches[i];
            if (!c || c->cfg.kind != KVC_KIND_SIMPLE) continue;
            if (c->offset <= quantized_kv_start) {
                waiting = true;
                continue;
            }
            DeviceGuard dg(c->device);
            kvc_cache *n = nullptr;
            try {
                if (prot[(size_t)i]) {
                    n = kvc::cache_to_quantized(c, 64, 8, as_stream(stream));
                } else {
                    // affine-K mode quantises keys in groups: resolve the group size against this layer's
                    // head dims up front and skip the layer when none of the supported sizes divides them
                    int key_group = 64;
                    if (key_bits == 8) {
                        key_group = c->k.allocated() ? kvc::resolved_group_size(64, (int)c->k.W, (int)c->v.W) : 0;
                        if (!key_group) continue;
                    }
                    n = kvc::cache_to_turbo(c, key_bits, value_bits, key_group, as_stream(stream));
                }
            } catch (const kvc::Error &) {
                n = nullptr;  // unsupported realised shape: the layer stays in full precision
            }
            if (n) {
                kvc_free(c);
                caches[i] = n;
            }
        }
        if (complete) *complete = waiting ? 0 : 1;
    });
}

kvc_status kvc_logical_view(kvc_cache *c, int64_t tail, void *stream, kvc_tensor *out_k, kvc_tensor *out_v) {
    KVC_CHECK_HANDLE(c);
    return guarded([&] {
        DeviceGuard dg(c->device);
        kvc::cache_logical_view(c, tail, as_stream(stream), out_k, out_v);
    });
}

// ---------------------------------------------------------------------
// staged rounds
// ---------------------------------------------------------------------
kvc_status kvc_round_begin(kvc_cache *c, int32_t max_positions, kvc_round **out) {
    KVC_CHECK_HANDLE(c);
    if (!out) return set_error(KVC_ERR_INVALID_ARG, "kvc_round_begin: null output");
    *out = nullptr;
    return guarded([&] { kvc::round_begin(c, max_positions, out); });
}

kvc_status kvc_round_update(kvc_round *r, const kvc_tensor *k, const kvc_tensor *v, void *stream,
                            kvc_tensor *out_k, kvc_tensor *out_v) {
    KVC_CHECK_HANDLE(r);
    if (!k || !v) return set_error(KVC_ERR_INVALID_ARG, "kvc_round_update: null tensor");
    return guarded([&] {
        if (!r->cache || r->closed) kvc::fail(KVC_ERR_INVALID_STATE, "round is closed");
        DeviceGuard dg(r->cache->device);
        kvc::round_update(r, *k, *v, as_stream(stream), out_k, out_v);
    });
}

kvc_status kvc_round_attention(kvc_round *r, const kvc_tensor *q, const kvc_tensor *k,
                               const kvc_tensor *v, float scale, int32_t mask_mode,
                               const kvc_tensor *mask, const kvc_tensor *out, void *stream) {
    KVC_CHECK_HANDLE(r);
    if (!q || !k || !v || !out) return set_error(KVC_ERR_INVALID_ARG, "kvc_round_attention: null tensor");
    return guarded([&] {
        if (!r->cache || r->closed) kvc::fail(KVC_ERR_INVALID_STATE, "round is closed");
        DeviceGuard dg(r->cache->device);
        cudaStream_t s = as_stream(stream);
        if (!r->rotating) {
            // write-through leaves use the cache's own fused path
            kvc_round *saved = r->cache->open_round;
            r->cache->open_round = nullptr;
            try {
                kvc::cache_attention(r->cache, *q, *k, *v, scale, mask_mode, mask, *out, s);
            } catch (...) {
                r->cache->open_round = saved;
                throw;
            }
            r->cache->open_round = saved;
            return;
        }
        kvc_tensor pk, pv;
        kvc::round_update(r, *k, *v, s, &pk, &pv);
        kvc::AttnArgs a = kvc::make_attn_args(*q, *out, scale, mask_mode, mask, pk.shape[2], (int)k->shape[1]);
        a.k = kvc::raw_source(pk);
        a.v = kvc::raw_source(pv);
        kvc::launch_attention(a, s);
    });
}

int64_t kvc_round_offset(const kvc_round *r) {
    if (!r || !r->cache) return -1;
    return r->rotating ? r->cache->offset + r->staged : r->cache->offset;
}

kvc_status kvc_round_commit(kvc_round *r, int32_t retain, void *stream) {
    KVC_CHECK_HANDLE(r);
    return guarded([&] {
        if (!r->cache || r->closed) kvc::fail(KVC_ERR_INVALID_STATE, "round is closed");
        DeviceGuard dg(r->cache->device);
        kvc::round_commit(r, retain, as_stream(stream));
    });
}

kvc_status kvc_round_rollback(kvc_round *r, void *stream) { return kvc_round_commit(r, 0, stream); }

kvc_status kvc_rewind_last_round(kvc_cache *c, int64_t count, void *stream, int64_t *out_rewound) {
    KVC_CHECK_HANDLE(c);
    return guarded([&] {
        DeviceGuard dg(c->device);
        const int64_t n = kvc::rewind_last_round(c, count, as_stream(stream));
        if (out_rewound) *out_rewound = n;
    });
}

void kvc_round_free(kvc_round *r) {
    if (!r) return;
    try {
        if (r->cache && r->cache->open_round == r) r->cache->open_round = nullptr;
        cudaStream_t s = r->cache ? r->cache->last_stream : nullptr;
        r->sk.release(s); r->sv.release(s); r->pk.release(s); r->pv.release(s);
        delete r;
    } catch (...) {
    }
}

// ---------------------------------------------------------------------
// TurboQuant codec pieces
// ---------------------------------------------------------------------
int32_t kvc_turbo_packed_width(int32_t count, int32_t bits) { return (count * bits + 31) / 32; }

kvc_status kvc_turbo_codebook(int32_t dim, int32_t bits, float *centroids, float *boundaries) {
    return guarded([&] {
        KVC_REQUIRE(dim >= 4 && bits >= 1 && bits <= 4, "kvc_turbo_codebook: dim >= 4 and bits in 1..4");
        std::vector<float> c, b;
        kvc::turbo_codebook(dim, bits, c, b);
        if (centroids) std::memcpy(centroids, c.data(), c.size() * sizeof(float));
        if (boundaries) std::memcpy(boundaries, b.data(), b.size() * sizeof(float));
    });
}

kvc_status kvc_turbo_signs(int32_t dim, uint64_t seed, float *signs) {
    return guarded([&] {
        KVC_REQUIRE(dim > 0 && signs, "kvc_turbo_signs: bad arguments");
        std::vector<float> s;
        kvc::turbo_signs(dim, seed, s);
        std::memcpy(signs, s.data(), s.size() * sizeof(float));
    });
}

kvc_status kvc_turbo_set_codec(kvc_cache *c, const float *key_centroids, const float *value_centroids,
                               const float *key_signs, const float *value_signs, int32_t dim) {
    KVC_CHECK_HANDLE(c);
    return guarded([&] {
        KVC_REQUIRE(c->cfg.kind == KVC_KIND_TURBO, "kvc_turbo_set_codec needs a TurboQuantKVCache");
        if (c->codec_ready) kvc::fail(KVC_ERR_INVALID_STATE, "kvc_turbo_set_codec: the codec is already in use");
        KVC_REQUIRE(dim > 0, "kvc_turbo_set_codec: bad dim");
        if (key_centroids && !c->raw_key && !c->affine_key)
            c->user_kc.assign(key_centroids, key_centroids + (1 << c->key_bits));
        if (value_centroids && !c->affine_value)
            c->user_vc.assign(value_centroids, value_centroids + (1 << c->value_bits));
        if (key_signs) c->user_ks.assign(key_signs, key_signs + dim);
        if (value_signs) c->user_vs.assign(value_signs, value_signs + dim);
    });
}

kvc_status kvc_turbo_rotation(int32_t dim, uint64_t seed, float *rotation) {
    return guarded([&] {
        KVC_REQUIRE(dim >= 2 && dim <= 1024 && rotation, "kvc_turbo_rotation: bad arguments");
        std::vector<float> r;
        kvc::turbo_rotation(dim, seed, r);
        std::memcpy(rotation, r.data(), r.size() * sizeof(float));
    });
}

kvc_status kvc_turbo_set_rotation(kvc_cache *c, const float *key_rotation, const float *value_rotation, int32_t dim) {
    KVC_CHECK_HANDLE(c);
    return guarded([&] {
        KVC_REQUIRE(c->cfg.kind == KVC_KIND_TURBO, "kvc_turbo_set_rotation needs a TurboQuantKVCache");
        if (c->codec_ready) kvc::fail(KVC_ERR_INVALID_STATE, "kvc_turbo_set_rotation: the codec is already in use");
        KVC_REQUIRE(dim >= 2 && dim <= 1024, "kvc_turbo_set_rotation: bad dim");
        const size_t n = (size_t)dim * dim;
        if (key_rotation) c->user_kr.assign(key_rotation, key_rotation + n);
        if (value_rotation) c->user_vr.assign(value_rotation, value_rotation + n);
    });
}

kvc_status kvc_turbo_encode(const kvc_tensor *rows, const float *signs_dev, const float *boundaries_host,
                            int32_t bits, const kvc_tensor *packed, const kvc_tensor *norms, void *stream) {
    if (!rows || !signs_dev || !boundaries_host || !packed || !norms)
        return set_error(KVC_ERR_INVALID_ARG, "kvc_turbo_encode: null argument");
    return guarded([&] {
        DeviceGuard dg(-1);
        KVC_REQUIRE(rows->ndim == 2 && is_contiguous(*rows) && is_contiguous(*packed) && is_contiguous(*norms),
                    "kvc_turbo_encode: rows must be a contiguous [rows, D] tensor");
        KVC_REQUIRE(bits >= 1 && bits <= 4, "kvc_turbo_encode: bits in 1..4");
        const int D = (int)rows->shape[1];
        const int pw = (D * bits + 31) / 32;
        KVC_REQUIRE(packed->dtype == KVC_U32 && packed->shape[packed->ndim - 1] == pw, "kvc_turbo_encode: packed must be uint32 [rows, PW]");
        KVC_REQUIRE(norms->dtype == KVC_F32, "kvc_turbo_encode: norms must be float32");
        kvc::TurboEncodeArgs a;
        a.src = rows->data; a.dtype = rows->dtype;
        a.s_sb = 0; a.s_sh = 0; a.s_ss = D; a.s_sd = 1;
        a.packed = (uint32_t *)packed->data; a.norms = (float *)norms->data;
        a.p_sb = 0; a.p_sh = 0; a.p_st = pw;
        a.n_sb = 0; a.n_sh = 0; a.n_st = 1;
        a.B = 1; a.H = 1; a.S = (int)rows->shape[0]; a.D = D; a.bits = bits; a.pos = 0;
        a.signs = signs_dev;
        for (int i = 0; i < (1 << bits) - 1; ++i) a.boundaries[i] = boundaries_host[i];
        kvc::launch_turbo_encode(a, as_stream(stream));
    });
}

kvc_status kvc_attention_varlen(kvc_cache *const *caches, int32_t count, const kvc_tensor *queries,
                                const kvc_tensor *keys, const kvc_tensor *values, float scale,
                                const kvc_tensor *outs, void *stream) {
    if (!caches || !queries || !keys || !values || !outs) return set_error(KVC_ERR_INVALID_ARG, "kvc_attention_varlen: null argument");
    if (count <= 0) return KVC_OK;
    for (int i = 0; i < count; ++i) KVC_CHECK_HANDLE(caches[i]);
    return guarded([&] {
        DeviceGuard dg(caches[0]->device);
        kvc::cache_attention_varlen(caches, count, queries, keys, values, scale, outs, as_stream(stream));
    });
}

kvc_status kvc_turbo_encode_new_token(kvc_cache *cache, const kvc_tensor *keys, const kvc_tensor *values,
                                      void *stream) {
    if (!cache || !keys || !values) return set_error(KVC_ERR_INVALID_ARG, "kvc_turbo_encode_new_token: null argument");
    return guarded([&] {
        DeviceGuard dg(cache->device);
        kvc::cache_turbo_encode_new_token(cache, *keys, *values, as_stream(stream));
    });
}

kvc_status kvc_attention_batch(kvc_cache *const *caches, int32_t count, const kvc_tensor *q,
                               const kvc_tensor *k, const kvc_tensor *v, float scale,
                               int32_t mask_mode, const kvc_tensor *outs, void *stream,
                               int32_t host, int32_t synchronize) {
    if (!caches || !q || !k || !v || !outs) return set_error(KVC_ERR_INVALID_ARG, "kvc_attention_batch: null argument");
    if (host && count > 0 && mask_mode != KVC_MASK_ARRAY) {
        for (int i = 0; i < count; ++i) KVC_CHECK_HANDLE(caches[i]);
        return guarded([&] {
            // Host buffers: every layer's inputs are known when the call is made, so their
            // copies run ahead on a copy stream while earlier layers compute, and each output
            // leaves on a third stream as soon as its layer is done. `stream` joins both at the end.
            DeviceGuard dg(caches[0]->device);
            cudaStream_t s = as_stream(stream);
            SidePipe &pipe = side_pipe(kvc::current_device(), 2 * (size_t)count + 2);  // the guard has bound it
            auto al = [](size_t x) { return (x + 255) / 256 * 256; };
            std::vector<char *> slabs((size_t)count);
            for (int i = 0; i < count; ++i) {
                KVC_REQUIRE(caches[i]->device == caches[0]->device, "kvc_attention_batch: caches live on different devices");
                KVC_REQUIRE(is_contiguous(q[i]) && is_contiguous(k[i]) && is_contiguous(v[i]) && is_contiguous(outs[i]),
                            "kvc_attention_batch: host tensors must be contiguous");
                slabs[(size_t)i] = (char *)stage_get(caches[i], 0,
                                                     al(tensor_bytes_contiguous(q[i])) + al(tensor_bytes_contiguous(k[i])) +
                                                         al(tensor_bytes_contiguous(v[i])) + al(tensor_bytes_contiguous(outs[i])), s);
            }
            cudaEvent_t start = pipe.events[0], done = pipe.events[1];
            KVC_CUDA(cudaEventRecord(start, s));              // earlier work on `stream` still reads the slabs
            KVC_CUDA(cudaStreamWaitEvent(pipe.h2d, start, 0));
            // Layers travel in groups: one event per group tells `stream` that the group's inputs have
            // arrived, and one tells the output stream that its results are ready. Inside a group the
            // layers' kernels follow one another with nothing in between, so a layer starts under the
            // tail of the one before it. Groups are small at both ends (the first kernel waits for
            // one layer's copies only, the last output copy is one layer's) and up to 8 layers between.
            std::vector<int> group_end;   // one past the last layer of each group
            {
                std::vector<int> front, back;
                int used = 0;
                for (int sz = 1; used + sz <= count / 2; sz = std::min(sz * 2, 8)) {
                    front.push_back(sz);
                    back.push_back(sz);
                    used += sz;
                }
                int pos = 0;
                for (int sz : front) group_end.push_back(pos += sz);
                for (int left = count - 2 * used; left > 0;) {
                    const int sz = std::min(left, 8);
                    group_end.push_back(pos += sz);
                    left -= sz;
                }
                for (auto it = back.rbegin(); it != back.rend(); ++it) group_end.push_back(pos += *it);
            }
            // The host issues a group's input copies one group ahead of its kernels: the copies of
            // all layers up front would keep the device idle while the host is still queueing them.
            auto issue_inputs = [&](size_t gi) {
                if (gi >= group_end.size()) return;
                for (int i = gi ? group_end[gi - 1] : 0; i < group_end[gi]; ++i) {
                    const size_t qb = tensor_bytes_contiguous(q[i]), kb = tensor_bytes_contiguous(k[i]),
                                 vb = tensor_bytes_contiguous(v[i]);
                    char *dq = slabs[(size_t)i], *dk = dq + al(qb), *dv = dk + al(kb);
                    KVC_CUDA(cudaMemcpyAsync(dq, q[i].data, qb, cudaMemcpyHostToDevice, pipe.h2d));
                    KVC_CUDA(cudaMemcpyAsync(dk, k[i].data, kb, cudaMemcpyHostToDevice, pipe.h2d));
                    KVC_CUDA(cudaMemcpyAsync(dv, v[i].data, vb, cudaMemcpyHostToDevice, pipe.h2d));
                }
                KVC_CUDA(cudaEventRecord(pipe.events[2 + 2 * gi], pipe.h2d));
            };
            issue_inputs(0);
            int first = 0;
            struct HintReset { ~HintReset() { kvc::set_batch_previous(nullptr); } } hint_reset;
            first = 0;
            for (size_t gi = 0; gi < group_end.size(); ++gi) {
                KVC_CUDA(cudaStreamWaitEvent(s, pipe.events[2 + 2 * gi], 0));
                for (int i = first; i < group_end[gi]; ++i) {
                    const size_t qb = tensor_bytes_contiguous(q[i]), kb = tensor_bytes_contiguous(k[i]),
                                 vb = tensor_bytes_contiguous(v[i]);
                    char *dq = slabs[(size_t)i], *dk = dq + al(qb), *dv = dk + al(kb), *dout = dv + al(vb);
                    kvc_tensor tq = q[i], tk = k[i], tv = v[i], to = outs[i];
                    tq.data = dq; tk.data = dk; tv.data = dv; to.data = dout;
                    // layer i's launches follow layer i - 1's on the stream with nothing in between
                    kvc::set_batch_previous(i > first ? caches[i - 1] : nullptr);
                    kvc::cache_attention(caches[i], tq, tk, tv, scale, mask_mode, nullptr, to, s);
                }
                kvc::set_batch_previous(nullptr);
                cudaEvent_t out_ready = pipe.events[3 + 2 * gi];
                KVC_CUDA(cudaEventRecord(out_ready, s));
                KVC_CUDA(cudaStreamWaitEvent(pipe.d2h, out_ready, 0));
                for (int i = first; i < group_end[gi]; ++i) {
                    const size_t qb = tensor_bytes_contiguous(q[i]), kb = tensor_bytes_contiguous(k[i]),
                                 vb = tensor_bytes_contiguous(v[i]), ob = tensor_bytes_contiguous(outs[i]);
                    char *dout = slabs[(size_t)i] + al(qb) + al(kb) + al(vb);
                    KVC_CUDA(cudaMemcpyAsync(outs[i].data, dout, ob, cudaMemcpyDeviceToHost, pipe.d2h));
                }
                first = group_end[gi];
                issue_inputs(gi + 1);
            }
            KVC_CUDA(cudaEventRecord(done, pipe.d2h));
            KVC_CUDA(cudaStreamWaitEvent(s, done, 0));
            if (synchronize) KVC_CUDA(cudaStreamSynchronize(s));
        });
    }
    for (int i = 0; i < count; ++i) {
        // layer i's launches follow layer i - 1's on the stream with nothing in between
        kvc::set_batch_previous(!host && i > 0 ? caches[i - 1] : nullptr);
        kvc_status st = host ? kvc_attention_host(caches[i], &q[i], &k[i], &v[i], scale, mask_mode, nullptr,
                                                  &outs[i], stream, 0)
                             : kvc_attention(caches[i], &q[i], &k[i], &v[i], scale, mask_mode, nullptr,
                                             &outs[i], stream);
        kvc::set_batch_previous(nullptr);
        if (st != KVC_OK) return st;
    }
    if (synchronize) {
        return guarded([&] { KVC_CUDA(cudaStreamSynchronize(as_stream(stream))); });
    }
    return KVC_OK;
}

int32_t kvc_device_status(void) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        (void)cudaGetLastError();
        return -1;
    }
    return kvc::device_status(dev);
}

// ---------------------------------------------------------------------
// rotary positions at the cache offset; speculative rounds over a layer list
// ---------------------------------------------------------------------
namespace {
kvc::RopeTensor rope_tensor(const kvc_tensor &x, void *dst, int64_t d_sb, int64_t d_sh, int64_t d_sl) {
    kvc::RopeTensor t;
    t.src = x.data; t.dst = dst;
    t.s_sb = x.stride[0]; t.s_sh = x.stride[1]; t.s_sl = x.stride[2];
    t.d_sb = d_sb; t.d_sh = d_sh; t.d_sl = d_sl;
    t.B = (int32_t)x.shape[0]; t.H = (int32_t)x.shape[1]; t.L = (int32_t)x.shape[2];
    return t;
}

void rope_check(const kvc_tensor &x, const kvc_rope_config &r, const char *what) {
    KVC_REQUIRE(x.ndim == 4 && x.stride[3] == 1, std::string(what) + ": tensors must be [B, H, L, D] with inner stride 1");
    KVC_REQUIRE(x.dtype == KVC_F32 || x.dtype == KVC_F16 || x.dtype == KVC_BF16, std::string(what) + ": floating dtype needed");
    KVC_REQUIRE(r.dims >= 2 && r.dims % 2 == 0 && r.dims <= x.shape[3] && x.shape[3] % 2 == 0,
                std::string(what) + ": rope dims must be even and at most the head dim");
    KVC_REQUIRE(r.base > 0.f, std::string(what) + ": rope base must be positive");
}

kvc::RopeArgs rope_args(const kvc_rope_config &r, int32_t dtype, int D, int64_t offset) {
    kvc::RopeArgs a;
    a.dtype = dtype; a.D = D; a.dims = r.dims; a.traditional = r.traditional ? 1 : 0;
    a.log2_base_over_half = std::log2((double)r.base) / (double)(r.dims / 2);
    a.scale = r.scale;
    a.offset = offset;
    return a;
}
}  // namespace

kvc_status kvc_rope(const kvc_tensor *x, int64_t offset, const kvc_rope_config *rope, const kvc_tensor *out, void *stream) {
    if (!x || !rope || !out) return set_error(KVC_ERR_INVALID_ARG, "kvc_rope: null argument");
    return guarded([&] {
        rope_check(*x, *rope, "kvc_rope");
        KVC_REQUIRE(out->ndim == 4 && out->stride[3] == 1 && out->dtype == x->dtype, "kvc_rope: out must match x");
        for (int i = 0; i < 4; ++i) KVC_REQUIRE(out->shape[i] == x->shape[i], "kvc_rope: out must match x");
        kvc::RopeArgs a = rope_args(*rope, x->dtype, (int)x->shape[3], offset);
        a.q = rope_tensor(*x, out->data, out->stride[0], out->stride[1], out->stride[2]);
        kvc::launch_rope(a, as_stream(stream));
    });
}

kvc_status kvc_attention_rope(kvc_cache *cache, const kvc_tensor *q, const kvc_tensor *k, const kvc_tensor *v,
                              const kvc_rope_config *rope, float scale, int32_t mask_mode, const kvc_tensor *mask,
                              const kvc_tensor *out, void *stream) {
    if (!q || !k || !v || !rope || !out) return set_error(KVC_ERR_INVALID_ARG, "kvc_attention_rope: null argument");
    return guarded([&] {
        cudaStream_t s = as_stream(stream);
        rope_check(*q, *rope, "kvc_attention_rope");
        rope_check(*k, *rope, "kvc_attention_rope");
        KVC_REQUIRE(q->dtype == k->dtype && q->shape[3] == k->shape[3] && q->shape[2] == k->shape[2] && q->shape[0] == k->shape[0],
                    "kvc_attention_rope: queries and keys disagree");
        DeviceGuard dg(cache ? cache->device : -1);
        // cache?.ropeOffset: the scalar cache offset (KVCache.swift:107-109), 0 without a cache
        const int64_t offset = cache ? cache->offset : 0;
        const size_t es = kvc::dtype_size(q->dtype);
        const int64_t D = q->shape[3], L = q->shape[2];
        const size_t qn = (size_t)(q->shape[0] * q->shape[1] * L * D), kn = (size_t)(k->shape[0] * k->shape[1] * L * D);
        char *buf = (char *)kvc::dev_alloc((qn + kn) * es + 256, s);
        struct Free { char *p; cudaStream_t s; ~Free() { kvc::dev_free(p, s); } } freer{buf, s};
        kvc_tensor rq = *q, rk = *k;
        rq.data = buf;
        rk.data = buf + ((qn * es + 255) / 256) * 256;
        for (kvc_tensor *t : {&rq, &rk}) {
            t->stride[3] = 1; t->stride[2] = D; t->stride[1] = L * D; t->stride[0] = t->shape[1] * L * D;
        }
        kvc::RopeArgs a = rope_args(*rope, q->dtype, (int)D, offset);
        a.q = rope_tensor(*q, rq.data, rq.stride[0], rq.stride[1], rq.stride[2]);
        a.k = rope_tensor(*k, rk.data, rk.stride[0], rk.stride[1], rk.stride[2]);
        kvc::launch_rope(a, s);
        if (cache) {
            kvc::cache_attention(cache, rq, rk, *v, scale, mask_mode, mask, *out, s);
        } else {
            // attentionWithCacheUpdate without a cache: plain SDPA (AttentionUtils.swift:46-52)
            kvc_status st = kvc_sdpa(&rq, &rk, v, scale, mask_mode, mask, out, stream);
            if (st != KVC_OK) kvc::fail(st, kvc_last_error_message());
        }
    });
}

kvc_status kvc_storage_begin_round(kvc_cache *const *caches, int32_t count, int32_t max_positions, kvc_round **out_rounds) {
    if (!caches || !out_rounds || count <= 0) return set_error(KVC_ERR_INVALID_ARG, "kvc_storage_begin_round: bad argument");
    for (int i = 0; i < count; ++i) out_rounds[i] = nullptr;
    for (int i = 0; i < count; ++i) {
        // nested lists expand to more leaves than slots and are refused (KVCachePlan.swift:226-231)
        kvc_status st = (caches[i] && caches[i]->cfg.kind == KVC_KIND_LIST)
                            ? set_error(KVC_ERR_NOT_TRIMMABLE, "a CacheList entry cannot take part in a staged round")
                            : kvc_round_begin(caches[i], max_positions, &out_rounds[i]);
        if (st != KVC_OK) {
            // all or nothing: close what was opened (nothing has been written through them yet)
            const std::string msg = kvc_last_error_message() ? kvc_last_error_message() : "";
            for (int j = 0; j < i; ++j) {
                (void)kvc_round_rollback(out_rounds[j], nullptr);
                kvc_round_free(out_rounds[j]);
                out_rounds[j] = nullptr;
            }
            return set_error(st, msg.c_str());
        }
    }
    return KVC_OK;
}

kvc_status kvc_storage_round_attention(kvc_round *const *rounds, int32_t count, const kvc_tensor *q, const kvc_tensor *k,
                                       const kvc_tensor *v, float scale, int32_t mask_mode, const kvc_tensor *outs, void *stream) {
    if (!rounds || !q || !k || !v || !outs) return set_error(KVC_ERR_INVALID_ARG, "kvc_storage_round_attention: null argument");
    for (int i = 0; i < count; ++i) {
        kvc_status st = kvc_round_attention(rounds[i], &q[i], &k[i], &v[i], scale, mask_mode, nullptr, &outs[i], stream);
        if (st != KVC_OK) return st;
    }
    return KVC_OK;
}

kvc_status kvc_storage_commit(kvc_round **rounds, int32_t count, int32_t retaining, void *stream) {
    if (!rounds) return set_error(KVC_ERR_INVALID_ARG, "kvc_storage_commit: null argument");
    kvc_status first = KVC_OK;
    for (int i = 0; i < count; ++i) {
        if (!rounds[i]) continue;
        kvc_status st = kvc_round_commit(rounds[i], retaining, stream);
        if (st != KVC_OK && first == KVC_OK) first = st;
        kvc_round_free(rounds[i]);
        rounds[i] = nullptr;
    }
    return first;
}

kvc_status kvc_speculate_rewind(kvc_cache *const *caches, int32_t count, int32_t num_draft, int32_t accepted, int32_t is_draft,
                                int64_t *out_trimmed) {
    if (!caches || num_draft < 0 || accepted < 0 || accepted > num_draft)
        return set_error(KVC_ERR_INVALID_ARG, "kvc_speculate_rewind: need 0 <= accepted <= num_draft");
    // Evaluate.swift:1262-1264
    const int64_t n = is_draft ? std::max(num_draft - accepted - 1, 0) : num_draft - accepted;
    int64_t trimmed = 0;
    kvc_status st = n > 0 ? kvc_trim_prompt_cache(caches, count, n, &trimmed) : KVC_OK;
    if (out_trimmed) *out_trimmed = trimmed;
    return st;
}

kvc_status kvc_device_status_reset(void) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || !kvc::device_status_reset(dev)) {
        (void)cudaGetLastError();
        return set_error(KVC_ERR_CUDA, "kvc_device_status_reset: the status word could not be cleared");
    }
    return KVC_OK;
}

kvc_status kvc_device_wait_probe(uint32_t iterations, void *stream) {
    return guarded([&] {
        KVC_REQUIRE(iterations > 0 && iterations <= (1u << 24), "kvc_device_wait_probe: iterations must be in [1, 2^24]");
        kvc::device_wait_probe(kvc::current_device(), iterations, as_stream(stream));
    });
}

void kvc_timing_enable(int32_t on) { kvc::timing_set(on != 0); }

kvc_status kvc_timing_read(double *total_ms, int64_t *launches, int32_t reset) {
    return guarded([&] { kvc::timing_read(total_ms, launches, reset != 0); });
}

int64_t kvc_launch_count(int32_t reset) {
    const int64_t n = kvc::g_launch_count;
    if (reset) kvc::g_launch_count = 0;
    return n;
}

}  // extern "C"
