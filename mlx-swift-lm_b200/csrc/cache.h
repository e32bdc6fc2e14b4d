// Host-side cache objects: the state machines of KVCacheSimple,
// RotatingKVCache, QuantizedKVCache and TurboQuantKVCache re-stated over
// device arrays that this library owns.
#pragma once

#include "common.h"

#include <memory>
#include <string>
#include <vector>

namespace kvc {

// A device array shaped [B, H, cap, W] (W = 1 for per-token norms).
struct Array4 {
    void *ptr = nullptr;
    int32_t dtype = KVC_BF16;
    int64_t B = 0, H = 0, cap = 0, W = 0;

    bool allocated() const { return ptr != nullptr; }
    int64_t sb() const { return H * cap * W; }
    int64_t sh() const { return cap * W; }
    int64_t st() const { return W; }
    size_t esize() const { return dtype_size(dtype); }
    size_t bytes() const { return (size_t)(B * H * cap * W) * esize(); }

    void alloc(int64_t b, int64_t h, int64_t c, int64_t w, int32_t dt, cudaStream_t s);
    void release(cudaStream_t s);
    // Grow to at least `need` token rows, preserving the first `keep_rows`.
    void ensure(int64_t need, int64_t keep_rows, int64_t step, cudaStream_t s);
    kvc_tensor view(int64_t tokens, int64_t first = 0) const;
};

struct TurboCodec {
    int dim = 0, bits = 0;
    std::vector<float> centroids, boundaries, signs;
    float *signs_dev = nullptr;
    // Key-calibration scale (keys only; empty = none): TurboQuantKVCache.keyCalibScale
    // (TurboQuantKVCache.swift:688, computed at :867-886).
    std::vector<float> calib;
    float *calib_dev = nullptr;
    // Dense rotation Pi, row-major [dim, dim], for head dims that are not powers of two
    // (TurboQuantRotation.rotationMatrix, TurboQuantKVCache.swift:246-259); empty on the Walsh-Hadamard path.
    std::vector<float> rotation;
    float *rotation_dev = nullptr;
};

struct RestorePoint {
    bool valid = false;
    Array4 k, v;            // snapshot of the physical ring
    int64_t len = 0, offset = 0, idx = 0;
    Array4 rk, rv;          // staged rows to replay
    int64_t committed = 0;
};

}  // namespace kvc

struct kvc_round;

// Records a failure for kvc_last_error_message() on the calling thread.
extern "C" kvc_status kvc_internal_set_error(kvc_status code, const char *msg);

struct kvc_cache {
    kvc_config cfg{};
    int device = 0;
    int64_t offset = 0;
    // The stream of the last call that enqueued work on this handle's arrays: buffers the handle gives
    // up without being handed a stream (the destructor, trim to empty) are freed in that stream's order,
    // so the pool cannot hand them out again under kernels still queued there.
    cudaStream_t last_stream = nullptr;

    // simple / rotating / turbo raw phase
    kvc::Array4 k, v;
    // rotating
    int64_t len = 0;   // the reference's keys.dim(2)
    int64_t idx = 0;
    std::string origin = "modelNative";
    // chunked: ChunkedKVCache.startPosition (KVCache.swift:1215); `len` is the reference's keys.dim(2)
    int64_t start_position = 0;
    // list: CacheList children (owned)
    std::vector<kvc_cache *> children;
    kvc::Array4 k_alt, v_alt;       // ping-pong target for re-order / trim
    kvc::Array4 k_view, v_view;     // scratch for logical views
    kvc::RestorePoint restore;
    kvc_round *open_round = nullptr;

    // quantized (and turbo affine-K): codes / scales / biases
    kvc::Array4 kq, ks, kb, vq, vs, vb;
    int32_t group_size = 64, bits = 8;
    bool group_resolved = false;

    // turbo
    bool compressed = false;
    int32_t key_bits = 4, value_bits = 4, key_group = 64;
    bool raw_key = false, affine_key = false, affine_value = false;
    kvc::Array4 kp, kn, vp, vn;     // packed indices + norms
    kvc::TurboCodec kcodec, vcodec;
    bool codec_ready = false;
    std::vector<float> user_kc, user_vc, user_ks, user_vs;  // overrides
    std::vector<float> user_kr, user_vr;                    // dense-rotation overrides [D * D]

    // host-call staging
    void *stage[4] = {nullptr, nullptr, nullptr, nullptr};
    size_t stage_bytes[4] = {0, 0, 0, 0};

    ~kvc_cache();
};

struct kvc_round {
    kvc_cache *cache = nullptr;
    int32_t max_positions = 0;
    bool rotating = false;
    int64_t start_offset = 0;
    kvc::Array4 sk, sv;   // staged rows [B, H, max_positions, D]
    int64_t staged = 0;
    kvc::Array4 pk, pv;   // presentation buffers
    bool closed = false;
};

namespace kvc {

// Operations (throw kvc::Error).
void cache_update(kvc_cache *c, const kvc_tensor &k, const kvc_tensor &v, cudaStream_t s,
                  kvc_tensor *out_k, kvc_tensor *out_v);
void cache_update_quantized(kvc_cache *c, const kvc_tensor &k, const kvc_tensor &v, cudaStream_t s,
                            kvc_tensor out_k[3], kvc_tensor out_v[3], bool defer_quantize = false);
// attentionWithCacheUpdate for a list of independent caches, one new token each: two launches for
// the whole list when they are affine caches of one layout, otherwise one call per cache.
void cache_attention_varlen(kvc_cache *const *caches, int n, const kvc_tensor *q, const kvc_tensor *k,
                            const kvc_tensor *v, float scale, const kvc_tensor *outs, cudaStream_t s);
void cache_attention(kvc_cache *c, const kvc_tensor &q, const kvc_tensor &k, const kvc_tensor &v,
                     float scale, int32_t mask_mode, const kvc_tensor *mask, const kvc_tensor &out,
                     cudaStream_t s);
int64_t cache_trim(kvc_cache *c, int64_t n);
bool cache_is_trimmable_after(const kvc_cache *c, int64_t positions);
int cache_state_count(const kvc_cache *c);
kvc_tensor cache_state_get(kvc_cache *c, int index);
void cache_state_set(kvc_cache *c, const kvc_tensor *arrays, int count, cudaStream_t s);
std::vector<std::string> cache_meta_state(const kvc_cache *c);
void cache_set_meta_state(kvc_cache *c, const std::vector<std::string> &m);
// prompt-cache files (promptcache.cu)
void save_prompt_cache(const char *path, kvc_cache *const *caches, int count, const char *const *keys,
                       const char *const *values, int meta_count, cudaStream_t s);
void load_prompt_cache(const char *path, int device, std::vector<kvc_cache *> &out,
                       std::vector<std::pair<std::string, std::string>> &user_meta, cudaStream_t s);
kvc_cache *cache_copy(const kvc_cache *c, cudaStream_t s);
kvc_cache *cache_to_quantized(const kvc_cache *c, int group, int bits, cudaStream_t s);
kvc_cache *cache_to_unquantized(const kvc_cache *c, cudaStream_t s);
void cache_turbo_encode_new_token(kvc_cache *c, const kvc_tensor &k, const kvc_tensor &v, cudaStream_t s);
kvc_cache *cache_to_turbo(const kvc_cache *c, int kb, int vb, int kg, cudaStream_t s);
void cache_logical_view(kvc_cache *c, int64_t tail, cudaStream_t s, kvc_tensor *ok, kvc_tensor *ov);
void cache_maybe_trim_front(kvc_cache *c, cudaStream_t s);
const char *cache_class_name(const kvc_cache *c);
void cache_make_mask(const kvc_cache *c, int n, int64_t window, bool return_array, int32_t *mode,
                     int64_t *rows, int64_t *cols, void *out_mask, cudaStream_t s);
int resolved_group_size(int requested, int kd, int vd);  // 0 when none fits
void ensure_codecs(kvc_cache *c, int head_dim, cudaStream_t s);
void turbo_codebook(int dim, int bits, std::vector<float> &centroids, std::vector<float> &bounds);
void turbo_signs(int dim, uint64_t seed, std::vector<float> &signs);
void turbo_rotation(int dim, uint64_t seed, std::vector<float> &rotation);   // row-major [dim, dim]

// attention over explicit tensors
AttnArgs make_attn_args(const kvc_tensor &q, const kvc_tensor &out, float scale, int32_t mask_mode,
                        const kvc_tensor *mask, int64_t T, int Hkv);
KVSource raw_source(const kvc_tensor &t);

// Batched entry points: names the cache whose kernels were launched just before the next
// cache_attention call on the same stream (nullptr = unknown / none).
void set_batch_previous(const kvc_cache *prev);

}  // namespace kvc
