// Header-only C++ mirror of MLXLMCommon's KVCache protocol surface
// (Libraries/MLXLMCommon/KVCache.swift:46-104, :156-181) over the C ABI in
// include/kvcache_b200.h. Same member names and argument meaning as the Swift
// classes; programmer errors throw kvc::host::Error where the reference traps.
#pragma once

#include <cstdint>
#include <map>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "../../include/kvcache_b200.h"

namespace kvc::host {

struct Error : std::runtime_error {
    kvc_status status;
    Error(kvc_status s, const std::string &m) : std::runtime_error(m), status(s) {}
};

inline void check(kvc_status s) {
    if (s != KVC_OK) {
        const char *m = kvc_last_error_message();
        throw Error(s, m ? m : "unknown error");
    }
}

enum class MaskKind { none, causal, array };
struct Mask {
    MaskKind kind = MaskKind::none;
    kvc_tensor array{};
};

class KVCache {
  public:
    virtual ~KVCache() { if (h_) kvc_free(h_); }
    KVCache(const KVCache &) = delete;
    KVCache &operator=(const KVCache &) = delete;

    int64_t offset() const { return kvc_offset(h_); }
    void setOffset(int64_t n) { check(kvc_set_offset(h_, n)); }
    std::optional<int64_t> maxSize() const {
        const int64_t m = kvc_max_size(h_);
        return m < 0 ? std::nullopt : std::optional<int64_t>(m);
    }

    // update(keys:values:) -> (keys, values)
    std::pair<kvc_tensor, kvc_tensor> update(const kvc_tensor &keys, const kvc_tensor &values) {
        kvc_tensor k{}, v{};
        check(kvc_update(h_, &keys, &values, stream, &k, &v));
        return {k, v};
    }

    std::vector<kvc_tensor> state() {
        std::vector<kvc_tensor> out((size_t)kvc_state_count(h_));
        for (size_t i = 0; i < out.size(); ++i) check(kvc_state_get(h_, (int32_t)i, &out[i]));
        return out;
    }
    void setState(const std::vector<kvc_tensor> &arrays) {
        check(kvc_state_set(h_, arrays.data(), (int32_t)arrays.size(), stream));
    }

    std::vector<std::string> metaState() const {
        size_t n = 0;
        check(kvc_meta_state(h_, nullptr, 0, &n));
        std::string buf(n, '\0');
        check(kvc_meta_state(h_, buf.data(), n, &n));
        buf.resize(n ? n - 1 : 0);
        std::vector<std::string> out;
        size_t start = 0;
        for (;;) {
            const size_t p = buf.find('\n', start);
            out.push_back(buf.substr(start, p == std::string::npos ? std::string::npos : p - start));
            if (p == std::string::npos) break;
            start = p + 1;
        }
        return out;
    }
    void setMetaState(const std::vector<std::string> &m) {
        std::string joined;
        for (size_t i = 0; i < m.size(); ++i) joined += (i ? "\n" : "") + m[i];
        check(kvc_set_meta_state(h_, joined.c_str()));
    }

    bool isTrimmable() const { return kvc_is_trimmable(h_) != 0; }
    bool isTrimmable(int64_t afterPositions) const { return kvc_is_trimmable_after(h_, afterPositions) != 0; }
    int64_t trim(int64_t n) {
        int64_t t = 0;
        check(kvc_trim(h_, n, &t));
        return t;
    }

    // attentionWithCacheUpdate(queries:keys:values:cache:scale:mask:) for this cache
    void attention(const kvc_tensor &queries, const kvc_tensor &keys, const kvc_tensor &values, float scale,
                   const Mask &mask, const kvc_tensor &out) {
        const int32_t mode = mask.kind == MaskKind::none ? KVC_MASK_NONE
                             : mask.kind == MaskKind::causal ? KVC_MASK_CAUSAL : KVC_MASK_ARRAY;
        check(kvc_attention(h_, &queries, &keys, &values, scale, mode,
                            mask.kind == MaskKind::array ? &mask.array : nullptr, &out, stream));
    }

    // makeMask(n:windowSize:returnArray:): the mode, and for array masks the [rows, cols] shape;
    // `maskOut` (device, bool, rows * cols bytes) may be null to query the shape only.
    struct MaskInfo {
        MaskKind kind;
        int64_t rows, cols;
    };
    MaskInfo makeMask(int n, std::optional<int64_t> windowSize, bool returnArray, void *maskOut = nullptr) const {
        int32_t mode = KVC_MASK_NONE;
        int64_t rows = 0, cols = 0;
        check(kvc_make_mask(h_, n, windowSize ? *windowSize : -1, returnArray ? 1 : 0, &mode, &rows, &cols,
                            maskOut, stream));
        return {mode == KVC_MASK_NONE ? MaskKind::none : mode == KVC_MASK_CAUSAL ? MaskKind::causal : MaskKind::array,
                rows, cols};
    }

    // copy(): a deep copy of the same class
    std::unique_ptr<KVCache> copy() const {
        kvc_cache *out = nullptr;
        check(kvc_copy(h_, stream, &out));
        return wrap(out);
    }

    // prepare(lengths:rightPadding:) / finalize(): no-ops for the caches of this path, as in the reference
    void prepare(const std::vector<int32_t> &lengths) { check(kvc_prepare(h_, lengths.data(), (int32_t)lengths.size())); }
    void finalize() { check(kvc_finalize(h_)); }

    int32_t kind() const { return kvc_kind_of(h_); }
    int64_t memoryBytes() const { return kvc_memory_bytes(h_); }
    // capacity hint (no reference counterpart): room for `tokens` rows without regrowth
    void reserve(int64_t tokens, int batch, int kvHeads, int headDim, int32_t dtype) {
        check(kvc_reserve(h_, tokens, batch, kvHeads, headDim, dtype, stream));
    }

    // Adopt a handle under the class its kind names (results of conversions and file loads).
    static std::unique_ptr<KVCache> wrap(kvc_cache *adopted);
    // Give the handle up (list-level calls that replace handles in place).
    kvc_cache *release() {
        kvc_cache *h = h_;
        h_ = nullptr;
        return h;
    }

    kvc_cache *handle() const { return h_; }
    void *stream = nullptr;

  protected:
    explicit KVCache(const kvc_config &cfg) { check(kvc_create(&cfg, &h_)); }
    explicit KVCache(kvc_cache *adopted) : h_(adopted) {}
    static kvc_config defaults(int32_t kind) {
        kvc_config c;
        kvc_config_default(&c, kind);
        return c;
    }
    kvc_cache *h_ = nullptr;
};

class QuantizedKVCache;

class KVCacheSimple : public KVCache {
  public:
    explicit KVCacheSimple(int step = 256) : KVCache(make(step)) {}
    explicit KVCacheSimple(kvc_cache *adopted) : KVCache(adopted) {}
    // toQuantized(groupSize:bits:)
    std::unique_ptr<KVCache> toQuantized(int groupSize = 64, int bits = 4) const {
        kvc_cache *out = nullptr;
        check(kvc_to_quantized(h_, groupSize, bits, stream, &out));
        return wrap(out);
    }
    // the per-layer conversion of maybeTurboQuantizeKVCache
    std::unique_ptr<KVCache> toTurbo(int keyBits, int valueBits, int keyGroupSize = 64) const {
        kvc_cache *out = nullptr;
        check(kvc_to_turbo(h_, keyBits, valueBits, keyGroupSize, stream, &out));
        return wrap(out);
    }

  private:
    static kvc_config make(int step) {
        kvc_config c = defaults(KVC_KIND_SIMPLE);
        c.step = step;
        return c;
    }
};

class RotatingKVCache : public KVCache {
  public:
    RotatingKVCache(int maxSize, int keep = 0, int step = 256) : KVCache(make(maxSize, keep, step)) {}
    explicit RotatingKVCache(kvc_cache *adopted) : KVCache(adopted) {}
    int64_t idx() const { return kvc_ring_index(h_); }
    // logicalView(tail:); nullopt before the first write
    std::optional<std::pair<kvc_tensor, kvc_tensor>> logicalView(int64_t tail) {
        kvc_tensor k{}, v{};
        const kvc_status s = kvc_logical_view(h_, tail, stream, &k, &v);
        if (s == KVC_ERR_INVALID_STATE) return std::nullopt;
        check(s);
        return std::make_pair(k, v);
    }

  private:
    static kvc_config make(int maxSize, int keep, int step) {
        kvc_config c = defaults(KVC_KIND_ROTATING);
        c.max_size = maxSize;
        c.keep = keep;
        c.step = step;
        return c;
    }
};

class QuantizedKVCache : public KVCache {
  public:
    explicit QuantizedKVCache(int groupSize = 64, int bits = 8) : KVCache(make(groupSize, bits)) {}
    explicit QuantizedKVCache(kvc_cache *adopted) : KVCache(adopted) {}
    int groupSize() const { return kvc_group_size(h_); }
    int bits() const { return kvc_bits(h_); }
    // updateQuantized(keys:values:) -> ((w, scales, biases), (w, scales, biases))
    void updateQuantized(const kvc_tensor &keys, const kvc_tensor &values, kvc_tensor outK[3], kvc_tensor outV[3]) {
        check(kvc_update_quantized(h_, &keys, &values, stream, outK, outV));
    }
    // getQuantizedState()
    void getQuantizedState(kvc_tensor outK[3], kvc_tensor outV[3]) { check(kvc_quantized_state(h_, outK, outV)); }
    // toUnquantized()
    std::unique_ptr<KVCache> toUnquantized() const {
        kvc_cache *out = nullptr;
        check(kvc_to_unquantized(h_, stream, &out));
        return wrap(out);
    }

  private:
    static kvc_config make(int g, int b) {
        kvc_config c = defaults(KVC_KIND_QUANTIZED);
        c.group_size = g;
        c.bits = b;
        return c;
    }
};

class TurboQuantKVCache : public KVCache {
  public:
    explicit TurboQuantKVCache(int bits = 4, int keyBits = -1, int valueBits = -1, uint64_t seed = 42,
                               int keyGroupSize = 64)
        : KVCache(make(bits, keyBits, valueBits, seed, keyGroupSize)) {}
    explicit TurboQuantKVCache(kvc_cache *adopted) : KVCache(adopted) {}
    bool isCompressed() const { return kvc_is_compressed(h_) != 0; }
    // compressRawCache + encodeNewToken without the attention (chunked compressed prefill)
    void encodeNewToken(const kvc_tensor &keys, const kvc_tensor &values) {
        check(kvc_turbo_encode_new_token(h_, &keys, &values, stream));
    }

  private:
    static kvc_config make(int bits, int kb, int vb, uint64_t seed, int kg) {
        kvc_config c = defaults(KVC_KIND_TURBO);
        c.bits = bits;
        c.key_bits = kb;
        c.value_bits = vb;
        c.seed = seed;
        c.key_group_size = kg;
        return c;
    }
};

// ChunkedKVCache(chunkSize:): a KVCacheSimple whose front can be dropped chunk by chunk.
class ChunkedKVCache : public KVCache {
  public:
    explicit ChunkedKVCache(std::optional<int64_t> chunkSize = std::nullopt) : KVCache(config(chunkSize)) {}
    explicit ChunkedKVCache(kvc_cache *adopted) : KVCache(adopted) {}
    void maybeTrimFront() { check(kvc_maybe_trim_front(h_, stream)); }
    int64_t startPosition() const { return kvc_start_position(h_); }

  private:
    static kvc_config config(std::optional<int64_t> chunkSize) {
        kvc_config c = defaults(KVC_KIND_CHUNKED);
        c.max_size = chunkSize ? (int32_t)*chunkSize : -1;   // the chunk size travels in max_size; -1 = nil
        return c;
    }
};

// CacheList(caches...): a composite whose state / metaState / trim span its children in order. The
// children are handed over to the list; subscript(index:) gives a borrowed view of one of them.
class CacheList : public KVCache {
  public:
    explicit CacheList(std::vector<std::unique_ptr<KVCache>> children) : KVCache(make(children)) {}
    explicit CacheList(kvc_cache *adopted) : KVCache(adopted) {}
    int count() const { return kvc_list_count(h_); }
    kvc_cache *operator[](int index) const { return kvc_list_child(h_, index); }

  private:
    static kvc_cache *make(std::vector<std::unique_ptr<KVCache>> &children) {
        std::vector<kvc_cache *> h;
        for (auto &c : children) h.push_back(c->handle());
        kvc_cache *out = nullptr;
        check(kvc_list_create(h.data(), (int32_t)h.size(), &out));
        for (auto &c : children) c->release();   // the list owns them now
        return out;
    }
};

// createCausalMask(n:offset:windowSize:lengths:): `maskOut` is device memory, one byte per element,
// [n, offset + n] without lengths and [batch, 1, n, offset + n] with them (device int32 [batch]).
inline void createCausalMask(int n, int64_t offset, std::optional<int64_t> windowSize, const int32_t *lengthsDev,
                             int batch, void *maskOut, void *stream = nullptr) {
    check(kvc_create_causal_mask(n, offset, windowSize ? *windowSize : -1, lengthsDev, batch, maskOut, stream));
}

// RoPE(dimensions:traditional:base:scale:) as the attention blocks apply it.
struct RoPE {
    int dimensions;
    bool traditional = false;
    float base = 10000.f;
    float scale = 1.f;
    kvc_rope_config config() const { return kvc_rope_config{dimensions, traditional ? 1 : 0, base, scale}; }
    // applyRotaryPosition(rope, to: x, offset:)
    void operator()(const kvc_tensor &x, int64_t offset, const kvc_tensor &out, void *stream = nullptr) const {
        const kvc_rope_config c = config();
        check(kvc_rope(&x, offset, &c, &out, stream));
    }
};

// The cache step of an attention block: rotary positions at the cache offset, then update + attention.
inline void attentionWithRope(const kvc_tensor &queries, const kvc_tensor &keys, const kvc_tensor &values,
                              KVCache *cache, const RoPE &rope, float scale, const Mask &mask, const kvc_tensor &out,
                              void *stream = nullptr) {
    const kvc_rope_config c = rope.config();
    const int32_t mode = mask.kind == MaskKind::none ? KVC_MASK_NONE
                         : mask.kind == MaskKind::causal ? KVC_MASK_CAUSAL : KVC_MASK_ARRAY;
    check(kvc_attention_rope(cache ? cache->handle() : nullptr, &queries, &keys, &values, &c, scale, mode,
                             mask.kind == MaskKind::array ? &mask.array : nullptr, &out, cache ? cache->stream : stream));
}

inline void attentionWithCacheUpdate(const kvc_tensor &queries, const kvc_tensor &keys, const kvc_tensor &values,
                                     KVCache *cache, float scale, const Mask &mask, const kvc_tensor &out,
                                     void *stream = nullptr) {
    if (cache) {
        cache->attention(queries, keys, values, scale, mask, out);
        return;
    }
    const int32_t mode = mask.kind == MaskKind::none ? KVC_MASK_NONE
                         : mask.kind == MaskKind::causal ? KVC_MASK_CAUSAL : KVC_MASK_ARRAY;
    check(kvc_sdpa(&queries, &keys, &values, scale, mode, mask.kind == MaskKind::array ? &mask.array : nullptr,
                   &out, stream));
}

inline std::unique_ptr<KVCache> KVCache::wrap(kvc_cache *adopted) {
    switch (kvc_kind_of(adopted)) {
        case KVC_KIND_SIMPLE: return std::make_unique<KVCacheSimple>(adopted);
        case KVC_KIND_ROTATING: return std::make_unique<RotatingKVCache>(adopted);
        case KVC_KIND_QUANTIZED: return std::make_unique<QuantizedKVCache>(adopted);
        case KVC_KIND_TURBO: return std::make_unique<TurboQuantKVCache>(adopted);
        case KVC_KIND_CHUNKED: return std::make_unique<ChunkedKVCache>(adopted);
        case KVC_KIND_LIST: return std::make_unique<CacheList>(adopted);
        default: kvc_free(adopted); throw Error(KVC_ERR_INTERNAL, "unknown cache kind");
    }
}

// quantizedScaledDotProductAttention(queries:quantizedKeys:quantizedValues:scale:mask:groupSize:bits:)
inline void quantizedScaledDotProductAttention(const kvc_tensor &queries, const kvc_tensor qk[3], const kvc_tensor qv[3],
                                               float scale, const Mask &mask, int groupSize, int bits,
                                               const kvc_tensor &out, void *stream = nullptr) {
    const int32_t mode = mask.kind == MaskKind::none ? KVC_MASK_NONE
                         : mask.kind == MaskKind::causal ? KVC_MASK_CAUSAL : KVC_MASK_ARRAY;
    check(kvc_quantized_sdpa(&queries, qk, qv, scale, mode, mask.kind == MaskKind::array ? &mask.array : nullptr,
                             groupSize, bits, &out, stream));
}

// [KVCache]: the per-layer cache array the iterators carry
using CacheArray = std::vector<std::unique_ptr<KVCache>>;

namespace detail {
inline std::vector<kvc_cache *> handles(const CacheArray &caches) {
    std::vector<kvc_cache *> h;
    for (const auto &c : caches) h.push_back(c->handle());
    return h;
}
// Re-adopt the handles a list-level conversion left in `h` (converted slots hold new handles, the old
// ones were freed by the library).
inline void readopt(CacheArray &caches, const std::vector<kvc_cache *> &h) {
    for (size_t i = 0; i < caches.size(); ++i)
        if (caches[i]->handle() != h[i]) {
            void *stream = caches[i]->stream;
            caches[i]->release();
            caches[i] = KVCache::wrap(h[i]);
            caches[i]->stream = stream;
        }
}
}  // namespace detail

// canTrimPromptCache / trimPromptCache
inline bool canTrimPromptCache(const CacheArray &caches) {
    const auto h = detail::handles(caches);
    return kvc_can_trim_prompt_cache(h.data(), (int32_t)h.size()) != 0;
}
inline int64_t trimPromptCache(const CacheArray &caches, int64_t numTokens) {
    const auto h = detail::handles(caches);
    int64_t t = 0;
    check(kvc_trim_prompt_cache(h.data(), (int32_t)h.size(), numTokens, &t));
    return t;
}

// resolveTurboScheme / resolveAffineScheme: (keyBits, valueBits) / (bits, groupSize), or nullopt
inline std::optional<std::pair<int, int>> resolveTurboScheme(const std::string &scheme) {
    int32_t a = 0, b = 0;
    if (!kvc_resolve_turbo_scheme(scheme.c_str(), &a, &b)) return std::nullopt;
    return std::make_pair((int)a, (int)b);
}
inline std::optional<std::pair<int, int>> resolveAffineScheme(const std::string &scheme) {
    int32_t a = 0, b = 0;
    if (!kvc_resolve_affine_scheme(scheme.c_str(), &a, &b)) return std::nullopt;
    return std::make_pair((int)a, (int)b);
}

// maybeAffineQuantizeKVCache / maybeTurboQuantizeKVCache over a flat layer list; returns whether every
// eligible layer has been converted.
inline bool maybeAffineQuantizeKVCache(CacheArray &caches, int bits, int groupSize, int64_t compressionStart,
                                       void *stream = nullptr) {
    auto h = detail::handles(caches);
    int32_t complete = 0;
    check(kvc_maybe_affine_quantize(h.data(), (int32_t)h.size(), bits, groupSize, compressionStart, stream, &complete));
    detail::readopt(caches, h);
    return complete != 0;
}
inline bool maybeTurboQuantizeKVCache(CacheArray &caches, int keyBits, int valueBits, int64_t quantizedKVStart,
                                      void *stream = nullptr) {
    auto h = detail::handles(caches);
    int32_t complete = 0;
    check(kvc_maybe_turbo_quantize(h.data(), (int32_t)h.size(), keyBits, valueBits, quantizedKVStart, stream, &complete));
    detail::readopt(caches, h);
    return complete != 0;
}

// savePromptCache(url:cache:metadata:) / loadPromptCache(url:)
inline void savePromptCache(const std::string &path, const CacheArray &caches,
                            const std::map<std::string, std::string> &metadata = {}, void *stream = nullptr) {
    const auto h = detail::handles(caches);
    std::vector<const char *> keys, values;
    for (const auto &kv : metadata) {
        keys.push_back(kv.first.c_str());
        values.push_back(kv.second.c_str());
    }
    check(kvc_save_prompt_cache(path.c_str(), h.data(), (int32_t)h.size(), keys.data(), values.data(),
                                (int32_t)keys.size(), stream));
}
inline std::pair<CacheArray, std::map<std::string, std::string>> loadPromptCache(const std::string &path, int device = -1,
                                                                                 void *stream = nullptr) {
    int32_t count = 0;
    size_t need = 0;
    check(kvc_load_prompt_cache(path.c_str(), device, nullptr, 0, &count, nullptr, 0, &need, stream));
    std::vector<kvc_cache *> h((size_t)count);
    std::string buf(need ? need : 1, '\0');
    check(kvc_load_prompt_cache(path.c_str(), device, h.data(), count, &count, buf.data(), buf.size(), &need, stream));
    CacheArray caches;
    for (int32_t i = 0; i < count; ++i) caches.push_back(KVCache::wrap(h[(size_t)i]));
    std::map<std::string, std::string> meta;
    for (size_t p = 0; p < buf.size() && buf[p] != '\0';) {   // key NUL value NUL ... closed by an empty key
        const std::string key(buf.c_str() + p);
        p += key.size() + 1;
        const std::string value(buf.c_str() + p);
        p += value.size() + 1;
        meta[key] = value;
    }
    return {std::move(caches), std::move(meta)};
}

// One cache's share of a speculative verify round (KVCacheRound: beginRound / commit / rollback).
class StagedRound {
  public:
    StagedRound(KVCache &cache, int maxPositions) : stream(cache.stream) {
        check(kvc_round_begin(cache.handle(), maxPositions, &r_));
    }
    ~StagedRound() { if (r_) kvc_round_free(r_); }
    StagedRound(const StagedRound &) = delete;
    StagedRound &operator=(const StagedRound &) = delete;

    int64_t offset() const { return kvc_round_offset(r_); }
    std::pair<kvc_tensor, kvc_tensor> update(const kvc_tensor &keys, const kvc_tensor &values) {
        kvc_tensor k{}, v{};
        check(kvc_round_update(r_, &keys, &values, stream, &k, &v));
        return {k, v};
    }
    void attention(const kvc_tensor &queries, const kvc_tensor &keys, const kvc_tensor &values, float scale,
                   const Mask &mask, const kvc_tensor &out) {
        const int32_t mode = mask.kind == MaskKind::none ? KVC_MASK_NONE
                             : mask.kind == MaskKind::causal ? KVC_MASK_CAUSAL : KVC_MASK_ARRAY;
        check(kvc_round_attention(r_, &queries, &keys, &values, scale, mode,
                                  mask.kind == MaskKind::array ? &mask.array : nullptr, &out, stream));
    }
    void commit(int retain) { check(kvc_round_commit(r_, retain, stream)); }
    void rollback() { check(kvc_round_rollback(r_, stream)); }

    void *stream = nullptr;

  private:
    kvc_round *r_ = nullptr;
};

// KVCacheStorage.beginRound / commit over the whole layer array: one staged round per cache, all or
// nothing (throws Error with KVC_ERR_NOT_TRIMMABLE when some cache cannot stage the round).
class StorageRound {
  public:
    StorageRound(const CacheArray &caches, int maxPositions) : rounds_(caches.size(), nullptr) {
        const auto h = detail::handles(caches);
        check(kvc_storage_begin_round(h.data(), (int32_t)h.size(), maxPositions, rounds_.data()));
    }
    ~StorageRound() {
        for (kvc_round *r : rounds_)
            if (r) kvc_round_free(r);
    }
    StorageRound(const StorageRound &) = delete;
    StorageRound &operator=(const StorageRound &) = delete;
    // the verify pass of every layer: queries[i], keys[i], values[i], outs[i] belong to layer i
    void attention(const std::vector<kvc_tensor> &queries, const std::vector<kvc_tensor> &keys,
                   const std::vector<kvc_tensor> &values, float scale, const Mask &mask,
                   const std::vector<kvc_tensor> &outs, void *stream = nullptr) {
        const int32_t mode = mask.kind == MaskKind::none ? KVC_MASK_NONE : KVC_MASK_CAUSAL;
        check(kvc_storage_round_attention(rounds_.data(), (int32_t)rounds_.size(), queries.data(), keys.data(),
                                          values.data(), scale, mode, outs.data(), stream));
    }
    // commit(retaining:): keeps the first `retaining` positions of the round in every cache (0 = rollback)
    void commit(int retaining, void *stream = nullptr) {
        check(kvc_storage_commit(rounds_.data(), (int32_t)rounds_.size(), retaining, stream));
    }

  private:
    std::vector<kvc_round *> rounds_;
};

// The rewind at the end of a speculative round without staged rounds: the main model's caches give back
// numDraft - accepted positions, the draft model's max(numDraft - accepted - 1, 0).
inline int64_t speculateRewind(const CacheArray &caches, int numDraft, int accepted, bool isDraft) {
    const auto h = detail::handles(caches);
    int64_t t = 0;
    check(kvc_speculate_rewind(h.data(), (int32_t)h.size(), numDraft, accepted, isDraft ? 1 : 0, &t));
    return t;
}

// rewindLastRound(count) -> positions taken back
inline int64_t rewindLastRound(KVCache &cache, int64_t count) {
    int64_t n = 0;
    check(kvc_rewind_last_round(cache.handle(), count, cache.stream, &n));
    return n;
}

}  // namespace kvc::host
