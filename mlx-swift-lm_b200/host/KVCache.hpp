// Header-only C++ mirror of MLXLMCommon's KVCache protocol surface
// (Libraries/MLXLMCommon/KVCache.swift:46-104, :156-181) over the C ABI in
// include/kvcache_b200.h. Same member names and argument meaning as the Swift
// classes; programmer errors throw kvc::host::Error where the reference traps.
#pragma once

#include <cstdint>
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
    virtual ~KVCache() { kvc_free(h_); }
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
    bool isCompressed() const { return kvc_is_compressed(h_) != 0; }

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

}  // namespace kvc::host
