// Prompt-cache files: the safetensors layout that savePromptCache / loadPromptCache use
// (KVCache.swift:1797-1846, :1859-1987, restoreCacheFromMetaState :2031-2138), shared with the
// Python mlx-lm cache files:
//   tensors   "i.j"      = array j of cache i's `state`
//   metadata  "0.i.j"    = string j of cache i's `metaState`
//             "1.<key>"  = user metadata
//             "2.i"      = class name of cache i ("KVCache", "RotatingKVCache", "QuantizedKVCache",
//                          "TurboQuantKVCache")
// A safetensors file is an 8-byte little-endian header length, a JSON header
// {"name": {"dtype", "shape", "data_offsets"}, ..., "__metadata__": {...}} and the raw tensors.
// Files that carry model state (class names with the state marker) are refused: this library
// holds caches, not model state.
#include "cache.h"

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "../../include/kvcache_b200.h"

namespace kvc {
namespace {

// ---------------- a small JSON reader: objects, arrays, strings, integers ----------------
struct Json {
    enum Kind { OBJ, ARR, STR, NUM } kind = STR;
    std::string str;
    double num = 0;
    std::vector<std::pair<std::string, Json>> obj;
    std::vector<Json> arr;
    const Json *get(const std::string &k) const {
        for (const auto &e : obj)
            if (e.first == k) return &e.second;
        return nullptr;
    }
};

struct JsonReader {
    const char *p, *end;
    void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
    [[noreturn]] void bad(const char *what) { fail(KVC_ERR_INVALID_ARG, std::string("prompt cache header: ") + what); }
    std::string string() {
        if (p >= end || *p != '"') bad("expected a string");
        ++p;
        std::string out;
        while (p < end && *p != '"') {
            if (*p == '\\') {
                if (++p >= end) bad("truncated escape");
                switch (*p) {
                    case 'n': out += '\n'; break;
                    case 't': out += '\t'; break;
                    case 'r': out += '\r'; break;
                    case 'b': out += '\b'; break;
                    case 'f': out += '\f'; break;
                    case 'u': {
                        if (end - p < 5) bad("truncated \\u escape");
                        unsigned cp = 0;
                        for (int i = 1; i <= 4; ++i) {
                            const char ch = p[i];
                            cp = cp * 16 + (ch >= '0' && ch <= '9' ? ch - '0' : (ch | 32) >= 'a' && (ch | 32) <= 'f' ? (ch | 32) - 'a' + 10 : 0);
                        }
                        p += 4;
                        if (cp < 0x80) out += (char)cp;
                        else if (cp < 0x800) { out += (char)(0xC0 | (cp >> 6)); out += (char)(0x80 | (cp & 0x3F)); }
                        else { out += (char)(0xE0 | (cp >> 12)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
                        break;
                    }
                    default: out += *p;
                }
                ++p;
            } else {
                out += *p++;
            }
        }
        if (p >= end) bad("unterminated string");
        ++p;
        return out;
    }
    Json value(int depth = 0) {
        if (depth > 8) bad("nesting too deep");
        ws();
        if (p >= end) bad("truncated");
        Json j;
        if (*p == '{') {
            j.kind = Json::OBJ;
            ++p;
            ws();
            if (p < end && *p == '}') { ++p; return j; }
            for (;;) {
                ws();
                std::string k = string();
                ws();
                if (p >= end || *p != ':') bad("expected ':'");
                ++p;
                j.obj.emplace_back(std::move(k), value(depth + 1));
                ws();
                if (p < end && *p == ',') { ++p; continue; }
                if (p < end && *p == '}') { ++p; break; }
                bad("expected ',' or '}'");
            }
        } else if (*p == '[') {
            j.kind = Json::ARR;
            ++p;
            ws();
            if (p < end && *p == ']') { ++p; return j; }
            for (;;) {
                j.arr.push_back(value(depth + 1));
                ws();
                if (p < end && *p == ',') { ++p; continue; }
                if (p < end && *p == ']') { ++p; break; }
                bad("expected ',' or ']'");
            }
        } else if (*p == '"') {
            j.kind = Json::STR;
            j.str = string();
        } else {
            j.kind = Json::NUM;
            char *e = nullptr;
            j.num = std::strtod(p, &e);
            if (e == p || e > end) bad("expected a value");
            p = e;
        }
        return j;
    }
};

void json_escape(std::string &out, const std::string &s) {
    out += '"';
    for (unsigned char ch : s) {
        switch (ch) {
            case '"': out += "\\\""; break;
            case '\\': out += "\\\\"; break;
            case '\n': out += "\\n"; break;
            case '\t': out += "\\t"; break;
            case '\r': out += "\\r"; break;
            default:
                if (ch < 0x20) {
                    char buf[8];
                    std::snprintf(buf, sizeof buf, "\\u%04x", ch);
                    out += buf;
                } else {
                    out += (char)ch;
                }
        }
    }
    out += '"';
}

const char *st_dtype(int32_t d) {
    switch (d) {
        case KVC_F32: return "F32";
        case KVC_F16: return "F16";
        case KVC_BF16: return "BF16";
        case KVC_U32: return "U32";
        case KVC_BOOL: return "BOOL";
        default: fail(KVC_ERR_UNSUPPORTED, "prompt cache: unsupported dtype");
    }
}

int32_t kvc_dtype(const std::string &s) {
    if (s == "F32") return KVC_F32;
    if (s == "F16") return KVC_F16;
    if (s == "BF16") return KVC_BF16;
    if (s == "U32") return KVC_U32;
    if (s == "BOOL") return KVC_BOOL;
    fail(KVC_ERR_UNSUPPORTED, "prompt cache: unsupported tensor dtype '" + s + "'");
}

const char *class_name(int32_t kind) {
    switch (kind) {
        case KVC_KIND_SIMPLE: return "KVCache";
        case KVC_KIND_ROTATING: return "RotatingKVCache";
        case KVC_KIND_QUANTIZED: return "QuantizedKVCache";
        case KVC_KIND_TURBO: return "TurboQuantKVCache";
        case KVC_KIND_CHUNKED: return "ChunkedKVCache";
        case KVC_KIND_LIST: return "CacheList";
        default: fail(KVC_ERR_UNSUPPORTED, "prompt cache: unknown cache kind");
    }
}

std::vector<std::string> split_lines(const std::string &joined) {
    std::vector<std::string> out;
    size_t a = 0;
    for (;;) {
        const size_t b = joined.find('\n', a);
        out.push_back(joined.substr(a, b == std::string::npos ? std::string::npos : b - a));
        if (b == std::string::npos) break;
        a = b + 1;
    }
    return out;
}

void must(kvc_status st) {
    if (st != KVC_OK) fail(st, kvc_last_error_message());
}

int64_t parse_int(const std::string &s, const char *cls) {
    char *e = nullptr;
    const long long v = std::strtoll(s.c_str(), &e, 10);
    if (s.empty() || *e) fail(KVC_ERR_INVALID_ARG, std::string("Corrupt prompt cache: ") + cls + " metadata '" + s + "' is not an integer.");
    return v;
}

struct FileCloser {
    FILE *f;
    ~FileCloser() { if (f) std::fclose(f); }
};

// restoreCacheFromMetaState (KVCache.swift:2031-2138): a cache of class `cls` from its state arrays
// (device tensors, copied) and metaState strings. CacheList recurses (CacheList.fromState :1689-1725).
kvc_cache *restore_cache(const std::string &cls, const std::vector<kvc_tensor> &tens, const std::vector<std::string> &ms,
                         int device, cudaStream_t s) {
    auto require_counts = [&](const char *name, std::initializer_list<size_t> sc, std::initializer_list<size_t> mc) {
        bool s_ok = false, m_ok = false;
        for (size_t x : sc) s_ok = s_ok || tens.size() == x;
        for (size_t x : mc) m_ok = m_ok || ms.size() == x;
        if (!s_ok) fail(KVC_ERR_INVALID_ARG, std::string("Corrupt prompt cache: ") + name + " has " + std::to_string(tens.size()) + " state arrays.");
        for (const kvc_tensor &t : tens)
            if (t.ndim != 4) fail(KVC_ERR_INVALID_ARG, std::string("Corrupt prompt cache: invalid ") + name + " state shape.");
        if (!m_ok) fail(KVC_ERR_INVALID_ARG, std::string("Corrupt prompt cache: ") + name + " has " + std::to_string(ms.size()) + " metadata entries.");
    };
    if (cls.rfind("__mlx_lm_state", 0) == 0) fail(KVC_ERR_UNSUPPORTED, "Prompt cache contains model state; this library restores caches only");
    if (cls == "CacheList") {
        if (ms.empty()) fail(KVC_ERR_INVALID_ARG, "CacheList metaState missing child count");
        const int64_t child_count = parse_int(ms[0], "CacheList");
        std::vector<kvc_cache *> children;
        struct Guard { std::vector<kvc_cache *> &v; bool armed = true; ~Guard() { if (armed) for (kvc_cache *c : v) kvc_free(c); } } guard{children};
        size_t mi = 1, si = 0;
        for (int64_t k = 0; k < child_count; ++k) {
            if (mi + 2 >= ms.size()) fail(KVC_ERR_INVALID_ARG, "CacheList metaState truncated");
            const std::string child_cls = ms[mi];
            const int64_t state_count = parse_int(ms[mi + 1], "CacheList");
            const int64_t meta_count = parse_int(ms[mi + 2], "CacheList");
            mi += 3;
            std::vector<std::string> child_meta;
            for (int64_t j = 0; j < meta_count && mi + (size_t)j < ms.size(); ++j) child_meta.push_back(ms[mi + (size_t)j]);
            mi += (size_t)meta_count;
            std::vector<kvc_tensor> child_state;
            for (int64_t j = 0; j < state_count && si + (size_t)j < tens.size(); ++j) child_state.push_back(tens[si + (size_t)j]);
            si += (size_t)state_count;
            children.push_back(restore_cache(child_cls, child_state, child_meta, device, s));
        }
        kvc_cache *list = nullptr;
        must(kvc_list_create(children.data(), (int32_t)children.size(), &list));
        guard.armed = false;   // the list owns them now
        return list;
    }
    kvc_config cfg;
    bool set_meta = true;
    if (cls == "KVCache" || cls == "KVCacheSimple") {
        require_counts("KVCacheSimple", {0, 2}, {1});
        if (!ms[0].empty()) fail(KVC_ERR_INVALID_ARG, "Corrupt prompt cache: KVCacheSimple metadata must contain its single empty placeholder.");
        kvc_config_default(&cfg, KVC_KIND_SIMPLE);
        set_meta = false;
    } else if (cls == "RotatingKVCache") {
        require_counts("RotatingKVCache", {0, 2}, {5, 6});
        for (int j = 0; j < 5; ++j) (void)parse_int(ms[(size_t)j], "RotatingKVCache");
        kvc_config_default(&cfg, KVC_KIND_ROTATING);
        cfg.max_size = parse_int(ms[1], "RotatingKVCache");
    } else if (cls == "QuantizedKVCache") {
        require_counts("QuantizedKVCache", {0, 4, 6}, {4});
        for (const std::string &m : ms) (void)parse_int(m, "QuantizedKVCache");
        kvc_config_default(&cfg, KVC_KIND_QUANTIZED);
        cfg.group_size = (int32_t)parse_int(ms[2], "QuantizedKVCache");
        cfg.bits = (int32_t)parse_int(ms[3], "QuantizedKVCache");
    } else if (cls == "ChunkedKVCache") {
        require_counts("ChunkedKVCache", {0, 2}, {2});
        kvc_config_default(&cfg, KVC_KIND_CHUNKED);
        cfg.max_size = ms[0] == "None" ? -1 : (int32_t)parse_int(ms[0], "ChunkedKVCache");
        (void)parse_int(ms[1], "ChunkedKVCache");
    } else if (cls == "TurboQuantKVCache") {
        if (ms.size() < 5) fail(KVC_ERR_INVALID_ARG, "Invalid TurboQuantKVCache metaState");
        kvc_config_default(&cfg, KVC_KIND_TURBO);
        cfg.bits = (int32_t)parse_int(ms[1], "TurboQuantKVCache");
        cfg.key_bits = (int32_t)parse_int(ms[2], "TurboQuantKVCache");
        cfg.value_bits = (int32_t)parse_int(ms[3], "TurboQuantKVCache");
        cfg.seed = (uint64_t)std::strtoull(ms[4].c_str(), nullptr, 10);
    } else {
        fail(KVC_ERR_UNSUPPORTED, "Unknown cache class: " + cls);
    }
    cfg.device = device;
    kvc_cache *c = nullptr;
    must(kvc_create(&cfg, &c));
    struct One { kvc_cache *c; bool armed = true; ~One() { if (armed) kvc_free(c); } } one{c};
    if (!tens.empty()) must(kvc_state_set(c, tens.data(), (int32_t)tens.size(), (void *)s));
    if (set_meta) {
        std::string joined;
        for (size_t j = 0; j < ms.size(); ++j) {
            if (j) joined += '\n';
            joined += ms[j];
        }
        must(kvc_set_meta_state(c, joined.c_str()));
    }
    one.armed = false;
    return c;
}

}  // namespace

void save_prompt_cache(const char *path, kvc_cache *const *caches, int count, const char *const *keys,
                       const char *const *values, int meta_count, cudaStream_t s) {
    struct Entry { std::string name; kvc_tensor desc; std::vector<char> bytes; };
    std::vector<Entry> tensors;
    std::vector<std::pair<std::string, std::string>> meta;
    for (int i = 0; i < count; ++i) {
        kvc_cache *c = caches[i];
        const int n = kvc_state_count(c);
        for (int j = 0; j < n; ++j) {
            kvc_tensor view;
            must(kvc_state_get(c, j, &view));
            size_t elems = 1;
            for (int d = 0; d < view.ndim; ++d) elems *= (size_t)view.shape[d];
            Entry e;
            e.name = std::to_string(i) + "." + std::to_string(j);
            e.bytes.resize(elems * dtype_size(view.dtype));
            must(kvc_state_export(c, j, e.bytes.data(), e.bytes.size(), &e.desc, (void *)s));
            tensors.push_back(std::move(e));
        }
        size_t need = 0;
        must(kvc_meta_state(c, nullptr, 0, &need));
        std::string joined(need ? need : 1, '\0');
        must(kvc_meta_state(c, &joined[0], joined.size(), &need));
        joined.resize(std::strlen(joined.c_str()));
        const std::vector<std::string> lines = split_lines(joined);
        for (size_t j = 0; j < lines.size(); ++j) meta.emplace_back("0." + std::to_string(i) + "." + std::to_string(j), lines[j]);
        meta.emplace_back("2." + std::to_string(i), class_name(kvc_kind_of(c)));
    }
    for (int i = 0; i < meta_count; ++i) {
        if (std::strncmp(keys[i], "__mlx_lm_state_", 15) == 0)
            fail(KVC_ERR_INVALID_ARG, "User metadata uses the reserved prompt cache state namespace");
        meta.emplace_back(std::string("1.") + keys[i], values[i]);
    }

    std::string header = "{";
    size_t offset = 0;
    for (const Entry &e : tensors) {
        json_escape(header, e.name);
        header += ":{\"dtype\":\"";
        header += st_dtype(e.desc.dtype);
        header += "\",\"shape\":[";
        for (int d = 0; d < e.desc.ndim; ++d) {
            if (d) header += ',';
            header += std::to_string(e.desc.shape[d]);
        }
        header += "],\"data_offsets\":[" + std::to_string(offset) + "," + std::to_string(offset + e.bytes.size()) + "]},";
        offset += e.bytes.size();
    }
    header += "\"__metadata__\":{";
    for (size_t i = 0; i < meta.size(); ++i) {
        if (i) header += ',';
        json_escape(header, meta[i].first);
        header += ':';
        json_escape(header, meta[i].second);
    }
    header += "}}";
    while (header.size() % 8) header += ' ';  // tensor data starts 8-byte aligned

    FileCloser fc{std::fopen(path, "wb")};
    if (!fc.f) fail(KVC_ERR_INVALID_ARG, std::string("prompt cache: cannot open '") + path + "' for writing");
    const uint64_t hlen = header.size();
    unsigned char le[8];
    for (int i = 0; i < 8; ++i) le[i] = (unsigned char)(hlen >> (8 * i));
    bool ok = std::fwrite(le, 1, 8, fc.f) == 8 && std::fwrite(header.data(), 1, header.size(), fc.f) == header.size();
    for (const Entry &e : tensors) ok = ok && (e.bytes.empty() || std::fwrite(e.bytes.data(), 1, e.bytes.size(), fc.f) == e.bytes.size());
    if (!ok) fail(KVC_ERR_INVALID_STATE, std::string("prompt cache: short write to '") + path + "'");
}

// Returns the caches of the file (ownership passes to the caller) and the user metadata.
void load_prompt_cache(const char *path, int device, std::vector<kvc_cache *> &out,
                       std::vector<std::pair<std::string, std::string>> &user_meta, cudaStream_t s) {
    FileCloser fc{std::fopen(path, "rb")};
    if (!fc.f) fail(KVC_ERR_INVALID_ARG, std::string("prompt cache: cannot open '") + path + "'");
    unsigned char le[8];
    if (std::fread(le, 1, 8, fc.f) != 8) fail(KVC_ERR_INVALID_ARG, "prompt cache: file too short");
    uint64_t hlen = 0;
    for (int i = 0; i < 8; ++i) hlen |= (uint64_t)le[i] << (8 * i);
    if (hlen == 0 || hlen > (1ull << 28)) fail(KVC_ERR_INVALID_ARG, "prompt cache: implausible header length");
    std::string header(hlen, '\0');
    if (std::fread(&header[0], 1, hlen, fc.f) != hlen) fail(KVC_ERR_INVALID_ARG, "prompt cache: truncated header");
    JsonReader rd{header.data(), header.data() + header.size()};
    const Json root = rd.value();
    if (root.kind != Json::OBJ) fail(KVC_ERR_INVALID_ARG, "prompt cache header: not an object");

    std::map<int, std::vector<std::string>> meta_state;   // cache -> metaState strings
    std::map<int, std::string> classes;
    if (const Json *m = root.get("__metadata__")) {
        for (const auto &kv : m->obj) {
            const std::string &k = kv.first;
            if (k.rfind("0.", 0) == 0) {
                const size_t dot = k.find('.', 2);
                if (dot == std::string::npos) continue;
                const int i = (int)parse_int(k.substr(2, dot - 2), "metadata key");
                const int j = (int)parse_int(k.substr(dot + 1), "metadata key");
                auto &v = meta_state[i];
                if ((int)v.size() <= j) v.resize((size_t)j + 1);
                v[(size_t)j] = kv.second.str;
            } else if (k.rfind("1.", 0) == 0) {
                if (k.compare(2, 15, "__mlx_lm_state_") == 0)
                    fail(KVC_ERR_UNSUPPORTED, "Prompt cache contains model state; this library restores caches only");
                user_meta.emplace_back(k.substr(2), kv.second.str);
            } else if (k.rfind("2.", 0) == 0) {
                classes[(int)parse_int(k.substr(2), "metadata key")] = kv.second.str;
            }
        }
    }
    struct Ten { int j; int32_t dtype; std::vector<int64_t> shape; uint64_t a, b; };
    std::map<int, std::vector<Ten>> state;
    for (const auto &kv : root.obj) {
        if (kv.first == "__metadata__") continue;
        if (kv.first.rfind("__mlx_lm_state_tensor_", 0) == 0)
            fail(KVC_ERR_UNSUPPORTED, "Prompt cache contains model state; this library restores caches only");
        const size_t dot = kv.first.find('.');
        if (dot == std::string::npos) fail(KVC_ERR_UNSUPPORTED, "prompt cache: unexpected tensor '" + kv.first + "'");
        Ten t;
        const int i = (int)parse_int(kv.first.substr(0, dot), "tensor name");
        t.j = (int)parse_int(kv.first.substr(dot + 1), "tensor name");
        const Json *dt = kv.second.get("dtype"), *sh = kv.second.get("shape"), *off = kv.second.get("data_offsets");
        if (!dt || !sh || !off || off->arr.size() != 2) fail(KVC_ERR_INVALID_ARG, "prompt cache header: incomplete tensor entry");
        t.dtype = kvc_dtype(dt->str);
        for (const Json &d : sh->arr) t.shape.push_back((int64_t)d.num);
        t.a = (uint64_t)off->arr[0].num;
        t.b = (uint64_t)off->arr[1].num;
        state[i].push_back(std::move(t));
    }

    const int n = (int)classes.size();
    if ((int)meta_state.size() != n) fail(KVC_ERR_INVALID_ARG, "Mismatch in cache counts");
    for (const auto &kv : state)
        if (kv.first < 0 || kv.first >= n)
            fail(KVC_ERR_INVALID_ARG, "Corrupt prompt cache: array of cache " + std::to_string(kv.first) + " has no class entry.");
    struct Cleanup {
        std::vector<kvc_cache *> &v;
        bool armed = true;
        ~Cleanup() { if (armed) for (kvc_cache *c : v) kvc_free(c); if (armed) v.clear(); }
    } cleanup{out};
    for (int i = 0; i < n; ++i) {
        if (!classes.count(i)) fail(KVC_ERR_INVALID_ARG, "Corrupt prompt cache: class names are not contiguous");
        const std::string &cls = classes[i];
        if (cls.rfind("__mlx_lm_state", 0) == 0) fail(KVC_ERR_UNSUPPORTED, "Prompt cache contains model state; this library restores caches only");
        std::vector<Ten> &tens = state[i];
        std::sort(tens.begin(), tens.end(), [](const Ten &x, const Ten &y) { return x.j < y.j; });
        for (size_t j = 0; j < tens.size(); ++j)
            if (tens[j].j != (int)j) fail(KVC_ERR_INVALID_ARG, "Corrupt prompt cache: state arrays are not contiguous");
        const std::vector<std::string> &ms = meta_state[i];
        // the entry's arrays, on the device for the duration of the restore
        std::vector<void *> dev_bufs;
        std::vector<kvc_tensor> descs;
        struct Free { std::vector<void *> &b; ~Free() { for (void *p : b) cudaFree(p); } } freer{dev_bufs};
        for (const Ten &t : tens) {
            kvc_tensor d = {};
            d.dtype = t.dtype;
            d.ndim = (int32_t)t.shape.size();
            if (d.ndim < 1 || d.ndim > 5) fail(KVC_ERR_INVALID_ARG, "prompt cache: tensor rank out of range");
            size_t elems = 1;
            for (int k = 0; k < d.ndim; ++k) {
                d.shape[k] = t.shape[(size_t)k];
                elems *= (size_t)t.shape[(size_t)k];
            }
            int64_t stride = 1;
            for (int k = d.ndim - 1; k >= 0; --k) {
                d.stride[k] = stride;
                stride *= d.shape[k];
            }
            const size_t bytes = elems * dtype_size(t.dtype);
            if (t.b < t.a || t.b - t.a != bytes) fail(KVC_ERR_INVALID_ARG, "Corrupt prompt cache: tensor size does not match its shape");
            std::vector<char> host(bytes);
            if (std::fseek(fc.f, (long)(8 + hlen + t.a), SEEK_SET) != 0 || (bytes && std::fread(host.data(), 1, bytes, fc.f) != bytes))
                fail(KVC_ERR_INVALID_ARG, "prompt cache: truncated tensor data");
            void *dp = nullptr;
            KVC_CUDA(cudaMalloc(&dp, bytes ? bytes : 16));
            dev_bufs.push_back(dp);
            KVC_CUDA(cudaMemcpyAsync(dp, host.data(), bytes, cudaMemcpyHostToDevice, s));
            KVC_CUDA(cudaStreamSynchronize(s));   // `host` goes out of scope
            d.data = dp;
            descs.push_back(d);
        }
        out.push_back(restore_cache(cls, descs, ms, device, s));
        if (!descs.empty()) KVC_CUDA(cudaStreamSynchronize(s));   // the staging buffers are freed at the end of the iteration
    }
    cleanup.armed = false;
}

}  // namespace kvc
