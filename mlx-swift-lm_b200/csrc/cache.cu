// Cache state machines. Every function here follows the bookkeeping of the
// reference class it replaces (cited per function); the arithmetic and the row
// movement run in the CUDA kernels of this library.
#include "cache.h"

#include <algorithm>
#include <limits>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <vector>

namespace kvc {

// Set by the batched entry points around each layer's call: the cache of the layer launched just
// before on the same stream (nullptr outside a batched call or for its first layer).
static thread_local const kvc_cache *tl_batch_prev = nullptr;
void set_batch_previous(const kvc_cache *prev) { tl_batch_prev = prev; }

int launch_attention(const AttnArgs &a, cudaStream_t stream);

namespace {

int64_t round_up(int64_t x, int64_t q) { return ((x + q - 1) / q) * q; }

void require4(const kvc_tensor &t, const char *what) {
    if (t.ndim != 4) fail(KVC_ERR_INVALID_ARG, std::string(what) + ": expected a 4-d tensor [B, H, S, D]");
    if (!t.data && t.shape[0] * t.shape[1] * t.shape[2] * t.shape[3] != 0)
        fail(KVC_ERR_INVALID_ARG, std::string(what) + ": null data pointer");
    for (int i = 0; i < 4; ++i)
        if (t.shape[i] < 0) fail(KVC_ERR_INVALID_ARG, std::string(what) + ": negative dimension");
}

void zero_rows(Array4 &a, int64_t first, int64_t count, cudaStream_t s) {
    if (count <= 0 || !a.ptr) return;
    const size_t pitch = (size_t)a.cap * a.W * a.esize();
    KVC_CUDA(cudaMemset2DAsync((char *)a.ptr + (size_t)first * a.W * a.esize(), pitch, 0,
                               (size_t)count * a.W * a.esize(), (size_t)(a.B * a.H), s));
}

void copy_rows(const Array4 &src, int64_t src_first, Array4 &dst, int64_t dst_first, int64_t count,
               cudaStream_t s) {
    if (count <= 0) return;
    GatherArgs g;
    g.src = src.ptr;
    g.dst = dst.ptr;
    g.s_sb = src.sb(); g.s_sh = src.sh(); g.s_st = src.st();
    g.d_sb = dst.sb(); g.d_sh = dst.sh(); g.d_st = dst.st();
    g.B = (int)src.B; g.H = (int)src.H; g.W = (int)src.W;
    g.esize = (int)src.esize();
    g.nseg = 1;
    g.seg[0] = {src_first, count};
    g.dst_start = dst_first;
    launch_gather(g, s);
}

void gather_rows(const Array4 &src, Array4 &dst, const std::vector<GatherSeg> &segs, cudaStream_t s) {
    if (segs.size() > 4) fail(KVC_ERR_INTERNAL, "ring re-order produced more than 4 segments");
    GatherArgs g;
    g.src = src.ptr;
    g.dst = dst.ptr;
    g.s_sb = src.sb(); g.s_sh = src.sh(); g.s_st = src.st();
    g.d_sb = dst.sb(); g.d_sh = dst.sh(); g.d_st = dst.st();
    g.B = (int)src.B; g.H = (int)src.H; g.W = (int)src.W;
    g.esize = (int)src.esize();
    g.nseg = (int)segs.size();
    for (size_t i = 0; i < segs.size(); ++i) g.seg[i] = segs[i];
    g.dst_start = 0;
    launch_gather(g, s);
}

// Append the rows of `t` ([B, H, S, W], any strides) to `dst` at token `pos`.
void append_pair(Array4 &kd, Array4 &vd, const kvc_tensor &k, const kvc_tensor &v, int64_t pos,
                 cudaStream_t s) {
    AppendArgs a;
    a.k_src = k.data; a.v_src = v.data;
    a.ks_sb = k.stride[0]; a.ks_sh = k.stride[1]; a.ks_ss = k.stride[2]; a.ks_sd = k.stride[3];
    a.vs_sb = v.stride[0]; a.vs_sh = v.stride[1]; a.vs_ss = v.stride[2]; a.vs_sd = v.stride[3];
    a.k_dst = kd.ptr; a.v_dst = vd.ptr;
    a.kd_sb = kd.sb(); a.kd_sh = kd.sh(); a.kd_st = kd.st();
    a.vd_sb = vd.sb(); a.vd_sh = vd.sh(); a.vd_st = vd.st();
    a.B = (int)k.shape[0]; a.H = (int)k.shape[1]; a.S = (int)k.shape[2];
    a.Dk = (int)k.shape[3]; a.Dv = (int)v.shape[3];
    a.pos = pos;
    a.esize = (int)dtype_size(k.dtype);
    launch_append(a, s);
}

int64_t seg_total(const std::vector<GatherSeg> &v) {
    int64_t n = 0;
    for (auto &g : v) n += g.count;
    return n;
}

void seg_push(std::vector<GatherSeg> &out, int64_t start, int64_t count) {
    if (count <= 0) return;
    if (!out.empty() && out.back().src_start + out.back().count == start) out.back().count += count;
    else out.push_back({start, count});
}

// Sub-range [begin, end) of the sequence described by `in`.
std::vector<GatherSeg> seg_slice(const std::vector<GatherSeg> &in, int64_t begin, int64_t end) {
    std::vector<GatherSeg> out;
    int64_t pos = 0;
    for (auto &g : in) {
        const int64_t lo = std::max(begin, pos), hi = std::min(end, pos + g.count);
        if (hi > lo) seg_push(out, g.src_start + (lo - pos), hi - lo);
        pos += g.count;
    }
    return out;
}

std::vector<GatherSeg> seg_concat(std::vector<GatherSeg> a, const std::vector<GatherSeg> &b) {
    for (auto &g : b) seg_push(a, g.src_start, g.count);
    return a;
}

// RotatingKVCache.temporalOrder (KVCache.swift:592-606) as a row mapping.
std::vector<GatherSeg> rot_temporal(const kvc_cache *c) {
    std::vector<GatherSeg> t;
    if (c->idx < 0) fail(KVC_ERR_INVALID_STATE, "rotating cache: ring index is negative (trim past the ring start)");
    if (c->idx == c->len) {
        seg_push(t, 0, c->len);
    } else if (c->idx < c->offset) {
        const int64_t k0 = std::min<int64_t>(c->cfg.keep, c->len);
        const int64_t id = std::min(c->idx, c->len);
        seg_push(t, 0, k0);
        seg_push(t, id, c->len - id);
        seg_push(t, std::min<int64_t>(c->cfg.keep, id), id - std::min<int64_t>(c->cfg.keep, id));
    } else {
        seg_push(t, 0, std::min(c->idx, c->len));
    }
    return t;
}

// RotatingKVCache.trim(trimSize:_:) (KVCache.swift:576-590) applied to a sequence.
std::vector<GatherSeg> rot_front_trim(const std::vector<GatherSeg> &seq, int64_t trim_size, int64_t keep) {
    if (trim_size <= 0) return seq;
    const int64_t n = seg_total(seq);
    auto head = seg_slice(seq, 0, std::min(keep, n));
    auto tail = seg_slice(seq, std::min(trim_size + keep, n), n);
    return seg_concat(head, tail);
}

void ensure_like(Array4 &dst, const Array4 &like, int64_t need_cap, cudaStream_t s) {
    if (dst.allocated() && dst.cap >= need_cap && dst.B == like.B && dst.H == like.H &&
        dst.W == like.W && dst.dtype == like.dtype)
        return;
    dst.release(s);
    dst.alloc(like.B, like.H, need_cap, like.W, like.dtype, s);
}

// Replace the ring contents by the rows `segs` selects (in that order).
void rot_rebuild(kvc_cache *c, const std::vector<GatherSeg> &segs, int64_t extra_cap, cudaStream_t s) {
    const int64_t n = seg_total(segs);
    const int64_t need = std::max<int64_t>(std::max<int64_t>(n + extra_cap, c->cfg.max_size), c->k.cap);
    ensure_like(c->k_alt, c->k, need, s);
    ensure_like(c->v_alt, c->v, need, s);
    gather_rows(c->k, c->k_alt, segs, s);
    gather_rows(c->v, c->v_alt, segs, s);
    std::swap(c->k, c->k_alt);
    std::swap(c->v, c->v_alt);
    c->len = n;
}

void check_new_rows(const kvc_cache *c, const Array4 &ka, const Array4 &va, const kvc_tensor &k,
                    const kvc_tensor &v) {
    if (!ka.allocated()) return;
    if (k.shape[0] != ka.B || k.shape[1] != ka.H)
        fail(KVC_ERR_INVALID_ARG, "update: batch / head count differs from the cached arrays");
    (void)c; (void)va; (void)v;
}

}  // namespace

// ---------------------------------------------------------------------
// Array4
// ---------------------------------------------------------------------
void Array4::alloc(int64_t b, int64_t h, int64_t c, int64_t w, int32_t dt, cudaStream_t s) {
    // capacity in whole 256-token steps (the reference's allocation step): the TMA-staged attention
    // kernels copy full stages of up to 256 tokens, and a stage must never reach past the (batch, head) slab
    B = b; H = h; cap = round_up(std::max<int64_t>(c, 1), 256); W = w; dtype = dt;
    ptr = dev_alloc(bytes(), s);
    KVC_CUDA(cudaMemsetAsync(ptr, 0, bytes(), s));
}

void Array4::release(cudaStream_t s) {
    if (ptr) dev_free(ptr, s);
    ptr = nullptr;
    cap = 0;
}

void Array4::ensure(int64_t need, int64_t keep_rows, int64_t step, cudaStream_t s) {
    if (!ptr) fail(KVC_ERR_INTERNAL, "Array4::ensure on an unallocated array");
    if (need <= cap) return;
    step = std::max<int64_t>(step, 1);
    const int64_t grown = round_up(cap + cap / 2, step);
    const int64_t new_cap = std::max(round_up(need, step), grown);
    Array4 next;
    next.alloc(B, H, new_cap, W, dtype, s);
    copy_rows(*this, 0, next, 0, std::min(keep_rows, cap), s);
    dev_free(ptr, s);
    *this = next;
}

kvc_tensor Array4::view(int64_t tokens, int64_t first) const {
    kvc_tensor t{};
    t.data = ptr ? (void *)((char *)ptr + (size_t)first * W * esize()) : nullptr;
    t.dtype = dtype;
    t.ndim = 4;
    t.shape[0] = B; t.shape[1] = H; t.shape[2] = tokens; t.shape[3] = W;
    t.stride[0] = sb(); t.stride[1] = sh(); t.stride[2] = st(); t.stride[3] = 1;
    return t;
}

static kvc_tensor view3(const Array4 &a, int64_t tokens) {
    kvc_tensor t = a.view(tokens);
    t.ndim = 3;
    t.shape[3] = 0;
    t.stride[3] = 0;
    return t;
}


void turbo_rotation(int dim, uint64_t seed, std::vector<float> &rotation) {
    // TurboQuantRotation.rotationMatrix (TurboQuantKVCache.swift:246-259): QR of a seeded Gaussian matrix,
    // the columns of Q flipped by the signs of R's diagonal. The reference draws the matrix from MLXRandom
    // and factors it with MLX's QR, neither of which is reproducible outside MLX; this library defines its
    // own: Box-Muller normals from the splitmix64 stream seeded with `seed` (row-major fill), Householder QR
    // in double precision, result rounded to float32.
    const int n = dim;
    std::vector<double> a((size_t)n * n);
    uint64_t x = seed;
    auto next_u = [&]() {
        x += 0x9E3779B97F4A7C15ull;
        uint64_t z = x;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        z = z ^ (z >> 31);
        return ((double)(z >> 11) + 0.5) / 9007199254740992.0;   // (0, 1)
    };
    for (size_t i = 0; i < a.size(); i += 2) {
        const double u1 = next_u(), u2 = next_u();
        const double r = std::sqrt(-2.0 * std::log(u1)), t = 6.283185307179586476925286766559 * u2;
        a[i] = r * std::cos(t);
        if (i + 1 < a.size()) a[i + 1] = r * std::sin(t);
    }
    // Householder: A = Q R; accumulate Q explicitly
    std::vector<double> q((size_t)n * n, 0.0), v(n);
    for (int i = 0; i < n; ++i) q[(size_t)i * n + i] = 1.0;
    std::vector<double> rdiag(n, 0.0);
    for (int k = 0; k < n; ++k) {
        double norm = 0.0;
        for (int i = k; i < n; ++i) norm += a[(size_t)i * n + k] * a[(size_t)i * n + k];
        norm = std::sqrt(norm);
        const double akk = a[(size_t)k * n + k];
        const double alpha = akk > 0 ? -norm : norm;
        for (int i = 0; i < n; ++i) v[i] = 0.0;
        for (int i = k; i < n; ++i) v[i] = a[(size_t)i * n + k];
        v[k] -= alpha;
        double vnorm2 = 0.0;
        for (int i = k; i < n; ++i) vnorm2 += v[i] * v[i];
        if (vnorm2 > 0.0) {
            for (int j = 0; j < n; ++j) {      // A <- (I - 2 v v^T / v^T v) A
                double dot = 0.0;
                for (int i = k; i < n; ++i) dot += v[i] * a[(size_t)i * n + j];
                const double f = 2.0 * dot / vnorm2;
                for (int i = k; i < n; ++i) a[(size_t)i * n + j] -= f * v[i];
            }
            for (int i = 0; i < n; ++i) {      // Q <- Q (I - 2 v v^T / v^T v)
                double dot = 0.0;
                for (int j = k; j < n; ++j) dot += q[(size_t)i * n + j] * v[j];
                const double f = 2.0 * dot / vnorm2;
                for (int j = k; j < n; ++j) q[(size_t)i * n + j] -= f * v[j];
            }
        }
        rdiag[k] = a[(size_t)k * n + k];
    }
    rotation.resize((size_t)n * n);
    for (int i = 0; i < n; ++i)
        for (int j = 0; j < n; ++j)
            rotation[(size_t)i * n + j] = (float)(q[(size_t)i * n + j] * (rdiag[j] < 0 ? -1.0 : 1.0));
}

}  // namespace kvc

kvc_cache::~kvc_cache() {
    // free in the order of the stream that last used the arrays, on the handle's device
    cudaStream_t s = last_stream;
    int prev = -1;
    const bool switched = device >= 0 && cudaGetDevice(&prev) == cudaSuccess && prev != device && cudaSetDevice(device) == cudaSuccess;
    kvc::Array4 *arrays[] = {&k, &v, &k_alt, &v_alt, &k_view, &v_view, &kq, &ks, &kb, &vq, &vs, &vb,
                             &kp, &kn, &vp, &vn, &restore.k, &restore.v, &restore.rk, &restore.rv};
    for (auto *a : arrays) a->release(s);
    for (int i = 0; i < 4; ++i)
        if (stage[i]) kvc::dev_free(stage[i], s);
    if (kcodec.signs_dev) kvc::dev_free(kcodec.signs_dev, s);
    if (vcodec.signs_dev) kvc::dev_free(vcodec.signs_dev, s);
    if (kcodec.calib_dev) kvc::dev_free(kcodec.calib_dev, s);
    if (kcodec.rotation_dev) kvc::dev_free(kcodec.rotation_dev, s);
    if (vcodec.rotation_dev) kvc::dev_free(vcodec.rotation_dev, s);
    for (kvc_cache *child : children) delete child;
    if (switched) (void)cudaSetDevice(prev);
}

namespace kvc {

int resolved_group_size(int requested, int kd, int vd) {
    // resolvedKVQuantizationGroupSize (KVCache.swift:902-920): nearest of
    // {32, 64, 128} dividing both head dims, ties to the smaller.
    requested = std::max(1, requested);
    int best = 0;
    for (int g : {32, 64, 128}) {
        if (kd % g || vd % g) continue;
        if (!best) { best = g; continue; }
        const int db = std::abs(best - requested), dg = std::abs(g - requested);
        if (dg < db || (dg == db && g < best)) best = g;
    }
    return best;
}

// ---------------------------------------------------------------------
// update
// ---------------------------------------------------------------------

// KVCacheSimple.update (KVCache.swift:404-447) and the raw prefill phase of
// TurboQuantKVCache.update (TurboQuantKVCache.swift:802-846). Capacity grows
// ahead of need, which the protocol surface cannot observe: every getter
// exposes rows [0, offset) only.
static void linear_update(kvc_cache *c, const kvc_tensor &k, const kvc_tensor &v, cudaStream_t s,
                          bool defer_append = false) {
    const int64_t S = k.shape[2];
    const int64_t step = std::max<int32_t>(c->cfg.step, 1);
    if (!c->k.allocated()) {
        const int64_t cap = std::max<int64_t>(c->cfg.reserve_tokens, round_up(c->offset + std::max<int64_t>(S, 1), step));
        c->k.alloc(k.shape[0], k.shape[1], cap, k.shape[3], k.dtype, s);
        c->v.alloc(v.shape[0], v.shape[1], cap, v.shape[3], v.dtype, s);
    } else {
        KVC_REQUIRE(k.shape[0] == c->k.B && k.shape[1] == c->k.H && k.shape[3] == c->k.W &&
                        v.shape[3] == c->v.W && k.dtype == c->k.dtype,
                    "update: new keys/values do not match the cached shape or dtype");
        c->k.ensure(c->offset + S, c->offset, step, s);
        c->v.ensure(c->offset + S, c->offset, step, s);
    }
    if (S > 0 && !defer_append) append_pair(c->k, c->v, k, v, c->offset, s);
    c->offset += S;
}

// RotatingKVCache.updateInPlace (KVCache.swift:684-740), S == 1.
// With `slot` the new row is NOT written: the caller (the fused decode kernel) stores it at *slot.
static void rotating_update_in_place(kvc_cache *c, const kvc_tensor &k, const kvc_tensor &v,
                                     cudaStream_t s, kvc_tensor *ok, kvc_tensor *ov, int64_t *slot = nullptr) {
    const int64_t max_size = c->cfg.max_size, keep = c->cfg.keep;
    const int64_t prev = c->offset;
    if (!c->k.allocated() || (prev >= c->len && c->len < max_size)) {
        const int64_t new_size = std::min<int64_t>(c->cfg.step, max_size - prev);
        if (new_size <= 0)
            fail(KVC_ERR_INVALID_STATE, "rotating cache: cannot grow (offset is past maxSize while the buffer is short)");
        if (!c->k.allocated()) {
            const int64_t cap = std::max<int64_t>(max_size, new_size);
            c->k.alloc(k.shape[0], k.shape[1], cap, k.shape[3], k.dtype, s);
            c->v.alloc(v.shape[0], v.shape[1], cap, v.shape[3], v.dtype, s);
            c->len = 0;
        } else {
            c->k.ensure(c->len + new_size, c->len, c->cfg.step, s);
            c->v.ensure(c->len + new_size, c->len, c->cfg.step, s);
            zero_rows(c->k, c->len, new_size, s);
            zero_rows(c->v, c->len, new_size, s);
        }
        c->len += new_size;
        c->idx = prev;
    }
    KVC_REQUIRE(k.shape[0] == c->k.B && k.shape[1] == c->k.H && k.shape[3] == c->k.W &&
                    v.shape[3] == c->v.W && k.dtype == c->k.dtype,
                "update: new keys/values do not match the cached shape or dtype");
    const int64_t trim_size = c->len - max_size;
    if (trim_size > 0) {
        std::vector<GatherSeg> all;
        seg_push(all, 0, c->len);
        rot_rebuild(c, rot_front_trim(all, trim_size, keep), 0, s);
        c->idx = max_size;
    }
    if (c->idx == max_size) c->idx = keep;
    if (c->idx < 0 || c->idx + 1 > c->len)
        fail(KVC_ERR_INVALID_STATE, "rotating cache: ring index outside the buffer");
    if (slot) *slot = c->idx;
    else append_pair(c->k, c->v, k, v, c->idx, s);
    c->offset += 1;
    c->idx += 1;
    const int64_t rows = c->offset < max_size ? std::min(c->offset, c->len) : c->len;
    if (ok) *ok = c->k.view(rows);
    if (ov) *ov = c->v.view(rows);
}

// RotatingKVCache.updateConcat (KVCache.swift:660-682), S > 1.
static void rotating_update_concat(kvc_cache *c, const kvc_tensor &k, const kvc_tensor &v,
                                   cudaStream_t s, kvc_tensor *ok, kvc_tensor *ov) {
    const int64_t S = k.shape[2];
    const int64_t max_size = c->cfg.max_size, keep = c->cfg.keep;
    if (!c->k.allocated()) {
        const int64_t cap = std::max<int64_t>(S, max_size);
        c->k.alloc(k.shape[0], k.shape[1], cap, k.shape[3], k.dtype, s);
        c->v.alloc(v.shape[0], v.shape[1], cap, v.shape[3], v.dtype, s);
        append_pair(c->k, c->v, k, v, 0, s);
        c->len = S;
    } else {
        KVC_REQUIRE(k.shape[0] == c->k.B && k.shape[1] == c->k.H && k.shape[3] == c->k.W &&
                        v.shape[3] == c->v.W && k.dtype == c->k.dtype,
                    "update: new keys/values do not match the cached shape or dtype");
        auto ordered = rot_temporal(c);
        c->idx = seg_total(ordered);
        const int64_t trim_size = c->idx - max_size + 1;
        auto segs = rot_front_trim(ordered, trim_size, keep);
        const int64_t n = seg_total(segs);
        if (segs.size() == 1 && segs[0].src_start == 0) {
            c->len = n;  // already in place: a prefix of the buffer
            c->k.ensure(n + S, n, c->cfg.step, s);
            c->v.ensure(n + S, n, c->cfg.step, s);
        } else {
            rot_rebuild(c, segs, S, s);
        }
        append_pair(c->k, c->v, k, v, n, s);
        c->len = n + S;
    }
    c->offset += S;
    c->idx = c->len;
    if (ok) *ok = c->k.view(c->len);
    if (ov) *ov = c->v.view(c->len);
}

// ChunkedKVCache.update (KVCache.swift:1234-1269). `len` follows the reference's buffer length
// keys.dim(2) (whole `step`s of zero rows are appended when the new rows do not fit; a buffer whose
// fill is not a multiple of `step` is first cut back to its fill), because maybeTrimFront and the
// state getter work on that length, zero padding included.
static void chunked_update(kvc_cache *c, const kvc_tensor &k, const kvc_tensor &v, cudaStream_t s) {
    const int64_t S = k.shape[2];
    const int64_t step = std::max<int32_t>(c->cfg.step, 1);
    const int64_t prev = c->offset - c->start_position;
    if (prev < 0) fail(KVC_ERR_INVALID_STATE, "chunked cache: offset is before startPosition");
    if (!c->k.allocated() || prev + S > c->len) {
        const int64_t n_steps = (step + S - 1) / step;
        if (!c->k.allocated()) {
            c->len = n_steps * step;
            c->k.alloc(k.shape[0], k.shape[1], c->len, k.shape[3], k.dtype, s);
            c->v.alloc(v.shape[0], v.shape[1], c->len, v.shape[3], v.dtype, s);
        } else {
            int64_t kept = c->len;
            if (prev % step != 0) kept = prev;          // currentKeys[..<prev]
            const int64_t new_len = kept + n_steps * step;
            c->k.ensure(new_len, kept, step, s);
            c->v.ensure(new_len, kept, step, s);
            zero_rows(c->k, kept, new_len - kept, s);    // the appended rows are zeros in the reference
            zero_rows(c->v, kept, new_len - kept, s);
            c->len = new_len;
        }
    }
    KVC_REQUIRE(k.shape[0] == c->k.B && k.shape[1] == c->k.H && k.shape[3] == c->k.W && v.shape[3] == c->v.W &&
                    k.dtype == c->k.dtype,
                "update: new keys/values do not match the cached shape or dtype");
    if (S > 0) append_pair(c->k, c->v, k, v, prev, s);
    c->offset += S;
}

// ChunkedKVCache.maybeTrimFront (KVCache.swift:1222-1232).
void cache_maybe_trim_front(kvc_cache *c, cudaStream_t s) {
    c->last_stream = s;
    KVC_REQUIRE(c->cfg.kind == KVC_KIND_CHUNKED, "maybeTrimFront needs a ChunkedKVCache");
    const int64_t chunk = c->cfg.max_size;
    if (!c->k.allocated() || chunk <= 0 || c->len < chunk) return;
    const int64_t drop = c->len - chunk;
    c->start_position += drop;
    if (drop > 0) {
        std::vector<GatherSeg> keep;
        seg_push(keep, drop, chunk);
        ensure_like(c->k_alt, c->k, std::max<int64_t>(chunk, c->k.cap), s);
        ensure_like(c->v_alt, c->v, std::max<int64_t>(chunk, c->v.cap), s);
        gather_rows(c->k, c->k_alt, keep, s);
        gather_rows(c->v, c->v_alt, keep, s);
        std::swap(c->k, c->k_alt);
        std::swap(c->v, c->v_alt);
    }
    c->len = chunk;
}

void cache_update(kvc_cache *c, const kvc_tensor &k, const kvc_tensor &v, cudaStream_t s,
                  kvc_tensor *out_k, kvc_tensor *out_v) {
    c->last_stream = s;
    require4(k, "keys");
    require4(v, "values");
    KVC_REQUIRE(is_float_dtype(k.dtype) && k.dtype == v.dtype, "update: keys/values must share a floating dtype");
    KVC_REQUIRE(k.shape[0] == v.shape[0] && k.shape[1] == v.shape[1] && k.shape[2] == v.shape[2],
                "update: keys and values disagree on batch, heads or length");
    if (c->open_round) fail(KVC_ERR_INVALID_STATE, "update: a staged round is open on this cache");
    c->restore.valid = false;
    switch (c->cfg.kind) {
        case KVC_KIND_SIMPLE:
            linear_update(c, k, v, s);
            if (out_k) *out_k = c->k.view(c->offset);
            if (out_v) *out_v = c->v.view(c->offset);
            return;
        case KVC_KIND_TURBO:
            if (c->compressed)
                fail(KVC_ERR_INVALID_STATE, "update: the raw path is gone once a TurboQuant cache is compressed; use attention");
            linear_update(c, k, v, s);
            if (out_k) *out_k = c->k.view(c->offset);
            if (out_v) *out_v = c->v.view(c->offset);
            return;
        case KVC_KIND_ROTATING:
            check_new_rows(c, c->k, c->v, k, v);
            if (k.shape[2] == 1) rotating_update_in_place(c, k, v, s, out_k, out_v);
            else rotating_update_concat(c, k, v, s, out_k, out_v);
            return;
        case KVC_KIND_QUANTIZED:
            // KVCache.swift:1106-1110
            fail(KVC_ERR_INVALID_STATE, "`update` was called on `QuantizedKVCache`. Use `updateQuantized` instead.");
        case KVC_KIND_CHUNKED: {
            chunked_update(c, k, v, s);
            const int64_t end = c->offset - c->start_position;
            if (out_k) *out_k = c->k.view(end);
            if (out_v) *out_v = c->v.view(end);
            return;
        }
        case KVC_KIND_LIST:
            // KVCache.swift:1576-1578
            fail(KVC_ERR_INVALID_STATE, "CacheList should not use update(keys:values:) - use subscript access instead");
        default: fail(KVC_ERR_INVALID_ARG, "unknown cache kind");
    }
}

// ---------------------------------------------------------------------
// QuantizedKVCache.updateQuantized (KVCache.swift:1011-1102)
// ---------------------------------------------------------------------
static QuantAppendArgs quant_args(const kvc_tensor &x, Array4 &codes, Array4 &scales, Array4 &biases,
                                  int group, int bits, int64_t pos) {
    QuantAppendArgs a;
    a.src = x.data; a.dtype = x.dtype;
    a.s_sb = x.stride[0]; a.s_sh = x.stride[1]; a.s_ss = x.stride[2]; a.s_sd = x.stride[3];
    a.codes = (uint32_t *)codes.ptr;
    a.scales = scales.ptr; a.biases = biases.ptr;
    a.c_sb = codes.sb(); a.c_sh = codes.sh(); a.c_st = codes.st();
    a.g_sb = scales.sb(); a.g_sh = scales.sh(); a.g_st = scales.st();
    a.B = (int)x.shape[0]; a.H = (int)x.shape[1]; a.S = (int)x.shape[2]; a.D = (int)x.shape[3];
    a.group = group; a.bits = bits; a.pos = pos;
    return a;
}

static void quant_triple_alloc(Array4 &q, Array4 &sc, Array4 &bi, int64_t B, int64_t H, int64_t cap,
                               int D, int group, int bits, int32_t dtype, cudaStream_t s) {
    q.alloc(B, H, cap, (int64_t)D * bits / 32, KVC_U32, s);
    sc.alloc(B, H, cap, D / group, dtype, s);
    bi.alloc(B, H, cap, D / group, dtype, s);
}

void cache_update_quantized(kvc_cache *c, const kvc_tensor &k, const kvc_tensor &v, cudaStream_t s,
                            kvc_tensor out_k[3], kvc_tensor out_v[3], bool defer_quantize) {
    c->last_stream = s;
    KVC_REQUIRE(c->cfg.kind == KVC_KIND_QUANTIZED, "updateQuantized needs a QuantizedKVCache");
    require4(k, "keys");
    require4(v, "values");
    KVC_REQUIRE(is_float_dtype(k.dtype) && k.dtype == v.dtype, "updateQuantized: keys/values must share a floating dtype");
    KVC_REQUIRE(k.shape[0] == v.shape[0] && k.shape[1] == v.shape[1] && k.shape[2] == v.shape[2],
                "updateQuantized: keys and values disagree on batch, heads or length");
    const int kd = (int)k.shape[3], vd = (int)v.shape[3];
    const int eff = resolved_group_size(c->group_size, kd, vd);
    if (!eff)
        fail(KVC_ERR_INVALID_ARG,
             "KV cache quantization requires head dimensions divisible by one of the supported group sizes (32, 64, 128).");
    if (eff != c->group_size && !c->kq.allocated() && c->offset == 0) c->group_size = eff;
    KVC_REQUIRE(kd % c->group_size == 0 && vd % c->group_size == 0,
                "updateQuantized: head dims are not multiples of the cache's group size");
    const int64_t S = k.shape[2], prev = c->offset;
    const int64_t step = std::max<int32_t>(c->cfg.step, 1);
    if (!c->kq.allocated()) {
        const int64_t cap = std::max<int64_t>(c->cfg.reserve_tokens, round_up(prev + std::max<int64_t>(S, 1), step));
        quant_triple_alloc(c->kq, c->ks, c->kb, k.shape[0], k.shape[1], cap, kd, c->group_size, c->bits, k.dtype, s);
        quant_triple_alloc(c->vq, c->vs, c->vb, v.shape[0], v.shape[1], cap, vd, c->group_size, c->bits, v.dtype, s);
    } else {
        KVC_REQUIRE(k.shape[0] == c->kq.B && k.shape[1] == c->kq.H &&
                        (int64_t)kd * c->bits / 32 == c->kq.W && (int64_t)vd * c->bits / 32 == c->vq.W &&
                        k.dtype == c->ks.dtype,
                    "updateQuantized: new keys/values do not match the cached shape or dtype");
        for (Array4 *a : {&c->kq, &c->ks, &c->kb, &c->vq, &c->vs, &c->vb}) a->ensure(prev + S, prev, step, s);
    }
    if (S > 0 && !defer_quantize) {
        QuantAppendArgs qa = quant_args(k, c->kq, c->ks, c->kb, c->group_size, c->bits, prev);
        QuantAppendArgs qv = quant_args(v, c->vq, c->vs, c->vb, c->group_size, c->bits, prev);
        launch_affine_quantize2(qa, &qv, s);
    }
    c->offset = prev + S;
    if (out_k) { out_k[0] = c->kq.view(c->offset); out_k[1] = c->ks.view(c->offset); out_k[2] = c->kb.view(c->offset); }
    if (out_v) { out_v[0] = c->vq.view(c->offset); out_v[1] = c->vs.view(c->offset); out_v[2] = c->vb.view(c->offset); }
}

// ---------------------------------------------------------------------
// attention
// ---------------------------------------------------------------------
int launch_attention_decode(const AttnArgs &a, cudaStream_t stream);

KVSource raw_source(const kvc_tensor &t) {
    KVSource s;
    s.kind = SRC_RAW;
    s.dtype = t.dtype;
    s.data = t.data;
    s.sb = t.stride[0]; s.sh = t.stride[1]; s.st = t.stride[2];
    return s;
}

static KVSource affine_source(const kvc_tensor &w, const kvc_tensor &sc, const kvc_tensor &bi, int group, int bits) {
    KVSource s;
    s.kind = SRC_AFFINE;
    s.dtype = sc.dtype;
    s.data = w.data; s.scales = sc.data; s.biases = bi.data;
    s.sb = w.stride[0]; s.sh = w.stride[1]; s.st = w.stride[2];
    s.gsb = sc.stride[0]; s.gsh = sc.stride[1]; s.gst = sc.stride[2];
    s.bits = bits; s.group = group; s.words = (int)w.shape[3];
    return s;
}

static KVSource turbo_source(const Array4 &p, const Array4 &n, const TurboCodec &codec) {
    KVSource s;
    s.kind = SRC_TURBO;
    s.data = p.ptr; s.norms = (const float *)n.ptr;
    s.sb = p.sb(); s.sh = p.sh(); s.st = p.st();
    s.gsb = n.sb(); s.gsh = n.sh(); s.gst = n.st();
    s.bits = codec.bits; s.words = (int)p.W;
    for (size_t i = 0; i < codec.centroids.size() && i < 16; ++i) s.codebook[i] = codec.centroids[i];
    return s;
}

AttnArgs make_attn_args(const kvc_tensor &q, const kvc_tensor &out, float scale, int32_t mask_mode,
                        const kvc_tensor *mask, int64_t T, int Hkv) {
    require4(q, "queries");
    require4(out, "out");
    KVC_REQUIRE(is_float_dtype(q.dtype) && out.dtype == q.dtype, "attention: output dtype must equal the query dtype");
    KVC_REQUIRE(q.stride[3] == 1 && out.stride[3] == 1, "attention: queries/out must be contiguous along the head dim");
    for (int i = 0; i < 4; ++i) KVC_REQUIRE(q.shape[i] == out.shape[i], "attention: out shape differs from queries");
    AttnArgs a;
    a.q = q.data; a.out = out.data; a.q_dtype = q.dtype;
    a.q_sb = q.stride[0]; a.q_sh = q.stride[1]; a.q_sl = q.stride[2];
    a.o_sb = out.stride[0]; a.o_sh = out.stride[1]; a.o_sl = out.stride[2];
    a.B = (int)q.shape[0]; a.Hq = (int)q.shape[1]; a.L = (int)q.shape[2]; a.D = (int)q.shape[3];
    a.Hkv = Hkv; a.T = T; a.scale = scale;
    a.device = current_device();
    a.mask.mode = mask_mode;
    if (mask_mode == KVC_MASK_CAUSAL) {
        a.mask.causal_offset = T - a.L;
    } else if (mask_mode == KVC_MASK_ARRAY) {
        KVC_REQUIRE(mask && mask->data, "attention: array mask mode needs a mask tensor");
        KVC_REQUIRE(mask->ndim >= 1 && mask->ndim <= 4, "attention: mask must have 1..4 dims");
        KVC_REQUIRE(mask->dtype == KVC_BOOL || is_float_dtype(mask->dtype), "attention: mask must be bool or floating");
        a.mask.dtype = mask->dtype;
        a.mask.data = mask->data;
        const int64_t want[4] = {a.B, a.Hq, a.L, T};
        int64_t st[4] = {0, 0, 0, 0};
        for (int i = 0; i < mask->ndim; ++i) {
            const int dst = 4 - mask->ndim + i;
            if (mask->shape[i] == want[dst]) st[dst] = mask->stride[i];
            else if (mask->shape[i] == 1) st[dst] = 0;
            else fail(KVC_ERR_INVALID_ARG, "attention: mask is not broadcastable to [B, Hq, L, T]");
        }
        a.mask.sb = st[0]; a.mask.sh = st[1]; a.mask.sl = st[2]; a.mask.st = st[3];
    } else if (mask_mode != KVC_MASK_NONE) {
        fail(KVC_ERR_INVALID_ARG, "attention: unknown mask mode");
    }
    return a;
}

static void upload_signs(TurboCodec &codec, cudaStream_t s) {
    if (codec.signs_dev) dev_free(codec.signs_dev, s);
    codec.signs_dev = (float *)dev_alloc(codec.signs.size() * sizeof(float), s);
    KVC_CUDA(cudaMemcpyAsync(codec.signs_dev, codec.signs.data(), codec.signs.size() * sizeof(float),
                             cudaMemcpyHostToDevice, s));
}

void ensure_codecs(kvc_cache *c, int head_dim, cudaStream_t s) {
    // TurboQuantKVCache.ensureCodecs (TurboQuantKVCache.swift:753-759): key codec
    // seeded with `seed`, value codec with `seed + 1`. MSECodec.init (:459-486): the randomised
    // Walsh-Hadamard rotation for power-of-two head dims up to 1024, a dense random rotation otherwise.
    if (c->codec_ready && c->vcodec.dim == head_dim) return;
    KVC_REQUIRE(head_dim >= 2 && head_dim <= 1024, "TurboQuant: head dim must be in [2, 1024]");
    const bool wht = (head_dim & (head_dim - 1)) == 0;
    if (wht && head_dim < 32)
        fail(KVC_ERR_UNSUPPORTED, "TurboQuant: power-of-two head dims below 32 (Walsh-Hadamard over less than a warp) are not built");
    if (!wht) KVC_REQUIRE(head_dim <= 256, "TurboQuant: the dense-rotation path is built for head dims up to 256");
    auto build = [&](TurboCodec &codec, int bits, uint64_t seed, const std::vector<float> &uc,
                     const std::vector<float> &us, const std::vector<float> &ur) {
        codec.dim = head_dim;
        codec.bits = bits;
        if (!uc.empty()) {
            KVC_REQUIRE((int)uc.size() == (1 << bits), "TurboQuant: codebook override has the wrong length");
            codec.centroids = uc;
            codec.boundaries.clear();
            for (size_t i = 0; i + 1 < uc.size(); ++i) codec.boundaries.push_back((uc[i] + uc[i + 1]) / 2.0f);
        } else {
            turbo_codebook(head_dim, bits, codec.centroids, codec.boundaries);
        }
        if (wht) {
            if (!us.empty()) {
                KVC_REQUIRE((int)us.size() == head_dim, "TurboQuant: sign override has the wrong length");
                codec.signs = us;
            } else {
                turbo_signs(head_dim, seed, codec.signs);
            }
            upload_signs(codec, s);
        } else {
            if (!ur.empty()) {
                KVC_REQUIRE((int64_t)ur.size() == (int64_t)head_dim * head_dim, "TurboQuant: rotation override has the wrong size");
                codec.rotation = ur;
            } else {
                turbo_rotation(head_dim, seed, codec.rotation);
            }
            if (codec.rotation_dev) dev_free(codec.rotation_dev, s);
            codec.rotation_dev = (float *)dev_alloc(codec.rotation.size() * sizeof(float), s);
            KVC_CUDA(cudaMemcpyAsync(codec.rotation_dev, codec.rotation.data(), codec.rotation.size() * sizeof(float),
                                     cudaMemcpyHostToDevice, s));
        }
    };
    if (!c->raw_key && !c->affine_key) build(c->kcodec, c->key_bits, c->cfg.seed, c->user_kc, c->user_ks, c->user_kr);
    if (!c->affine_value) build(c->vcodec, c->value_bits, c->cfg.seed + 1, c->user_vc, c->user_vs, c->user_vr);
    else c->vcodec.dim = head_dim;
    c->codec_ready = true;
}

static TurboEncodeArgs turbo_args(const kvc_tensor &x, Array4 &packed, Array4 &norms,
                                  const TurboCodec &codec, int64_t pos) {
    TurboEncodeArgs a;
    a.src = x.data; a.dtype = x.dtype;
    a.s_sb = x.stride[0]; a.s_sh = x.stride[1]; a.s_ss = x.stride[2]; a.s_sd = x.stride[3];
    a.packed = (uint32_t *)packed.ptr; a.norms = (float *)norms.ptr;
    a.p_sb = packed.sb(); a.p_sh = packed.sh(); a.p_st = packed.st();
    a.n_sb = norms.sb(); a.n_sh = norms.sh(); a.n_st = norms.st();
    a.B = (int)x.shape[0]; a.H = (int)x.shape[1]; a.S = (int)x.shape[2]; a.D = (int)x.shape[3];
    a.bits = codec.bits; a.pos = pos; a.signs = codec.signs_dev;
    for (size_t i = 0; i < codec.boundaries.size() && i < 15; ++i) a.boundaries[i] = codec.boundaries[i];
    a.calib = codec.calib_dev;
    a.rotation = codec.rotation_dev;
    if (a.calib || a.rotation)
        for (size_t i = 0; i < codec.centroids.size() && i < 16; ++i) a.centroids[i] = codec.centroids[i];
    return a;
}

static void set_key_calibration(kvc_cache *c, const std::vector<float> &scale, cudaStream_t s) {
    TurboCodec &codec = c->kcodec;
    if (codec.calib_dev) { dev_free(codec.calib_dev, s); codec.calib_dev = nullptr; }
    codec.calib = scale;
    if (scale.empty()) return;
    codec.calib_dev = (float *)dev_alloc(scale.size() * sizeof(float), s);
    KVC_CUDA(cudaMemcpyAsync(codec.calib_dev, codec.calib.data(), scale.size() * sizeof(float), cudaMemcpyHostToDevice, s));
}

// computeKeyCalibrationScale (TurboQuantKVCache.swift:867-886): per-dimension standard deviation of
// the rotated unit keys over every cached (batch, head, token), divided by its mean over the
// dimensions, clamped to [0.25, 4]; none when fewer than 32 rows or when no dimension is 10 % off 1.
// The two moments are accumulated on the device as fixed-point integers (order-free, so a CPU
// restatement reaches the same bits), the rest is a handful of host operations per dimension. The
// host reads the sums back, so this call waits for the stream like the reference's eval/item does.
static std::vector<float> compute_key_calibration(kvc_cache *c, const kvc_tensor &keys, cudaStream_t s) {
    const int D = (int)keys.shape[3];
    const int64_t rows = keys.shape[0] * keys.shape[1] * keys.shape[2];
    if (rows < 32) return {};
    Array4 dummy_p, dummy_n;
    TurboEncodeArgs a = turbo_args(keys, dummy_p, dummy_n, c->kcodec, 0);
    a.calib = nullptr;   // the statistic is taken on the uncalibrated rotation
    long long *sums = (long long *)dev_alloc((size_t)2 * D * sizeof(long long), s);
    KVC_CUDA(cudaMemsetAsync(sums, 0, (size_t)2 * D * sizeof(long long), s));
    launch_turbo_calib_stats(a, sums, s);
    std::vector<long long> host(2 * D);
    KVC_CUDA(cudaMemcpyAsync(host.data(), sums, host.size() * sizeof(long long), cudaMemcpyDeviceToHost, s));
    KVC_CUDA(cudaStreamSynchronize(s));
    dev_free(sums, s);
    std::vector<float> sd(D);
    double sd_sum = 0.0;
    for (int d = 0; d < D; ++d) {
        const double mean = (double)host[d] / 1073741824.0 / (double)rows;
        const double ex2 = (double)host[D + d] / 68719476736.0 / (double)rows;
        const double var = std::max(ex2 - mean * mean, 0.0);
        sd[d] = (float)std::sqrt(var);
        sd_sum += (double)sd[d];
    }
    const float mean_sd = std::max((float)(sd_sum / (double)D), 1e-8f);
    float max_dev = 0.0f;
    for (int d = 0; d < D; ++d) {
        sd[d] = std::min(std::max(sd[d] / mean_sd, 0.25f), 4.0f);
        max_dev = std::max(max_dev, std::fabs(sd[d] - 1.0f));
    }
    if (!(max_dev >= 0.1f)) return {};
    return sd;
}

static int turbo_pw(int count, int bits) { return (count * bits + 31) / 32; }

// Encode S rows of K and V into the compressed arrays at token `pos`
// (the kernel work of compressRawCacheInternal :924-1002 and encodeNewToken :1010-1147).
static void turbo_encode_rows(kvc_cache *c, const kvc_tensor &k, const kvc_tensor &v, int64_t pos, cudaStream_t s) {
    if (k.shape[2] == 0) return;
    const bool k_turbo = !c->raw_key && !c->affine_key;
    const bool v_turbo = !c->affine_value;
    if (k_turbo && v_turbo) {
        TurboEncodeArgs ka = turbo_args(k, c->kp, c->kn, c->kcodec, pos);
        TurboEncodeArgs va = turbo_args(v, c->vp, c->vn, c->vcodec, pos);
        launch_turbo_encode2(ka, &va, s);
    } else {
        if (k_turbo) launch_turbo_encode(turbo_args(k, c->kp, c->kn, c->kcodec, pos), s);
        if (v_turbo) launch_turbo_encode(turbo_args(v, c->vp, c->vn, c->vcodec, pos), s);
    }
    if (c->affine_key)
        launch_affine_quantize(quant_args(k, c->kq, c->ks, c->kb, c->key_group, 8, pos), s);
    if (c->affine_value)
        launch_affine_quantize(quant_args(v, c->vq, c->vs, c->vb, c->key_group, c->value_bits, pos), s);
    if (c->raw_key) {
        // raw keys keep living in c->k; V of the raw pair is unused, append K only
        AppendArgs a;
        a.k_src = k.data; a.v_src = k.data;
        a.ks_sb = k.stride[0]; a.ks_sh = k.stride[1]; a.ks_ss = k.stride[2]; a.ks_sd = k.stride[3];
        a.vs_sb = a.ks_sb; a.vs_sh = a.ks_sh; a.vs_ss = a.ks_ss; a.vs_sd = a.ks_sd;
        a.k_dst = c->k.ptr; a.v_dst = c->k.ptr;
        a.kd_sb = c->k.sb(); a.kd_sh = c->k.sh(); a.kd_st = c->k.st();
        a.vd_sb = a.kd_sb; a.vd_sh = a.kd_sh; a.vd_st = a.kd_st;
        a.B = (int)k.shape[0]; a.H = (int)k.shape[1]; a.S = (int)k.shape[2];
        a.Dk = (int)k.shape[3]; a.Dv = 0;
        a.pos = pos; a.esize = (int)dtype_size(k.dtype);
        launch_append(a, s);
    }
}

static void turbo_alloc_compressed(kvc_cache *c, int64_t B, int64_t H, int D, int32_t dtype, int64_t cap, cudaStream_t s) {
    const bool k_turbo = !c->raw_key && !c->affine_key;
    if (k_turbo) {
        c->kp.alloc(B, H, cap, turbo_pw(D, c->key_bits), KVC_U32, s);
        c->kn.alloc(B, H, cap, 1, KVC_F32, s);
    }
    if (c->affine_key) {
        const int g = resolved_group_size(c->key_group, D, D);
        if (!g) fail(KVC_ERR_INVALID_ARG, "TurboQuant affine key quantization requires head dimensions divisible by 32, 64 or 128");
        c->key_group = g;
        quant_triple_alloc(c->kq, c->ks, c->kb, B, H, cap, D, g, 8, dtype, s);
    }
    if (c->affine_value) {
        const int g = resolved_group_size(c->key_group, D, D);
        if (!g) fail(KVC_ERR_INVALID_ARG, "affine value quantization requires head dimensions divisible by 32, 64 or 128");
        c->key_group = g;
        quant_triple_alloc(c->vq, c->vs, c->vb, B, H, cap, D, g, c->value_bits, dtype, s);
    } else {
        c->vp.alloc(B, H, cap, turbo_pw(D, c->value_bits), KVC_U32, s);
        c->vn.alloc(B, H, cap, 1, KVC_F32, s);
    }
}

static void turbo_ensure_compressed(kvc_cache *c, int64_t need, int64_t keep_rows, cudaStream_t s) {
    const int64_t step = 256;
    for (Array4 *a : {&c->kp, &c->kn, &c->vp, &c->vn, &c->kq, &c->ks, &c->kb, &c->vq, &c->vs, &c->vb})
        if (a->allocated()) a->ensure(need, keep_rows, step, s);
    if (c->raw_key && c->k.allocated()) c->k.ensure(need, keep_rows, step, s);
}

// TurboQuantKVCache.compressRawCache (TurboQuantKVCache.swift:895-918).
static void turbo_compress_raw(kvc_cache *c, cudaStream_t s) {
    if (c->compressed || !c->k.allocated() || c->offset <= 0) return;
    const int D = (int)c->k.W;
    KVC_REQUIRE(c->v.W == c->k.W, "TurboQuant: key and value head dims must match");
    ensure_codecs(c, D, s);
    // whole 256-row steps, like the reference's allocations: the decode kernels stream whole stages
    const int64_t cap = round_up(std::max<int64_t>(std::max<int64_t>(c->cfg.reserve_tokens, c->k.cap), round_up(c->offset, 256)), 256);
    turbo_alloc_compressed(c, c->k.B, c->k.H, D, c->k.dtype, cap, s);
    kvc_tensor kt = c->k.view(c->offset), vt = c->v.view(c->offset);
    if (c->raw_key) {
        // keys stay where they are (raw, in c->k); only values are encoded
        (void)kt;
        if (!c->affine_value) launch_turbo_encode(turbo_args(vt, c->vp, c->vn, c->vcodec, 0), s);
        else launch_affine_quantize(quant_args(vt, c->vq, c->vs, c->vb, c->key_group, c->value_bits, 0), s);
        c->v.release(s);
    } else {
        // standard mode: the calibration scale is derived once from the whole raw key cache and
        // reused by every later encode on this cache (TurboQuantKVCache.swift:960-962)
        if (!c->affine_key) set_key_calibration(c, compute_key_calibration(c, kt, s), s);
        turbo_encode_rows(c, kt, vt, 0, s);
        c->k.release(s);
        c->v.release(s);
    }
    c->compressed = true;
}

// The cache-side half of compressedAttention: compress a raw prefix if there is one, then
// encode the new rows and append them in the compressed domain
// (TurboQuantKVCache.swift:1176-1200 -> compressRawCache :895, encodeNewToken :1010-1147).
void cache_turbo_encode_new_token(kvc_cache *c, const kvc_tensor &k, const kvc_tensor &v, cudaStream_t s) {
    c->last_stream = s;
    KVC_REQUIRE(c->cfg.kind == KVC_KIND_TURBO, "encode_new_token: not a TurboQuant cache");
    if (c->open_round) fail(KVC_ERR_INVALID_STATE, "encode_new_token: a staged round is open on this cache");
    require4(k, "keys");
    require4(v, "values");
    const int D = (int)k.shape[3];
    KVC_REQUIRE(v.shape[3] == D, "TurboQuant: query, key and value head dims must match");
    if (!c->compressed) turbo_compress_raw(c, s);
    ensure_codecs(c, D, s);
    const int64_t S = k.shape[2], prev = c->offset;
    if (!c->compressed) {
        // nothing was cached yet: start directly in the compressed phase
        const int64_t cap = round_up(std::max<int64_t>(c->cfg.reserve_tokens, round_up(std::max<int64_t>(S, 1), 256)), 256);
        turbo_alloc_compressed(c, k.shape[0], k.shape[1], D, k.dtype, cap, s);
        if (c->raw_key) c->k.alloc(k.shape[0], k.shape[1], cap, D, k.dtype, s);
        c->compressed = true;
    }
    turbo_ensure_compressed(c, prev + S, prev, s);
    turbo_encode_rows(c, k, v, prev, s);
    c->offset = prev + S;
}

// TurboQuantKVCache.compressedAttention (TurboQuantKVCache.swift:1164-1446).
static void turbo_compressed_attention(kvc_cache *c, const kvc_tensor &q, const kvc_tensor &k,
                                       const kvc_tensor &v, float scale, int32_t mask_mode,
                                       const kvc_tensor *mask, const kvc_tensor &out, cudaStream_t s) {
    const int D = (int)k.shape[3];
    KVC_REQUIRE(q.shape[3] == D, "TurboQuant: query, key and value head dims must match");
    cache_turbo_encode_new_token(c, k, v, s);

    const int64_t T = c->offset;
    const int L = (int)q.shape[2];
    int32_t mode = mask_mode;
    if (L == 1 && mode == KVC_MASK_CAUSAL) mode = KVC_MASK_NONE;
    AttnArgs a = make_attn_args(q, out, scale, mode, mask, T, (int)k.shape[1]);
    if (c->raw_key) {
        a.k = raw_source(c->k.view(T));
    } else if (c->affine_key) {
        a.k = affine_source(c->kq.view(T), c->ks.view(T), c->kb.view(T), c->key_group, 8);
    } else {
        a.k = turbo_source(c->kp, c->kn, c->kcodec);
        a.q_signs = c->kcodec.rotation_dev ? nullptr : c->kcodec.signs_dev;
        a.q_rot = c->kcodec.rotation_dev;
        a.q_calib = c->kcodec.calib_dev;   // folded into the rotated query (TurboQuantKVCache.swift:1348-1352)
    }
    if (c->affine_value) {
        a.v = affine_source(c->vq.view(T), c->vs.view(T), c->vb.view(T), c->key_group, c->value_bits);
    } else {
        a.v = turbo_source(c->vp, c->vn, c->vcodec);
        a.o_signs = c->vcodec.rotation_dev ? nullptr : c->vcodec.signs_dev;
        a.o_rot = c->vcodec.rotation_dev;
    }
    launch_attention(a, s);
}

void cache_attention(kvc_cache *c, const kvc_tensor &q, const kvc_tensor &k, const kvc_tensor &v,
                     float scale, int32_t mask_mode, const kvc_tensor *mask, const kvc_tensor &out,
                     cudaStream_t s) {
    c->last_stream = s;
    require4(q, "queries");
    require4(k, "keys");
    require4(v, "values");
    KVC_REQUIRE(q.shape[0] == k.shape[0], "attention: query and key batch differ");
    KVC_REQUIRE(k.shape[1] > 0 && q.shape[1] % k.shape[1] == 0, "attention: Hq must be a multiple of Hkv");
    KVC_REQUIRE(q.dtype == k.dtype, "attention: queries and keys must share a dtype");
    const int Hkv = (int)k.shape[1];
    switch (c->cfg.kind) {
        case KVC_KIND_TURBO: {
            const int L = (int)q.shape[2];
            if (L > 1 && !c->compressed) {
                // AttentionUtils.swift:56-63: raw prefill + plain SDPA
                kvc_tensor ck, cv;
                cache_update(c, k, v, s, &ck, &cv);
                AttnArgs a = make_attn_args(q, out, scale, mask_mode, mask, ck.shape[2], Hkv);
                a.k = raw_source(ck);
                a.v = raw_source(cv);
                launch_attention(a, s);
            } else {
                if (c->open_round) fail(KVC_ERR_INVALID_STATE, "attention: a staged round is open on this cache");
                turbo_compressed_attention(c, q, k, v, scale, mask_mode, mask, out, s);
            }
            return;
        }
        case KVC_KIND_QUANTIZED: {
            kvc_tensor qk[3], qv[3];
            cache_update_quantized(c, k, v, s, qk, qv);
            AttnArgs a = make_attn_args(q, out, scale, mask_mode, mask, c->offset, Hkv);
            a.k = affine_source(qk[0], qk[1], qk[2], c->group_size, c->bits);
            a.v = affine_source(qv[0], qv[1], qv[2], c->group_size, c->bits);
            launch_attention(a, s);
            return;
        }
        default: {
            // Decode on a KVCacheSimple: the attention kernel appends the new row itself when it can
            // (one launch per layer); otherwise the append runs first as its own launch.
            static const bool fuse_off = [] {
                const char *e = std::getenv("KVC_FUSED_APPEND");
                return e && e[0] == '0';
            }();
            if (!fuse_off && c->cfg.kind == KVC_KIND_SIMPLE && k.shape[2] == 1 && q.shape[2] == 1 && !c->open_round &&
                mask_mode != KVC_MASK_ARRAY && k.stride[3] == 1 && v.stride[3] == 1 &&
                (k.dtype == KVC_BF16 || k.dtype == KVC_F16)) {
                require4(k, "keys");
                require4(v, "values");
                KVC_REQUIRE(k.dtype == v.dtype && k.shape[0] == v.shape[0] && k.shape[1] == v.shape[1] && v.shape[2] == 1,
                            "update: keys and values disagree on batch, heads or length");
                c->restore.valid = false;
                const int64_t prev = c->offset;
                const void *k_before = c->k.allocated() ? c->k.view(c->offset).data : nullptr;
                linear_update(c, k, v, s, /*defer_append=*/true);
                kvc_tensor ck = c->k.view(c->offset), cv = c->v.view(c->offset);
                AttnArgs a = make_attn_args(q, out, scale, KVC_MASK_NONE, nullptr, ck.shape[2], Hkv);
                a.k = raw_source(ck);
                a.v = raw_source(cv);
                a.new_k = k.data; a.new_v = v.data;
                // inside a batched call the launch before this one belongs to the previous layer's cache;
                // a growth copy in linear_update would be a write to this one
                a.stored_rows_settled = tl_batch_prev != nullptr && tl_batch_prev != c && k_before == ck.data;
                a.nk_sb = k.stride[0]; a.nk_sh = k.stride[1];
                a.nv_sb = v.stride[0]; a.nv_sh = v.stride[1];
                if (launch_attention_decode(a, s) > 0) return;
                append_pair(c->k, c->v, k, v, prev, s);
                a.new_k = a.new_v = nullptr;
                launch_attention(a, s);
                return;
            }
            // The same for a RotatingKVCache's single-token update (updateInPlace): the kernel writes
            // the row into the ring slot and leaves the row it replaces out of the scores.
            if (!fuse_off && c->cfg.kind == KVC_KIND_ROTATING && k.shape[2] == 1 && q.shape[2] == 1 && !c->open_round &&
                mask_mode == KVC_MASK_NONE && k.stride[3] == 1 && v.stride[3] == 1 && k.ndim == 4 && v.ndim == 4 &&
                (k.dtype == KVC_BF16 || k.dtype == KVC_F16) && k.dtype == v.dtype && k.shape[0] == v.shape[0] &&
                k.shape[1] == v.shape[1] && v.shape[2] == 1) {
                check_new_rows(c, c->k, c->v, k, v);
                c->restore.valid = false;
                const int64_t launches_before = g_launch_count;
                const void *k_before = c->k.allocated() ? c->k.view(1).data : nullptr;
                kvc_tensor ck, cv;
                int64_t slot = -1;
                rotating_update_in_place(c, k, v, s, &ck, &cv, &slot);
                AttnArgs a = make_attn_args(q, out, scale, KVC_MASK_NONE, nullptr, ck.shape[2], Hkv);
                a.k = raw_source(ck);
                a.v = raw_source(cv);
                a.new_k = k.data; a.new_v = v.data;
                a.new_slot = slot;
                a.nk_sb = k.stride[0]; a.nk_sh = k.stride[1];
                a.nv_sb = v.stride[0]; a.nv_sh = v.stride[1];
                // no growth copy and no ring rebuild in this call: the stored rows are as the last step left them
                a.stored_rows_settled = tl_batch_prev != nullptr && tl_batch_prev != c && k_before == ck.data &&
                                        launches_before == g_launch_count;
                if (slot >= 0 && slot < ck.shape[2] && launch_attention_decode(a, s) > 0) return;
                append_pair(c->k, c->v, k, v, slot, s);
                a.new_k = a.new_v = nullptr;
                a.new_slot = -1;
                a.stored_rows_settled = false;
                launch_attention(a, s);
                return;
            }
            kvc_tensor ck, cv;
            cache_update(c, k, v, s, &ck, &cv);
            AttnArgs a = make_attn_args(q, out, scale, mask_mode, mask, ck.shape[2], Hkv);
            a.k = raw_source(ck);
            a.v = raw_source(cv);
            launch_attention(a, s);
            return;
        }
    }
}

int launch_attention_affine_varlen(const AttnArgs *args, int n, cudaStream_t stream);

void cache_attention_varlen(kvc_cache *const *caches, int n, const kvc_tensor *q, const kvc_tensor *k,
                            const kvc_tensor *v, float scale, const kvc_tensor *outs, cudaStream_t s) {
    auto one_by_one = [&](int from, int to) {
        for (int i = from; i < to; ++i) cache_attention(caches[i], q[i], k[i], v[i], scale, KVC_MASK_NONE, nullptr, outs[i], s);
    };
    auto row_contiguous = [](const kvc_tensor &t) {
        return t.ndim == 4 && t.stride[3] == 1 && t.stride[1] == t.shape[3] * t.shape[2];
    };
    for (int from = 0; from < n; from += KVC_VARLEN_MAX) {
        const int to = std::min(n, from + KVC_VARLEN_MAX), m = to - from;
        bool fits = m > 1;
        for (int i = from; i < to && fits; ++i) {
            const kvc_cache *c = caches[i];
            fits = c && c->cfg.kind == KVC_KIND_QUANTIZED && !c->open_round && c->device == caches[from]->device &&
                   c->bits == caches[from]->bits && q[i].ndim == 4 && row_contiguous(k[i]) && row_contiguous(v[i]) &&
                   k[i].shape[0] == 1 && k[i].shape[2] == 1 && q[i].shape[0] == 1 && q[i].shape[2] == 1 &&
                   k[i].shape[1] == k[from].shape[1] && k[i].shape[3] == k[from].shape[3] &&
                   v[i].shape[3] == k[from].shape[3] && k[i].dtype == k[from].dtype && q[i].dtype == k[i].dtype &&
                   k[i].stride[1] == k[from].stride[1] && v[i].stride[1] == k[from].stride[1];
        }
        if (!fits) {
            one_by_one(from, to);
            continue;
        }
        // bookkeeping + growth per cache (no launch), then ONE quantise-append launch for all of them
        VarlenQuantArgs qa = {};
        qa.n = m;
        qa.H = (int)k[from].shape[1];
        qa.D = (int)k[from].shape[3];
        qa.dtype = k[from].dtype;
        qa.src_sh = k[from].stride[1];
        std::vector<AttnArgs> args((size_t)m);
        bool same_group = true;
        for (int i = from; i < to; ++i) {
            kvc_cache *c = caches[i];
            const int64_t prev = c->offset;
            kvc_tensor qk[3], qv[3];
            cache_update_quantized(c, k[i], v[i], s, qk, qv, /*defer_quantize=*/true);
            same_group = same_group && c->group_size == caches[from]->group_size;
            VarlenQuantSeq &sq = qa.seq[i - from];
            sq.ksrc = k[i].data; sq.vsrc = v[i].data;
            sq.kcodes = (uint32_t *)c->kq.ptr + prev * c->kq.st();
            sq.vcodes = (uint32_t *)c->vq.ptr + prev * c->vq.st();
            const size_t es = dtype_size(c->ks.dtype);
            sq.kscales = (char *)c->ks.ptr + prev * c->ks.st() * es;
            sq.kbiases = (char *)c->kb.ptr + prev * c->kb.st() * es;
            sq.vscales = (char *)c->vs.ptr + prev * c->vs.st() * es;
            sq.vbiases = (char *)c->vb.ptr + prev * c->vb.st() * es;
            sq.c_sh = c->kq.sh(); sq.g_sh = c->ks.sh();
            same_group = same_group && c->vq.sh() == c->kq.sh() && c->vs.sh() == c->ks.sh();
            AttnArgs a = make_attn_args(q[i], outs[i], scale, KVC_MASK_NONE, nullptr, c->offset, qa.H);
            a.k = affine_source(qk[0], qk[1], qk[2], c->group_size, c->bits);
            a.v = affine_source(qv[0], qv[1], qv[2], c->group_size, c->bits);
            args[(size_t)(i - from)] = a;
        }
        qa.group = caches[from]->group_size;
        qa.bits = caches[from]->bits;
        if (!same_group || !launch_affine_quantize_varlen(qa, s)) {
            for (int i = from; i < to; ++i) {
                kvc_cache *c = caches[i];
                const int64_t prev = c->offset - 1;
                QuantAppendArgs ka = quant_args(k[i], c->kq, c->ks, c->kb, c->group_size, c->bits, prev);
                QuantAppendArgs va = quant_args(v[i], c->vq, c->vs, c->vb, c->group_size, c->bits, prev);
                launch_affine_quantize2(ka, &va, s);
            }
        }
        if (!same_group || launch_attention_affine_varlen(args.data(), m, s) == 0)
            for (int i = 0; i < m; ++i) launch_attention(args[(size_t)i], s);
    }
}

// ---------------------------------------------------------------------
// trim / trimmable
// ---------------------------------------------------------------------
int64_t cache_trim(kvc_cache *c, int64_t n) {
    if (c->open_round) fail(KVC_ERR_INVALID_STATE, "trim: a staged round is open on this cache");
    c->restore.valid = false;
    switch (c->cfg.kind) {
        case KVC_KIND_ROTATING: {
            // KVCache.swift:826-831: no validity check, idx moves with offset.
            const int64_t t = std::min(c->offset, std::max<int64_t>(n, 0));
            c->offset -= t;
            c->idx -= t;
            return t;
        }
        case KVC_KIND_TURBO: {
            // TurboQuantKVCache.swift:1583-1603
            if (n <= 0 || c->offset <= 0) return 0;
            const int64_t t = std::min(n, c->offset);
            c->offset -= t;
            if (c->offset == 0) {
                cudaStream_t s = c->last_stream;   // trim carries no stream: free behind the last work on the arrays
                for (Array4 *a : {&c->k, &c->v, &c->kp, &c->kn, &c->vp, &c->vn, &c->kq, &c->ks, &c->kb,
                                  &c->vq, &c->vs, &c->vb})
                    a->release(s);
                set_key_calibration(c, {}, s);   // keyCalibScale = nil (:1598)
                c->compressed = false;
            }
            return t;
        }
        case KVC_KIND_CHUNKED: {
            // KVCache.swift:1271-1276
            const int64_t t = std::min(c->offset - c->start_position, n);
            c->offset -= t;
            return t;
        }
        case KVC_KIND_LIST: {
            // KVCache.swift:1653-1660: every child trims, the last child's count is returned
            int64_t result = 0;
            for (kvc_cache *child : c->children) result = cache_trim(child, n);
            return result;
        }
        default: {
            const int64_t t = std::min(c->offset, std::max<int64_t>(n, 0));
            c->offset -= t;
            return t;
        }
    }
}

bool cache_is_trimmable_after(const kvc_cache *c, int64_t positions) {
    if (c->cfg.kind == KVC_KIND_ROTATING) return c->offset + positions < c->cfg.max_size;  // KVCache.swift:821-823
    if (c->cfg.kind == KVC_KIND_LIST) {  // KVCache.swift:1645-1651
        for (const kvc_cache *child : c->children)
            if (!cache_is_trimmable_after(child, positions)) return false;
        return true;
    }
    return true;
}

const char *cache_class_name(const kvc_cache *c) {
    // cacheClassName (KVCache.swift:1739-1751)
    switch (c->cfg.kind) {
        case KVC_KIND_SIMPLE: return "KVCache";
        case KVC_KIND_ROTATING: return "RotatingKVCache";
        case KVC_KIND_QUANTIZED: return "QuantizedKVCache";
        case KVC_KIND_TURBO: return "TurboQuantKVCache";
        case KVC_KIND_CHUNKED: return "ChunkedKVCache";
        case KVC_KIND_LIST: return "CacheList";
        default: return "KVCache";
    }
}

// ---------------------------------------------------------------------
// state / metaState
// ---------------------------------------------------------------------
int cache_state_count(const kvc_cache *c) {
    switch (c->cfg.kind) {
        case KVC_KIND_LIST: {
            int n = 0;
            for (const kvc_cache *child : c->children) n += cache_state_count(child);
            return n;
        }
        case KVC_KIND_CHUNKED:
        case KVC_KIND_SIMPLE:
        case KVC_KIND_ROTATING: return c->k.allocated() ? 2 : 0;
        case KVC_KIND_QUANTIZED: return c->kq.allocated() ? 6 : 0;
        case KVC_KIND_TURBO:
            if (c->offset <= 0) return 0;
            if (!c->compressed) return c->k.allocated() ? 2 : 0;
            if (c->affine_value) return c->raw_key ? 4 : (c->affine_key ? 6 : 5);
            if (c->affine_key) return 5;
            if (c->raw_key) return 3;
            return c->kcodec.calib_dev ? 5 : 4;
        default: return 0;
    }
}

kvc_tensor cache_state_get(kvc_cache *c, int index) {
    const int n = cache_state_count(c);
    if (index < 0 || index >= n) fail(KVC_ERR_INVALID_ARG, "state index out of range");
    switch (c->cfg.kind) {
        case KVC_KIND_LIST: {
            // state = caches.flatMap { $0.state } (KVCache.swift:1580-1581)
            for (kvc_cache *child : c->children) {
                const int m = cache_state_count(child);
                if (index < m) return cache_state_get(child, index);
                index -= m;
            }
            fail(KVC_ERR_INTERNAL, "CacheList state index");
        }
        case KVC_KIND_CHUNKED:
            // the inherited getter slices [..<offset] with the ABSOLUTE offset (KVCache.swift:449-459); a slice
            // past the end of the buffer clamps to it, zero padding rows included
            return (index == 0 ? c->k : c->v).view(std::min(c->offset, c->len));
        case KVC_KIND_SIMPLE: return (index == 0 ? c->k : c->v).view(c->offset);
        case KVC_KIND_ROTATING: {
            // KVCache.swift:752-763: rows [0, offset) while the buffer is longer, else the whole ring
            const int64_t rows = c->offset < c->len ? std::max<int64_t>(c->offset, 0) : c->len;
            return (index == 0 ? c->k : c->v).view(rows);
        }
        case KVC_KIND_QUANTIZED: {
            Array4 *arr[6] = {&c->kq, &c->ks, &c->kb, &c->vq, &c->vs, &c->vb};
            return arr[index]->view(c->offset);
        }
        case KVC_KIND_TURBO: {
            if (!c->compressed) return (index == 0 ? c->k : c->v).view(c->offset);
            std::vector<kvc_tensor> st;
            if (c->affine_key) { st.push_back(c->kq.view(c->offset)); st.push_back(c->ks.view(c->offset)); st.push_back(c->kb.view(c->offset)); }
            else if (c->raw_key) st.push_back(c->k.view(c->offset));
            else { st.push_back(c->kp.view(c->offset)); st.push_back(view3(c->kn, c->offset)); }
            if (c->affine_value) { st.push_back(c->vq.view(c->offset)); st.push_back(c->vs.view(c->offset)); st.push_back(c->vb.view(c->offset)); }
            else { st.push_back(c->vp.view(c->offset)); st.push_back(view3(c->vn, c->offset)); }
            if (!c->affine_key && !c->raw_key && !c->affine_value && c->kcodec.calib_dev) {
                // fifth array of the standard state: the calibration scale, shape [D] (:1509-1511)
                kvc_tensor t{};
                t.data = c->kcodec.calib_dev; t.dtype = KVC_F32; t.ndim = 1;
                t.shape[0] = (int64_t)c->kcodec.calib.size(); t.stride[0] = 1;
                st.push_back(t);
            }
            return st[index];
        }
        default: fail(KVC_ERR_INVALID_ARG, "unknown cache kind");
    }
}

// Copy a strided [B, H, T, W] (or [B, H, T]) device tensor into a fresh array.
// `step` > 1 rounds the capacity up to whole steps (the rows beyond the copied ones stay unused).
static void adopt(Array4 &dst, const kvc_tensor &t, cudaStream_t s, int64_t step = 1) {
    kvc_tensor x = t;
    if (x.ndim == 3) { x.ndim = 4; x.shape[3] = 1; x.stride[3] = 1; }
    require4(x, "state array");
    dst.release(s);
    dst.alloc(x.shape[0], x.shape[1], round_up(std::max<int64_t>(x.shape[2], 1), step), x.shape[3], x.dtype, s);
    if (x.shape[2] == 0) return;
    AppendArgs a;
    a.k_src = x.data; a.v_src = x.data;
    a.ks_sb = x.stride[0]; a.ks_sh = x.stride[1]; a.ks_ss = x.stride[2]; a.ks_sd = x.stride[3];
    a.vs_sb = a.ks_sb; a.vs_sh = a.ks_sh; a.vs_ss = a.ks_ss; a.vs_sd = a.ks_sd;
    a.k_dst = dst.ptr; a.v_dst = dst.ptr;
    a.kd_sb = dst.sb(); a.kd_sh = dst.sh(); a.kd_st = dst.st();
    a.vd_sb = a.kd_sb; a.vd_sh = a.kd_sh; a.vd_st = a.kd_st;
    a.B = (int)x.shape[0]; a.H = (int)x.shape[1]; a.S = (int)x.shape[2];
    a.Dk = (int)x.shape[3]; a.Dv = 0;
    a.pos = 0; a.esize = (int)dtype_size(x.dtype);
    launch_append(a, s);
}

void cache_state_set(kvc_cache *c, const kvc_tensor *arrays, int count, cudaStream_t s) {
    c->last_stream = s;
    if (c->open_round) fail(KVC_ERR_INVALID_STATE, "state: a staged round is open on this cache");
    c->restore.valid = false;
    switch (c->cfg.kind) {
        case KVC_KIND_LIST: {
            // KVCache.swift:1582-1590: every child takes as many arrays as its state currently has
            int start = 0;
            for (kvc_cache *child : c->children) {
                const int m = cache_state_count(child);
                KVC_REQUIRE(start + m <= count, "CacheList state: too few arrays for the children's current state counts");
                cache_state_set(child, arrays + start, m, s);
                start += m;
            }
            return;
        }
        case KVC_KIND_CHUNKED:
            KVC_REQUIRE(count == 2, "KVCacheSimple state must have exactly 2 arrays (keys, values)");
            adopt(c->k, arrays[0], s);
            adopt(c->v, arrays[1], s);
            c->offset = arrays[0].shape[2];
            c->len = arrays[0].shape[2];
            return;
        case KVC_KIND_SIMPLE:
            KVC_REQUIRE(count == 2, "KVCacheSimple state must have exactly 2 arrays (keys, values)");
            adopt(c->k, arrays[0], s);
            adopt(c->v, arrays[1], s);
            c->offset = arrays[0].shape[2];  // KVCache.swift:467
            return;
        case KVC_KIND_ROTATING:
            KVC_REQUIRE(count == 2, "RotatingKVCache state must have exactly 2 arrays");
            adopt(c->k, arrays[0], s);
            adopt(c->v, arrays[1], s);
            c->len = arrays[0].shape[2];  // offset and idx travel in metaState (KVCache.swift:770-771)
            return;
        case KVC_KIND_QUANTIZED: {
            if (count == 4) fail(KVC_ERR_UNSUPPORTED, "QuantizedKVCache state without biases (non-affine modes) is not built");
            KVC_REQUIRE(count == 6, "QuantizedKVCache state must have exactly 6 or 4 arrays (3/2 for keys, 3/2 for values)");
            Array4 *arr[6] = {&c->kq, &c->ks, &c->kb, &c->vq, &c->vs, &c->vb};
            for (int i = 0; i < 6; ++i) adopt(*arr[i], arrays[i], s);
            return;
        }
        case KVC_KIND_TURBO: {
            // TurboQuantKVCache.swift:1519-1567
            for (Array4 *a : {&c->k, &c->v, &c->kp, &c->kn, &c->vp, &c->vn, &c->kq, &c->ks, &c->kb, &c->vq, &c->vs, &c->vb})
                a->release(s);
            if (c->affine_key && count == 5 && !c->affine_value) {
                adopt(c->kq, arrays[0], s); adopt(c->ks, arrays[1], s); adopt(c->kb, arrays[2], s);
                adopt(c->vp, arrays[3], s, 256); adopt(c->vn, arrays[4], s, 256);
                c->compressed = true;
            } else if (c->raw_key && count == 3 && !c->affine_value) {
                adopt(c->k, arrays[0], s); adopt(c->vp, arrays[1], s, 256); adopt(c->vn, arrays[2], s, 256);
                c->compressed = true;
            } else if (!c->affine_key && !c->raw_key && c->affine_value && count == 5) {
                adopt(c->kp, arrays[0], s, 256); adopt(c->kn, arrays[1], s, 256);
                adopt(c->vq, arrays[2], s); adopt(c->vs, arrays[3], s); adopt(c->vb, arrays[4], s);
                c->compressed = true;
            } else if (!c->affine_key && !c->raw_key && count == 5) {
                // [keyPacked, keyNorms, valPacked, valNorms, keyCalibScale] (:1539-1550)
                const kvc_tensor &cs = arrays[4];
                KVC_REQUIRE(cs.ndim == 1 && cs.dtype == KVC_F32 && cs.stride[0] == 1 && cs.shape[0] > 0 && cs.shape[0] <= 1024,
                            "TurboQuantKVCache state: the key-calibration scale must be a contiguous float32 [D] array");
                std::vector<float> scale((size_t)cs.shape[0]);
                KVC_CUDA(cudaMemcpyAsync(scale.data(), cs.data, scale.size() * sizeof(float), cudaMemcpyDeviceToHost, s));
                KVC_CUDA(cudaStreamSynchronize(s));
                adopt(c->kp, arrays[0], s, 256); adopt(c->kn, arrays[1], s, 256);
                adopt(c->vp, arrays[2], s, 256); adopt(c->vn, arrays[3], s, 256);
                set_key_calibration(c, scale, s);
                c->compressed = true;
            } else if (count == 4 && !c->affine_value) {
                adopt(c->kp, arrays[0], s, 256); adopt(c->kn, arrays[1], s, 256);
                adopt(c->vp, arrays[2], s, 256); adopt(c->vn, arrays[3], s, 256);
                c->compressed = true;
            } else if (count == 2) {
                adopt(c->k, arrays[0], s); adopt(c->v, arrays[1], s);
                c->compressed = false;
            } else {
                fail(KVC_ERR_INVALID_ARG, "TurboQuantKVCache state: unexpected number of arrays");
            }
            c->offset = arrays[0].shape[2];
            return;
        }
        default: fail(KVC_ERR_INVALID_ARG, "unknown cache kind");
    }
}

std::vector<std::string> cache_meta_state(const kvc_cache *c) {
    auto S = [](int64_t v) { return std::to_string(v); };
    switch (c->cfg.kind) {
        case KVC_KIND_SIMPLE: return {""};  // BaseKVCache default (KVCache.swift:207-214)
        case KVC_KIND_ROTATING:  // KVCache.swift:775-781
            return {S(c->cfg.keep), S(c->cfg.max_size), S(c->cfg.step), S(c->offset), S(c->idx), c->origin};
        case KVC_KIND_QUANTIZED:  // KVCache.swift:1148-1149
            return {S(c->cfg.step), S(c->offset), S(c->group_size), S(c->bits)};
        case KVC_KIND_TURBO:  // TurboQuantKVCache.swift:1570-1573
            return {S(c->offset), S(c->cfg.bits), S(c->key_bits), S(c->value_bits), std::to_string(c->cfg.seed)};
        case KVC_KIND_CHUNKED:  // KVCache.swift:1289-1293
            return {c->cfg.max_size > 0 ? S(c->cfg.max_size) : std::string("None"), S(c->start_position)};
        case KVC_KIND_LIST: {   // KVCache.swift:1673-1685: [childCount, (className, stateCount, metaCount, meta...)*]
            std::vector<std::string> out{S((int64_t)c->children.size())};
            for (const kvc_cache *child : c->children) {
                const std::vector<std::string> meta = cache_meta_state(child);
                out.push_back(cache_class_name(child));
                out.push_back(S(cache_state_count(child)));
                out.push_back(S((int64_t)meta.size()));
                out.insert(out.end(), meta.begin(), meta.end());
            }
            return out;
        }
        default: return {};
    }
}

static bool parse_int(const std::string &s, int64_t &out) {
    if (s.empty()) return false;
    char *end = nullptr;
    const long long v = std::strtoll(s.c_str(), &end, 10);
    if (!end || *end != '\0') return false;
    out = v;
    return true;
}

void cache_set_meta_state(kvc_cache *c, const std::vector<std::string> &m) {
    if (c->open_round) fail(KVC_ERR_INVALID_STATE, "metaState: a staged round is open on this cache");
    c->restore.valid = false;
    switch (c->cfg.kind) {
        case KVC_KIND_SIMPLE:
            KVC_REQUIRE(m.size() == 1 && m[0].empty(), "This cache has no meta_state but a meta_state was set.");
            return;
        case KVC_KIND_ROTATING: {
            KVC_REQUIRE(m.size() == 5 || m.size() == 6, "RotatingKVCache metaState must have 5 or 6 values");
            int64_t keep, step, off, idx, mx;
            KVC_REQUIRE(parse_int(m[0], keep) && parse_int(m[2], step) && parse_int(m[3], off) && parse_int(m[4], idx),
                        "Failed to convert metaState values to integers");
            KVC_REQUIRE(m[1] != "None", "RotatingKVCache requires a non-nil maxSize. Cannot load cache with maxSize=None.");
            KVC_REQUIRE(parse_int(m[1], mx), "Failed to convert maxCacheSize to integer");
            std::string origin = "modelNative";
            if (m.size() == 6) {
                KVC_REQUIRE(m[5] == "modelNative" || m[5] == "requested", "Invalid RotatingKVCache capacity origin");
                origin = m[5];
            }
            c->cfg.keep = (int32_t)keep; c->cfg.max_size = (int32_t)mx; c->cfg.step = (int32_t)step;
            c->offset = off; c->idx = idx; c->origin = origin;
            return;
        }
        case KVC_KIND_QUANTIZED: {
            KVC_REQUIRE(m.size() == 4, "QuantizedKVCache metaState must have exactly 4 values");
            int64_t off, g, b;
            KVC_REQUIRE(parse_int(m[1], off) && parse_int(m[2], g) && parse_int(m[3], b),
                        "Failed to convert QuantizedKVCache metaState values to integers");
            c->offset = off; c->group_size = (int32_t)g; c->bits = (int32_t)b;
            return;
        }
        case KVC_KIND_TURBO: {
            int64_t off;
            if (m.size() >= 5 && parse_int(m[0], off)) c->offset = off;  // TurboQuantKVCache.swift:1574-1579
            return;
        }
        case KVC_KIND_CHUNKED: {
            // KVCache.swift:1294-1303
            KVC_REQUIRE(m.size() == 2, "ChunkedKVCache metaState must have exactly 2 values");
            int64_t v = 0;
            if (m[0] == "None") c->cfg.max_size = -1;
            else if (parse_int(m[0], v)) c->cfg.max_size = (int32_t)v;
            else c->cfg.max_size = -1;   // Int(newValue[0]) gives nil
            c->start_position = parse_int(m[1], v) ? v : 0;
            return;
        }
        case KVC_KIND_LIST:
            // KVCache.swift:1686-1689
            fail(KVC_ERR_INVALID_STATE, "CacheList.metaState should not be set directly. Use CacheList.fromState() instead");
        default: fail(KVC_ERR_INVALID_ARG, "unknown cache kind");
    }
}

// ---------------------------------------------------------------------
// copy / conversions
// ---------------------------------------------------------------------
static void clone_array(const Array4 &src, Array4 &dst, int64_t rows, cudaStream_t s, int64_t step = 1) {
    if (!src.allocated()) return;
    dst.alloc(src.B, src.H, round_up(std::max<int64_t>(rows, 1), step), src.W, src.dtype, s);
    copy_rows(src, 0, dst, 0, std::min(rows, src.cap), s);
}

kvc_cache *cache_copy(const kvc_cache *c, cudaStream_t s) {
    // copy() (KVCache.swift:525-533, :877-885, :1177-1185): the new object adopts
    // the `state` arrays and the metaState.
    std::unique_ptr<kvc_cache> n(new kvc_cache());
    if (c->cfg.kind == KVC_KIND_LIST) {
        // KVCache.swift:1592-1596
        n->cfg = c->cfg;
        n->device = c->device;
        for (const kvc_cache *child : c->children) n->children.push_back(cache_copy(child, s));
        return n.release();
    }
    n->cfg = c->cfg;
    n->cfg.reserve_tokens = 0;
    n->device = c->device;
    n->offset = c->offset;
    n->len = c->len; n->idx = c->idx; n->origin = c->origin;
    n->group_size = c->group_size; n->bits = c->bits; n->group_resolved = c->group_resolved;
    n->compressed = c->compressed;
    n->key_bits = c->key_bits; n->value_bits = c->value_bits; n->key_group = c->key_group;
    n->raw_key = c->raw_key; n->affine_key = c->affine_key; n->affine_value = c->affine_value;
    n->user_kc = c->user_kc; n->user_vc = c->user_vc; n->user_ks = c->user_ks; n->user_vs = c->user_vs;
    n->user_kr = c->user_kr; n->user_vr = c->user_vr;
    int64_t rows = c->offset;
    if (c->cfg.kind == KVC_KIND_CHUNKED) {
        // KVCache.swift:1278-1287: the copy adopts `state` (rows up to the absolute offset, clamped to the
        // buffer) and then the metaState; its offset becomes the adopted row count
        rows = c->k.allocated() ? std::min(c->offset, c->len) : 0;
        n->offset = c->k.allocated() ? rows : 0;
        n->len = rows;
        n->start_position = c->start_position;
    }
    if (c->cfg.kind == KVC_KIND_ROTATING) {
        rows = c->offset < c->len ? std::max<int64_t>(c->offset, 0) : c->len;
        n->len = c->k.allocated() ? rows : 0;
    }
    clone_array(c->k, n->k, rows, s); clone_array(c->v, n->v, rows, s);
    clone_array(c->kq, n->kq, rows, s); clone_array(c->ks, n->ks, rows, s); clone_array(c->kb, n->kb, rows, s);
    clone_array(c->vq, n->vq, rows, s); clone_array(c->vs, n->vs, rows, s); clone_array(c->vb, n->vb, rows, s);
    // packed TurboQuant arrays in whole 256-row steps (what the reference allocates; the decode kernels stream whole stages)
    clone_array(c->kp, n->kp, rows, s, 256); clone_array(c->kn, n->kn, rows, s, 256);
    clone_array(c->vp, n->vp, rows, s, 256); clone_array(c->vn, n->vn, rows, s, 256);
    if (!c->kcodec.calib.empty()) set_key_calibration(n.get(), c->kcodec.calib, s);
    return n.release();
}

static kvc_cache *new_cache(int kind) {
    kvc_cache *n = new kvc_cache();
    kvc_config_default(&n->cfg, kind);
    return n;
}

kvc_cache *cache_to_quantized(const kvc_cache *c, int group, int bits, cudaStream_t s) {
    // KVCacheSimple.toQuantized (KVCache.swift:486-523); RotatingKVCache.toQuantized always throws (:894-899).
    if (c->cfg.kind == KVC_KIND_ROTATING)
        fail(KVC_ERR_UNSUPPORTED, "RotatingKVCache quantization is not implemented because its temporal ordering requires dedicated handling.");
    KVC_REQUIRE(c->cfg.kind == KVC_KIND_SIMPLE, "toQuantized needs a KVCacheSimple");
    std::unique_ptr<kvc_cache> n(new_cache(KVC_KIND_QUANTIZED));
    n->device = c->device;
    n->bits = bits; n->cfg.bits = bits;
    n->group_size = group; n->cfg.group_size = group;
    n->offset = c->offset;
    if (!c->k.allocated()) return n.release();
    const int kd = (int)c->k.W, vd = (int)c->v.W;
    const int eff = resolved_group_size(group, kd, vd);
    if (!eff)
        fail(KVC_ERR_INVALID_ARG,
             "KV cache quantization requires head dimensions divisible by one of the supported group sizes (32, 64, 128).");
    n->group_size = eff;
    const int64_t rows = c->offset;
    quant_triple_alloc(n->kq, n->ks, n->kb, c->k.B, c->k.H, rows, kd, eff, bits, c->k.dtype, s);
    quant_triple_alloc(n->vq, n->vs, n->vb, c->v.B, c->v.H, rows, vd, eff, bits, c->v.dtype, s);
    if (rows > 0) {
        kvc_tensor kt = c->k.view(rows), vt = c->v.view(rows);
        QuantAppendArgs qa = quant_args(kt, n->kq, n->ks, n->kb, eff, bits, 0);
        QuantAppendArgs qv = quant_args(vt, n->vq, n->vs, n->vb, eff, bits, 0);
        launch_affine_quantize2(qa, &qv, s);
    }
    return n.release();
}

kvc_cache *cache_to_unquantized(const kvc_cache *c, cudaStream_t s) {
    // QuantizedKVCache.toUnquantized (KVCache.swift:1188-1209)
    KVC_REQUIRE(c->cfg.kind == KVC_KIND_QUANTIZED, "toUnquantized needs a QuantizedKVCache");
    std::unique_ptr<kvc_cache> n(new_cache(KVC_KIND_SIMPLE));
    n->device = c->device;
    n->offset = c->offset;
    if (!c->kq.allocated()) return n.release();
    const int64_t rows = c->offset;
    const int kd = (int)(c->kq.W * 32 / c->bits), vd = (int)(c->vq.W * 32 / c->bits);
    n->k.alloc(c->kq.B, c->kq.H, std::max<int64_t>(rows, 1), kd, c->ks.dtype, s);
    n->v.alloc(c->vq.B, c->vq.H, std::max<int64_t>(rows, 1), vd, c->vs.dtype, s);
    // one launch per (batch, head) plane keeps the row strides simple
    for (int which = 0; which < 2; ++which) {
        const Array4 &q = which ? c->vq : c->kq, &sc = which ? c->vs : c->ks, &bi = which ? c->vb : c->kb;
        Array4 &o = which ? n->v : n->k;
        for (int64_t bh = 0; bh < q.B * q.H; ++bh) {
            DequantArgs d;
            d.codes = (const uint32_t *)q.ptr + bh * q.sh();
            d.scales = (const char *)sc.ptr + (size_t)bh * sc.sh() * sc.esize();
            d.biases = (const char *)bi.ptr + (size_t)bh * bi.sh() * bi.esize();
            d.out = (char *)o.ptr + (size_t)bh * o.sh() * o.esize();
            d.dtype = sc.dtype; d.rows = rows;
            d.c_srow = q.st(); d.g_srow = sc.st(); d.o_srow = o.st();
            d.D = (int)o.W; d.group = c->group_size; d.bits = c->bits;
            launch_affine_dequantize(d, s);
        }
    }
    return n.release();
}

kvc_cache *cache_to_turbo(const kvc_cache *c, int kb, int vb, int kg, cudaStream_t s) {
    // maybeTurboQuantizeKVCache per-layer conversion (TurboQuantKVCache.swift:1748-1759)
    KVC_REQUIRE(c->cfg.kind == KVC_KIND_SIMPLE, "turbo conversion needs a KVCacheSimple");
    kvc_config cfg;
    kvc_config_default(&cfg, KVC_KIND_TURBO);
    cfg.bits = std::max(kb, vb); cfg.key_bits = kb; cfg.value_bits = vb; cfg.key_group_size = kg;
    kvc_cache *raw = nullptr;
    if (kvc_create(&cfg, &raw) != KVC_OK) fail(KVC_ERR_INVALID_ARG, kvc_last_error_message());
    std::unique_ptr<kvc_cache> n(raw);
    if (c->k.allocated() && c->offset > 0) {
        kvc_tensor kt = c->k.view(c->offset), vt = c->v.view(c->offset);
        cache_update(n.get(), kt, vt, s, nullptr, nullptr);
    }
    return n.release();
}

// ---------------------------------------------------------------------
// logical view / masks
// ---------------------------------------------------------------------
void cache_logical_view(kvc_cache *c, int64_t tail, cudaStream_t s, kvc_tensor *ok, kvc_tensor *ov) {
    c->last_stream = s;
    // RotatingKVCache.logicalView(tail:) (KVCache.swift:631-658)
    KVC_REQUIRE(c->cfg.kind == KVC_KIND_ROTATING, "logicalView needs a RotatingKVCache");
    if (!c->k.allocated()) fail(KVC_ERR_INVALID_STATE, "logicalView: nothing has been written yet");
    auto ordered = rot_temporal(c);
    const int64_t available = seg_total(ordered);
    const int64_t keep = c->cfg.keep;
    const int64_t requested = std::min(std::max<int64_t>(tail, 0), available);
    const int64_t bound = std::max(requested, std::min(keep, available));
    const int64_t trim_size = available - bound;
    std::vector<GatherSeg> segs = ordered;
    if (trim_size > 0) {
        if (keep == 0) segs = seg_slice(ordered, trim_size, available);
        else segs = rot_front_trim(ordered, trim_size, keep);
    }
    const int64_t n = seg_total(segs);
    if (segs.size() <= 1) {
        const int64_t first = segs.empty() ? 0 : segs[0].src_start;
        if (ok) *ok = c->k.view(n, first);
        if (ov) *ov = c->v.view(n, first);
        return;
    }
    ensure_like(c->k_view, c->k, std::max<int64_t>(n, c->cfg.max_size), s);
    ensure_like(c->v_view, c->v, std::max<int64_t>(n, c->cfg.max_size), s);
    gather_rows(c->k, c->k_view, segs, s);
    gather_rows(c->v, c->v_view, segs, s);
    if (ok) *ok = c->k_view.view(n);
    if (ov) *ov = c->v_view.view(n);
}

void cache_make_mask(const kvc_cache *c, int n, int64_t window, bool return_array, int32_t *mode,
                     int64_t *rows, int64_t *cols, void *out_mask, cudaStream_t s) {
    *rows = 0; *cols = 0;
    if (c->cfg.kind == KVC_KIND_ROTATING) {
        // RotatingKVCache.makeMask (KVCache.swift:834-871)
        const int64_t max_size = c->cfg.max_size;
        if (n > 1) {
            const int64_t actual = window >= 0 ? window : max_size;
            const int64_t capped = std::min(max_size - 1, c->offset);
            if (capped + n > actual || return_array) {
                *mode = KVC_MASK_ARRAY; *rows = n; *cols = capped + n;
                if (out_mask) launch_causal_mask((uint8_t *)out_mask, n, capped, actual, s);
                return;
            }
            *mode = KVC_MASK_CAUSAL;
            return;
        }
        if (window < 0) { *mode = KVC_MASK_NONE; return; }
        if (c->offset >= window && max_size > window) {
            int64_t cur = c->idx;
            if (cur >= max_size) cur = 0;
            const int64_t size = c->offset < max_size ? c->offset + 1 : max_size;
            *mode = KVC_MASK_ARRAY; *rows = 1; *cols = size;
            if (out_mask) launch_rolled_mask((uint8_t *)out_mask, size, window, cur + 1, s);
            return;
        }
        *mode = KVC_MASK_NONE;
        return;
    }
    // BaseKVCache.makeMask (KVCache.swift:236-250)
    if (n == 1) { *mode = KVC_MASK_NONE; return; }
    if (return_array || (window >= 0 && n > window)) {
        *mode = KVC_MASK_ARRAY; *rows = n; *cols = c->offset + n;
        if (out_mask) launch_causal_mask((uint8_t *)out_mask, n, c->offset, window, s);
        return;
    }
    *mode = KVC_MASK_CAUSAL;
}

// ---------------------------------------------------------------------
// TurboQuant codebooks and sign vectors
// ---------------------------------------------------------------------
namespace {
// The Lloyd-Max centroids the reference ships as data for its common (head dim, bits) pairs
// (TurboQuantCodebook.precomputed, TurboQuantKVCache.swift:57-94). The reference reads this
// table before it falls back to its generator (codebook(dim:bits:), :134-147), and the values
// are not exactly symmetric, so packed codes only match the reference's when the very same
// numbers set the boundaries.
struct ShippedCentroids {
    int dim, bits;
    float c[16];
};
const ShippedCentroids kShippedCentroids[] = {
    {64, 2, {-0.18745463f, -0.05649366f, 0.05649367f, 0.18745449f}},
    {64, 3, {-0.26375133f, -0.16599470f, -0.09368263f, -0.03040462f, 0.03040464f, 0.09368261f, 0.16599482f, 0.26375186f}},
    {64, 4, {-0.32913971f, -0.25096416f, -0.19681059f, -0.15295772f, -0.11478586f, -0.08000945f, -0.04726735f, -0.01563822f, 0.01563822f, 0.04723797f, 0.07994876f, 0.11472529f, 0.15289739f, 0.19675052f, 0.25090477f, 0.32908401f}},
    {128, 2, {-0.13302007f, -0.03998107f, 0.03998102f, 0.13302033f}},
    {128, 3, {-0.18828832f, -0.11801215f, -0.06648001f, -0.02156330f, 0.02156329f, 0.06648005f, 0.11801218f, 0.18828897f}},
    {128, 4, {-0.23639172f, -0.17934021f, -0.14023653f, -0.10881814f, -0.08157559f, -0.05678632f, -0.03350975f, -0.01108178f, 0.01108178f, 0.03350975f, 0.05678631f, 0.08157560f, 0.10881804f, 0.14023650f, 0.17934017f, 0.23639278f}},
    {256, 2, {-0.09420358f, -0.02827190f, 0.02827190f, 0.09420330f}},
    {256, 3, {-0.13371243f, -0.08361249f, -0.04704370f, -0.01524900f, 0.01524901f, 0.04704368f, 0.08361248f, 0.13371260f}},
    {256, 4, {-0.16852295f, -0.12754069f, -0.09961203f, -0.07719406f, -0.05781249f, -0.04021866f, -0.02370371f, -0.00783269f, 0.00783269f, 0.02370371f, 0.04021868f, 0.05781246f, 0.07719407f, 0.09961203f, 0.12754090f, 0.16852276f}},
};
}  // namespace

void turbo_codebook(int dim, int bits, std::vector<float> &centroids, std::vector<float> &bounds) {
    const int levels = 1 << bits;
    centroids.assign(levels, 0.0f);
    bool found = false;
    for (const ShippedCentroids &e : kShippedCentroids)
        if (e.dim == dim && e.bits == bits) {
            for (int k = 0; k < levels; ++k) centroids[k] = e.c[k];
            found = true;
        }
    if (!found) {
        // Any other pair: the Lloyd-Max quantiser for one coordinate of a random unit vector in
        // R^dim (density proportional to (1 - x^2)^((dim-3)/2) on [-1, 1]) by weighted k-means on
        // a 32768-point grid, 100 sweeps from a quantile start, in single precision and in the
        // order of operations of TurboQuantCodebook.generateCentroids (TurboQuantKVCache.swift:174-233),
        // so that the same host produces the same floats.
        const int grid_n = 32768;
        std::vector<float> grid(grid_n), w(grid_n);
        const float expo = (float)(dim - 3) / 2.0f;
        float total = 0.0f;
        for (int i = 0; i < grid_n; ++i) {
            const float x = -1.0f + 2.0f * (float)i / (float)(grid_n - 1);
            grid[i] = x;
            w[i] = std::pow(std::max(1.0f - x * x, 1e-30f), expo);
            total += w[i];
        }
        std::vector<float> cen(levels, 0.0f);
        int filled = 0;
        float cum = 0.0f;
        for (int i = 0; i < grid_n; ++i) {
            cum += w[i];
            if (filled < levels && cum >= ((float)filled + 0.5f) / (float)levels * total) cen[filled++] = grid[i];
        }
        const float sigma = 1.0f / std::sqrt((float)dim);
        for (; filled < levels; ++filled) cen[filled] = (filled ? cen[filled - 1] : 0.0f) + sigma;
        std::vector<float> sums(levels), cnt(levels);
        for (int it = 0; it < 100; ++it) {
            std::fill(sums.begin(), sums.end(), 0.0f);
            std::fill(cnt.begin(), cnt.end(), 0.0f);
            for (int i = 0; i < grid_n; ++i) {
                int best = 0;
                float best_d = std::numeric_limits<float>::infinity();
                for (int j = 0; j < levels; ++j) {
                    const float d = std::fabs(grid[i] - cen[j]);
                    if (d < best_d) { best_d = d; best = j; }
                }
                sums[best] += grid[i] * w[i];
                cnt[best] += w[i];
            }
            for (int j = 0; j < levels; ++j)
                if (cnt[j] > 0.0f) cen[j] = sums[j] / cnt[j];
        }
        std::sort(cen.begin(), cen.end());
        centroids = cen;
    }
    bounds.resize(levels - 1);
    for (int k = 0; k + 1 < levels; ++k) bounds[k] = (centroids[k] + centroids[k + 1]) / 2.0f;
}

void turbo_signs(int dim, uint64_t seed, std::vector<float> &signs) {
    // The reference draws the signs from MLXRandom (TurboQuantKVCache.swift:289-298),
    // whose stream is not reproducible outside MLX. This library defines its own:
    // splitmix64 seeded with `seed`, one draw per dimension, top bit set -> +1.
    signs.resize(dim);
    uint64_t x = seed;
    for (int i = 0; i < dim; ++i) {
        x += 0x9E3779B97F4A7C15ull;
        uint64_t z = x;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        z = z ^ (z >> 31);
        signs[i] = (z >> 63) ? 1.0f : -1.0f;
    }
}

}  // namespace kvc
