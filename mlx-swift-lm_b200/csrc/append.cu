// Cache row movement: linear append, ring scatter and the segment gather the
// rotating cache uses for temporal re-ordering, front trims and logical views.
// All of it is pure data movement (bit-exact by construction) and HBM-bound:
// one thread moves one 16-byte vector, consecutive threads touch consecutive
// vectors of a row, K and V travel in the same launch.
#include "common.h"

namespace kvc {

namespace {

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename V>
__global__ void append_kernel(AppendArgs a, int64_t k_units, int64_t total_units,
                              int k_upr, int v_upr /* units per row */) {
    // lets a dependent kernel launched with programmatic serialization begin its prologue now
    asm volatile("griddepcontrol.launch_dependents;");
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total_units) return;
    const bool is_v = i >= k_units;
    if (is_v) i -= k_units;
    const int upr = is_v ? v_upr : k_upr;
    const int u = (int)(i % upr);
    int64_t row = i / upr;
    const int s = (int)(row % a.S);
    row /= a.S;
    const int h = (int)(row % a.H);
    const int b = (int)(row / a.H);
    constexpr int VB = sizeof(V);
    if (!is_v) {
        const char *src = (const char *)a.k_src +
                          (b * a.ks_sb + h * a.ks_sh + s * a.ks_ss) * (int64_t)a.esize + (int64_t)u * VB;
        char *dst = (char *)a.k_dst +
                    (b * a.kd_sb + h * a.kd_sh + (a.pos + s) * a.kd_st) * (int64_t)a.esize + (int64_t)u * VB;
        *(V *)dst = *(const V *)src;
    } else {
        const char *src = (const char *)a.v_src +
                          (b * a.vs_sb + h * a.vs_sh + s * a.vs_ss) * (int64_t)a.esize + (int64_t)u * VB;
        char *dst = (char *)a.v_dst +
                    (b * a.vd_sb + h * a.vd_sh + (a.pos + s) * a.vd_st) * (int64_t)a.esize + (int64_t)u * VB;
        *(V *)dst = *(const V *)src;
    }
}

// Element-wise fallback for sources whose inner stride is not 1 or whose rows
// are not 16-byte aligned.
template <typename E>
__global__ void append_strided_kernel(AppendArgs a, int64_t k_elems, int64_t total) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const bool is_v = i >= k_elems;
    if (is_v) i -= k_elems;
    const int D = is_v ? a.Dv : a.Dk;
    const int d = (int)(i % D);
    int64_t row = i / D;
    const int s = (int)(row % a.S);
    row /= a.S;
    const int h = (int)(row % a.H);
    const int b = (int)(row / a.H);
    if (!is_v) {
        const E *src = (const E *)a.k_src + b * a.ks_sb + h * a.ks_sh + s * a.ks_ss + d * a.ks_sd;
        E *dst = (E *)a.k_dst + b * a.kd_sb + h * a.kd_sh + (a.pos + s) * a.kd_st + d;
        *dst = *src;
    } else {
        const E *src = (const E *)a.v_src + b * a.vs_sb + h * a.vs_sh + s * a.vs_ss + d * a.vs_sd;
        E *dst = (E *)a.v_dst + b * a.vd_sb + h * a.vd_sh + (a.pos + s) * a.vd_st + d;
        *dst = *src;
    }
}

// Rotary positions for queries and keys in one launch (applyRotaryPosition,
// MLXLMCommon/RoPEApplication.swift:58-69; the rotation itself is MLX's published RoPE: pair i of a
// head at position p turns by p * scale * base^(-2i/dims)). One thread per (row, pair); features past
// `dims` are copied. Arithmetic in float32, results rounded to the element type.
template <typename T>
__global__ void rope_kernel(RopeArgs a, int64_t q_items, int64_t total_items) {
    asm volatile("griddepcontrol.launch_dependents;");
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total_items) return;
    const bool is_k = i >= q_items;
    if (is_k) i -= q_items;
    const RopeTensor &t = is_k ? a.k : a.q;
    const int half = a.D / 2;            // items per row: D / 2 (rotated pairs first, then pass-through pairs)
    const int p = (int)(i % half);
    int64_t row = i / half;
    const int l = (int)(row % t.L);
    row /= t.L;
    const int h = (int)(row % t.H);
    const int b = (int)(row / t.H);
    const T *src = (const T *)t.src + b * t.s_sb + h * t.s_sh + l * t.s_sl;
    T *dst = (T *)t.dst + b * t.d_sb + h * t.d_sh + l * t.d_sl;
    const int rp = a.dims / 2;           // rotated pairs
    if (p < rp) {
        const int i0 = a.traditional ? 2 * p : p, i1 = a.traditional ? 2 * p + 1 : p + rp;
        const float x0 = to_float<T>(src[i0]), x1 = to_float<T>(src[i1]);
        // the frequency in double precision, rounded once: at positions in the tens of thousands a float32
        // exp2 would already move the angle by 1e-3
        const float inv_freq = (float)exp2(-(double)p * a.log2_base_over_half);
        const float theta = __fmul_rn(__fmul_rn((float)(a.offset + l), a.scale), inv_freq);
        float sn, cs;
        sincosf(theta, &sn, &cs);
        dst[i0] = from_float<T>(x0 * cs - x1 * sn);
        dst[i1] = from_float<T>(x0 * sn + x1 * cs);
    } else {
        // the features past `dims`, two per item
        const int j = a.dims + 2 * (p - rp);
        dst[j] = src[j];
        if (j + 1 < a.D) dst[j + 1] = src[j + 1];
    }
}

template <typename V>
__global__ void gather_kernel(GatherArgs a, int64_t total_units, int upr, int64_t rows_per_bh) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total_units) return;
    const int u = (int)(i % upr);
    int64_t row = i / upr;
    int64_t j = row % rows_per_bh;
    row /= rows_per_bh;
    const int h = (int)(row % a.H);
    const int b = (int)(row / a.H);
    // Map destination-relative row j to its source token.
    int64_t src_t = -1;
    int64_t rem = j;
#pragma unroll
    for (int sgi = 0; sgi < 4; ++sgi) {
        if (sgi < a.nseg && src_t < 0) {
            if (rem < a.seg[sgi].count) src_t = a.seg[sgi].src_start + rem;
            else rem -= a.seg[sgi].count;
        }
    }
    if (src_t < 0) return;
    constexpr int VB = sizeof(V);
    const char *src = (const char *)a.src +
                      (b * a.s_sb + h * a.s_sh + src_t * a.s_st) * (int64_t)a.esize + (int64_t)u * VB;
    char *dst = (char *)a.dst +
                (b * a.d_sb + h * a.d_sh + (a.dst_start + j) * a.d_st) * (int64_t)a.esize + (int64_t)u * VB;
    *(V *)dst = *(const V *)src;
}

__global__ void causal_mask_kernel(uint8_t *out, int64_t n, int64_t offset, int64_t window) {
    // createCausalMask (KVCache.swift:253-275): rows are absolute positions
    // offset..offset+n-1, columns 0..offset+n-1; keep when row >= col and,
    // with a window, row < col + window.
    const int64_t cols = offset + n;
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n * cols) return;
    const int64_t r = offset + i / cols;
    const int64_t c = i % cols;
    bool keep = r >= c;
    if (window >= 0) keep = keep && (r < c + window);
    out[i] = keep ? 1 : 0;
}

// The same mask per batch entry with prepared lengths: entry b also requires col < lengths[b]
// (createCausalMask's `lengths` argument, KVCache.swift:268-271). out: [batch, 1, n, offset + n].
__global__ void causal_mask_lengths_kernel(uint8_t *out, int64_t n, int64_t offset, int64_t window,
                                           const int32_t *lengths, int64_t total) {
    const int64_t cols = offset + n;
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int64_t b = i / (n * cols), j = i % (n * cols);
    const int64_t r = offset + j / cols;
    const int64_t c = j % cols;
    bool keep = r >= c;
    if (window >= 0) keep = keep && (r < c + window);
    keep = keep && (c < (int64_t)lengths[b]);
    out[i] = keep ? 1 : 0;
}

__global__ void rolled_mask_kernel(uint8_t *out, int64_t size, int64_t window, int64_t shift) {
    // RotatingKVCache.makeMask single-token branch (KVCache.swift:861-865):
    // mask[i] = i >= size - window, rolled right by `shift`.
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= size) return;
    int64_t srci = ((i - shift) % size + size) % size;
    out[i] = (srci >= size - window) ? 1 : 0;
}

bool aligned16(const void *p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace

void launch_append(const AppendArgs &a, cudaStream_t stream) {
    if (a.B <= 0 || a.H <= 0 || a.S <= 0) return;
    const int64_t rows = (int64_t)a.B * a.H * a.S;
    const int64_t kb = (int64_t)a.Dk * a.esize, vb = (int64_t)a.Dv * a.esize;
    auto stride_ok = [&](int64_t s) { return (s * a.esize) % 16 == 0; };
    const bool vec = a.ks_sd == 1 && a.vs_sd == 1 && kb % 16 == 0 && vb % 16 == 0 &&
                     aligned16(a.k_src) && aligned16(a.v_src) && aligned16(a.k_dst) &&
                     aligned16(a.v_dst) && stride_ok(a.ks_sb) && stride_ok(a.ks_sh) &&
                     stride_ok(a.ks_ss) && stride_ok(a.vs_sb) && stride_ok(a.vs_sh) &&
                     stride_ok(a.vs_ss) && stride_ok(a.kd_sb) && stride_ok(a.kd_sh) &&
                     stride_ok(a.kd_st) && stride_ok(a.vd_sb) && stride_ok(a.vd_sh) &&
                     stride_ok(a.vd_st);
    const int threads = 256;
    if (vec) {
        const int k_upr = (int)(kb / 16), v_upr = (int)(vb / 16);
        const int64_t k_units = rows * k_upr, total = k_units + rows * v_upr;
        const int64_t blocks = (total + threads - 1) / threads;
        append_kernel<uint4><<<(unsigned)blocks, threads, 0, stream>>>(a, k_units, total, k_upr, v_upr);
    } else {
        const int64_t k_elems = rows * a.Dk, total = k_elems + rows * a.Dv;
        const int64_t blocks = (total + threads - 1) / threads;
        if (a.esize == 2)
            append_strided_kernel<uint16_t><<<(unsigned)blocks, threads, 0, stream>>>(a, k_elems, total);
        else if (a.esize == 4)
            append_strided_kernel<uint32_t><<<(unsigned)blocks, threads, 0, stream>>>(a, k_elems, total);
        else
            fail(KVC_ERR_INVALID_ARG, "append: unsupported element size");
    }
    KVC_CUDA(cudaGetLastError());
    ++g_launch_count;
}

void launch_gather(const GatherArgs &a, cudaStream_t stream) {
    int64_t rows_per_bh = 0;
    for (int i = 0; i < a.nseg; ++i) rows_per_bh += a.seg[i].count;
    if (rows_per_bh <= 0 || a.B <= 0 || a.H <= 0) return;
    const int64_t rb = (int64_t)a.W * a.esize;
    auto stride_ok = [&](int64_t s) { return (s * a.esize) % 16 == 0; };
    const bool vec = rb % 16 == 0 && aligned16(a.src) && aligned16(a.dst) && stride_ok(a.s_sb) &&
                     stride_ok(a.s_sh) && stride_ok(a.s_st) && stride_ok(a.d_sb) &&
                     stride_ok(a.d_sh) && stride_ok(a.d_st);
    const int threads = 256;
    const int64_t rows = (int64_t)a.B * a.H * rows_per_bh;
    if (vec) {
        const int upr = (int)(rb / 16);
        const int64_t total = rows * upr;
        gather_kernel<uint4><<<(unsigned)((total + threads - 1) / threads), threads, 0, stream>>>(
            a, total, upr, rows_per_bh);
    } else if (rb % 4 == 0 && ((uintptr_t)a.src & 3) == 0 && ((uintptr_t)a.dst & 3) == 0 &&
               (a.esize == 4 || (a.s_sb % 2 == 0 && a.s_sh % 2 == 0 && a.s_st % 2 == 0 &&
                                 a.d_sb % 2 == 0 && a.d_sh % 2 == 0 && a.d_st % 2 == 0))) {
        const int upr = (int)(rb / 4);
        const int64_t total = rows * upr;
        gather_kernel<uint32_t><<<(unsigned)((total + threads - 1) / threads), threads, 0, stream>>>(
            a, total, upr, rows_per_bh);
    } else if (a.esize == 2) {
        const int upr = (int)(rb / 2);
        const int64_t total = rows * upr;
        gather_kernel<uint16_t><<<(unsigned)((total + threads - 1) / threads), threads, 0, stream>>>(
            a, total, upr, rows_per_bh);
    } else {
        fail(KVC_ERR_INVALID_ARG, "gather: unsupported row layout");
    }
    KVC_CUDA(cudaGetLastError());
    ++g_launch_count;
}

void launch_rope(const RopeArgs &a, cudaStream_t s) {
    KVC_REQUIRE(a.dims >= 2 && a.dims % 2 == 0 && a.dims <= a.D && a.D % 2 == 0, "rope: dims must be even and at most the head dim");
    const int half = a.D / 2;
    const int64_t q_items = a.q.src ? (int64_t)a.q.B * a.q.H * a.q.L * half : 0;
    const int64_t k_items = a.k.src ? (int64_t)a.k.B * a.k.H * a.k.L * half : 0;
    const int64_t total = q_items + k_items;
    if (total <= 0) return;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    switch (a.dtype) {
        case KVC_F32: rope_kernel<float><<<blocks, 256, 0, s>>>(a, q_items, total); break;
        case KVC_F16: rope_kernel<__half><<<blocks, 256, 0, s>>>(a, q_items, total); break;
        case KVC_BF16: rope_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(a, q_items, total); break;
        default: fail(KVC_ERR_INVALID_ARG, "rope needs a floating dtype");
    }
    KVC_CUDA(cudaGetLastError());
    ++g_launch_count;
}

void launch_causal_mask(uint8_t *out, int64_t n, int64_t offset, int64_t window, cudaStream_t s) {
    const int64_t total = n * (offset + n);
    if (total <= 0) return;
    causal_mask_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(out, n, offset, window);
    KVC_CUDA(cudaGetLastError());
    ++g_launch_count;
}

void launch_causal_mask_lengths(uint8_t *out, int64_t n, int64_t offset, int64_t window, const int32_t *lengths,
                                int64_t batch, cudaStream_t s) {
    const int64_t total = batch * n * (offset + n);
    if (total <= 0) return;
    causal_mask_lengths_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(out, n, offset, window, lengths, total);
    KVC_CUDA(cudaGetLastError());
    ++g_launch_count;
}

void launch_rolled_mask(uint8_t *out, int64_t size, int64_t window, int64_t shift, cudaStream_t s) {
    if (size <= 0) return;
    rolled_mask_kernel<<<(unsigned)((size + 255) / 256), 256, 0, s>>>(out, size, window, shift);
    KVC_CUDA(cudaGetLastError());
    ++g_launch_count;
}

}  // namespace kvc
