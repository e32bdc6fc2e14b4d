// kvc_sdpa_noalloc: scaled-dot-product attention over raw K/V that never
// allocates.
//
// Who needs this: hosts that must not call into the CUDA allocator on the
// request path. A serving process that has handed the whole device budget to
// its own pool (MLX's wired-memory policy, a framework allocator that owns all
// of HBM) cannot afford a library that grows a private arena behind its back,
// and cudaMalloc/cudaFree synchronise the whole device, which stalls every
// other stream of a latency-sensitive decoder. The regular entry points keep
// their split-K partials in an arena that is cudaMalloc'ed and grown on
// demand; this variant keeps them in a fixed array that is part of the loaded
// module instead, so the only memory it touches is what the caller passed in
// plus that array.
//
// The array is a file-scope `static __device__` object, KVC_NOALLOC_SCRATCH_BYTES
// large; every GPU that loads this library carries one copy until the process
// exits. Host code cannot use the array's name as an address (on the host the
// name is only a handle for the runtime), so the first call on each device asks
// the runtime for the device address with cudaGetSymbolAddress, with that
// device current, and remembers it; that first call should therefore happen
// outside any stream capture. All calls share the one array: two calls whose
// kernels overlap on the GPU (different streams, no dependency) race on it.
// Nothing in it has to start at zero, because the first kernel writes every
// slot that the second one reads.
#include "common.h"

#include <algorithm>
#include <mutex>

#define KVC_NOALLOC_SCRATCH_BYTES (4u << 20)

extern "C" kvc_status kvc_internal_set_error(kvc_status code, const char *msg);

namespace {

static __device__ __align__(256) unsigned char g_noalloc_scratch[KVC_NOALLOC_SCRATCH_BYTES];

constexpr int NA_THREADS = 128;
constexpr int NA_TILE = 32;
constexpr int NA_ROWS = 8;

struct NoAllocArgs {
    const void *q, *k, *v;
    void *out;
    int32_t dtype;
    int64_t q_sb, q_sh, q_sl, o_sb, o_sh, o_sl;
    int64_t k_sb, k_sh, k_st, v_sb, v_sh, v_st;
    int32_t B, Hq, Hkv, L, D;
    int64_t T;
    float scale;
    int32_t causal;
    int64_t causal_offset;
    int32_t splits;
    int64_t tokens_per_split;
    int32_t row_chunks;
};

__device__ __forceinline__ float na_ld(const void *p, int32_t dtype, int64_t i) {
    switch (dtype) {
        case KVC_F32: return ((const float *)p)[i];
        case KVC_F16: return __half2float(((const __half *)p)[i]);
        default: return __bfloat162float(((const __nv_bfloat16 *)p)[i]);
    }
}

__device__ __forceinline__ void na_st(void *p, int32_t dtype, int64_t i, float v) {
    switch (dtype) {
        case KVC_F32: ((float *)p)[i] = v; break;
        case KVC_F16: ((__half *)p)[i] = __float2half_rn(v); break;
        default: ((__nv_bfloat16 *)p)[i] = __float2bfloat16_rn(v); break;
    }
}

// One CTA per (token split, KV head x row chunk, batch): fp32 tiles of K and V in
// shared memory, online softmax per query row, un-normalised partial written to
// `scratch` (layout: [query row][split][D] floats, then [query row][split] (m, l)).
__global__ void __launch_bounds__(NA_THREADS)
noalloc_partial_kernel(const NoAllocArgs a, unsigned char *scratch, size_t ml_offset) {
    extern __shared__ float na_smem[];
    const int D = a.D, KS = D + 1;
    float *Qs = na_smem;
    float *Ks = Qs + NA_ROWS * D;
    float *Vs = Ks + NA_TILE * KS;
    float *Ps = Vs + NA_TILE * KS;
    float *row_m = Ps + NA_ROWS * NA_TILE;
    float *row_l = row_m + NA_ROWS;
    float *row_alpha = row_l + NA_ROWS;
    float *o_part = (float *)scratch;
    float2 *ml_part = (float2 *)(scratch + ml_offset);

    const int tid = threadIdx.x;
    const int split = blockIdx.x;
    const int hk = blockIdx.y / a.row_chunks, rc = blockIdx.y % a.row_chunks;
    const int b = blockIdx.z;
    const int rep = a.Hq / a.Hkv;
    const int row0 = rc * NA_ROWS;
    const int nrows = min(NA_ROWS, rep * a.L - row0);

    if (tid < NA_ROWS) {
        row_m[tid] = -INFINITY;
        row_l[tid] = 0.f;
        row_alpha[tid] = 1.f;
    }
    for (int i = tid; i < NA_ROWS * D; i += NA_THREADS) {
        const int r = i / D, d = i % D;
        float qv = 0.f;
        if (r < nrows) {
            const int ri = row0 + r;
            const int hq = hk * rep + ri / a.L, l = ri % a.L;
            qv = na_ld(a.q, a.dtype, b * a.q_sb + hq * a.q_sh + l * a.q_sl + d) * a.scale;
        }
        Qs[i] = qv;
    }
    __syncthreads();

    const int64_t t_begin = (int64_t)split * a.tokens_per_split;
    const int64_t t_end = min(a.T, t_begin + a.tokens_per_split);
    float acc[NA_ROWS][2];
#pragma unroll
    for (int r = 0; r < NA_ROWS; ++r) acc[r][0] = acc[r][1] = 0.f;

    for (int64_t t0 = t_begin; t0 < t_end; t0 += NA_TILE) {
        const int nt = (int)min((int64_t)NA_TILE, t_end - t0);
        for (int i = tid; i < NA_TILE * D; i += NA_THREADS) {
            const int tt = i / D, d = i % D;
            float kv = 0.f, vv = 0.f;
            if (tt < nt) {
                kv = na_ld(a.k, a.dtype, b * a.k_sb + hk * a.k_sh + (t0 + tt) * a.k_st + d);
                vv = na_ld(a.v, a.dtype, b * a.v_sb + hk * a.v_sh + (t0 + tt) * a.v_st + d);
            }
            Ks[tt * KS + d] = kv;
            Vs[tt * KS + d] = vv;
        }
        __syncthreads();
        {
            const int tt = tid & 31, r0 = tid >> 5;
            float s0 = 0.f, s1 = 0.f;
            for (int d = 0; d < D; ++d) {
                const float kv = Ks[tt * KS + d];
                s0 = fmaf(Qs[r0 * D + d], kv, s0);
                s1 = fmaf(Qs[(r0 + 4) * D + d], kv, s1);
            }
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const int r = r0 + 4 * k;
                float sc = k ? s1 : s0;
                bool keep = r < nrows && tt < nt;
                if (keep && a.causal) keep = (t0 + tt) <= a.causal_offset + (row0 + r) % a.L;
                Ps[r * NA_TILE + tt] = keep ? sc : -INFINITY;
            }
        }
        __syncthreads();
        {
            const int lane = tid & 31, w = tid >> 5;
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const int r = w + 4 * k;
                const float sc = Ps[r * NA_TILE + lane];
                float mx = sc;
#pragma unroll
                for (int o = 16; o >= 1; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                const float m_old = row_m[r], m_new = fmaxf(m_old, mx);
                float p = 0.f, alpha = 1.f;
                if (m_new != -INFINITY) {
                    p = expf(sc - m_new);
                    alpha = expf(m_old - m_new);
                }
                float sum = p;
#pragma unroll
                for (int o = 16; o >= 1; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
                Ps[r * NA_TILE + lane] = p;
                __syncwarp();
                if (lane == 0) {
                    row_m[r] = m_new;
                    row_l[r] = row_l[r] * alpha + sum;
                    row_alpha[r] = alpha;
                }
            }
        }
        __syncthreads();
#pragma unroll
        for (int dd = 0; dd < 2; ++dd) {
            const int d = tid + dd * NA_THREADS;
            if (d < D) {
#pragma unroll
                for (int r = 0; r < NA_ROWS; ++r) acc[r][dd] *= row_alpha[r];
                for (int tt = 0; tt < nt; ++tt) {
                    const float vv = Vs[tt * KS + d];
#pragma unroll
                    for (int r = 0; r < NA_ROWS; ++r) acc[r][dd] = fmaf(Ps[r * NA_TILE + tt], vv, acc[r][dd]);
                }
            }
        }
        __syncthreads();
    }
    for (int r = 0; r < nrows; ++r) {
        const int ri = row0 + r;
        const int hq = hk * rep + ri / a.L, l = ri % a.L;
        const int64_t base = (((int64_t)b * a.Hq + hq) * a.L + l) * a.splits + split;
#pragma unroll
        for (int dd = 0; dd < 2; ++dd) {
            const int d = tid + dd * NA_THREADS;
            if (d < D) o_part[base * D + d] = acc[r][dd];
        }
        if (tid == 0) ml_part[base] = make_float2(row_m[r], row_l[r]);
    }
}

__global__ void noalloc_merge_kernel(const NoAllocArgs a, const unsigned char *scratch, size_t ml_offset) {
    const float *o_part = (const float *)scratch;
    const float2 *ml_part = (const float2 *)(scratch + ml_offset);
    const int64_t qrow = blockIdx.x;
    const int l = (int)(qrow % a.L);
    const int hq = (int)((qrow / a.L) % a.Hq);
    const int b = (int)(qrow / ((int64_t)a.L * a.Hq));
    float m = -INFINITY;
    for (int s = 0; s < a.splits; ++s) m = fmaxf(m, ml_part[qrow * a.splits + s].x);
    float lsum = 0.f;
    for (int s = 0; s < a.splits; ++s) {
        const float2 ml = ml_part[qrow * a.splits + s];
        if (ml.y > 0.f && ml.x != -INFINITY) lsum += ml.y * expf(ml.x - m);
    }
    const float inv_l = lsum > 0.f ? 1.f / lsum : 0.f;
    for (int d = threadIdx.x; d < a.D; d += blockDim.x) {
        float o = 0.f;
        for (int s = 0; s < a.splits; ++s) {
            const float2 ml = ml_part[qrow * a.splits + s];
            if (ml.y > 0.f && ml.x != -INFINITY)
                o = fmaf(o_part[(qrow * a.splits + s) * a.D + d], expf(ml.x - m), o);
        }
        na_st(a.out, a.dtype, b * a.o_sb + hq * a.o_sh + l * a.o_sl + d, o * inv_l);
    }
}

// Device address of the static array, looked up once per device.
unsigned char *noalloc_scratch_address(int device) {
    static std::mutex mu;
    static unsigned char *ptrs[64] = {nullptr};
    static bool attr_done[64] = {false};
    if (device < 0 || device >= 64) kvc::fail(KVC_ERR_INVALID_ARG, "kvc_sdpa_noalloc: device ordinal out of range");
    std::lock_guard<std::mutex> lock(mu);
    if (!ptrs[device]) {
        unsigned char *ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void **)&ptr, g_noalloc_scratch);
        if (e != cudaSuccess || !ptr) {
            (void)cudaGetLastError();
            kvc::fail(KVC_ERR_CUDA, std::string("kvc_sdpa_noalloc: cudaGetSymbolAddress failed: ") +
                                        cudaGetErrorString(e));
        }
        ptrs[device] = ptr;
    }
    if (!attr_done[device]) {
        cudaError_t e = cudaFuncSetAttribute(noalloc_partial_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             100 * 1024);
        if (e != cudaSuccess) {
            (void)cudaGetLastError();
            kvc::fail(KVC_ERR_CUDA, std::string("kvc_sdpa_noalloc: cudaFuncSetAttribute failed: ") +
                                        cudaGetErrorString(e));
        }
        attr_done[device] = true;
    }
    return ptrs[device];
}

}  // namespace

extern "C" kvc_status kvc_sdpa_noalloc(const kvc_tensor *q, const kvc_tensor *k, const kvc_tensor *v,
                                       float scale, int32_t mask_mode, const kvc_tensor *out, void *stream) {
    if (!q || !k || !v || !out) return kvc_internal_set_error(KVC_ERR_INVALID_ARG, "kvc_sdpa_noalloc: null tensor");
    try {
        KVC_REQUIRE(q->ndim == 4 && k->ndim == 4 && v->ndim == 4 && out->ndim == 4,
                    "kvc_sdpa_noalloc: tensors must be 4-d ([B, H, L or T, D])");
        KVC_REQUIRE(kvc::is_float_dtype(q->dtype) && k->dtype == q->dtype && v->dtype == q->dtype &&
                        out->dtype == q->dtype,
                    "kvc_sdpa_noalloc: q, k, v and out must share one floating dtype");
        KVC_REQUIRE(q->stride[3] == 1 && k->stride[3] == 1 && v->stride[3] == 1 && out->stride[3] == 1,
                    "kvc_sdpa_noalloc: tensors must be contiguous along the head dim");
        KVC_REQUIRE(mask_mode == KVC_MASK_NONE || mask_mode == KVC_MASK_CAUSAL,
                    "kvc_sdpa_noalloc: only the none and causal mask modes are available");
        for (int i = 0; i < 4; ++i) KVC_REQUIRE(q->shape[i] == out->shape[i], "kvc_sdpa_noalloc: out shape differs from q");
        NoAllocArgs a;
        a.q = q->data; a.k = k->data; a.v = v->data; a.out = out->data; a.dtype = q->dtype;
        a.q_sb = q->stride[0]; a.q_sh = q->stride[1]; a.q_sl = q->stride[2];
        a.o_sb = out->stride[0]; a.o_sh = out->stride[1]; a.o_sl = out->stride[2];
        a.k_sb = k->stride[0]; a.k_sh = k->stride[1]; a.k_st = k->stride[2];
        a.v_sb = v->stride[0]; a.v_sh = v->stride[1]; a.v_st = v->stride[2];
        a.B = (int)q->shape[0]; a.Hq = (int)q->shape[1]; a.L = (int)q->shape[2]; a.D = (int)q->shape[3];
        a.Hkv = (int)k->shape[1]; a.T = k->shape[2];
        KVC_REQUIRE(k->shape[0] == a.B && v->shape[0] == a.B && v->shape[1] == a.Hkv && v->shape[2] == a.T &&
                        k->shape[3] == a.D && v->shape[3] == a.D,
                    "kvc_sdpa_noalloc: key/value shapes do not match the queries");
        KVC_REQUIRE(a.Hkv > 0 && a.Hq % a.Hkv == 0, "kvc_sdpa_noalloc: Hq must be a multiple of Hkv");
        KVC_REQUIRE(a.D >= 1 && a.D <= 2 * NA_THREADS, "kvc_sdpa_noalloc: head dim must be in [1, 256]");
        a.scale = scale;
        a.causal = mask_mode == KVC_MASK_CAUSAL ? 1 : 0;
        a.causal_offset = a.T - a.L;
        const int64_t qrows = (int64_t)a.B * a.Hq * a.L;
        if (qrows == 0) return KVC_OK;

        // split the token axis as far as the fixed scratch allows
        const size_t per_split = (size_t)qrows * ((size_t)a.D * sizeof(float) + sizeof(float2)) + 256;
        if (per_split > KVC_NOALLOC_SCRATCH_BYTES) {
            return kvc_internal_set_error(
                KVC_ERR_INVALID_ARG,
                "kvc_sdpa_noalloc: B*Hq*L*(4*D+8) bytes of partials exceed the static scratch "
                "(KVC_NOALLOC_SCRATCH_BYTES = 4 MiB); use kvc_sdpa for larger calls");
        }
        const int rep = a.Hq / a.Hkv;
        a.row_chunks = (rep * a.L + NA_ROWS - 1) / NA_ROWS;
        const int64_t tiles = std::max<int64_t>(1, (a.T + NA_TILE - 1) / NA_TILE);
        int device = 0;
        KVC_CUDA(cudaGetDevice(&device));
        int sms = 0;
        KVC_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
        const int64_t base_ctas = (int64_t)a.B * a.Hkv * a.row_chunks;
        int64_t splits = std::max<int64_t>(1, std::min<int64_t>((4LL * sms + base_ctas - 1) / base_ctas, tiles));
        splits = std::min<int64_t>(splits, (int64_t)(KVC_NOALLOC_SCRATCH_BYTES / per_split));
        splits = std::max<int64_t>(1, std::min<int64_t>(splits, 128));
        const int64_t tiles_per_split = (tiles + splits - 1) / splits;
        splits = (tiles + tiles_per_split - 1) / tiles_per_split;
        a.splits = (int)splits;
        a.tokens_per_split = tiles_per_split * NA_TILE;
        KVC_REQUIRE(a.Hkv * a.row_chunks <= 65535 && a.B <= 65535, "kvc_sdpa_noalloc: grid too large");

        unsigned char *scratch = noalloc_scratch_address(device);
        const size_t o_bytes = (size_t)qrows * splits * a.D * sizeof(float);
        const size_t ml_offset = (o_bytes + 255) / 256 * 256;
        const size_t smem = (size_t)(NA_ROWS * a.D + 2 * NA_TILE * (a.D + 1) + NA_ROWS * NA_TILE + 3 * NA_ROWS) *
                            sizeof(float);
        cudaStream_t s = (cudaStream_t)stream;
        dim3 grid((unsigned)splits, (unsigned)(a.Hkv * a.row_chunks), (unsigned)a.B);
        noalloc_partial_kernel<<<grid, NA_THREADS, smem, s>>>(a, scratch, ml_offset);
        KVC_CUDA(cudaGetLastError());
        const int threads = std::min(256, std::max(32, ((a.D + 31) / 32) * 32));
        noalloc_merge_kernel<<<(unsigned)qrows, threads, 0, s>>>(a, scratch, ml_offset);
        KVC_CUDA(cudaGetLastError());
        kvc::g_launch_count += 2;
        return KVC_OK;
    } catch (const kvc::Error &e) {
        return kvc_internal_set_error(e.code, e.what());
    }
}
