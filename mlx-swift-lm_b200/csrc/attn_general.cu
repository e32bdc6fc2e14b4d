// General split-K flash attention over any cache representation.
//
// This is the path that accepts every combination the library exposes: raw
// f32/f16/bf16 rows, affine-packed rows (2/4/8 bit), TurboQuant codebook rows,
// mixed K/V representations, any head dim, explicit boolean or additive masks,
// multi-token query chunks. A CTA owns one (batch, KV head, query-row chunk,
// token split): it stages a tile of K and V as fp32 in shared memory
// (dequantising on the way), scores the GQA group's query rows against it,
// keeps an online softmax per row and writes un-normalised partials that the
// merge kernel combines with a log-sum-exp reduction. The specialised decode
// kernels (attn_decode.cu) take over for the shapes the benchmarks run; this
// one is the reference point they are tested against on the device.
#include "common.h"

#include <algorithm>
#include <cmath>

namespace kvc {

namespace {

constexpr int G_THREADS = 128;
constexpr int G_TILE = 32;  // tokens per tile (one per lane in the score phase)
constexpr int G_RC = 8;     // query rows per CTA

__device__ __forceinline__ float ld_elem(const void *p, int32_t dtype, int64_t i) {
    switch (dtype) {
        case KVC_F32: return ((const float *)p)[i];
        case KVC_F16: return __half2float(((const __half *)p)[i]);
        default: return __bfloat162float(((const __nv_bfloat16 *)p)[i]);
    }
}

__device__ __forceinline__ void st_elem(void *p, int32_t dtype, int64_t i, float v) {
    switch (dtype) {
        case KVC_F32: ((float *)p)[i] = v; break;
        case KVC_F16: ((__half *)p)[i] = __float2half_rn(v); break;
        default: ((__nv_bfloat16 *)p)[i] = __float2bfloat16_rn(v); break;
    }
}

// One element of a cached row, dequantised to fp32.
__device__ __forceinline__ float load_kv(const KVSource &s, const float *cb, int b, int h,
                                         int64_t t, int d) {
    if (s.kind == SRC_RAW) {
        return ld_elem(s.data, s.dtype, b * s.sb + h * s.sh + t * s.st + d);
    } else if (s.kind == SRC_AFFINE) {
        const uint32_t *row = (const uint32_t *)s.data + b * s.sb + h * s.sh + t * s.st;
        const int bit = d * s.bits;
        const uint32_t code = (row[bit >> 5] >> (bit & 31)) & ((1u << s.bits) - 1u);
        const int64_t gi = b * s.gsb + h * s.gsh + t * s.gst + d / s.group;
        const float sc = ld_elem(s.scales, s.dtype, gi);
        const float bi = ld_elem(s.biases, s.dtype, gi);
        return fmaf(sc, (float)code, bi);
    } else {
        const uint32_t *row = (const uint32_t *)s.data + b * s.sb + h * s.sh + t * s.st;
        const int bit = d * s.bits;
        const int w = bit >> 5, sh = bit & 31;
        uint32_t val = row[w] >> sh;
        if (sh + s.bits > 32) val |= row[w + 1] << (32 - sh);
        val &= (1u << s.bits) - 1u;
        return cb[val] * s.norms[b * s.gsb + h * s.gsh + t * s.gst];
    }
}

__device__ __forceinline__ bool mask_allows(const MaskDesc &m, int b, int hq, int l, int64_t t,
                                            float &additive) {
    additive = 0.f;
    if (m.mode == KVC_MASK_NONE) return true;
    if (m.mode == KVC_MASK_CAUSAL) return t <= m.causal_offset + l;
    const int64_t i = b * m.sb + hq * m.sh + l * m.sl + t * m.st;
    if (m.dtype == KVC_BOOL) return ((const uint8_t *)m.data)[i] != 0;
    additive = ld_elem(m.data, m.dtype, i);
    return true;
}

// In-place unnormalised Walsh-Hadamard transform of `rows` rows of length D in
// shared memory (D a power of two).
__device__ void smem_fwht(float *buf, int rows, int D, int stride) {
    for (int half = 1; half < D; half <<= 1) {
        __syncthreads();
        for (int p = threadIdx.x; p < rows * (D / 2); p += blockDim.x) {
            const int r = p / (D / 2), j = p % (D / 2);
            const int i0 = ((j / half) * 2 * half) + (j % half);
            const int i1 = i0 + half;
            const float a = buf[r * stride + i0], c = buf[r * stride + i1];
            buf[r * stride + i0] = a + c;
            buf[r * stride + i1] = a - c;
        }
    }
    __syncthreads();
}

__global__ void __launch_bounds__(G_THREADS)
attn_general_partial(const __grid_constant__ AttnArgs a, float *o_part, float2 *ml_part,
                     int splits, int64_t tokens_per_split, int row_chunks) {
    extern __shared__ float smem[];
    const int D = a.D;
    const int KS = D + 1;
    float *Qs = smem;                       // [G_RC][D]
    float *Ks = Qs + G_RC * D;              // [G_TILE][D+1]
    float *Vs = Ks + G_TILE * KS;           // [G_TILE][D+1]
    float *Ps = Vs + G_TILE * KS;           // [G_RC][G_TILE]
    float *row_m = Ps + G_RC * G_TILE;      // [G_RC]
    float *row_l = row_m + G_RC;            // [G_RC]
    float *row_alpha = row_l + G_RC;        // [G_RC]
    float *kcb = row_alpha + G_RC;          // [16]
    float *vcb = kcb + 16;                  // [16]

    const int tid = threadIdx.x;
    const int split = blockIdx.x;
    const int hk = blockIdx.y / row_chunks;
    const int rc = blockIdx.y % row_chunks;
    const int b = blockIdx.z;
    const int rep = a.Hq / a.Hkv;
    const int rows_total = rep * a.L;
    const int row0 = rc * G_RC;
    const int nrows = min(G_RC, rows_total - row0);

    if (tid < 16) {
        kcb[tid] = a.k.codebook[tid];
        vcb[tid] = a.v.codebook[tid];
    }
    if (tid < G_RC) {
        row_m[tid] = -INFINITY;
        row_l[tid] = 0.f;
        row_alpha[tid] = 1.f;
    }
    // Stage the query rows (fp32). TurboQuant keys are scored in the rotated
    // basis: q' = H(signs * q)/sqrt(D), then the scale (and calibration).
    for (int i = tid; i < G_RC * D; i += G_THREADS) {
        const int r = i / D, d = i % D;
        float qv = 0.f;
        if (r < nrows) {
            const int ri = row0 + r;
            const int hq = hk * rep + ri / a.L, l = ri % a.L;
            qv = ld_elem(a.q, a.q_dtype, b * a.q_sb + hq * a.q_sh + l * a.q_sl + d);
            if (a.q_signs) qv *= a.q_signs[d];
            else if (!a.q_rot) qv *= a.scale;
        }
        Qs[r * D + d] = qv;
    }
    if (a.q_rot) {
        // dense rotation: q'[d] = sum_j Pi[d][j] q[j], then the scale (and calibration); two dims per thread
        __syncthreads();
        float rq[G_RC][2];
#pragma unroll
        for (int r = 0; r < G_RC; ++r) rq[r][0] = rq[r][1] = 0.f;
        for (int dd = 0; dd < 2; ++dd) {
            const int d = tid + dd * G_THREADS;
            if (d >= D) continue;
            const float *rot = a.q_rot + (int64_t)d * D;
            for (int j = 0; j < D; ++j) {
                const float m = rot[j];
#pragma unroll
                for (int r = 0; r < G_RC; ++r) rq[r][dd] = fmaf(m, Qs[r * D + j], rq[r][dd]);
            }
        }
        __syncthreads();
        for (int dd = 0; dd < 2; ++dd) {
            const int d = tid + dd * G_THREADS;
            if (d >= D) continue;
            const float f = a.scale * (a.q_calib ? a.q_calib[d] : 1.f);
#pragma unroll
            for (int r = 0; r < G_RC; ++r) Qs[r * D + d] = rq[r][dd] * f;
        }
    }
    if (a.q_signs) {
        smem_fwht(Qs, G_RC, D, D);
        const float f = rsqrtf((float)D) * a.scale;
        for (int i = tid; i < G_RC * D; i += G_THREADS) {
            float qv = Qs[i] * f;
            if (a.q_calib) qv *= a.q_calib[i % D];
            Qs[i] = qv;
        }
    }
    __syncthreads();

    const int64_t t_begin = (int64_t)split * tokens_per_split;
    const int64_t t_end = min(a.T, t_begin + tokens_per_split);

    // Output accumulators: thread owns dims d = tid, tid + 128 for every row.
    float acc[G_RC][2];
#pragma unroll
    for (int r = 0; r < G_RC; ++r) acc[r][0] = acc[r][1] = 0.f;

    for (int64_t t0 = t_begin; t0 < t_end; t0 += G_TILE) {
        const int nt = (int)min((int64_t)G_TILE, t_end - t0);
        // stage K and V tile
        for (int i = tid; i < G_TILE * D; i += G_THREADS) {
            const int tt = i / D, d = i % D;
            float kv = 0.f, vv = 0.f;
            if (tt < nt) {
                kv = load_kv(a.k, kcb, b, hk, t0 + tt, d);
                vv = load_kv(a.v, vcb, b, hk, t0 + tt, d);
            }
            Ks[tt * KS + d] = kv;
            Vs[tt * KS + d] = vv;
        }
        __syncthreads();
        // scores: thread (r = tid/32 + {0,4}, t = tid%32)
        {
            const int tt = tid & 31;
            const int r0 = tid >> 5;
            float s0 = 0.f, s1 = 0.f;
            const float *kr = Ks + tt * KS;
            const float *q0 = Qs + r0 * D;
            const float *q1 = Qs + (r0 + 4) * D;
            for (int d = 0; d < D; ++d) {
                const float kv = kr[d];
                s0 = fmaf(q0[d], kv, s0);
                s1 = fmaf(q1[d], kv, s1);
            }
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const int r = r0 + 4 * k;
                float sc = k ? s1 : s0;
                if (r < nrows && tt < nt) {
                    const int ri = row0 + r;
                    const int hq = hk * rep + ri / a.L, l = ri % a.L;
                    float add;
                    if (mask_allows(a.mask, b, hq, l, t0 + tt, add)) sc += add;
                    else sc = -INFINITY;
                } else {
                    sc = -INFINITY;
                }
                Ps[r * G_TILE + tt] = sc;
            }
        }
        __syncthreads();
        // online softmax: warp w handles rows w and w+4, one token per lane
        {
            const int lane = tid & 31, w = tid >> 5;
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const int r = w + 4 * k;
                const float sc = Ps[r * G_TILE + lane];
                float mx = sc;
#pragma unroll
                for (int o = 16; o >= 1; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                const float m_old = row_m[r];
                const float m_new = fmaxf(m_old, mx);
                float p = 0.f, alpha = 1.f;
                if (m_new != -INFINITY) {
                    p = expf(sc - m_new);
                    alpha = expf(m_old - m_new);
                }
                float sum = p;
#pragma unroll
                for (int o = 16; o >= 1; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
                Ps[r * G_TILE + lane] = p;
                __syncwarp();
                if (lane == 0) {
                    row_m[r] = m_new;
                    row_l[r] = row_l[r] * alpha + sum;
                    row_alpha[r] = alpha;
                }
            }
        }
        __syncthreads();
        // PV
#pragma unroll
        for (int dd = 0; dd < 2; ++dd) {
            const int d = tid + dd * G_THREADS;
            if (d < D) {
#pragma unroll
                for (int r = 0; r < G_RC; ++r) acc[r][dd] *= row_alpha[r];
                for (int tt = 0; tt < nt; ++tt) {
                    const float vv = Vs[tt * KS + d];
#pragma unroll
                    for (int r = 0; r < G_RC; ++r) acc[r][dd] = fmaf(Ps[r * G_TILE + tt], vv, acc[r][dd]);
                }
            }
        }
        __syncthreads();
    }

    // write partials
    for (int r = 0; r < nrows; ++r) {
        const int ri = row0 + r;
        const int hq = hk * rep + ri / a.L, l = ri % a.L;
        const int64_t qrow = ((int64_t)b * a.Hq + hq) * a.L + l;
        const int64_t base = (qrow * splits + split);
#pragma unroll
        for (int dd = 0; dd < 2; ++dd) {
            const int d = tid + dd * G_THREADS;
            if (d < D) o_part[base * D + d] = acc[r][dd];
        }
        if (tid == 0) ml_part[base] = make_float2(row_m[r], row_l[r]);
    }
}

// Log-sum-exp merge of the split partials; one CTA per query row. With
// `o_signs` the merged vector (still in the rotated basis of TurboQuant values)
// is rotated back: out = signs * H(o) / sqrt(D).
__global__ void attn_merge_kernel(const float *o_part, const float2 *ml_part, int splits, int D,
                                  void *out, int32_t out_dtype, int Hq, int L, int64_t o_sb,
                                  int64_t o_sh, int64_t o_sl, const float *o_signs, const float *o_rot) {
    extern __shared__ float sm[];  // [D] when rotating
    const int64_t qrow = blockIdx.x;
    const int l = (int)(qrow % L);
    const int hq = (int)((qrow / L) % Hq);
    const int b = (int)(qrow / ((int64_t)L * Hq));
    float m = -INFINITY;
    for (int s = 0; s < splits; ++s) m = fmaxf(m, ml_part[qrow * splits + s].x);
    float lsum = 0.f;
    for (int s = 0; s < splits; ++s) {
        const float2 ml = ml_part[qrow * splits + s];
        if (ml.y > 0.f && ml.x != -INFINITY) lsum += ml.y * expf(ml.x - m);
    }
    const float inv_l = lsum > 0.f ? 1.f / lsum : 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float o = 0.f;
        for (int s = 0; s < splits; ++s) {
            const float2 ml = ml_part[qrow * splits + s];
            if (ml.y > 0.f && ml.x != -INFINITY)
                o = fmaf(o_part[(qrow * splits + s) * D + d], expf(ml.x - m), o);
        }
        o *= inv_l;
        if (o_signs || o_rot) sm[d] = o;
        else st_elem(out, out_dtype, b * o_sb + hq * o_sh + l * o_sl + d, o);
    }
    if (o_rot) {
        // dense inverse rotation: out[j] = sum_d o'[d] Pi[d][j]
        __syncthreads();
        for (int j = threadIdx.x; j < D; j += blockDim.x) {
            float acc = 0.f;
            for (int d = 0; d < D; ++d) acc = fmaf(sm[d], o_rot[(int64_t)d * D + j], acc);
            st_elem(out, out_dtype, b * o_sb + hq * o_sh + l * o_sl + j, acc);
        }
        return;
    }
    if (o_signs) {
        smem_fwht(sm, 1, D, D);
        const float f = rsqrtf((float)D);
        for (int d = threadIdx.x; d < D; d += blockDim.x)
            st_elem(out, out_dtype, b * o_sb + hq * o_sh + l * o_sl + d, sm[d] * f * o_signs[d]);
    }
}

}  // namespace

void launch_merge(const float *o_part, const float2 *ml_part, int splits, const AttnArgs &a,
                  cudaStream_t stream) {
    const int64_t qrows = (int64_t)a.B * a.Hq * a.L;
    const int threads = std::min(256, std::max(32, ((a.D + 31) / 32) * 32));
    const size_t smem = (a.o_signs || a.o_rot) ? (size_t)a.D * sizeof(float) : 0;
    attn_merge_kernel<<<(unsigned)qrows, threads, smem, stream>>>(
        o_part, ml_part, splits, a.D, a.out, a.q_dtype, a.Hq, a.L, a.o_sb, a.o_sh, a.o_sl, a.o_signs, a.o_rot);
    KVC_CUDA(cudaGetLastError());
    ++g_launch_count;
}

int launch_attention_general(const AttnArgs &a, cudaStream_t stream) {
    KVC_REQUIRE(a.D > 0 && a.D <= 2 * G_THREADS, "attention: head dim must be in [1, 256]");
    KVC_REQUIRE(a.Hkv > 0 && a.Hq % a.Hkv == 0, "attention: Hq must be a multiple of Hkv");
    if (a.q_signs || a.o_signs)
        KVC_REQUIRE((a.D & (a.D - 1)) == 0, "attention: rotation needs a power-of-two head dim");
    if ((int64_t)a.B * a.Hq * a.L == 0) return 0;
    const int rep = a.Hq / a.Hkv;
    const int rows_total = rep * a.L;
    const int row_chunks = (rows_total + G_RC - 1) / G_RC;
    const int64_t tiles = std::max<int64_t>(1, (a.T + G_TILE - 1) / G_TILE);
    const int64_t base_ctas = (int64_t)a.B * a.Hkv * row_chunks;
    const int sms = sm_count(a.device);
    int64_t want = (4LL * sms + base_ctas - 1) / base_ctas;
    int splits = (int)std::max<int64_t>(1, std::min<int64_t>(std::min<int64_t>(want, tiles), 128));
    int64_t tiles_per_split = (tiles + splits - 1) / splits;
    splits = (int)((tiles + tiles_per_split - 1) / tiles_per_split);
    const int64_t tokens_per_split = tiles_per_split * G_TILE;

    const int64_t qrows = (int64_t)a.B * a.Hq * a.L;
    const size_t o_bytes = (size_t)qrows * splits * a.D * sizeof(float);
    const size_t ml_bytes = (size_t)qrows * splits * sizeof(float2);
    char *scratch = (char *)scratch_get(a.device, o_bytes + ml_bytes + 256, stream);
    float *o_part = (float *)scratch;
    float2 *ml_part = (float2 *)(scratch + ((o_bytes + 255) / 256) * 256);

    const size_t smem = (size_t)(G_RC * a.D + 2 * G_TILE * (a.D + 1) + G_RC * G_TILE + 3 * G_RC + 32) *
                        sizeof(float);
    static bool attr_set = false;
    if (!attr_set) {
        KVC_CUDA(cudaFuncSetAttribute(attn_general_partial,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
        attr_set = true;
    }
    KVC_REQUIRE(a.Hkv * row_chunks <= 65535 && a.B <= 65535, "attention: grid too large");
    dim3 grid((unsigned)splits, (unsigned)(a.Hkv * row_chunks), (unsigned)a.B);
    KernelTimer timer(stream);
    attn_general_partial<<<grid, G_THREADS, smem, stream>>>(a, o_part, ml_part, splits,
                                                            tokens_per_split, row_chunks);
    timer.stop();
    KVC_CUDA(cudaGetLastError());
    ++g_launch_count;
    launch_merge(o_part, ml_part, splits, a, stream);
    return 2;
}

}  // namespace kvc
