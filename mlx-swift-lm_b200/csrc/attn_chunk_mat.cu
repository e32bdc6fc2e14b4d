// Prefill chunks over the quantised caches on the tcgen05 chunk kernel.
//
// quantizedScaledDotProductAttention (KVCache.swift:2351-2447) and TurboQuantKVCache.compressedAttention
// (TurboQuantKVCache.swift:1164-1446) for a chunk of many query positions per head are contractions
// of 4 * rows * keys * D flops over a cache that is a few bytes per element: the work belongs on the
// tensor cores, and the dequantisation is small beside it. This path therefore
//
//   1. writes the visible rows of K and V once as 16-bit tiles into scratch memory, one 16-byte store
//      per eight elements: affine rows as scale * code + bias in the cache's dtype (what MLX's
//      dequantized() hands the matmul); TurboQuant rows as norm * centroid[index] in f16 whatever the
//      caller's dtype, i.e. the rows in the rotated basis at eleven significant bits (the product is
//      formed in fp32 and saturates at the f16 range: a row norm beyond 1e5 clips instead of
//      overflowing),
//   2. for TurboQuant rotates the chunk's queries into the key basis (sign flip, Walsh-Hadamard
//      butterfly in registers, 1/sqrt(D), optional calibration scale), f16,
//   3. runs attn_chunk_tc_kernel (tcgen05.mma, accumulators in TMEM) on those arrays,
//   4. for TurboQuant rotates the output rows back in place (butterfly, 1/sqrt(D), value signs) and
//      stores them in the caller's dtype.
//
// Steps 1, 2 and 4 move B*Hkv*T*D*4 + B*Hq*L*D*4 bytes through HBM; on a 512-token chunk over an
// 8192-token prefix that is a tenth of the time the contraction takes on the tensor cores, and a
// fifth of what the mma.sync kernel that dequantises inside its tile loop needs for the whole call.
// Batches whose scratch would pass a fixed bound are cut into slices of whole sequences.
#include "attn_common.cuh"
#include "common.h"

#include <algorithm>
#include <cstdio>
#include <cstdlib>

namespace kvc {

int launch_attention_chunk_tc(const AttnArgs &a, cudaStream_t stream);
bool attention_chunk_tc_accepts(const AttnArgs &a);

namespace {

using namespace dev;

constexpr size_t MAT_SCRATCH_LIMIT = (size_t)3 << 30;   // bytes of materialised K + V (+ Q') per slice

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    const T a = from_f32<T>(lo), b = from_f32<T>(hi);
    return (uint32_t)(*(const uint16_t *)&a) | ((uint32_t)(*(const uint16_t *)&b) << 16);
}

struct MatSource {
    const uint32_t *codes;      // packed words [B, H, cap, words]
    const void *scales, *biases;  // affine: [B, H, cap, D / group]
    const float *norms;         // turbo: [B, H, cap]
    int64_t sb, sh, st;         // word strides of codes
    int64_t gsb, gsh, gst;      // element strides of scales / biases / norms
    int32_t bits, group;
    float codebook[16];
};

struct MatParams {
    MatSource k, v;
    void *k_out, *v_out;        // [B, H, T, D] contiguous
    int32_t B, H, D;
    int64_t T;
    int32_t turbo;
};

// One thread = eight consecutive head dims of one token of K or V (blockIdx.z = 2 * b + which).
// T: dtype of the affine scales / biases; TO: dtype of the rows written (T for affine, f16 for TurboQuant).
template <typename T, typename TO>
__global__ void __launch_bounds__(256) materialize_kernel(const __grid_constant__ MatParams p) {
    const int which = blockIdx.z & 1, b = blockIdx.z >> 1, h = blockIdx.y;
    const MatSource &s = which ? p.v : p.k;
    const int per_row = p.D / 8;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= p.T * per_row) return;
    const int64_t t = i / per_row;
    const int d0 = (int)(i % per_row) * 8;
    const uint32_t *row = s.codes + b * s.sb + h * s.sh + t * s.st;
    float x[8];
    if (!p.turbo) {
        const int g = d0 / s.group;
        const int64_t gi = b * s.gsb + h * s.gsh + t * s.gst + g;
        const float sc = to_f32<T>(((const T *)s.scales)[gi]), bi = to_f32<T>(((const T *)s.biases)[gi]);
        if (s.bits == 4) {
            const uint32_t w = row[d0 / 8];
#pragma unroll
            for (int j = 0; j < 8; ++j) x[j] = fmaf(sc, (float)((w >> (4 * j)) & 15u), bi);
        } else if (s.bits == 8) {
            const uint32_t w0 = row[d0 / 4], w1 = row[d0 / 4 + 1];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                x[j] = fmaf(sc, (float)((w0 >> (8 * j)) & 255u), bi);
                x[4 + j] = fmaf(sc, (float)((w1 >> (8 * j)) & 255u), bi);
            }
        } else {  // 2 bits
            const uint32_t w = row[d0 / 16] >> ((d0 % 16) * 2);
#pragma unroll
            for (int j = 0; j < 8; ++j) x[j] = fmaf(sc, (float)((w >> (2 * j)) & 3u), bi);
        }
    } else {
        // indices are a low-bit-first stream of `bits` per dim; eight of them start at bit d0 * bits
        const float nrm = s.norms[b * s.gsb + h * s.gsh + t * s.gst];
        const int bit0 = d0 * s.bits, w0 = bit0 >> 5, sh = bit0 & 31;
        const int words = (p.D * s.bits + 31) / 32;
        uint64_t win = row[w0];
        if (w0 + 1 < words) win |= (uint64_t)row[w0 + 1] << 32;
        win >>= sh;
        const uint32_t m = (1u << s.bits) - 1u;
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = fminf(fmaxf(nrm * s.codebook[(uint32_t)(win >> (j * s.bits)) & m], -65504.f), 65504.f);
    }
    uint4 o;
    o.x = pack2<TO>(x[0], x[1]); o.y = pack2<TO>(x[2], x[3]); o.z = pack2<TO>(x[4], x[5]); o.w = pack2<TO>(x[6], x[7]);
    TO *out = (TO *)(which ? p.v_out : p.k_out) + (((int64_t)b * p.H + h) * p.T + t) * p.D + d0;
    *(uint4 *)out = o;
}

struct RotParams {
    const void *in;
    void *out;
    int64_t i_sb, i_sh, i_sl, o_sb, o_sh, o_sl;
    int32_t B, H, L;
    const float *pre;    // optional [D]: multiplied in before the butterfly
    const float *post;   // optional [D]: multiplied in after it
    const float *post2;  // optional second factor after it (calibration scale)
};

// out[row] = post * H(pre * in[row]) / sqrt(D), one warp per row, lane l holds dims E*l .. E*l + E - 1.
template <typename TI, typename TO, int D>
__global__ void __launch_bounds__(256) rotate_rows_kernel(const __grid_constant__ RotParams p) {
    constexpr int E = D / 32;
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= (int64_t)p.B * p.H * p.L) return;
    const int l = (int)(row % p.L), h = (int)((row / p.L) % p.H), b = (int)(row / ((int64_t)p.L * p.H));
    const TI *src = (const TI *)p.in + b * p.i_sb + h * p.i_sh + l * p.i_sl + E * lane;
    float x[E];
#pragma unroll
    for (int j = 0; j < E; ++j) {
        x[j] = to_f32<TI>(src[j]);
        if (p.pre) x[j] *= p.pre[E * lane + j];
    }
#pragma unroll
    for (int hh = 1; hh < E; hh <<= 1)
#pragma unroll
        for (int i = 0; i < E; ++i)
            if ((i & hh) == 0) {
                const float a = x[i], c = x[i + hh];
                x[i] = a + c;
                x[i + hh] = a - c;
            }
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {
        const bool upper = (lane & m) != 0;
#pragma unroll
        for (int j = 0; j < E; ++j) {
            const float y = __shfl_xor_sync(0xffffffffu, x[j], m);
            x[j] = upper ? y - x[j] : x[j] + y;
        }
    }
    const float fs = rsqrtf((float)D);
    TO *dst = (TO *)p.out + b * p.o_sb + h * p.o_sh + l * p.o_sl + E * lane;
#pragma unroll
    for (int j = 0; j < E; ++j) {
        float v = x[j] * fs;
        if (p.post) v *= p.post[E * lane + j];
        if (p.post2) v *= p.post2[E * lane + j];
        dst[j] = from_f32<TO>(v);
    }
}

bool source_ok(const KVSource &s, int D, bool turbo) {
    if (((uintptr_t)s.data & 3) != 0) return false;
    if (turbo) return s.kind == SRC_TURBO && s.bits >= 2 && s.bits <= 4 && s.norms != nullptr;
    if (s.kind != SRC_AFFINE || !s.scales || !s.biases) return false;
    if (s.bits != 2 && s.bits != 4 && s.bits != 8) return false;
    return s.group >= 8 && D % s.group == 0 && s.group % 8 == 0;
}

MatSource to_mat(const KVSource &s, int b0) {
    MatSource m = {};
    m.codes = (const uint32_t *)s.data + (int64_t)b0 * s.sb;
    const size_t es = 2;
    m.scales = s.scales ? (const char *)s.scales + (int64_t)b0 * s.gsb * es : nullptr;
    m.biases = s.biases ? (const char *)s.biases + (int64_t)b0 * s.gsb * es : nullptr;
    m.norms = s.norms ? s.norms + (int64_t)b0 * s.gsb : nullptr;
    m.sb = s.sb; m.sh = s.sh; m.st = s.st;
    m.gsb = s.gsb; m.gsh = s.gsh; m.gst = s.gst;
    m.bits = s.bits; m.group = s.group;
    for (int i = 0; i < 16; ++i) m.codebook[i] = s.codebook[i];
    return m;
}

template <typename TI, typename TO>
void rotate_rows(const RotParams &p, int D, cudaStream_t stream) {
    const int64_t rows = (int64_t)p.B * p.H * p.L;
    const unsigned blocks = (unsigned)((rows + 7) / 8);
    if (D == 128) rotate_rows_kernel<TI, TO, 128><<<blocks, 256, 0, stream>>>(p);
    else rotate_rows_kernel<TI, TO, 64><<<blocks, 256, 0, stream>>>(p);
    KVC_CUDA(cudaGetLastError());
    ++g_launch_count;
}

}  // namespace

// out[row] = post * H(pre * in[row]) / sqrt(D) over [B, H, L, D] rows (D 64 or 128); f16 / bf16 in and out.
void launch_rotate_rows_f16(const void *in, void *out, int32_t in_dtype, int32_t out_dtype, int64_t i_sb, int64_t i_sh, int64_t i_sl,
                            int64_t o_sb, int64_t o_sh, int64_t o_sl, int B, int H, int L, int D, const float *pre,
                            const float *post, cudaStream_t stream) {
    RotParams rp = {};
    rp.in = in; rp.out = out;
    rp.i_sb = i_sb; rp.i_sh = i_sh; rp.i_sl = i_sl; rp.o_sb = o_sb; rp.o_sh = o_sh; rp.o_sl = o_sl;
    rp.B = B; rp.H = H; rp.L = L;
    rp.pre = pre; rp.post = post; rp.post2 = nullptr;
    if (in_dtype == KVC_F16 && out_dtype == KVC_BF16) rotate_rows<__half, __nv_bfloat16>(rp, D, stream);
    else if (in_dtype == KVC_F16) rotate_rows<__half, __half>(rp, D, stream);
    else if (out_dtype == KVC_F16) rotate_rows<__nv_bfloat16, __half>(rp, D, stream);
    else rotate_rows<__nv_bfloat16, __nv_bfloat16>(rp, D, stream);
}

// Returns the number of kernels launched, 0 when the call is left to the other chunk kernels.
// KVC_CHUNK_MAT=0 turns the path off.
int launch_attention_chunk_materialized(const AttnArgs &a, cudaStream_t stream) {
    static const bool off = [] {
        const char *e = std::getenv("KVC_CHUNK_MAT");
        return e && e[0] == '0';
    }();
    if (off) return 0;
    if ((a.D != 128 && a.D != 64) || (a.q_dtype != KVC_BF16 && a.q_dtype != KVC_F16)) return 0;
    if (a.mask.mode == KVC_MASK_ARRAY || a.new_k || a.q_rot || a.o_rot) return 0;
    const bool turbo = a.k.kind == SRC_TURBO && a.v.kind == SRC_TURBO;
    const bool affine = a.k.kind == SRC_AFFINE && a.v.kind == SRC_AFFINE;
    if (!turbo && !affine) return 0;
    if (turbo && (!a.q_signs || !a.o_signs)) return 0;
    if (affine && (a.q_signs || a.o_signs || a.q_calib || a.k.dtype != a.q_dtype || a.v.dtype != a.q_dtype)) return 0;
    if (!source_ok(a.k, a.D, turbo) || !source_ok(a.v, a.D, turbo)) return 0;
    if (a.T < 1 || a.T > (int64_t)1 << 30 || a.B < 1) return 0;

    // the contraction as the tcgen05 kernel would see it: raw K / V of the query dtype, contiguous
    AttnArgs r = a;
    r.k = KVSource();
    r.v = KVSource();
    r.k.kind = r.v.kind = SRC_RAW;
    // TurboQuant runs in f16 whatever the caller's dtype
    const int32_t work_dtype = turbo ? KVC_F16 : a.q_dtype;
    r.q_dtype = work_dtype;
    r.k.dtype = r.v.dtype = work_dtype;
    r.k.st = r.v.st = a.D;
    r.k.sh = r.v.sh = a.T * a.D;
    r.k.sb = r.v.sb = (int64_t)a.Hkv * a.T * a.D;
    r.q_signs = r.o_signs = r.q_calib = nullptr;
    r.k.data = r.v.data = a.q;   // any 16-byte aligned address: only the shape is judged here
    if (((uintptr_t)a.q & 15) != 0 || !attention_chunk_tc_accepts(r)) return 0;

    const size_t es = 2;
    const size_t kv_per_b = (size_t)2 * a.Hkv * a.T * a.D * es;
    const size_t q_per_b = turbo ? (size_t)a.Hq * a.L * a.D * es : 0;
    const size_t per_b = kv_per_b + q_per_b + 512;
    if (per_b > MAT_SCRATCH_LIMIT) return 0;
    // whole sequences per slice, the slices as even as they come; every slice must still fill the part
    const int fit = (int)std::min<size_t>((size_t)a.B, MAT_SCRATCH_LIMIT / per_b);
    const int nslices = (a.B + fit - 1) / fit;
    const int slice = (a.B + nslices - 1) / nslices;
    {
        AttnArgs probe = r;
        probe.B = a.B - (nslices - 1) * slice;   // the last, smallest slice
        if (probe.B < 1 || !attention_chunk_tc_accepts(probe)) return 0;
        probe.B = slice;
        if (!attention_chunk_tc_accepts(probe)) return 0;
    }
    char *scratch = (char *)scratch_get(a.device, (size_t)slice * per_b + 1024, stream);
    int launches = 0;
    for (int b0 = 0; b0 < a.B; b0 += slice) {
        const int nb = std::min(slice, a.B - b0);
        char *k_out = scratch;
        char *v_out = k_out + (((size_t)nb * a.Hkv * a.T * a.D * es + 255) / 256) * 256;
        char *q_out = v_out + (((size_t)nb * a.Hkv * a.T * a.D * es + 255) / 256) * 256;
        MatParams mp = {};
        mp.k = to_mat(a.k, b0);
        mp.v = to_mat(a.v, b0);
        mp.k_out = k_out; mp.v_out = v_out;
        mp.B = nb; mp.H = a.Hkv; mp.D = a.D; mp.T = a.T;
        mp.turbo = turbo ? 1 : 0;
        const int64_t per_head = a.T * (a.D / 8);
        const dim3 grid((unsigned)((per_head + 255) / 256), (unsigned)a.Hkv, (unsigned)(2 * nb));
        if (turbo) materialize_kernel<__half, __half><<<grid, 256, 0, stream>>>(mp);
        else if (a.q_dtype == KVC_BF16) materialize_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, stream>>>(mp);
        else materialize_kernel<__half, __half><<<grid, 256, 0, stream>>>(mp);
        KVC_CUDA(cudaGetLastError());
        ++g_launch_count;
        ++launches;

        AttnArgs call = r;
        call.B = nb;
        call.q = (const char *)a.q + (int64_t)b0 * a.q_sb * es;
        call.out = (char *)a.out + (int64_t)b0 * a.o_sb * es;
        call.k.data = k_out;
        call.v.data = v_out;
        if (turbo) {
            RotParams rp = {};
            rp.in = call.q; rp.out = q_out;
            rp.i_sb = a.q_sb; rp.i_sh = a.q_sh; rp.i_sl = a.q_sl;
            rp.o_sb = (int64_t)a.Hq * a.L * a.D; rp.o_sh = (int64_t)a.L * a.D; rp.o_sl = a.D;
            rp.B = nb; rp.H = a.Hq; rp.L = a.L;
            rp.pre = a.q_signs; rp.post = a.q_calib; rp.post2 = nullptr;
            if (a.q_dtype == KVC_BF16) rotate_rows<__nv_bfloat16, __half>(rp, a.D, stream);
            else rotate_rows<__half, __half>(rp, a.D, stream);
            ++launches;
            call.q = q_out;
            call.q_sb = rp.o_sb; call.q_sh = rp.o_sh; call.q_sl = rp.o_sl;
        }
        const int n = launch_attention_chunk_tc(call, stream);
        if (n <= 0) fail(KVC_ERR_INTERNAL, "the tensor-core chunk kernel refused a call it had accepted");
        launches += n;
        if (turbo) {
            RotParams rp = {};
            rp.in = call.out; rp.out = call.out;
            rp.i_sb = rp.o_sb = a.o_sb; rp.i_sh = rp.o_sh = a.o_sh; rp.i_sl = rp.o_sl = a.o_sl;
            rp.B = nb; rp.H = a.Hq; rp.L = a.L;
            rp.pre = nullptr; rp.post = a.o_signs; rp.post2 = nullptr;
            if (a.q_dtype == KVC_BF16) rotate_rows<__half, __nv_bfloat16>(rp, a.D, stream);   // f16 rows in, caller's dtype out
            else rotate_rows<__half, __half>(rp, a.D, stream);
            ++launches;
        }
    }
    if (trace_dispatch())
        fprintf(stderr, "[kvc] chunk_mat: %s rows written out for the tcgen05 kernel, %d sequences per slice\n",
                turbo ? "TurboQuant" : "affine", slice);
    return launches;
}

}  // namespace kvc
