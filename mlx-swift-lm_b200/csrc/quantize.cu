// Group-wise affine quantisation (MLX `quantized` / `dequantized`, affine mode)
// and the TurboQuant fused Walsh-Hadamard encode.
//
// Both produce integer codes that must be bit-identical to the CPU oracle, so
// every floating-point step uses the explicit round-to-nearest intrinsics
// (never contracted into FMAs) and one fixed reduction tree:
//   * a row of D elements is owned by 32 lanes, lane l holding the E = D/32
//     contiguous elements [l*E, l*E+E);
//   * sums run sequentially over a lane's own elements, then over the xor
//     butterfly 16, 8, 4, 2, 1 across lanes.
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

// MLX affine quantisation of one group given its min and max:
//   scale = max((max-min)/(2^b-1), 1e-7); the sign of the scale and the
//   anchoring edge follow the larger-magnitude end, the scale is re-derived so
//   that the edge maps to an integer code, and codes are
//   rint((w - bias)/scale) clamped to [0, 2^b-1].
__device__ __forceinline__ void affine_params(float w_min, float w_max, float n_bins,
                                              float &scale, float &bias) {
    scale = fmaxf(__fdiv_rn(__fsub_rn(w_max, w_min), n_bins), 1e-7f);
    const bool side = fabsf(w_min) > fabsf(w_max);
    scale = side ? scale : -scale;
    const float edge = side ? w_min : w_max;
    const float q0 = rintf(__fdiv_rn(edge, scale));
    bias = 0.f;
    if (q0 != 0.f) {
        scale = __fdiv_rn(edge, q0);
        bias = edge;
    }
}

__device__ __forceinline__ uint32_t affine_code(float w, float scale, float bias, float n_bins) {
    float q = rintf(__fdiv_rn(__fsub_rn(w, bias), scale));
    q = fminf(fmaxf(q, 0.f), n_bins);
    return (uint32_t)q;
}

// One row (D = 32 E elements) by one warp: group min/max by shuffles, MLX affine parameters,
// codes packed low bits first. `src` points at the row's first element, `dst` at its first code
// word, `scales` / `biases` at its first group.
template <typename T, int E>
__device__ __forceinline__ void quantize_row_warp(const T *src, int64_t s_sd, uint32_t *dst, T *scales, T *biases,
                                                  int group, int bits, int lane) {
    float v[E];
#pragma unroll
    for (int i = 0; i < E; ++i) v[i] = to_float<T>(src[(int64_t)(lane * E + i) * s_sd]);

    float w_min = v[0], w_max = v[0];
#pragma unroll
    for (int i = 1; i < E; ++i) {
        w_min = fminf(w_min, v[i]);
        w_max = fmaxf(w_max, v[i]);
    }
    const int lanes_per_group = group / E;  // power of two, <= 32
    for (int m = lanes_per_group >> 1; m >= 1; m >>= 1) {
        w_min = fminf(w_min, __shfl_xor_sync(0xffffffffu, w_min, m));
        w_max = fmaxf(w_max, __shfl_xor_sync(0xffffffffu, w_max, m));
    }
    const float n_bins = (float)((1 << bits) - 1);
    float scale, bias;
    affine_params(w_min, w_max, n_bins, scale, bias);

    if ((lane % lanes_per_group) == 0) {
        const int g = lane / lanes_per_group;
        scales[g] = from_float<T>(scale);
        biases[g] = from_float<T>(bias);
    }

    // Pack: the lane's E codes occupy E*bits consecutive bits starting at bit
    // lane*E*bits of the row (low bits first).
    const int nbits = E * bits;  // a power of two in [2, 64]
    uint64_t acc = 0;
#pragma unroll
    for (int i = 0; i < E; ++i)
        acc |= (uint64_t)affine_code(v[i], scale, bias, n_bins) << (i * bits);
    if (nbits == 64) {
        dst[lane * 2] = (uint32_t)acc;
        dst[lane * 2 + 1] = (uint32_t)(acc >> 32);
    } else if (nbits == 32) {
        dst[lane] = (uint32_t)acc;
    } else {
        const uint32_t part = (uint32_t)acc;
        const int lpw = 32 / nbits;  // lanes per word
        uint32_t word = part;
        for (int k = 1; k < lpw; ++k) {
            const uint32_t other = __shfl_down_sync(0xffffffffu, part, k);
            word |= other << (k * nbits);
        }
        if ((lane % lpw) == 0) dst[lane / lpw] = word;
    }
}

// One warp per (tensor, b, h, s) row; E elements per lane.
template <typename T, int E>
__global__ void affine_quantize_warp_kernel(QuantAppendArgs ka, QuantAppendArgs va, int64_t k_rows,
                                            int64_t total_rows) {
    // lets a dependent kernel launched with programmatic serialization begin its prologue now
    asm volatile("griddepcontrol.launch_dependents;");
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= total_rows) return;
    const bool is_v = row >= k_rows;
    const QuantAppendArgs &a = is_v ? va : ka;
    int64_t r = is_v ? row - k_rows : row;
    const int s = (int)(r % a.S);
    r /= a.S;
    const int h = (int)(r % a.H);
    const int b = (int)(r / a.H);
    const int64_t t = a.pos + s;
    quantize_row_warp<T, E>((const T *)a.src + b * a.s_sb + h * a.s_sh + s * a.s_ss, a.s_sd,
                            a.codes + b * a.c_sb + h * a.c_sh + t * a.c_st,
                            (T *)a.scales + b * a.g_sb + h * a.g_sh + t * a.g_st,
                            (T *)a.biases + b * a.g_sb + h * a.g_sh + t * a.g_st, a.group, a.bits, lane);
}

// Codes of VEC values of one group. The correctly rounded quotient (w - bias) / scale lies between
// the products of (w - bias) with the reciprocal scaled by 1 -+ 4e-7. Each product is rounded to an
// integer by a fused multiply-add with 1.5 * 2^23 (one rounding, ties to even, like rint): when both
// ends give the same integer that is rint of the quotient as well; when they differ for any value
// the lane redoes its values with the division itself. So the codes are those of affine_code bit for
// bit. The clamps run on the biased floats (a NaN becomes code 0, as fmaxf(NaN, 0) makes it), and
// the words accumulate the float bit patterns by multiply-add; MAGIC_SUM removes the bias's share.
template <int VEC, int BITS>
__device__ __forceinline__ uint64_t affine_codes_vec(const float (&v)[VEC], float scale, float bias) {
    constexpr float n_bins = (float)((1 << BITS) - 1);
    constexpr float MAGIC = 12582912.f;          // 1.5 * 2^23: x + MAGIC leaves rint(x) in the low mantissa bits
    constexpr uint32_t MAGIC_BITS = 0x4B400000u;
    constexpr int PER_WORD = (VEC * BITS > 32) ? 32 / BITS : VEC;   // values per 32-bit word
    uint32_t magic_sum = 0;
#pragma unroll
    for (int i = 0; i < PER_WORD; ++i) magic_sum += MAGIC_BITS << (i * BITS);
    const float inv = __frcp_rn(scale);
    const float inv_lo = fmaf(inv, -4e-7f, inv), inv_hi = fmaf(inv, 4e-7f, inv);
    uint32_t w[2] = {0u, 0u};
    uint32_t differ = 0;
#pragma unroll
    for (int i = VEC - 1; i >= 0; --i) {
        const float x = __fsub_rn(v[i], bias);
        const float u_lo = __fmaf_rn(x, inv_lo, MAGIC), u_hi = __fmaf_rn(x, inv_hi, MAGIC);
        differ |= __float_as_uint(u_lo) ^ __float_as_uint(u_hi);
        const float u = fminf(fmaxf(u_lo, MAGIC), MAGIC + n_bins);
        w[i / PER_WORD] = (w[i / PER_WORD] << BITS) + __float_as_uint(u);
    }
    w[0] -= magic_sum;
    if (VEC * BITS > 32) w[1] -= magic_sum;
    // (products beyond 2^22 leave the integer grid of the biased floats but are far outside the code
    // range, so the clamps settle them.) A reciprocal below 1e-30 has lost bits to the subnormal
    // range: exact path, like a straddled tie.
    if (differ != 0u || !(fabsf(inv) > 1e-30f) || !(fabsf(inv) < 1e30f)) {
        w[0] = w[1] = 0u;
#pragma unroll
        for (int i = VEC - 1; i >= 0; --i)
            w[i / PER_WORD] = (w[i / PER_WORD] << BITS) | affine_code(v[i], scale, bias, n_bins);
    }
    return (uint64_t)w[0] | ((uint64_t)w[1] << 32);
}

// Contiguous rows, 16 bytes per lane: a row takes LPR = D / VEC lanes (VEC = 8 for 16-bit types, 4 for
// fp32), a warp covers 32 / LPR rows per pass and keeps U passes of loads in flight. Grid: x = chunks
// of consecutive tokens, y = head, z = batch (keys first, then values), so a block works on one
// (tensor, batch, head) and its pointers are uniform. Same parameters and codes as quantize_row_warp
// (min / max are order-free).
template <typename T, int LPR, int BITS, int U>
__device__ __forceinline__ void affine_quantize_vec_body(const QuantAppendArgs &a, int b, int lpg_log2) {
    constexpr int VEC = 16 / (int)sizeof(T);
    constexpr int RPP = 32 / LPR;
    constexpr int NBITS = VEC * BITS;   // code bits per lane: 8, 16, 32 or 64
    constexpr float n_bins = (float)((1 << BITS) - 1);
    const int lane = threadIdx.x & 31;
    const int sub = lane / LPR, l = lane % LPR;
    const int h = blockIdx.y;
    const int s0 = (blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * (RPP * U) + sub;
    if (s0 - sub >= a.S) return;   // whole warp
    const T *src = (const T *)a.src + b * a.s_sb + h * a.s_sh + l * VEC;
    uint32_t *codes = a.codes + b * a.c_sb + h * a.c_sh + a.pos * a.c_st;
    const int64_t g0 = b * a.g_sb + h * a.g_sh + a.pos * a.g_st;
    T *scales = (T *)a.scales + g0, *biases = (T *)a.biases + g0;

    uint4 raw[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int sr = s0 + u * RPP;
        raw[u] = sr < a.S ? __ldg(reinterpret_cast<const uint4 *>(src + sr * a.s_ss)) : make_uint4(0u, 0u, 0u, 0u);
    }
    const int lpg = 1 << lpg_log2;   // lanes per group
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int sr = s0 + u * RPP;
        float v[VEC];
        const T *e = reinterpret_cast<const T *>(&raw[u]);
#pragma unroll
        for (int i = 0; i < VEC; ++i) v[i] = to_float<T>(e[i]);
        float w_min = v[0], w_max = v[0];
#pragma unroll
        for (int i = 1; i < VEC; ++i) {
            w_min = fminf(w_min, v[i]);
            w_max = fmaxf(w_max, v[i]);
        }
        for (int m = lpg >> 1; m >= 1; m >>= 1) {
            w_min = fminf(w_min, __shfl_xor_sync(0xffffffffu, w_min, m));
            w_max = fmaxf(w_max, __shfl_xor_sync(0xffffffffu, w_max, m));
        }
        float scale, bias;
        affine_params(w_min, w_max, n_bins, scale, bias);
        const uint64_t acc = affine_codes_vec<VEC, BITS>(v, scale, bias);
        uint32_t word = (uint32_t)acc;
        if (NBITS < 32) {
            constexpr int LPW = NBITS < 32 ? 32 / NBITS : 1;   // lanes per word
#pragma unroll
            for (int k = 1; k < LPW; ++k) word |= __shfl_down_sync(0xffffffffu, (uint32_t)acc, k) << (k * NBITS);
        }
        if (sr < a.S) {
            if ((l & (lpg - 1)) == 0) {
                scales[sr * a.g_st + (l >> lpg_log2)] = from_float<T>(scale);
                biases[sr * a.g_st + (l >> lpg_log2)] = from_float<T>(bias);
            }
            uint32_t *row = codes + sr * a.c_st;
            if (NBITS == 64) {
                *reinterpret_cast<uint2 *>(row + l * 2) = make_uint2((uint32_t)acc, (uint32_t)(acc >> 32));
            } else if (NBITS == 32) {
                row[l] = word;
            } else {
                constexpr int LPW = NBITS < 32 ? 32 / NBITS : 1;
                if ((l % LPW) == 0) row[l / LPW] = word;
            }
        }
    }
}

template <typename T, int LPR, int BITS, int U>
__global__ void __launch_bounds__(256)
affine_quantize_vec_kernel(QuantAppendArgs ka, QuantAppendArgs va, int lpg_log2) {
    asm volatile("griddepcontrol.launch_dependents;");
    // keys and values share B, H and S; the branch is uniform over the block
    if ((int)blockIdx.z >= ka.B) affine_quantize_vec_body<T, LPR, BITS, U>(va, (int)blockIdx.z - ka.B, lpg_log2);
    else affine_quantize_vec_body<T, LPR, BITS, U>(ka, (int)blockIdx.z, lpg_log2);
}

// The same rows for a list of independent caches (one new token each): row = (sequence, K or V,
// head); every pointer of the table already addresses head 0 at the sequence's append position.
template <typename T, int E>
__global__ void affine_quantize_varlen_kernel(const __grid_constant__ VarlenQuantArgs a) {
    asm volatile("griddepcontrol.launch_dependents;");
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= a.n * 2 * a.H) return;
    const int i = row / (2 * a.H), rr = row % (2 * a.H);
    const bool is_v = rr >= a.H;
    const int h = rr % a.H;
    const VarlenQuantSeq &q = a.seq[i];
    const T *src = (const T *)(is_v ? q.vsrc : q.ksrc) + (int64_t)h * a.src_sh;
    uint32_t *codes = (is_v ? q.vcodes : q.kcodes) + (int64_t)h * q.c_sh;
    T *scales = (T *)(is_v ? q.vscales : q.kscales) + (int64_t)h * q.g_sh;
    T *biases = (T *)(is_v ? q.vbiases : q.kbiases) + (int64_t)h * q.g_sh;
    quantize_row_warp<T, E>(src, 1, codes, scales, biases, a.group, a.bits, lane);
}

// General shapes: one thread per group.
template <typename T>
__global__ void affine_quantize_group_kernel(QuantAppendArgs ka, QuantAppendArgs va,
                                             int64_t k_groups, int64_t total_groups) {
    int64_t gidx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gidx >= total_groups) return;
    const bool is_v = gidx >= k_groups;
    const QuantAppendArgs &a = is_v ? va : ka;
    if (is_v) gidx -= k_groups;
    const int gpr = a.D / a.group;
    const int g = (int)(gidx % gpr);
    int64_t r = gidx / gpr;
    const int s = (int)(r % a.S);
    r /= a.S;
    const int h = (int)(r % a.H);
    const int b = (int)(r / a.H);
    const T *src = (const T *)a.src + b * a.s_sb + h * a.s_sh + s * a.s_ss + (int64_t)g * a.group * a.s_sd;
    float w_min = to_float<T>(src[0]), w_max = w_min;
    for (int i = 1; i < a.group; ++i) {
        const float x = to_float<T>(src[i * a.s_sd]);
        w_min = fminf(w_min, x);
        w_max = fmaxf(w_max, x);
    }
    const float n_bins = (float)((1 << a.bits) - 1);
    float scale, bias;
    affine_params(w_min, w_max, n_bins, scale, bias);
    const int64_t t = a.pos + s;
    const int64_t gi = b * a.g_sb + h * a.g_sh + t * a.g_st + g;
    ((T *)a.scales)[gi] = from_float<T>(scale);
    ((T *)a.biases)[gi] = from_float<T>(bias);
    uint32_t *dst = a.codes + b * a.c_sb + h * a.c_sh + t * a.c_st + (int64_t)g * a.group * a.bits / 32;
    const int per_word = 32 / a.bits;
    for (int w = 0; w < a.group / per_word; ++w) {
        uint32_t word = 0;
        for (int k = 0; k < per_word; ++k)
            word |= affine_code(to_float<T>(src[(int64_t)(w * per_word + k) * a.s_sd]), scale, bias, n_bins)
                    << (k * a.bits);
        dst[w] = word;
    }
}

template <typename T>
__global__ void affine_dequantize_kernel(DequantArgs a, int64_t total) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int d = (int)(i % a.D);
    const int64_t row = i / a.D;
    const uint32_t word = a.codes[row * a.c_srow + (d * a.bits) / 32];
    const uint32_t code = (word >> ((d * a.bits) % 32)) & ((1u << a.bits) - 1u);
    const int g = d / a.group;
    const float sc = to_float<T>(((const T *)a.scales)[row * a.g_srow + g]);
    const float bi = to_float<T>(((const T *)a.biases)[row * a.g_srow + g]);
    // MLX dequantises in the array dtype: scale * q + bias.
    const float val = __fadd_rn(__fmul_rn(sc, (float)code), bi);
    ((T *)a.out)[row * a.o_srow + d] = from_float<T>(val);
}

template <typename T>
void quantize_dispatch(const QuantAppendArgs &k, const QuantAppendArgs &v, bool have_v,
                       cudaStream_t stream) {
    const QuantAppendArgs &vv = have_v ? v : k;
    const int64_t k_rows = (int64_t)k.B * k.H * k.S;
    const int64_t v_rows = have_v ? (int64_t)v.B * v.H * v.S : 0;
    auto warp_ok = [](const QuantAppendArgs &a) {
        if (a.D % 32 != 0) return false;
        const int E = a.D / 32;
        if (!(E == 1 || E == 2 || E == 4 || E == 8)) return false;
        if (a.group % E != 0) return false;
        const int lpg = a.group / E;
        if (lpg < 1 || lpg > 32 || (lpg & (lpg - 1))) return false;
        const int nbits = E * a.bits;
        return (nbits >= 32) ? (nbits % 32 == 0) : (32 % nbits == 0);
    };
    const bool same_shape = !have_v || (k.D == v.D && k.group == v.group && k.bits == v.bits);
    // 16-byte lanes need contiguous, 16-byte aligned rows
    constexpr int VEC = 16 / (int)sizeof(T);
    auto vec_ok = [&](const QuantAppendArgs &a) {
        const int lpr = a.D / VEC;
        if (a.D % VEC != 0 || !(lpr == 8 || lpr == 16 || lpr == 32)) return false;
        if (a.group % VEC != 0 || a.group / VEC > lpr || ((a.group / VEC) & (a.group / VEC - 1))) return false;
        if (a.s_sd != 1 || a.s_sb % VEC || a.s_sh % VEC || a.s_ss % VEC) return false;
        if ((reinterpret_cast<uintptr_t>(a.src) & 15) || (reinterpret_cast<uintptr_t>(a.codes) & 7)) return false;
        return (a.c_sb % 2 == 0) && (a.c_sh % 2 == 0) && (a.c_st % 2 == 0);
    };
    const bool same_dims = !have_v || (k.B == v.B && k.H == v.H && k.S == v.S);
    if (same_shape && same_dims && vec_ok(k) && (!have_v || vec_ok(v)) && k.H <= 65535 && 2 * (int64_t)k.B <= 65535) {
        const int lpr = k.D / VEC, rpp = 32 / lpr;
        int lpg_log2 = 0;
        while ((1 << lpg_log2) < k.group / VEC) ++lpg_log2;
        const bool deep = (int64_t)k.S >= 8 * rpp * 4;   // a block of 8 warps fills up with 4 passes per warp
        const int rows_per_warp = rpp * (deep ? 4 : 1);
        const int warps = std::max(1, std::min(8, (k.S + rows_per_warp - 1) / rows_per_warp));
        const dim3 grid((unsigned)((k.S + warps * rows_per_warp - 1) / (warps * rows_per_warp)), (unsigned)k.H,
                        (unsigned)(k.B * (have_v ? 2 : 1)));
#define KVC_QVEC(LPR, BITS)                                                                                   \
    do {                                                                                                      \
        if (deep) affine_quantize_vec_kernel<T, LPR, BITS, 4><<<grid, warps * 32, 0, stream>>>(k, vv, lpg_log2); \
        else affine_quantize_vec_kernel<T, LPR, BITS, 1><<<grid, warps * 32, 0, stream>>>(k, vv, lpg_log2);      \
    } while (0)
#define KVC_QVEC_B(LPR)                                            \
    switch (k.bits) {                                              \
        case 2: KVC_QVEC(LPR, 2); break;                           \
        case 4: KVC_QVEC(LPR, 4); break;                           \
        default: KVC_QVEC(LPR, 8); break;                          \
    }
        switch (lpr) {
            case 8: KVC_QVEC_B(8); break;
            case 16: KVC_QVEC_B(16); break;
            default: KVC_QVEC_B(32); break;
        }
#undef KVC_QVEC_B
#undef KVC_QVEC
    } else if (same_shape && warp_ok(k)) {
        const int64_t total = k_rows + v_rows;
        const int warps = 8;
        const unsigned blocks = (unsigned)((total + warps - 1) / warps);
        switch (k.D / 32) {
            case 1: affine_quantize_warp_kernel<T, 1><<<blocks, warps * 32, 0, stream>>>(k, vv, k_rows, total); break;
            case 2: affine_quantize_warp_kernel<T, 2><<<blocks, warps * 32, 0, stream>>>(k, vv, k_rows, total); break;
            case 4: affine_quantize_warp_kernel<T, 4><<<blocks, warps * 32, 0, stream>>>(k, vv, k_rows, total); break;
            case 8: affine_quantize_warp_kernel<T, 8><<<blocks, warps * 32, 0, stream>>>(k, vv, k_rows, total); break;
        }
    } else {
        const int64_t k_groups = k_rows * (k.D / k.group);
        const int64_t v_groups = have_v ? v_rows * (v.D / v.group) : 0;
        const int64_t total = k_groups + v_groups;
        affine_quantize_group_kernel<T><<<(unsigned)((total + 127) / 128), 128, 0, stream>>>(
            k, vv, k_groups, total);
    }
    KVC_CUDA(cudaGetLastError());
    ++g_launch_count;
}

}  // namespace

bool launch_affine_quantize_varlen(const VarlenQuantArgs &a, cudaStream_t stream) {
    if (a.D % 32 != 0 || a.n < 1 || a.n > KVC_VARLEN_MAX) return false;
    const int E = a.D / 32;
    if (!(E == 1 || E == 2 || E == 4 || E == 8) || a.group % E != 0) return false;
    const int lpg = a.group / E;
    if (lpg < 1 || lpg > 32 || (lpg & (lpg - 1))) return false;
    const int nbits = E * a.bits;
    if (!((nbits >= 32) ? (nbits % 32 == 0) : (32 % nbits == 0))) return false;
    const int total = a.n * 2 * a.H, warps = 8;
    const unsigned blocks = (unsigned)((total + warps - 1) / warps);
#define KVC_QV(TT)                                                                                      \
    switch (E) {                                                                                        \
        case 1: affine_quantize_varlen_kernel<TT, 1><<<blocks, warps * 32, 0, stream>>>(a); break;     \
        case 2: affine_quantize_varlen_kernel<TT, 2><<<blocks, warps * 32, 0, stream>>>(a); break;     \
        case 4: affine_quantize_varlen_kernel<TT, 4><<<blocks, warps * 32, 0, stream>>>(a); break;     \
        default: affine_quantize_varlen_kernel<TT, 8><<<blocks, warps * 32, 0, stream>>>(a); break;    \
    }
    if (a.dtype == KVC_BF16) { KVC_QV(__nv_bfloat16) }
    else if (a.dtype == KVC_F16) { KVC_QV(__half) }
    else if (a.dtype == KVC_F32) { KVC_QV(float) }
    else return false;
#undef KVC_QV
    KVC_CUDA(cudaGetLastError());
    ++g_launch_count;
    return true;
}

void launch_affine_quantize2(const QuantAppendArgs &k, const QuantAppendArgs *v, cudaStream_t stream) {
    if ((int64_t)k.B * k.H * k.S == 0) return;
    auto check = [](const QuantAppendArgs &a) {
        KVC_REQUIRE(a.bits == 2 || a.bits == 4 || a.bits == 8,
                    "affine quantisation supports 2, 4 or 8 bits");
        KVC_REQUIRE(a.group > 0 && a.D % a.group == 0, "head dim must be a multiple of the group size");
        KVC_REQUIRE((a.group * a.bits) % 32 == 0, "group must fill whole 32-bit words");
    };
    check(k);
    if (v) {
        check(*v);
        KVC_REQUIRE(v->dtype == k.dtype, "keys and values must share a dtype");
    }
    const QuantAppendArgs dummy = k;
    switch (k.dtype) {
        case KVC_F32: quantize_dispatch<float>(k, v ? *v : dummy, v != nullptr, stream); break;
        case KVC_F16: quantize_dispatch<__half>(k, v ? *v : dummy, v != nullptr, stream); break;
        case KVC_BF16: quantize_dispatch<__nv_bfloat16>(k, v ? *v : dummy, v != nullptr, stream); break;
        default: fail(KVC_ERR_INVALID_ARG, "affine quantisation needs a floating dtype");
    }
}

void launch_affine_quantize(const QuantAppendArgs &a, cudaStream_t stream) {
    launch_affine_quantize2(a, nullptr, stream);
}

void launch_affine_dequantize(const DequantArgs &a, cudaStream_t stream) {
    const int64_t total = a.rows * a.D;
    if (total <= 0) return;
    KVC_REQUIRE(a.bits == 2 || a.bits == 4 || a.bits == 8, "affine dequantisation supports 2, 4 or 8 bits");
    const unsigned blocks = (unsigned)((total + 255) / 256);
    switch (a.dtype) {
        case KVC_F32: affine_dequantize_kernel<float><<<blocks, 256, 0, stream>>>(a, total); break;
        case KVC_F16: affine_dequantize_kernel<__half><<<blocks, 256, 0, stream>>>(a, total); break;
        case KVC_BF16: affine_dequantize_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(a, total); break;
        default: fail(KVC_ERR_INVALID_ARG, "affine dequantisation needs a floating dtype");
    }
    KVC_CUDA(cudaGetLastError());
    ++g_launch_count;
}

// ---------------------------------------------------------------------
// TurboQuant fused WHT encode
// ---------------------------------------------------------------------
namespace {

template <typename T, int E>
__global__ void turbo_encode_kernel(TurboEncodeArgs ka, TurboEncodeArgs va, int64_t k_rows,
                                    int64_t total_rows, float inv_sqrt_dim) {
    // lets a dependent kernel launched with programmatic serialization begin its prologue now
    asm volatile("griddepcontrol.launch_dependents;");
    extern __shared__ uint32_t s_words[];  // [warps][PWmax]
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp;
    if (row >= total_rows) return;  // whole warp exits together
    const bool is_v = row >= k_rows;
    const TurboEncodeArgs &a = is_v ? va : ka;
    int64_t r = is_v ? row - k_rows : row;
    const int s = (int)(r % a.S);
    r /= a.S;
    const int h = (int)(r % a.H);
    const int b = (int)(r / a.H);
    constexpr int D = E * 32;

    const T *src = (const T *)a.src + b * a.s_sb + h * a.s_sh + s * a.s_ss;
    float v[E];
#pragma unroll
    for (int i = 0; i < E; ++i) v[i] = to_float<T>(src[(int64_t)(lane * E + i) * a.s_sd]);

    // L2 norm over the fixed reduction tree.
    float sq = __fmul_rn(v[0], v[0]);
#pragma unroll
    for (int i = 1; i < E; ++i) sq = __fadd_rn(sq, __fmul_rn(v[i], v[i]));
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) sq = __fadd_rn(sq, __shfl_xor_sync(0xffffffffu, sq, m));
    const float norm = __fsqrt_rn(sq);
    const float inv_norm = (norm > 1e-8f) ? __fdiv_rn(1.0f, norm) : 0.0f;

    // unit-normalise and flip signs: x * (inv_norm * sign)
#pragma unroll
    for (int i = 0; i < E; ++i) v[i] = __fmul_rn(v[i], __fmul_rn(inv_norm, a.signs[lane * E + i]));

    // Walsh-Hadamard butterfly, stage s pairs elements 2^s apart: (a, b) -> (a+b, a-b).
#pragma unroll
    for (int st = 1; st < E; st <<= 1) {
#pragma unroll
        for (int i = 0; i < E; ++i) {
            if ((i & st) == 0) {
                const float lo = v[i], hi = v[i + st];
                v[i] = __fadd_rn(lo, hi);
                v[i + st] = __fsub_rn(lo, hi);
            }
        }
    }
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
        for (int i = 0; i < E; ++i) {
            const float other = __shfl_xor_sync(0xffffffffu, v[i], m);
            v[i] = (lane & m) ? __fsub_rn(other, v[i]) : __fadd_rn(other, v[i]);
        }
    }

    // boundary quantise + pack (low bits first, codes may straddle words)
    const int pw = (D * a.bits + 31) / 32;
    uint32_t *words = s_words + warp * ((1024 * 4 + 31) / 32);
    for (int w = lane; w < pw; w += 32) words[w] = 0;
    __syncwarp();
    const int levels_m1 = (1 << a.bits) - 1;
    const uint32_t mask = (uint32_t)levels_m1;
    float recon_sq = 0.f;  // calibrated rows: squared norm of centroid * scale, same reduction tree as the norm
#pragma unroll
    for (int i = 0; i < E; ++i) {
        float rotated = __fmul_rn(v[i], inv_sqrt_dim);
        float cal = 1.f;
        if (a.calib) {
            cal = a.calib[lane * E + i];
            rotated = __fdiv_rn(rotated, cal);
        }
        uint32_t idx = 0;
        for (int bd = 0; bd < levels_m1; ++bd) idx += (rotated > a.boundaries[bd]) ? 1u : 0u;
        idx &= mask;
        if (a.calib) {
            const float cv = __fmul_rn(a.centroids[idx], cal);
            const float sqv = __fmul_rn(cv, cv);
            recon_sq = i == 0 ? sqv : __fadd_rn(recon_sq, sqv);
        }
        const int bit = (lane * E + i) * a.bits;
        const int w = bit >> 5, sh = bit & 31;
        atomicOr(&words[w], idx << sh);
        if (sh + a.bits > 32) atomicOr(&words[w + 1], idx >> (32 - sh));
    }
    float stored = norm;
    if (a.calib) {
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) recon_sq = __fadd_rn(recon_sq, __shfl_xor_sync(0xffffffffu, recon_sq, m));
        const float recon = __fsqrt_rn(recon_sq);
        if (recon > 1e-8f) stored = __fdiv_rn(norm, recon);
    }
    __syncwarp();
    const int64_t t = a.pos + s;
    uint32_t *dst = a.packed + b * a.p_sb + h * a.p_sh + t * a.p_st;
    for (int w = lane; w < pw; w += 32) dst[w] = words[w];
    if (lane == 0) a.norms[b * a.n_sb + h * a.n_sh + t * a.n_st] = stored;
}

// Dense-rotation encode for head dims that are not powers of two (fusedEncodeSource,
// TurboQuantKernels.swift:103-204): one block per row, thread d owns dimension d. Norm over the fixed tree
// (32 lanes x ceil(D/32) contiguous elements, then the xor butterfly), rotated[d] = sum_j Pi[d][j] * unit[j]
// accumulated left to right with separate multiply and add, boundary count, packing, and the norm
// correction norm / ||centroids[idx]|| over the same tree. With `calib` the rotated value is divided by
// the scale first and the correction uses centroids[idx] * scale (TurboQuantKernels.swift:354-411).
template <typename T>
__global__ void turbo_encode_dense_kernel(TurboEncodeArgs a, int64_t total_rows) {
    asm volatile("griddepcontrol.launch_dependents;");
    extern __shared__ float s_f[];           // [D] unit row, [D] tree scratch, then the packed words
    const int D = a.D;
    float *unit = s_f;
    float *tree = s_f + D;
    uint32_t *words = (uint32_t *)(s_f + 2 * D + 1);   // tree has one slot past the row
    const int d = threadIdx.x;
    const int64_t row = blockIdx.x;
    if (row >= total_rows) return;
    int64_t r = row;
    const int s = (int)(r % a.S);
    r /= a.S;
    const int h = (int)(r % a.H);
    const int b = (int)(r / a.H);
    const T *src = (const T *)a.src + b * a.s_sb + h * a.s_sh + s * a.s_ss;
    const int E = (D + 31) / 32;
    const float val = d < D ? to_float<T>(src[(int64_t)d * a.s_sd]) : 0.f;

    // sum over the fixed tree of a per-dimension quantity held in `tree`
    auto tree_sum = [&](float mine) -> float {
        if (d < D) tree[d] = mine;
        __syncthreads();
        float lane_sum = 0.f;
        if (d < 32) {
            bool first = true;
            for (int i = 0; i < E; ++i) {
                const int idx = d * E + i;
                const float x = idx < D ? tree[idx] : 0.f;
                lane_sum = first ? x : __fadd_rn(lane_sum, x);
                first = false;
            }
#pragma unroll
            for (int m = 16; m >= 1; m >>= 1) lane_sum = __fadd_rn(lane_sum, __shfl_xor_sync(0xffffffffu, lane_sum, m));
            if (d == 0) tree[D] = lane_sum;      // one slot past the row
        }
        __syncthreads();
        const float total = tree[D];
        __syncthreads();
        return total;
    };

    const float norm = __fsqrt_rn(tree_sum(__fmul_rn(val, val)));
    const float inv_norm = (norm > 1e-8f) ? __fdiv_rn(1.0f, norm) : 0.0f;
    if (d < D) unit[d] = __fmul_rn(val, inv_norm);
    const int pw = (D * a.bits + 31) / 32;
    for (int w = d; w < pw; w += blockDim.x) words[w] = 0;
    __syncthreads();
    uint32_t idx = 0;
    float recon = 0.f;
    if (d < D) {
        const float *rot = a.rotation + (int64_t)d * D;
        float acc = 0.f;
        for (int j = 0; j < D; ++j) acc = __fadd_rn(acc, __fmul_rn(rot[j], unit[j]));
        float cal = 1.f;
        if (a.calib) {
            cal = a.calib[d];
            acc = __fdiv_rn(acc, cal);
        }
        const int levels_m1 = (1 << a.bits) - 1;
        for (int bd = 0; bd < levels_m1; ++bd) idx += (acc > a.boundaries[bd]) ? 1u : 0u;
        idx &= (uint32_t)levels_m1;
        const float cv = a.calib ? __fmul_rn(a.centroids[idx], cal) : a.centroids[idx];
        recon = __fmul_rn(cv, cv);
        const int bit = d * a.bits;
        const int w = bit >> 5, sh = bit & 31;
        atomicOr(&words[w], idx << sh);
        if (sh + a.bits > 32) atomicOr(&words[w + 1], idx >> (32 - sh));
    }
    const float recon_norm = __fsqrt_rn(tree_sum(recon));
    const int64_t t = a.pos + s;
    uint32_t *dst = a.packed + b * a.p_sb + h * a.p_sh + t * a.p_st;
    for (int w = d; w < pw; w += blockDim.x) dst[w] = words[w];
    if (d == 0) a.norms[b * a.n_sb + h * a.n_sh + t * a.n_st] = (recon_norm > 1e-8f) ? __fdiv_rn(norm, recon_norm) : norm;
}

// The calibration statistic on the dense path: thread d of a row's block adds its rotated value (computed
// exactly as turbo_encode_dense_kernel computes it) to the fixed-point sums of dimension d.
template <typename T>
__global__ void turbo_calib_stats_dense_kernel(TurboEncodeArgs a, int64_t total_rows, unsigned long long *sums) {
    extern __shared__ float s_f[];           // [D] unit row, [D + 1] tree scratch
    const int D = a.D;
    float *unit = s_f;
    float *tree = s_f + D;
    const int d = threadIdx.x;
    const int64_t row = blockIdx.x;
    if (row >= total_rows) return;
    int64_t r = row;
    const int s = (int)(r % a.S);
    r /= a.S;
    const int h = (int)(r % a.H);
    const int b = (int)(r / a.H);
    const T *src = (const T *)a.src + b * a.s_sb + h * a.s_sh + s * a.s_ss;
    const int E = (D + 31) / 32;
    const float val = d < D ? to_float<T>(src[(int64_t)d * a.s_sd]) : 0.f;
    if (d < D) tree[d] = __fmul_rn(val, val);
    __syncthreads();
    if (d < 32) {
        float lane_sum = 0.f;
        bool first = true;
        for (int i = 0; i < E; ++i) {
            const int idx = d * E + i;
            const float x = idx < D ? tree[idx] : 0.f;
            lane_sum = first ? x : __fadd_rn(lane_sum, x);
            first = false;
        }
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) lane_sum = __fadd_rn(lane_sum, __shfl_xor_sync(0xffffffffu, lane_sum, m));
        if (d == 0) tree[D] = lane_sum;
    }
    __syncthreads();
    const float norm = __fsqrt_rn(tree[D]);
    const float inv_norm = (norm > 1e-8f) ? __fdiv_rn(1.0f, norm) : 0.0f;
    if (d < D) unit[d] = __fmul_rn(val, inv_norm);
    __syncthreads();
    if (d < D) {
        const float *rot = a.rotation + (int64_t)d * D;
        float acc = 0.f;
        for (int j = 0; j < D; ++j) acc = __fadd_rn(acc, __fmul_rn(rot[j], unit[j]));
        atomicAdd(&sums[d], (unsigned long long)__float2ll_rn(__fmul_rn(acc, 1073741824.0f)));
        atomicAdd(&sums[D + d], (unsigned long long)__float2ll_rn(__fmul_rn(__fmul_rn(acc, acc), 68719476736.0f)));
    }
}

// Fixed-point per-dimension sums of the rotated unit rows (see launch_turbo_calib_stats). One warp per
// row at a time, rows strided over the grid; a block folds its warps in shared memory and adds once
// per dimension to the global sums. The rotated values are computed exactly as turbo_encode_kernel
// computes the ones it quantises.
template <typename T, int E>
__global__ void __launch_bounds__(256)
turbo_calib_stats_kernel(TurboEncodeArgs a, int64_t total_rows, float inv_sqrt_dim, unsigned long long *sums) {
    constexpr int D = E * 32;
    __shared__ unsigned long long s_sum[2 * D];
    for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) s_sum[i] = 0ull;
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int warps = blockDim.x >> 5;
    long long acc1[E], acc2[E];
#pragma unroll
    for (int i = 0; i < E; ++i) { acc1[i] = 0; acc2[i] = 0; }
    for (int64_t row = (int64_t)blockIdx.x * warps + (threadIdx.x >> 5); row < total_rows; row += (int64_t)gridDim.x * warps) {
        int64_t r = row;
        const int s = (int)(r % a.S);
        r /= a.S;
        const int h = (int)(r % a.H);
        const int b = (int)(r / a.H);
        const T *src = (const T *)a.src + b * a.s_sb + h * a.s_sh + s * a.s_ss;
        float v[E];
#pragma unroll
        for (int i = 0; i < E; ++i) v[i] = to_float<T>(src[(int64_t)(lane * E + i) * a.s_sd]);
        float sq = __fmul_rn(v[0], v[0]);
#pragma unroll
        for (int i = 1; i < E; ++i) sq = __fadd_rn(sq, __fmul_rn(v[i], v[i]));
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) sq = __fadd_rn(sq, __shfl_xor_sync(0xffffffffu, sq, m));
        const float norm = __fsqrt_rn(sq);
        const float inv_norm = (norm > 1e-8f) ? __fdiv_rn(1.0f, norm) : 0.0f;
#pragma unroll
        for (int i = 0; i < E; ++i) v[i] = __fmul_rn(v[i], __fmul_rn(inv_norm, a.signs[lane * E + i]));
#pragma unroll
        for (int st = 1; st < E; st <<= 1) {
#pragma unroll
            for (int i = 0; i < E; ++i) {
                if ((i & st) == 0) {
                    const float lo = v[i], hi = v[i + st];
                    v[i] = __fadd_rn(lo, hi);
                    v[i + st] = __fsub_rn(lo, hi);
                }
            }
        }
#pragma unroll
        for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
            for (int i = 0; i < E; ++i) {
                const float other = __shfl_xor_sync(0xffffffffu, v[i], m);
                v[i] = (lane & m) ? __fsub_rn(other, v[i]) : __fadd_rn(other, v[i]);
            }
        }
#pragma unroll
        for (int i = 0; i < E; ++i) {
            const float rot = __fmul_rn(v[i], inv_sqrt_dim);
            acc1[i] += __float2ll_rn(__fmul_rn(rot, 1073741824.0f));                       // 2^30
            acc2[i] += __float2ll_rn(__fmul_rn(__fmul_rn(rot, rot), 68719476736.0f));      // 2^36
        }
    }
#pragma unroll
    for (int i = 0; i < E; ++i) {
        atomicAdd(&s_sum[lane * E + i], (unsigned long long)acc1[i]);
        atomicAdd(&s_sum[D + lane * E + i], (unsigned long long)acc2[i]);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 2 * D; i += blockDim.x)
        if (s_sum[i]) atomicAdd(&sums[i], s_sum[i]);
}

// E consecutive elements of a contiguous row in as few loads as their size allows.
template <typename T, int E>
__device__ __forceinline__ void load_row_elems(const T *p, float (&v)[E]) {
    constexpr int BYTES = E * (int)sizeof(T);
    if constexpr (BYTES % 16 == 0) {
        uint4 raw[BYTES / 16];
#pragma unroll
        for (int i = 0; i < BYTES / 16; ++i) raw[i] = __ldg(reinterpret_cast<const uint4 *>(p) + i);
        const T *e = reinterpret_cast<const T *>(raw);
#pragma unroll
        for (int i = 0; i < E; ++i) v[i] = to_float<T>(e[i]);
    } else if constexpr (BYTES == 8) {
        const uint2 raw = __ldg(reinterpret_cast<const uint2 *>(p));
        const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
        for (int i = 0; i < E; ++i) v[i] = to_float<T>(e[i]);
    } else if constexpr (BYTES == 4) {
        const uint32_t raw = __ldg(reinterpret_cast<const uint32_t *>(p));
        const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
        for (int i = 0; i < E; ++i) v[i] = to_float<T>(e[i]);
    } else {
#pragma unroll
        for (int i = 0; i < E; ++i) v[i] = to_float<T>(p[i]);
    }
}

// The same encode for contiguous rows with E <= 8: vector loads, R rows per warp in flight, the
// boundary count as a binary search over a shared-memory copy when the boundaries ascend (`sorted`),
// the cross-lane butterfly as one fused multiply-add per value (x * (+-1) + other rounds once, like
// the add or subtract it replaces), and the packed words assembled by shuffles. Grid: x = chunks of
// consecutive tokens, y = head, z = batch (keys first, then values): a block works on one (tensor,
// batch, head). Arithmetic and reduction order are those of turbo_encode_kernel, so norms and codes
// are the same bits.
template <typename T, int E, int R>
__device__ __forceinline__ void turbo_encode_vec_body(const TurboEncodeArgs &a, int b, float inv_sqrt_dim, int sorted,
                                                      float *s_bnd) {
    const int lane = threadIdx.x & 31;
    const int bits = a.bits;
    const int levels_m1 = (1 << bits) - 1;
    // unused upper entries hold +inf, so a search of fixed depth 4 serves every bit width
    if (threadIdx.x < 15) s_bnd[threadIdx.x] = threadIdx.x < levels_m1 ? a.boundaries[threadIdx.x] : __int_as_float(0x7f800000);
    __syncthreads();
    const int h = blockIdx.y;
    const int s0 = (blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * R;
    if (s0 >= a.S) return;  // whole warp
    const T *src = (const T *)a.src + b * a.s_sb + h * a.s_sh + lane * E;
    uint32_t *packed = a.packed + b * a.p_sb + h * a.p_sh + a.pos * a.p_st;
    float *norms = a.norms + b * a.n_sb + h * a.n_sh + a.pos * a.n_st;

    float v[R][E];
    float sg[E];
    load_row_elems<float, E>(a.signs + lane * E, sg);
#pragma unroll
    for (int r = 0; r < R; ++r) {
#pragma unroll
        for (int i = 0; i < E; ++i) v[r][i] = 0.f;
        if (s0 + r < a.S) load_row_elems<T, E>(src + (s0 + r) * a.s_ss, v[r]);
    }

    // L2 norm over the fixed reduction tree
    float sq[R], norm[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        sq[r] = __fmul_rn(v[r][0], v[r][0]);
#pragma unroll
        for (int i = 1; i < E; ++i) sq[r] = __fadd_rn(sq[r], __fmul_rn(v[r][i], v[r][i]));
    }
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1)
#pragma unroll
        for (int r = 0; r < R; ++r) sq[r] = __fadd_rn(sq[r], __shfl_xor_sync(0xffffffffu, sq[r], m));
#pragma unroll
    for (int r = 0; r < R; ++r) {
        norm[r] = __fsqrt_rn(sq[r]);
        const float inv_norm = (norm[r] > 1e-8f) ? __frcp_rn(norm[r]) : 0.0f;
#pragma unroll
        for (int i = 0; i < E; ++i) v[r][i] = __fmul_rn(v[r][i], __fmul_rn(inv_norm, sg[i]));
        // in-lane butterfly stages
#pragma unroll
        for (int st = 1; st < E; st <<= 1)
#pragma unroll
            for (int i = 0; i < E; ++i)
                if ((i & st) == 0) {
                    const float lo = v[r][i], hi = v[r][i + st];
                    v[r][i] = __fadd_rn(lo, hi);
                    v[r][i + st] = __fsub_rn(lo, hi);
                }
    }
    // cross-lane stages: the upper lane of a pair takes other - own, the lower one other + own
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {
        const float sign = (lane & m) ? -1.f : 1.f;
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int i = 0; i < E; ++i) v[r][i] = __fmaf_rn(v[r][i], sign, __shfl_xor_sync(0xffffffffu, v[r][i], m));
    }

    const int nb = E * bits;               // bits per lane = words per row (<= 32)
#pragma unroll
    for (int r = 0; r < R; ++r) {
        uint32_t chunk = 0;
#pragma unroll
        for (int i = E - 1; i >= 0; --i) {
            const float rotated = __fmul_rn(v[r][i], inv_sqrt_dim);
            uint32_t idx = 0;
            if (sorted) {
#pragma unroll
                for (int step = 8; step >= 1; step >>= 1)
                    if (rotated > s_bnd[idx + step - 1]) idx += step;
            } else {
                for (int bd = 0; bd < levels_m1; ++bd) idx += (rotated > s_bnd[bd]) ? 1u : 0u;
            }
            chunk = (chunk << bits) | idx;
        }
        const bool live = s0 + r < a.S;
        uint32_t *dst = packed + (s0 + r) * a.p_st;
        if (nb == 32) {
            if (live) dst[lane] = chunk;
        } else if ((nb & (nb - 1)) == 0) {
            // 32 / nb lanes per word: fold neighbours in with a shuffle tree
            uint32_t word = chunk;
            for (int span = 1, sh = nb; sh < 32; span <<= 1, sh <<= 1)
                word |= __shfl_down_sync(0xffffffffu, word, span) << sh;
            const int lpw = 32 / nb;
            if (live && (lane & (lpw - 1)) == 0) dst[lane / lpw] = word;
        } else if (nb == 12) {
            // eight lanes hold 96 bits = three words: pairs (24 bits), quads (48 bits), then the octet
            const uint32_t pair = chunk | (__shfl_down_sync(0xffffffffu, chunk, 1) << 12);
            const uint64_t quad = (uint64_t)pair | ((uint64_t)__shfl_down_sync(0xffffffffu, pair, 2) << 24);
            const uint32_t hi_lo = __shfl_down_sync(0xffffffffu, (uint32_t)quad, 4);
            const uint32_t hi_hi = __shfl_down_sync(0xffffffffu, (uint32_t)(quad >> 32), 4);
            const uint64_t upper = (uint64_t)hi_lo | ((uint64_t)hi_hi << 32);   // bits 48..95 of the octet
            if (live && (lane & 7) == 0) {
                uint32_t *w = dst + (lane >> 3) * 3;
                w[0] = (uint32_t)quad;
                w[1] = (uint32_t)(quad >> 32) | (uint32_t)(upper << 16);
                w[2] = (uint32_t)(upper >> 16);
            }
        } else {
            // lane j holds bits [j nb, (j + 1) nb) of the row; lane w gathers word w
            const int j0 = (32 * lane) / nb;
            uint32_t word = 0;
            for (int k = 0; k <= 32 / nb + 1; ++k) {
                const int j = j0 + k;
                const uint32_t c = __shfl_sync(0xffffffffu, chunk, j & 31);
                const int lo = j * nb - 32 * lane;  // where lane j's chunk starts inside this word
                if (j < 32 && lo < 32) word |= lo >= 0 ? c << lo : c >> (-lo);
            }
            if (live && lane < nb) dst[lane] = word;
        }
        if (live && lane == 0) norms[(s0 + r) * a.n_st] = norm[r];
    }
}

template <typename T, int E, int R>
__global__ void __launch_bounds__(256)
turbo_encode_vec_kernel(TurboEncodeArgs ka, TurboEncodeArgs va, float inv_sqrt_dim, int sorted) {
    asm volatile("griddepcontrol.launch_dependents;");
    __shared__ float s_bnd[16];
    // keys and values share B, H and S; the branch is uniform over the block
    if ((int)blockIdx.z >= ka.B) turbo_encode_vec_body<T, E, R>(va, (int)blockIdx.z - ka.B, inv_sqrt_dim, sorted, s_bnd);
    else turbo_encode_vec_body<T, E, R>(ka, (int)blockIdx.z, inv_sqrt_dim, sorted, s_bnd);
}

template <typename T>
void turbo_dispatch(const TurboEncodeArgs &k, const TurboEncodeArgs &v, bool have_v, cudaStream_t stream) {
    const int64_t k_rows = (int64_t)k.B * k.H * k.S;
    const int64_t v_rows = have_v ? (int64_t)v.B * v.H * v.S : 0;
    const int64_t total = k_rows + v_rows;
    const int warps = 4;
    const unsigned blocks = (unsigned)((total + warps - 1) / warps);
    const size_t smem = warps * ((1024 * 4 + 31) / 32) * sizeof(uint32_t);
    const float inv_sqrt_dim = 1.0f / sqrtf((float)k.D);
    const int E = k.D / 32;
    auto vec_ok = [&](const TurboEncodeArgs &a) {
        if (a.s_sd != 1 || a.s_sb % E || a.s_sh % E || a.s_ss % E) return false;
        return (reinterpret_cast<uintptr_t>(a.src) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.signs) & 15) == 0;
    };
    auto ascending = [](const TurboEncodeArgs &a) {
        for (int i = 0; i + 2 < (1 << a.bits); ++i)
            if (!(a.boundaries[i] <= a.boundaries[i + 1])) return false;
        return true;
    };
    const bool same_dims = !have_v || (k.B == v.B && k.H == v.H && k.S == v.S);
    const bool calibrated = k.calib || (have_v && v.calib);   // calibrated rows take the generic kernel
    if (!calibrated && E <= 8 && same_dims && vec_ok(k) && (!have_v || vec_ok(v)) && k.H <= 65535 && 2 * (int64_t)k.B <= 65535) {
        const int sorted = ascending(k) && (!have_v || ascending(v)) ? 1 : 0;
        const bool deep = k.S >= 16;
        const int rpw = deep ? 2 : 1;
        const int vw = std::max(1, std::min(8, (k.S + rpw - 1) / rpw));
        const dim3 grid((unsigned)((k.S + vw * rpw - 1) / (vw * rpw)), (unsigned)k.H, (unsigned)(k.B * (have_v ? 2 : 1)));
#define KVC_TV(EE)                                                                                        \
    do {                                                                                                  \
        if (deep) turbo_encode_vec_kernel<T, EE, 2><<<grid, vw * 32, 0, stream>>>(k, v, inv_sqrt_dim, sorted); \
        else turbo_encode_vec_kernel<T, EE, 1><<<grid, vw * 32, 0, stream>>>(k, v, inv_sqrt_dim, sorted);      \
    } while (0)
        switch (E) {
            case 1: KVC_TV(1); break;
            case 2: KVC_TV(2); break;
            case 4: KVC_TV(4); break;
            default: KVC_TV(8); break;
        }
#undef KVC_TV
        KVC_CUDA(cudaGetLastError());
        ++g_launch_count;
        return;
    }
#define KVC_TE(EE)                                                                               \
    turbo_encode_kernel<T, EE><<<blocks, warps * 32, smem, stream>>>(k, v, k_rows, total, inv_sqrt_dim)
    switch (k.D / 32) {
        case 1: KVC_TE(1); break;
        case 2: KVC_TE(2); break;
        case 4: KVC_TE(4); break;
        case 8: KVC_TE(8); break;
        case 16: KVC_TE(16); break;
        case 32: KVC_TE(32); break;
        default: fail(KVC_ERR_UNSUPPORTED, "turbo encode: head dim must be a power of two in [32, 1024]");
    }
#undef KVC_TE
    KVC_CUDA(cudaGetLastError());
    ++g_launch_count;
}

}  // namespace

static void launch_turbo_encode_dense(const TurboEncodeArgs &a, cudaStream_t stream) {
    const int64_t rows = (int64_t)a.B * a.H * a.S;
    if (rows == 0) return;
    KVC_REQUIRE(a.bits >= 1 && a.bits <= 4, "turbo encode supports 1..4 bits");
    KVC_REQUIRE(a.D >= 2 && a.D <= 1024, "turbo encode (dense rotation) supports head dims up to 1024");
    const int threads = std::max(32, ((a.D + 31) / 32) * 32);
    const size_t smem = (size_t)(2 * a.D + 1) * sizeof(float) + (size_t)((a.D * a.bits + 31) / 32 + 1) * sizeof(uint32_t);
    switch (a.dtype) {
        case KVC_F32: turbo_encode_dense_kernel<float><<<(unsigned)rows, threads, smem, stream>>>(a, rows); break;
        case KVC_F16: turbo_encode_dense_kernel<__half><<<(unsigned)rows, threads, smem, stream>>>(a, rows); break;
        case KVC_BF16: turbo_encode_dense_kernel<__nv_bfloat16><<<(unsigned)rows, threads, smem, stream>>>(a, rows); break;
        default: fail(KVC_ERR_INVALID_ARG, "turbo encode needs a floating dtype");
    }
    KVC_CUDA(cudaGetLastError());
    ++g_launch_count;
}

void launch_turbo_encode2(const TurboEncodeArgs &k, const TurboEncodeArgs *v, cudaStream_t stream) {
    if ((int64_t)k.B * k.H * k.S == 0) return;
    if (k.rotation || (v && v->rotation)) {
        // dense rotations: one launch per tensor
        KVC_REQUIRE(k.rotation && (!v || v->rotation), "turbo encode: keys and values must both use the dense rotation");
        launch_turbo_encode_dense(k, stream);
        if (v) launch_turbo_encode_dense(*v, stream);
        return;
    }
    KVC_REQUIRE(k.bits >= 1 && k.bits <= 4, "turbo encode supports 1..4 bits");
    KVC_REQUIRE(k.D >= 32 && k.D <= 1024 && (k.D & (k.D - 1)) == 0,
                "turbo encode (Walsh-Hadamard path) needs a power-of-two head dim in [32, 1024]");
    if (v) {
        KVC_REQUIRE(v->D == k.D && v->dtype == k.dtype, "turbo encode: K and V must share dim and dtype");
        KVC_REQUIRE(v->bits >= 1 && v->bits <= 4, "turbo encode supports 1..4 bits");
    }
    const TurboEncodeArgs &vv = v ? *v : k;
    switch (k.dtype) {
        case KVC_F32: turbo_dispatch<float>(k, vv, v != nullptr, stream); break;
        case KVC_F16: turbo_dispatch<__half>(k, vv, v != nullptr, stream); break;
        case KVC_BF16: turbo_dispatch<__nv_bfloat16>(k, vv, v != nullptr, stream); break;
        default: fail(KVC_ERR_INVALID_ARG, "turbo encode needs a floating dtype");
    }
}

void launch_turbo_encode(const TurboEncodeArgs &a, cudaStream_t stream) {
    launch_turbo_encode2(a, nullptr, stream);
}

void launch_turbo_calib_stats(const TurboEncodeArgs &a, long long *sums, cudaStream_t stream) {
    const int64_t rows = (int64_t)a.B * a.H * a.S;
    if (rows == 0) return;
    if (a.rotation) {
        const int threads = std::max(32, ((a.D + 31) / 32) * 32);
        const size_t smem = (size_t)(2 * a.D + 1) * sizeof(float);
        unsigned long long *o = reinterpret_cast<unsigned long long *>(sums);
        switch (a.dtype) {
            case KVC_F32: turbo_calib_stats_dense_kernel<float><<<(unsigned)rows, threads, smem, stream>>>(a, rows, o); break;
            case KVC_F16: turbo_calib_stats_dense_kernel<__half><<<(unsigned)rows, threads, smem, stream>>>(a, rows, o); break;
            case KVC_BF16: turbo_calib_stats_dense_kernel<__nv_bfloat16><<<(unsigned)rows, threads, smem, stream>>>(a, rows, o); break;
            default: fail(KVC_ERR_INVALID_ARG, "key calibration needs a floating dtype");
        }
        KVC_CUDA(cudaGetLastError());
        ++g_launch_count;
        return;
    }
    KVC_REQUIRE(a.D >= 32 && a.D <= 1024 && (a.D & (a.D - 1)) == 0,
                "key calibration (Walsh-Hadamard path) needs a power-of-two head dim in [32, 1024]");
    const float inv_sqrt_dim = 1.0f / sqrtf((float)a.D);
    const int warps = 8;
    const unsigned blocks = (unsigned)std::min<int64_t>((rows + warps - 1) / warps, (int64_t)sm_count(current_device()) * 8);
    unsigned long long *out = reinterpret_cast<unsigned long long *>(sums);
#define KVC_CS(TT)                                                                                                \
    switch (a.D / 32) {                                                                                           \
        case 1: turbo_calib_stats_kernel<TT, 1><<<blocks, warps * 32, 0, stream>>>(a, rows, inv_sqrt_dim, out); break; \
        case 2: turbo_calib_stats_kernel<TT, 2><<<blocks, warps * 32, 0, stream>>>(a, rows, inv_sqrt_dim, out); break; \
        case 4: turbo_calib_stats_kernel<TT, 4><<<blocks, warps * 32, 0, stream>>>(a, rows, inv_sqrt_dim, out); break; \
        case 8: turbo_calib_stats_kernel<TT, 8><<<blocks, warps * 32, 0, stream>>>(a, rows, inv_sqrt_dim, out); break; \
        case 16: turbo_calib_stats_kernel<TT, 16><<<blocks, warps * 32, 0, stream>>>(a, rows, inv_sqrt_dim, out); break; \
        default: turbo_calib_stats_kernel<TT, 32><<<blocks, warps * 32, 0, stream>>>(a, rows, inv_sqrt_dim, out); break; \
    }
    switch (a.dtype) {
        case KVC_F32: KVC_CS(float) break;
        case KVC_F16: KVC_CS(__half) break;
        case KVC_BF16: KVC_CS(__nv_bfloat16) break;
        default: fail(KVC_ERR_INVALID_ARG, "key calibration needs a floating dtype");
    }
#undef KVC_CS
    KVC_CUDA(cudaGetLastError());
    ++g_launch_count;
}

}  // namespace kvc
