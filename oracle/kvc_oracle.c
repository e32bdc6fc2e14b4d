/*
 * kvc_oracle.c -- CPU restatement of the arithmetic on mlx-swift-lm's KV-cache
 * hot path. TEST INFRASTRUCTURE ONLY: it is the checker the CUDA library is
 * compared against (tests/, the smoke check) and the timed CPU baseline of the
 * benchmark; nothing in the shipped library links or calls it.
 *
 * Parity status. The cache state machines, bit packing, the Walsh-Hadamard
 * encode and the attention math follow source that is in the reference tree
 * and are pinned by the reference's own test expectations (see
 * tests/test_oracle_pins.py). The group-wise affine quantiser and the random
 * sign stream live in the un-vendored dependency ml-explore/mlx-swift
 * (Package.swift:64, .upToNextMinor(from: "0.31.6"), i.e. MLX core 0.31.x):
 * the quantiser below restates MLX's published `affine_quantize` algorithm and
 * is "parity unpinned" (no golden vector for it exists in the reference); the
 * sign stream is this project's own seeded generator.
 *
 * What each function follows (paths inside the reference project):
 *   orc_affine_quantize    MLX quantize(), affine mode; call sites
 *                          Libraries/MLXLMCommon/KVCache.swift:506-509, :1069-1070;
 *                          code layout pinned by TurboQuantKernels.swift:820-831
 *   orc_affine_dequantize  MLX dequantize(); KVCache.swift:1197-1202
 *   orc_turbo_encode       fusedEncodeWHT, TurboQuantKernels.swift:224-342 and
 *                          MSECodec.encode, TurboQuantKVCache.swift:517-566
 *   orc_pack / orc_unpack  TurboQuantPacking, TurboQuantKVCache.swift:351-424
 *   orc_fwht               whtButterfly, TurboQuantKVCache.swift:302-325
 *   orc_codebook           TurboQuantCodebook.generateCentroids, :174-233
 *   orc_turbo_encode_scaled / orc_turbo_calib_sums   key calibration, :867-886,
 *                          TurboQuantKernels.swift:354-411
 *   orc_attention          quantizedScaledDotProductAttention KVCache.swift:2351-2447,
 *                          MLXFast.scaledDotProductAttention as called at
 *                          AttentionUtils.swift:86-93, and the turbo flash kernels
 *                          TurboQuantKernels.swift:424-542, :879-1026, :1396-1519
 *
 * Floating-point contract shared with the CUDA kernels for the integer
 * outputs (codes must be bit-identical): IEEE single precision, no fused
 * multiply-add (build with -ffp-contract=off), and one reduction tree for the
 * sum of squares of a row: 32 "lanes" each own E = ceil(D/32) contiguous
 * elements summed left to right, then lanes combine over the xor butterfly
 * 16, 8, 4, 2, 1.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

enum { ORC_F32 = 0, ORC_F16 = 1, ORC_BF16 = 2 };

static inline float bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u); /* NaN */
    u += 0x7fffu + ((u >> 16) & 1u); /* round to nearest even */
    return (uint16_t)(u >> 16);
}

static inline float ld(const void *p, int dtype, int64_t i) {
    switch (dtype) {
        case ORC_F32: return ((const float *)p)[i];
        case ORC_F16: return (float)((const _Float16 *)p)[i];
        default: return bf16_to_f32(((const uint16_t *)p)[i]);
    }
}

static inline void st(void *p, int dtype, int64_t i, float v) {
    switch (dtype) {
        case ORC_F32: ((float *)p)[i] = v; break;
        case ORC_F16: ((_Float16 *)p)[i] = (_Float16)v; break;
        default: ((uint16_t *)p)[i] = f32_to_bf16(v); break;
    }
}

/* ------------------------------------------------------------------ */
/* affine group quantisation                                           */
/* ------------------------------------------------------------------ */

static void affine_params(float w_min, float w_max, float n_bins, float *scale, float *bias) {
    float s = fmaxf((w_max - w_min) / n_bins, 1e-7f);
    const int side = fabsf(w_min) > fabsf(w_max);
    s = side ? s : -s;
    const float edge = side ? w_min : w_max;
    const float q0 = rintf(edge / s);
    float b = 0.f;
    if (q0 != 0.f) {
        s = edge / q0;
        b = edge;
    }
    *scale = s;
    *bias = b;
}

void orc_affine_quantize(const void *x, int dtype, int64_t rows, int D, int group, int bits,
                         uint32_t *codes, void *scales, void *biases) {
    const int gpr = D / group;
    const int wpr = D * bits / 32;
    const int per_word = 32 / bits;
    const float n_bins = (float)((1 << bits) - 1);
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        for (int g = 0; g < gpr; ++g) {
            const int64_t base = r * D + (int64_t)g * group;
            float w_min = ld(x, dtype, base), w_max = w_min;
            for (int i = 1; i < group; ++i) {
                const float v = ld(x, dtype, base + i);
                w_min = fminf(w_min, v);
                w_max = fmaxf(w_max, v);
            }
            float scale, bias;
            affine_params(w_min, w_max, n_bins, &scale, &bias);
            st(scales, dtype, r * gpr + g, scale);
            st(biases, dtype, r * gpr + g, bias);
            uint32_t *dst = codes + r * wpr + (int64_t)g * group * bits / 32;
            for (int w = 0; w < group / per_word; ++w) {
                uint32_t word = 0;
                for (int k = 0; k < per_word; ++k) {
                    float q = rintf((ld(x, dtype, base + w * per_word + k) - bias) / scale);
                    q = fminf(fmaxf(q, 0.f), n_bins);
                    word |= (uint32_t)q << (k * bits);
                }
                dst[w] = word;
            }
        }
    }
}

void orc_affine_dequantize(const uint32_t *codes, const void *scales, const void *biases, int dtype,
                           int64_t rows, int D, int group, int bits, void *out) {
    const int gpr = D / group;
    const int wpr = D * bits / 32;
    const uint32_t mask = (1u << bits) - 1u;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        for (int d = 0; d < D; ++d) {
            const uint32_t code = (codes[r * wpr + (d * bits) / 32] >> ((d * bits) % 32)) & mask;
            const float sc = ld(scales, dtype, r * gpr + d / group);
            const float bi = ld(biases, dtype, r * gpr + d / group);
            st(out, dtype, r * D + d, sc * (float)code + bi);
        }
    }
}

/* ------------------------------------------------------------------ */
/* TurboQuant: packing, butterfly, encode, codebook                    */
/* ------------------------------------------------------------------ */

int orc_packed_width(int count, int bits) { return (count * bits + 31) / 32; }

void orc_pack(const uint32_t *idx, int64_t rows, int count, int bits, uint32_t *packed) {
    const int pw = orc_packed_width(count, bits);
    const uint32_t mask = (1u << bits) - 1u;
    for (int64_t r = 0; r < rows; ++r) {
        uint32_t *w = packed + r * pw;
        memset(w, 0, (size_t)pw * 4);
        for (int d = 0; d < count; ++d) {
            const int bit = d * bits, wi = bit / 32, off = bit % 32;
            const uint32_t v = idx[r * count + d] & mask;
            w[wi] |= v << off;
            if (off + bits > 32) w[wi + 1] |= v >> (32 - off);
        }
    }
}

void orc_unpack(const uint32_t *packed, int64_t rows, int count, int bits, uint32_t *idx) {
    const int pw = orc_packed_width(count, bits);
    const uint32_t mask = (1u << bits) - 1u;
    for (int64_t r = 0; r < rows; ++r) {
        const uint32_t *w = packed + r * pw;
        for (int d = 0; d < count; ++d) {
            const int bit = d * bits, wi = bit / 32, off = bit % 32;
            uint32_t v = w[wi] >> off;
            if (off + bits > 32) v |= w[wi + 1] << (32 - off);
            idx[r * count + d] = v & mask;
        }
    }
}

/* Unnormalised Walsh-Hadamard transform, stage s pairs elements 2^s apart. */
static void fwht_row(float *y, int D) {
    for (int half = 1; half < D; half <<= 1)
        for (int blk = 0; blk < D; blk += 2 * half)
            for (int j = 0; j < half; ++j) {
                const float a = y[blk + j], b = y[blk + j + half];
                y[blk + j] = a + b;
                y[blk + j + half] = a - b;
            }
}

void orc_fwht(float *x, int64_t rows, int D) {
    for (int64_t r = 0; r < rows; ++r) fwht_row(x + r * D, D);
}

static float sum_squares_tree(const float *v, int D) {
    const int E = (D + 31) / 32;
    float lane[32];
    for (int l = 0; l < 32; ++l) {
        float acc = 0.f;
        int first = 1;
        for (int i = 0; i < E; ++i) {
            const int d = l * E + i;
            const float x = d < D ? v[d] : 0.f;
            const float sq = x * x;
            if (first) { acc = sq; first = 0; }
            else acc = acc + sq;
        }
        lane[l] = acc;
    }
    for (int m = 16; m >= 1; m >>= 1) {
        float next[32];
        for (int l = 0; l < 32; ++l) next[l] = lane[l] + lane[l ^ m];
        memcpy(lane, next, sizeof(lane));
    }
    return lane[0];
}

void orc_turbo_encode(const void *x, int dtype, int64_t rows, int D, const float *signs,
                      const float *boundaries, int bits, uint32_t *packed, float *norms) {
    const int pw = orc_packed_width(D, bits);
    const int nb = (1 << bits) - 1;
    const float inv_sqrt_dim = 1.0f / sqrtf((float)D);
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        float v[1024];
        uint32_t idx[1024];
        for (int d = 0; d < D; ++d) v[d] = ld(x, dtype, r * D + d);
        const float norm = sqrtf(sum_squares_tree(v, D));
        const float inv_norm = norm > 1e-8f ? 1.0f / norm : 0.0f;
        for (int d = 0; d < D; ++d) v[d] = v[d] * (inv_norm * signs[d]);
        fwht_row(v, D);
        for (int d = 0; d < D; ++d) {
            const float rotated = v[d] * inv_sqrt_dim;
            uint32_t k = 0;
            for (int b = 0; b < nb; ++b) k += rotated > boundaries[b] ? 1u : 0u;
            idx[d] = k;
        }
        orc_pack(idx, 1, D, bits, packed + r * pw);
        norms[r] = norm;
    }
}

/* Calibrated encode: the row is rotated as above, divided by the per-dimension
 * calibration scale before the boundary count, and the stored norm is the raw
 * norm over the norm of (centroid[idx] * scale)
 * (fusedQuantizePackScaled, TurboQuantKernels.swift:354-411; MSECodec.encode
 * with a scale, TurboQuantKVCache.swift:527-544). The reconstruction norm uses
 * the same reduction tree as the row norm. */
void orc_turbo_encode_scaled(const void *x, int dtype, int64_t rows, int D, const float *signs,
                             const float *boundaries, const float *centroids, const float *scale,
                             int bits, uint32_t *packed, float *norms) {
    const int pw = orc_packed_width(D, bits);
    const int nb = (1 << bits) - 1;
    const float inv_sqrt_dim = 1.0f / sqrtf((float)D);
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        float v[1024], recon[1024];
        uint32_t idx[1024];
        for (int d = 0; d < D; ++d) v[d] = ld(x, dtype, r * D + d);
        const float norm = sqrtf(sum_squares_tree(v, D));
        const float inv_norm = norm > 1e-8f ? 1.0f / norm : 0.0f;
        for (int d = 0; d < D; ++d) v[d] = v[d] * (inv_norm * signs[d]);
        fwht_row(v, D);
        for (int d = 0; d < D; ++d) {
            const float rotated = v[d] * inv_sqrt_dim;
            const float calibrated = rotated / scale[d];
            uint32_t k = 0;
            for (int b = 0; b < nb; ++b) k += calibrated > boundaries[b] ? 1u : 0u;
            idx[d] = k;
            recon[d] = centroids[k] * scale[d];
        }
        orc_pack(idx, 1, D, bits, packed + r * pw);
        const float recon_norm = sqrtf(sum_squares_tree(recon, D));
        norms[r] = recon_norm > 1e-8f ? norm / recon_norm : norm;
    }
}

/* Dense-rotation encode for head dims that are not powers of two (fusedEncodeSource,
 * TurboQuantKernels.swift:103-204; MSECodec.encode dense branch, TurboQuantKVCache.swift:549-554):
 * rotated[d] = sum_j Pi[d][j] * unit[j] (left to right, separate multiply and add), boundary count,
 * stored norm = norm / ||centroids[idx]|| (norm itself when that is <= 1e-8). With `scale` the rotated
 * value is divided by it first and the correction uses centroids[idx] * scale. `scale` may be NULL. */
void orc_turbo_encode_dense(const void *x, int dtype, int64_t rows, int D, const float *rotation,
                            const float *boundaries, const float *centroids, const float *scale, int bits,
                            uint32_t *packed, float *norms) {
    const int pw = orc_packed_width(D, bits);
    const int nb = (1 << bits) - 1;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        float v[1024], recon[1024];
        uint32_t idx[1024];
        for (int d = 0; d < D; ++d) v[d] = ld(x, dtype, r * D + d);
        const float norm = sqrtf(sum_squares_tree(v, D));
        const float inv_norm = norm > 1e-8f ? 1.0f / norm : 0.0f;
        for (int d = 0; d < D; ++d) v[d] = v[d] * inv_norm;
        for (int d = 0; d < D; ++d) {
            const float *rot = rotation + (size_t)d * D;
            float acc = 0.f;
            for (int j = 0; j < D; ++j) acc = acc + rot[j] * v[j];
            if (scale) acc = acc / scale[d];
            uint32_t k = 0;
            for (int b = 0; b < nb; ++b) k += acc > boundaries[b] ? 1u : 0u;
            idx[d] = k;
            recon[d] = scale ? centroids[k] * scale[d] : centroids[k];
        }
        orc_pack(idx, 1, D, bits, packed + r * pw);
        const float recon_norm = sqrtf(sum_squares_tree(recon, D));
        norms[r] = recon_norm > 1e-8f ? norm / recon_norm : norm;
    }
}

/* The calibration statistic on the dense path (same fixed-point sums as orc_turbo_calib_sums). */
void orc_turbo_calib_sums_dense(const void *x, int dtype, int64_t rows, int D, const float *rotation, int64_t *sums) {
    memset(sums, 0, sizeof(int64_t) * 2 * (size_t)D);
#pragma omp parallel
    {
        int64_t *local = (int64_t *)calloc(2 * (size_t)D, sizeof(int64_t));
#pragma omp for schedule(static)
        for (int64_t r = 0; r < rows; ++r) {
            float v[1024];
            for (int d = 0; d < D; ++d) v[d] = ld(x, dtype, r * D + d);
            const float norm = sqrtf(sum_squares_tree(v, D));
            const float inv_norm = norm > 1e-8f ? 1.0f / norm : 0.0f;
            for (int d = 0; d < D; ++d) v[d] = v[d] * inv_norm;
            for (int d = 0; d < D; ++d) {
                const float *rot = rotation + (size_t)d * D;
                float acc = 0.f;
                for (int j = 0; j < D; ++j) acc = acc + rot[j] * v[j];
                const float sq = acc * acc;
                local[d] += (int64_t)llrintf(acc * 1073741824.0f);
                local[D + d] += (int64_t)llrintf(sq * 68719476736.0f);
            }
        }
#pragma omp critical
        for (int d = 0; d < 2 * D; ++d) sums[d] += local[d];
        free(local);
    }
}

/* First and second moments of the rotated unit rows per dimension, as
 * fixed-point integers (value * 2^30 and square * 2^36, each rounded to
 * nearest): the statistic under computeKeyCalibrationScale
 * (TurboQuantKVCache.swift:867-886). Integer sums do not depend on the order of
 * the rows. sums[0..D) first moments, sums[D..2D) second moments. */
void orc_turbo_calib_sums(const void *x, int dtype, int64_t rows, int D, const float *signs, int64_t *sums) {
    const float inv_sqrt_dim = 1.0f / sqrtf((float)D);
    memset(sums, 0, sizeof(int64_t) * 2 * (size_t)D);
#pragma omp parallel
    {
        int64_t *local = (int64_t *)calloc(2 * (size_t)D, sizeof(int64_t));
#pragma omp for schedule(static)
        for (int64_t r = 0; r < rows; ++r) {
            float v[1024];
            for (int d = 0; d < D; ++d) v[d] = ld(x, dtype, r * D + d);
            const float norm = sqrtf(sum_squares_tree(v, D));
            const float inv_norm = norm > 1e-8f ? 1.0f / norm : 0.0f;
            for (int d = 0; d < D; ++d) v[d] = v[d] * (inv_norm * signs[d]);
            fwht_row(v, D);
            for (int d = 0; d < D; ++d) {
                const float rot = v[d] * inv_sqrt_dim;
                const float sq = rot * rot;
                local[d] += (int64_t)llrintf(rot * 1073741824.0f);
                local[D + d] += (int64_t)llrintf(sq * 68719476736.0f);
            }
        }
#pragma omp critical
        for (int d = 0; d < 2 * D; ++d) sums[d] += local[d];
        free(local);
    }
}

/* Float32 restatement of the reference's centroid generator: weighted k-means
 * on a 32768-point grid of the density (1-x^2)^((dim-3)/2), quantile start,
 * 100 sweeps, sorted at the end. */
void orc_codebook(int dim, int bits, float *centroids) {
    const int levels = 1 << bits;
    const int n = 32768;
    float *grid = (float *)malloc(sizeof(float) * n);
    float *wt = (float *)malloc(sizeof(float) * n);
    const float sigma = 1.0f / sqrtf((float)dim);
    const float expo = (float)(dim - 3) / 2.0f;
    float total = 0.f;
    for (int i = 0; i < n; ++i) {
        const float x = -1.0f + 2.0f * (float)i / (float)(n - 1);
        grid[i] = x;
        wt[i] = powf(fmaxf(1.0f - x * x, 1e-30f), expo);
        total += wt[i];
    }
    float cen[16] = {0};
    float cum = 0.f;
    int ci = 0;
    for (int i = 0; i < n; ++i) {
        cum += wt[i];
        const float target = ((float)ci + 0.5f) / (float)levels * total;
        if (cum >= target && ci < levels) cen[ci++] = grid[i];
    }
    while (ci < levels) { cen[ci] = cen[ci - 1] + sigma; ++ci; }
    for (int it = 0; it < 100; ++it) {
        float sums[16] = {0}, cnt[16] = {0};
        for (int i = 0; i < n; ++i) {
            int best = 0;
            float bd = INFINITY;
            for (int j = 0; j < levels; ++j) {
                const float d = fabsf(grid[i] - cen[j]);
                if (d < bd) { bd = d; best = j; }
            }
            sums[best] += grid[i] * wt[i];
            cnt[best] += wt[i];
        }
        for (int j = 0; j < levels; ++j)
            if (cnt[j] > 0) cen[j] = sums[j] / cnt[j];
    }
    for (int i = 1; i < levels; ++i) { /* insertion sort */
        const float c = cen[i];
        int j = i - 1;
        while (j >= 0 && cen[j] > c) { cen[j + 1] = cen[j]; --j; }
        cen[j + 1] = c;
    }
    memcpy(centroids, cen, sizeof(float) * levels);
    free(grid);
    free(wt);
}

/* ------------------------------------------------------------------ */
/* attention                                                           */
/* ------------------------------------------------------------------ */

enum { SRC_RAW = 0, SRC_AFFINE = 1, SRC_TURBO = 2 };
enum { MASK_NONE = 0, MASK_CAUSAL = 1, MASK_ARRAY = 2 };

typedef struct orc_source {
    int32_t kind;
    int32_t dtype;
    const void *data;
    const void *scales;
    const void *biases;
    const float *norms;
    int64_t sb, sh, st;    /* element / word strides of data */
    int64_t gsb, gsh, gst; /* strides of scales/biases or norms */
    int32_t bits, group;
    float codebook[16];
} orc_source;

typedef struct orc_attn {
    const void *q;
    void *out;
    int32_t q_dtype;
    int32_t B, Hq, Hkv, L, D;
    int64_t T;
    float scale;
    orc_source k, v;
    int32_t mask_mode;
    int32_t mask_dtype; /* 4 = bool bytes, else float dtype */
    const void *mask;
    int64_t msb, msh, msl, mst;
    int64_t causal_offset;
    const float *q_signs;
    const float *q_calib;
    const float *o_signs;
    int32_t precise; /* 1: double accumulation (checker); 0: float (timed baseline) */
    const float *q_rot; /* dense key rotation Pi [D, D]: q' = Pi q (instead of q_signs) */
    const float *o_rot; /* dense value rotation: out = o' Pi (instead of o_signs) */
} orc_attn;

static inline float src_elem(const orc_source *s, int b, int h, int64_t t, int d) {
    if (s->kind == SRC_RAW) return ld(s->data, s->dtype, b * s->sb + h * s->sh + t * s->st + d);
    const uint32_t *row = (const uint32_t *)s->data + b * s->sb + h * s->sh + t * s->st;
    const int bit = d * s->bits, wi = bit / 32, off = bit % 32;
    uint32_t val = row[wi] >> off;
    if (off + s->bits > 32) val |= row[wi + 1] << (32 - off);
    val &= (1u << s->bits) - 1u;
    if (s->kind == SRC_AFFINE) {
        const int64_t gi = b * s->gsb + h * s->gsh + t * s->gst + d / s->group;
        return ld(s->scales, s->dtype, gi) * (float)val + ld(s->biases, s->dtype, gi);
    }
    return s->codebook[val] * s->norms[b * s->gsb + h * s->gsh + t * s->gst];
}

static void load_row(const orc_source *s, int b, int h, int64_t t, int D, float *dst) {
    if (s->kind == SRC_RAW && s->dtype == ORC_BF16) {
        const uint16_t *p = (const uint16_t *)s->data + b * s->sb + h * s->sh + t * s->st;
        for (int d = 0; d < D; ++d) dst[d] = bf16_to_f32(p[d]);
        return;
    }
    if (s->kind == SRC_TURBO) {
        /* one pass over the row's bit stream instead of a word lookup per element (same values) */
        const uint32_t *row = (const uint32_t *)s->data + b * s->sb + h * s->sh + t * s->st;
        const float norm = s->norms[b * s->gsb + h * s->gsh + t * s->gst];
        const int bits = s->bits;
        const uint32_t mask = (1u << bits) - 1u;
        uint64_t buf = 0;
        int have = 0, wi = 0;
        for (int d = 0; d < D; ++d) {
            if (have < bits) { buf |= (uint64_t)row[wi++] << have; have += 32; }
            dst[d] = s->codebook[(uint32_t)buf & mask] * norm;
            buf >>= bits;
            have -= bits;
        }
        return;
    }
    for (int d = 0; d < D; ++d) dst[d] = src_elem(s, b, h, t, d);
}

/* The timed baseline's form of the same attention (float accumulation, no array mask): one pass per
 * (batch, KV head) that decodes every cached K and V row once and serves all the query rows of the
 * head group from it, the way the reference's kernels share a KV head between its query heads
 * (TurboQuantKernels.swift:424-542) instead of decoding the row again for every query head. */
/* q' = Pi q (dense forward rotation), in place with a scratch row */
static void rotate_dense(const float *rot, float *x, int D, float *tmp) {
    for (int d = 0; d < D; ++d) {
        const float *r = rot + (size_t)d * D;
        double acc = 0.0;
        for (int j = 0; j < D; ++j) acc += (double)r[j] * (double)x[j];
        tmp[d] = (float)acc;
    }
    memcpy(x, tmp, sizeof(float) * (size_t)D);
}

/* out = o' Pi (dense inverse rotation) */
static void unrotate_dense(const float *rot, float *x, int D, float *tmp) {
    for (int j = 0; j < D; ++j) {
        double acc = 0.0;
        for (int d = 0; d < D; ++d) acc += (double)x[d] * (double)rot[(size_t)d * D + j];
        tmp[j] = (float)acc;
    }
    memcpy(x, tmp, sizeof(float) * (size_t)D);
}

static void attention_grouped(const orc_attn *a) {
    const int D = a->D, L = a->L;
    const int rep = a->Hq / a->Hkv;
    const int R = rep * L;
    const int64_t T = a->T;
    const int64_t units = (int64_t)a->B * a->Hkv;
#pragma omp parallel
    {
        float *kv = (float *)malloc(sizeof(float) * D);
        float *qv = (float *)malloc(sizeof(float) * (size_t)R * D);
        float *acc = (float *)malloc(sizeof(float) * (size_t)R * D);
        float *sc = (float *)malloc(sizeof(float) * (size_t)R * (size_t)(T > 0 ? T : 1));
        float *mx = (float *)malloc(sizeof(float) * R);
        float *lsum = (float *)malloc(sizeof(float) * R);
#pragma omp for schedule(dynamic, 1)
        for (int64_t u = 0; u < units; ++u) {
            const int hk = (int)(u % a->Hkv), b = (int)(u / a->Hkv);
            for (int r = 0; r < R; ++r) {
                const int hq = hk * rep + r / L, l = r % L;
                const int64_t qbase = (((int64_t)b * a->Hq + hq) * L + l) * D;
                float *q = qv + (size_t)r * D;
                for (int d = 0; d < D; ++d) q[d] = ld(a->q, a->q_dtype, qbase + d);
                if (a->q_signs) {
                    for (int d = 0; d < D; ++d) q[d] *= a->q_signs[d];
                    fwht_row(q, D);
                    const float f = 1.0f / sqrtf((float)D);
                    for (int d = 0; d < D; ++d) {
                        q[d] = q[d] * f * a->scale;
                        if (a->q_calib) q[d] *= a->q_calib[d];
                    }
                } else if (a->q_rot) {
                    rotate_dense(a->q_rot, q, D, kv);
                    for (int d = 0; d < D; ++d) {
                        q[d] = q[d] * a->scale;
                        if (a->q_calib) q[d] *= a->q_calib[d];
                    }
                } else {
                    for (int d = 0; d < D; ++d) q[d] *= a->scale;
                }
                mx[r] = -INFINITY;
                lsum[r] = 0.f;
                for (int d = 0; d < D; ++d) acc[(size_t)r * D + d] = 0.f;
            }
            for (int64_t t = 0; t < T; ++t) {
                load_row(&a->k, b, hk, t, D, kv);
                for (int r = 0; r < R; ++r) {
                    const int l = r % L;
                    float s2 = -INFINITY;
                    if (a->mask_mode != MASK_CAUSAL || t <= a->causal_offset + l) {
                        const float *q = qv + (size_t)r * D;
                        s2 = 0.f;
                        for (int d = 0; d < D; ++d) s2 += q[d] * kv[d];
                        if (s2 > mx[r]) mx[r] = s2;
                    }
                    sc[(size_t)r * T + t] = s2;
                }
            }
            for (int64_t t = 0; t < T; ++t) {
                load_row(&a->v, b, hk, t, D, kv);
                for (int r = 0; r < R; ++r) {
                    const float s2 = sc[(size_t)r * T + t];
                    if (s2 == -INFINITY) continue;
                    const float p = expf(s2 - mx[r]);
                    lsum[r] += p;
                    float *o = acc + (size_t)r * D;
                    for (int d = 0; d < D; ++d) o[d] += p * kv[d];
                }
            }
            for (int r = 0; r < R; ++r) {
                const int hq = hk * rep + r / L, l = r % L;
                const int64_t qbase = (((int64_t)b * a->Hq + hq) * L + l) * D;
                float *o = acc + (size_t)r * D;
                const float inv = lsum[r] > 0.f ? 1.0f / lsum[r] : 0.f;
                for (int d = 0; d < D; ++d) o[d] *= inv;
                if (a->o_signs) {
                    fwht_row(o, D);
                    const float f = 1.0f / sqrtf((float)D);
                    for (int d = 0; d < D; ++d) o[d] = o[d] * f * a->o_signs[d];
                } else if (a->o_rot) {
                    unrotate_dense(a->o_rot, o, D, kv);
                }
                for (int d = 0; d < D; ++d) st(a->out, a->q_dtype, qbase + d, o[d]);
            }
        }
        free(kv); free(qv); free(acc); free(sc); free(mx); free(lsum);
    }
}

void orc_attention(const orc_attn *a) {
    const int D = a->D, L = a->L;
    const int rep = a->Hq / a->Hkv;
    const int64_t T = a->T;
    const int64_t work = (int64_t)a->B * a->Hq * L;
    if (!a->precise && a->mask_mode != MASK_ARRAY) {
        attention_grouped(a);
        return;
    }
#pragma omp parallel
    {
        float *kv = (float *)malloc(sizeof(float) * D);
        float *qv = (float *)malloc(sizeof(float) * D);
        double *acc = (double *)malloc(sizeof(double) * D);
        float *accf = (float *)malloc(sizeof(float) * D);
        double *sc = (double *)malloc(sizeof(double) * (size_t)(T > 0 ? T : 1));
#pragma omp for schedule(dynamic, 1)
        for (int64_t w = 0; w < work; ++w) {
            const int l = (int)(w % L);
            const int hq = (int)((w / L) % a->Hq);
            const int b = (int)(w / ((int64_t)L * a->Hq));
            const int hk = hq / rep;
            const int64_t qbase = (((int64_t)b * a->Hq + hq) * L + l) * D;
            for (int d = 0; d < D; ++d) qv[d] = ld(a->q, a->q_dtype, qbase + d);
            if (a->q_signs) {
                for (int d = 0; d < D; ++d) qv[d] *= a->q_signs[d];
                fwht_row(qv, D);
                const float f = 1.0f / sqrtf((float)D);
                for (int d = 0; d < D; ++d) {
                    qv[d] = qv[d] * f * a->scale;
                    if (a->q_calib) qv[d] *= a->q_calib[d];
                }
            } else if (a->q_rot) {
                rotate_dense(a->q_rot, qv, D, kv);
                for (int d = 0; d < D; ++d) {
                    qv[d] = qv[d] * a->scale;
                    if (a->q_calib) qv[d] *= a->q_calib[d];
                }
            } else {
                for (int d = 0; d < D; ++d) qv[d] *= a->scale;
            }
            /* scores */
            double mx = -INFINITY;
            for (int64_t t = 0; t < T; ++t) {
                int keep = 1;
                double add = 0.0;
                if (a->mask_mode == MASK_CAUSAL) keep = t <= a->causal_offset + l;
                else if (a->mask_mode == MASK_ARRAY) {
                    const int64_t mi = b * a->msb + hq * a->msh + l * a->msl + t * a->mst;
                    if (a->mask_dtype == 4) keep = ((const uint8_t *)a->mask)[mi] != 0;
                    else add = ld(a->mask, a->mask_dtype, mi);
                }
                if (!keep) { sc[t] = -INFINITY; continue; }
                load_row(&a->k, b, hk, t, D, kv);
                double s;
                if (a->precise) {
                    double s2 = 0.0;
                    for (int d = 0; d < D; ++d) s2 += (double)qv[d] * (double)kv[d];
                    s = s2;
                } else {
                    float s2 = 0.f;
                    for (int d = 0; d < D; ++d) s2 += qv[d] * kv[d];
                    s = s2;
                }
                s += add;
                sc[t] = s;
                if (s > mx) mx = s;
            }
            /* softmax + weighted sum */
            double lsum = 0.0;
            for (int d = 0; d < D; ++d) { acc[d] = 0.0; accf[d] = 0.f; }
            if (mx != -INFINITY) {
                for (int64_t t = 0; t < T; ++t) {
                    if (sc[t] == -INFINITY) continue;
                    const double p = exp(sc[t] - mx);
                    lsum += p;
                    load_row(&a->v, b, hk, t, D, kv);
                    if (a->precise) for (int d = 0; d < D; ++d) acc[d] += p * (double)kv[d];
                    else { const float pf = (float)p; for (int d = 0; d < D; ++d) accf[d] += pf * kv[d]; }
                }
            }
            const double inv = lsum > 0.0 ? 1.0 / lsum : 0.0;
            for (int d = 0; d < D; ++d) qv[d] = (float)((a->precise ? acc[d] : (double)accf[d]) * inv);
            if (a->o_signs) {
                fwht_row(qv, D);
                const float f = 1.0f / sqrtf((float)D);
                for (int d = 0; d < D; ++d) qv[d] = qv[d] * f * a->o_signs[d];
            } else if (a->o_rot) {
                unrotate_dense(a->o_rot, qv, D, kv);
            }
            for (int d = 0; d < D; ++d) st(a->out, a->q_dtype, qbase + d, qv[d]);
        }
        free(kv); free(qv); free(acc); free(accf); free(sc);
    }
}

/* Row append used by the timed CPU baseline (the cache update of KVCacheSimple,
 * KVCache.swift:438-441): copies [B, H, S, W] rows into [B, H, cap, W] at `pos`. */
void orc_append(const void *src, void *dst, int esize, int B, int H, int S, int W, int64_t cap, int64_t pos) {
#pragma omp parallel for schedule(static)
    for (int64_t bh = 0; bh < (int64_t)B * H; ++bh)
        memcpy((char *)dst + ((size_t)bh * cap + pos) * W * esize, (const char *)src + (size_t)bh * S * W * esize,
               (size_t)S * W * esize);
}

/* Thread count of the following parallel regions (a launcher may have exported OMP_NUM_THREADS=1). */
void orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int orc_num_threads(void) {
    int n = 1;
#ifdef _OPENMP
#pragma omp parallel
    {
#pragma omp single
        n = omp_get_num_threads();
    }
#endif
    return n;
}
