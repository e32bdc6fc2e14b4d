// Multi-token chunks (prefill chunks over a quantised cache, speculative verify rounds)
// over the packed caches on sm_100a: more query rows per KV head than the decode kernels
// take (affine: > 16, TurboQuant: > 8), head dimension 128.
//
// With 16..64 rows per CTA the MMAs dominate and the codes are worth dequantising once per
// tile instead of once per row block: a producer lane streams packed 64-token tiles through
// the mbarrier ring (cp.async.bulk, as in the decode kernels); each of the four consumer
// warps dequantises 16 tokens of K and V into an f16 tile in shared memory, laid out exactly
// like the tiles the raw-cache kernels get from TMA (boxes of [64 tokens][64 elements], 16-byte
// chunk c of row r at chunk c ^ (r & 7)); after one barrier among the consumers every warp
// runs the row-split flash loop of the raw chunk kernel over the whole tile: warp w owns query
// rows 16w..16w+15 of the CTA's 64-row block. The f16 tile is double-buffered, so one barrier
// per tile is enough: a buffer is rewritten two tiles later, after every warp has passed the
// barrier of the tile in between.
//   * affine codes: n -> f16 exactly (exponent trick + one half2 add/fma), then s * n + b with
//     one half2 FMA. 4-bit words give the pairs (n_k, n_k+4): a 16-byte chunk holds its eight
//     elements in the order 0,4,1,5,2,6,3,7; the query fragments and the output columns use
//     the same order, so nothing is shuffled.
//   * TurboQuant rows: pair lookup in the lane-replicated table (see attn_turbo.cu), times the
//     row norm; queries are rotated once per CTA (sign flip + Walsh-Hadamard in shared memory),
//     outputs go back through signs * H(.) / sqrt(D) before they are written.
// Masks: none / causal (array masks stay on the general kernel). Under a causal mask a CTA
// only streams the tiles some row of its block can see.
#include "attn_common.cuh"

#include <algorithm>
#include <cstdio>
#include <cstdlib>

namespace kvc {

namespace {

using namespace dev;

constexpr int CP_WARPS = 4;
constexpr int CP_THREADS = (CP_WARPS + 1) * 32;
constexpr int CP_CONSUMERS = CP_WARPS * 32;
constexpr int CP_TILE = 64;
constexpr int CP_D = 128;
constexpr int CP_BOX = CP_TILE * 128;                 // [64 tokens][64 f16]
constexpr int CP_DQ_TILE = CP_TILE * CP_D * 2;        // one dequantised K (or V) tile
constexpr int CP_COUNTER_BYTES = 64 * 1024;

struct ChunkPackedParams {
    const void *q;
    void *out;
    int64_t q_sb, q_sh, q_sl, o_sb, o_sh, o_sl;
    // affine: codes + scales/biases (dtype T); turbo: packed indices + norms
    const uint32_t *kc, *vc;
    const void *ks, *kb, *vs, *vb;
    const float *kn, *vn;
    int64_t kc_sb, kc_sh, vc_sb, vc_sh;  // word strides of the code / index arrays
    int64_t kg_sb, kg_sh, vg_sb, vg_sh;  // element strides of scales/biases or norms
    const float *q_signs, *o_signs;      // turbo
    const float *q_calib;                // turbo: optional key-calibration scale folded into the rotated query
    float kcb[16], vcb[16];              // turbo centroids
    float *o_part;
    float2 *ml_part;
    int *counters;
    int *status;
    int32_t B, Hq, Hkv, L;
    int64_t T;
    int32_t splits, row_blocks, tiles_all;
    int32_t causal;
    int32_t out_dtype;
    int64_t causal_offset;
    float scale_log2;
};

__device__ __forceinline__ void mma_h(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t hfma2(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}

__device__ __forceinline__ uint32_t hmul2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

__device__ __forceinline__ uint32_t h2_bcast(float x) {
    return pack_h2(x, x);
}

// Per-warp flash state for 16 query rows x D head dims.
struct ChunkState {
    float m_run[2], l_run[2];
    float o_acc[CP_D / 8][4];
};

// One dequantised 64-token tile (f16, swizzled boxes) against the warp's 16 rows: the loop of
// the raw chunk kernel. Queries are pre-scaled, scores arrive in the exp2 domain.
__device__ __forceinline__ void chunk_tile(const unsigned char *kt, uint32_t vt_addr, const uint32_t (&qa)[CP_D / 16][4],
                                           const uint32_t (&k_off)[2], const uint32_t (&v_off)[4], int t_tile,
                                           int lim_max, int lim_min, const int (&row_limit)[2], int c,
                                           ChunkState &st) {
    constexpr int BOXES = CP_D / 64;
    constexpr int NT_O = CP_D / 8;
#pragma unroll 1
    for (int blk = 0; blk < 4; ++blk) {
        const int t_blk = t_tile + blk * 16;
        if (t_blk > lim_max) break;  // warp-uniform: nothing further in this tile is visible
        const uint32_t boff = blk * 16 * 128;
        float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int bx = 0; bx < BOXES; ++bx) {
#pragma unroll
            for (int ps = 0; ps < 2; ++ps) {
                const uint4 k0 = *(const uint4 *)(kt + bx * CP_BOX + boff + k_off[ps]);
                const uint4 k1 = *(const uint4 *)(kt + bx * CP_BOX + boff + k_off[ps] + 8 * 128);
                const int ks = bx * 4 + ps * 2;
                mma_h(sc[0], qa[ks], k0.x, k0.y);
                mma_h(sc[1], qa[ks], k1.x, k1.y);
                mma_h(sc[0], qa[ks + 1], k0.z, k0.w);
                mma_h(sc[1], qa[ks + 1], k1.z, k1.w);
            }
        }
        const bool edge = t_blk + 15 > lim_min;  // warp-uniform
        float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int half = e >> 1;
                float v = sc[j][e];
                if (edge) {
                    const int t = t_blk + j * 8 + 2 * c + (e & 1);
                    v = (t <= row_limit[half]) ? v : -INFINITY;
                }
                sc[j][e] = v;
                tmax[half] = fmaxf(tmax[half], v);
            }
        }
        float alpha[2];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            tmax[half] = fmaxf(tmax[half], __shfl_xor_sync(0xffffffffu, tmax[half], 1));
            tmax[half] = fmaxf(tmax[half], __shfl_xor_sync(0xffffffffu, tmax[half], 2));
            const float m_new = fmaxf(st.m_run[half], tmax[half]);
            alpha[half] = (m_new == -INFINITY) ? 1.f : fast_exp2(st.m_run[half] - m_new);
            st.m_run[half] = m_new;
        }
        uint32_t pa[4];
        {
            float pr[2][4];
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int half = e >> 1;
                    pr[j][e] = (st.m_run[half] == -INFINITY) ? 0.f : fast_exp2(sc[j][e] - st.m_run[half]);
                }
#pragma unroll
            for (int half = 0; half < 2; ++half)
                st.l_run[half] = st.l_run[half] * alpha[half] + pr[0][2 * half] + pr[0][2 * half + 1] +
                                 pr[1][2 * half] + pr[1][2 * half + 1];
            pa[0] = pack_h2(pr[0][0], pr[0][1]);
            pa[1] = pack_h2(pr[0][2], pr[0][3]);
            pa[2] = pack_h2(pr[1][0], pr[1][1]);
            pa[3] = pack_h2(pr[1][2], pr[1][3]);
        }
        if (__any_sync(0xffffffffu, (alpha[0] != 1.f) | (alpha[1] != 1.f))) {
#pragma unroll
            for (int nt = 0; nt < NT_O; ++nt) {
                st.o_acc[nt][0] *= alpha[0];
                st.o_acc[nt][1] *= alpha[0];
                st.o_acc[nt][2] *= alpha[1];
                st.o_acc[nt][3] *= alpha[1];
            }
        }
#pragma unroll
        for (int bx = 0; bx < BOXES; ++bx) {
#pragma unroll
            for (int cp = 0; cp < 4; ++cp) {
                uint32_t vf[4];
                ldmatrix_x4_trans(vf, vt_addr + bx * CP_BOX + boff + v_off[cp]);
                mma_h(st.o_acc[bx * 8 + 2 * cp], pa, vf[0], vf[1]);
                mma_h(st.o_acc[bx * 8 + 2 * cp + 1], pa, vf[2], vf[3]);
            }
        }
    }
}

// ---------------------------------------------------------------------
// Source policies: what a stage holds, how the producer fills it, how a lane turns
// (token tt of the tile, half hh of the row = 64 head dims) into eight 16-byte chunks of the
// f16 K and V tiles, and in which order a chunk holds its eight elements.
// ---------------------------------------------------------------------
template <typename T, int BITS, int GROUP>
struct AffineSrc {
    static constexpr int RB = CP_D * BITS / 8;          // code bytes per row
    static constexpr int WPR = RB / 4;                  // words per row
    static constexpr int G = CP_D / GROUP;              // groups per row
    static constexpr int CODE_TILE = CP_TILE * RB;
    static constexpr int SC_TILE = CP_TILE * G * 2;
    static constexpr int STAGE_BYTES = 2 * CODE_TILE + 4 * SC_TILE;
    static constexpr int TABLE_BYTES = 0;
    static constexpr bool ROTATED = false;
    static constexpr int HG = (GROUP >= 64) ? 1 : 64 / GROUP;  // groups inside one half row

    __device__ static void build_tables(const ChunkPackedParams &, unsigned char *, int) {}

    __device__ static void load(const ChunkPackedParams &p, int b, int hk, int64_t t0, unsigned char *st, uint64_t *bar) {
        const uint32_t *kc = p.kc + b * p.kc_sb + hk * p.kc_sh;
        const uint32_t *vc = p.vc + b * p.vc_sb + hk * p.vc_sh;
        const T *ks = (const T *)p.ks + b * p.kg_sb + hk * p.kg_sh;
        const T *kb = (const T *)p.kb + b * p.kg_sb + hk * p.kg_sh;
        const T *vs = (const T *)p.vs + b * p.vg_sb + hk * p.vg_sh;
        const T *vb = (const T *)p.vb + b * p.vg_sb + hk * p.vg_sh;
        bulk_load(st, kc + t0 * WPR, CODE_TILE, bar);
        bulk_load(st + CODE_TILE, vc + t0 * WPR, CODE_TILE, bar);
        bulk_load(st + 2 * CODE_TILE, ks + t0 * G, SC_TILE, bar);
        bulk_load(st + 2 * CODE_TILE + SC_TILE, kb + t0 * G, SC_TILE, bar);
        bulk_load(st + 2 * CODE_TILE + 2 * SC_TILE, vs + t0 * G, SC_TILE, bar);
        bulk_load(st + 2 * CODE_TILE + 3 * SC_TILE, vb + t0 * G, SC_TILE, bar);
    }

    // element (0..7) held at position pos of a chunk
    __device__ static constexpr int elem(int pos) {
        return BITS == 4 ? ((pos & 1) * 4 + (pos >> 1)) : pos;
    }

    // operand pair k of a code word as exact integer codes in f16
    __device__ static uint32_t exact(uint32_t w, uint32_t w8, int k) {
        uint32_t r;
        if (BITS == 4) {
            const uint32_t x = (k & 2) ? w8 : w;
            if (k & 1) {
                const uint32_t y = (x & 0x00F000F0u) | 0x54005400u;                       // 64 + n
                asm("add.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(y), "r"(0xD400D400u));
            } else {
                const uint32_t y = (x & 0x000F000Fu) | 0x54005400u;                       // 64 + n / 16
                asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(y), "r"(0x4C004C00u), "r"(0xE400E400u));
            }
        } else {
            const uint32_t y = __byte_perm(w, 0x64646464u, k ? 0x4342 : 0x4140);          // 1024 + n
            asm("add.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(y), "r"(0xE400E400u));
        }
        return r;
    }

    __device__ static void dequant_one(const uint32_t *words, const T *scales, const T *biases, int tt, int hh,
                                       unsigned char *dq) {
        uint32_t s2[HG], b2[HG];
#pragma unroll
        for (int i = 0; i < HG; ++i) {
            const int gr = (hh * 64) / GROUP + i;
            s2[i] = h2_bcast(to_f32<T>(scales[tt * G + gr]));
            b2[i] = h2_bcast(to_f32<T>(biases[tt * G + gr]));
        }
        constexpr int WPH = WPR / 2;  // words per half row
        const uint32_t *w = words + tt * WPR + hh * WPH;
        unsigned char *row = dq + hh * CP_BOX + tt * 128;
#pragma unroll
        for (int j = 0; j < 8; ++j) {  // chunk j of the half = 8 elements
            const int gi = (GROUP >= 64) ? 0 : (8 * j) / GROUP;
            uint4 o;
            if (BITS == 4) {
                const uint32_t x = w[j], x8 = x >> 8;
                o.x = hfma2(exact(x, x8, 0), s2[gi], b2[gi]);
                o.y = hfma2(exact(x, x8, 1), s2[gi], b2[gi]);
                o.z = hfma2(exact(x, x8, 2), s2[gi], b2[gi]);
                o.w = hfma2(exact(x, x8, 3), s2[gi], b2[gi]);
            } else {
                const uint32_t x0 = w[2 * j], x1 = w[2 * j + 1];
                o.x = hfma2(exact(x0, 0, 0), s2[gi], b2[gi]);
                o.y = hfma2(exact(x0, 0, 1), s2[gi], b2[gi]);
                o.z = hfma2(exact(x1, 0, 0), s2[gi], b2[gi]);
                o.w = hfma2(exact(x1, 0, 1), s2[gi], b2[gi]);
            }
            *(uint4 *)(row + ((j ^ (tt & 7)) << 4)) = o;
        }
    }

    __device__ static void dequant(const ChunkPackedParams &, const unsigned char *st, const unsigned char *, int tt,
                                   int hh, int, unsigned char *kdq, unsigned char *vdq) {
        dequant_one((const uint32_t *)st, (const T *)(st + 2 * CODE_TILE), (const T *)(st + 2 * CODE_TILE + SC_TILE), tt,
                    hh, kdq);
        dequant_one((const uint32_t *)(st + CODE_TILE), (const T *)(st + 2 * CODE_TILE + 2 * SC_TILE),
                    (const T *)(st + 2 * CODE_TILE + 3 * SC_TILE), tt, hh, vdq);
    }
};

template <int KB, int VB>
struct TurboSrc {
    static constexpr int KW = CP_D * KB / 32, VW = CP_D * VB / 32;
    static constexpr int K_TILE = CP_TILE * KW * 4, V_TILE = CP_TILE * VW * 4, N_TILE = CP_TILE * 4;
    static constexpr int STAGE_BYTES = K_TILE + V_TILE + 2 * N_TILE;
    static constexpr int KTAB = (1 << (2 * KB)) * 128, VTAB = (1 << (2 * VB)) * 128;
    static constexpr int TABLE_BYTES = KTAB + VTAB;
    static constexpr bool ROTATED = true;

    __device__ static void build_tables(const ChunkPackedParams &p, unsigned char *tab, int tid) {
        for (int w = tid; w < KTAB / 4; w += CP_THREADS) {
            const int j = w >> 5;
            ((uint32_t *)tab)[w] = pack_h2(p.kcb[j & ((1 << KB) - 1)], p.kcb[j >> KB]);
        }
        for (int w = tid; w < VTAB / 4; w += CP_THREADS) {
            const int j = w >> 5;
            ((uint32_t *)(tab + KTAB))[w] = pack_h2(p.vcb[j & ((1 << VB) - 1)], p.vcb[j >> VB]);
        }
    }

    __device__ static void load(const ChunkPackedParams &p, int b, int hk, int64_t t0, unsigned char *st, uint64_t *bar) {
        const uint32_t *kp = p.kc + b * p.kc_sb + hk * p.kc_sh;
        const uint32_t *vp = p.vc + b * p.vc_sb + hk * p.vc_sh;
        const float *kn = p.kn + b * p.kg_sb + hk * p.kg_sh;
        const float *vn = p.vn + b * p.vg_sb + hk * p.vg_sh;
        bulk_load(st, kp + t0 * KW, K_TILE, bar);
        bulk_load(st + K_TILE, vp + t0 * VW, V_TILE, bar);
        bulk_load(st + K_TILE + V_TILE, kn + t0, N_TILE, bar);
        bulk_load(st + K_TILE + V_TILE + N_TILE, vn + t0, N_TILE, bar);
    }

    __device__ static constexpr int elem(int pos) { return pos; }

    template <int BITS, int NW>
    __device__ static uint32_t pair_entry(const uint32_t (&w)[NW], int j, uint32_t lane_bits) {
        constexpr int B2 = 2 * BITS;
        constexpr uint32_t MASK = ((1u << B2) - 1u) << 7;
        const int bit = B2 * j, k = bit >> 5, s = bit & 31;
        uint32_t x;
        if (s + B2 <= 32) x = (s >= 7) ? (w[k] >> (s - 7)) : (w[k] << (7 - s));
        else x = __funnelshift_r(w[k], w[(k + 1 < NW) ? k + 1 : k], s - 7);
        return (x & MASK) | lane_bits;
    }

    template <int BITS>
    __device__ static void dequant_one(const uint32_t *words, const float *norms, const unsigned char *tab, int tt, int hh,
                                       uint32_t lane_bits, unsigned char *dq) {
        constexpr int WPH = CP_D * BITS / 64;  // words per half row
        uint32_t w[WPH];
#pragma unroll
        for (int i = 0; i < WPH; ++i) w[i] = words[tt * (2 * WPH) + hh * WPH + i];
        const uint32_t n2 = h2_bcast(norms[tt]);
        unsigned char *row = dq + hh * CP_BOX + tt * 128;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            uint4 o;
            o.x = hmul2(*(const uint32_t *)(tab + pair_entry<BITS, WPH>(w, 4 * j, lane_bits)), n2);
            o.y = hmul2(*(const uint32_t *)(tab + pair_entry<BITS, WPH>(w, 4 * j + 1, lane_bits)), n2);
            o.z = hmul2(*(const uint32_t *)(tab + pair_entry<BITS, WPH>(w, 4 * j + 2, lane_bits)), n2);
            o.w = hmul2(*(const uint32_t *)(tab + pair_entry<BITS, WPH>(w, 4 * j + 3, lane_bits)), n2);
            *(uint4 *)(row + ((j ^ (tt & 7)) << 4)) = o;
        }
    }

    __device__ static void dequant(const ChunkPackedParams &, const unsigned char *st, const unsigned char *tab, int tt,
                                   int hh, int lane, unsigned char *kdq, unsigned char *vdq) {
        const uint32_t lane_bits = (uint32_t)lane << 2;
        dequant_one<KB>((const uint32_t *)st, (const float *)(st + K_TILE + V_TILE), tab, tt, hh, lane_bits, kdq);
        dequant_one<VB>((const uint32_t *)(st + K_TILE), (const float *)(st + K_TILE + V_TILE + N_TILE), tab + KTAB, tt, hh,
                        lane_bits, vdq);
    }
};

template <typename T, typename SRC, int NSTAGE>
__global__ void __launch_bounds__(CP_THREADS, (SRC::TABLE_BYTES == 0 ? 2 : 1))
attn_chunk_packed_kernel(const __grid_constant__ ChunkPackedParams p) {
    constexpr int D = CP_D;
    constexpr int KSTEPS = D / 16;
    constexpr int NT_O = D / 8;
    constexpr int STAGE_BYTES = SRC::STAGE_BYTES;

    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char *dq = base;                                  // 2 x (K tile | V tile), f16, swizzled boxes
    unsigned char *tab = dq + 4 * CP_DQ_TILE;                  // lookup tables (TurboQuant)
    unsigned char *stages = tab + SRC::TABLE_BYTES;            // packed ring
    uint64_t *full = (uint64_t *)(stages + ((NSTAGE * STAGE_BYTES + 15) / 16) * 16);
    uint64_t *empty = full + NSTAGE;
    int *is_last = (int *)(empty + NSTAGE);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x % p.splits;
    const int unit = blockIdx.x / p.splits;
    const int rb = unit % p.row_blocks;
    const int bh = unit / p.row_blocks;
    const int hk = bh % p.Hkv, b = bh / p.Hkv;
    const int rep = p.Hq / p.Hkv;
    const int R = rep * p.L;
    const int r_lo = rb * 64, r_hi = min(R, r_lo + 64) - 1;

    int tiles_needed = p.tiles_all;
    if (p.causal) {
        const int max_l = (r_lo / p.L == r_hi / p.L) ? (r_hi % p.L) : (p.L - 1);
        const int64_t lim = min(p.T - 1, p.causal_offset + max_l);
        tiles_needed = (int)min((int64_t)p.tiles_all, lim / CP_TILE + 1);
    }
    const int t_base = tiles_needed / p.splits, t_rem = tiles_needed % p.splits;
    const int tile_begin = split * t_base + min(split, t_rem);
    const int ntiles = t_base + (split < t_rem ? 1 : 0);

    if (tid == 0) {
        for (int s = 0; s < NSTAGE; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], CP_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    SRC::build_tables(p, tab, tid);
    __syncthreads();
    pdl_wait();  // everything below reads what earlier kernels on the stream wrote

    bool ok = true;
    if (warp == CP_WARPS) {
        if (lane == 0) {
            for (int it = 0; it < ntiles && ok; ++it) {
                const int s = it % NSTAGE;
                if (it >= NSTAGE) ok = mbar_wait(&empty[s], ((it / NSTAGE) - 1) & 1);
                if (!ok) break;
                unsigned char *st = stages + (size_t)s * STAGE_BYTES;
                mbar_expect_tx(&full[s], STAGE_BYTES);
                SRC::load(p, b, hk, (int64_t)(tile_begin + it) * CP_TILE, st, &full[s]);
            }
            if (!ok) atomicExch(p.status, 11);
        }
        return;
    }

    // ---------------- consumers ----------------
    const int g = lane >> 2, c = lane & 3;
    // Query rows of the block, pre-scaled (and rotated for TurboQuant), staged as f32 in the
    // f16 tile area before the first tile is dequantised: qs[64][D].
    float *qs = (float *)dq;
    {
        const float sc = SRC::ROTATED ? 1.f : p.scale_log2;
        for (int i = tid; i < 64 * D; i += CP_CONSUMERS) {
            const int rr = i / D, d = i % D;
            const int r = r_lo + rr;
            float x = 0.f;
            if (r < R) {
                const int hq = hk * rep + r / p.L, l = r % p.L;
                x = to_f32<T>(((const T *)p.q)[b * p.q_sb + hq * p.q_sh + l * p.q_sl + d]);
                x *= SRC::ROTATED ? p.q_signs[d] : sc;
            }
            qs[i] = x;
        }
        if (SRC::ROTATED) {
            for (int half = 1; half < D; half <<= 1) {
                consumer_bar<CP_WARPS>();
                for (int pi = tid; pi < 64 * (D / 2); pi += CP_CONSUMERS) {
                    const int rr = pi / (D / 2), j = pi % (D / 2);
                    const int i0 = ((j / half) * 2 * half) + (j % half), i1 = i0 + half;
                    const float xa = qs[rr * D + i0], ya = qs[rr * D + i1];
                    qs[rr * D + i0] = xa + ya;
                    qs[rr * D + i1] = xa - ya;
                }
            }
            if (p.q_calib) {
                consumer_bar<CP_WARPS>();
                for (int i = tid; i < 64 * D; i += CP_CONSUMERS) qs[i] *= p.q_calib[i % D];
            }
        }
        consumer_bar<CP_WARPS>();
    }
    const int r_warp = r_lo + 16 * warp;
    uint32_t qa[KSTEPS][4];
    {
        const float qf = SRC::ROTATED ? rsqrtf((float)D) * p.scale_log2 : 1.f;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            // k-step ks = (box bx, pass ps, half h): lane c covers chunk 2c + ps of the box, positions 4h..4h+3
            const int bx = ks / 4, ps = (ks >> 1) & 1, h = ks & 1;
            const int dch = bx * 64 + (2 * c + ps) * 8;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const float *qr = qs + (16 * warp + g + 8 * half) * D + dch;
                qa[ks][half] = pack_h2(qr[SRC::elem(4 * h)] * qf, qr[SRC::elem(4 * h + 1)] * qf);
                qa[ks][2 + half] = pack_h2(qr[SRC::elem(4 * h + 2)] * qf, qr[SRC::elem(4 * h + 3)] * qf);
            }
        }
    }
    consumer_bar<CP_WARPS>();  // the staging area becomes the f16 tiles

    int row_limit[2];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = r_warp + g + 8 * half;
        const int l = r % p.L;
        row_limit[half] = (r < R) ? (int)(p.causal ? min(p.T - 1, p.causal_offset + l) : p.T - 1) : -1;
    }
    int lim_max = max(row_limit[0], row_limit[1]);
    int lim_min = min(row_limit[0] < 0 ? 0x7fffffff : row_limit[0], row_limit[1] < 0 ? 0x7fffffff : row_limit[1]);
#pragma unroll
    for (int o = 4; o <= 16; o <<= 1) {
        lim_max = max(lim_max, __shfl_xor_sync(0xffffffffu, lim_max, o));
        lim_min = min(lim_min, __shfl_xor_sync(0xffffffffu, lim_min, o));
    }
    uint32_t k_off[2];
#pragma unroll
    for (int ps = 0; ps < 2; ++ps) k_off[ps] = (uint32_t)(g * 128 + (((2 * c + ps) ^ g) << 4));
    uint32_t v_off[4];
    {
        const int mi = lane >> 3, rr = lane & 7;
#pragma unroll
        for (int cp = 0; cp < 4; ++cp)
            v_off[cp] = (uint32_t)(((mi & 1) * 8 + rr) * 128 + (((2 * cp + (mi >> 1)) ^ rr) << 4));
    }
    ChunkState st;
    st.m_run[0] = st.m_run[1] = -INFINITY;
    st.l_run[0] = st.l_run[1] = 0.f;
#pragma unroll
    for (int i = 0; i < NT_O; ++i) st.o_acc[i][0] = st.o_acc[i][1] = st.o_acc[i][2] = st.o_acc[i][3] = 0.f;

    // this lane's share of a tile's dequantisation: token 16 warp + lane / 2, half row lane & 1
    const int dq_tok = 16 * warp + (lane >> 1), dq_half = lane & 1;
    for (int it = 0; it < ntiles; ++it) {
        unsigned char *kdq = dq + (size_t)(it & 1) * 2 * CP_DQ_TILE;
        unsigned char *vdq = kdq + CP_DQ_TILE;
        if (ok) {
            const int s = it % NSTAGE;
            ok = mbar_wait(&full[s], (it / NSTAGE) & 1);
            if (ok) {
                SRC::dequant(p, stages + (size_t)s * STAGE_BYTES, tab, dq_tok, dq_half, lane, kdq, vdq);
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
            } else if (lane == 0) {
                atomicExch(p.status, 12);
            }
        }
        consumer_bar<CP_WARPS>();  // every warp reaches it, whether or not its wait ran out
        if (ok)
            chunk_tile(kdq, smem_u32(vdq), qa, k_off, v_off, (tile_begin + it) * CP_TILE, lim_max, lim_min, row_limit, c,
                       st);
    }

    // ---------------- rows out ----------------
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        st.l_run[half] += __shfl_xor_sync(0xffffffffu, st.l_run[half], 1);
        st.l_run[half] += __shfl_xor_sync(0xffffffffu, st.l_run[half], 2);
    }
    const int64_t qrow0 = ((int64_t)b * p.Hq + hk * rep) * p.L;
    consumer_bar<CP_WARPS>();  // all tiles consumed: the f16 tile area is free again
    float *rows = (float *)dq;  // [64][D] staging for the inverse rotation / the merged rows
    if (p.splits == 1) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int rr = 16 * warp + g + 8 * half, r = r_lo + rr;
            if (r >= R) continue;
            const float inv = st.l_run[half] > 0.f ? 1.f / st.l_run[half] : 0.f;
            const int hq = hk * rep + r / p.L, lq = r % p.L;
            const int64_t obase = b * p.o_sb + hq * p.o_sh + lq * p.o_sl;
#pragma unroll
            for (int nt = 0; nt < NT_O; ++nt) {
                const int d0 = 8 * nt + SRC::elem(2 * c), d1 = 8 * nt + SRC::elem(2 * c + 1);
                const float v0 = st.o_acc[nt][2 * half] * inv, v1 = st.o_acc[nt][2 * half + 1] * inv;
                if (SRC::ROTATED) {
                    rows[rr * D + d0] = v0;
                    rows[rr * D + d1] = v1;
                } else {
                    store_out(p.out, p.out_dtype, obase + d0, v0);
                    store_out(p.out, p.out_dtype, obase + d1, v1);
                }
            }
        }
        if (!SRC::ROTATED) return;
    } else {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = r_warp + g + 8 * half;
            if (r >= R) continue;
            const int64_t pbase = (qrow0 + r) * p.splits + split;
#pragma unroll
            for (int nt = 0; nt < NT_O; ++nt) {
                __stcg(&p.o_part[pbase * D + 8 * nt + SRC::elem(2 * c)], st.o_acc[nt][2 * half]);
                __stcg(&p.o_part[pbase * D + 8 * nt + SRC::elem(2 * c + 1)], st.o_acc[nt][2 * half + 1]);
            }
            if (c == 0) __stcg(&p.ml_part[pbase], make_float2(st.m_run[half], st.l_run[half]));
        }
        __threadfence();
        consumer_bar<CP_WARPS>();
        if (tid == 0) {
            const int ticket = atomicAdd(&p.counters[unit], 1);
            const int last = (ticket == p.splits - 1) ? 1 : 0;
            if (last) p.counters[unit] = 0;
            *is_last = last;
        }
        consumer_bar<CP_WARPS>();
        if (!*is_last) return;
        __threadfence();
        float *work = (float *)(dq + 64 * D * 4);  // [rows of the block][splits] merge weights
        const int nrows = r_hi - r_lo + 1;
        for (int rr = warp; rr < nrows; rr += CP_WARPS) {
            const int64_t row = qrow0 + r_lo + rr;
            float m = -INFINITY;
            for (int s = lane; s < p.splits; s += 32) m = fmaxf(m, __ldcg(&p.ml_part[row * p.splits + s]).x);
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            float lsum = 0.f;
            for (int s = lane; s < p.splits; s += 32) {
                const float2 ml = __ldcg(&p.ml_part[row * p.splits + s]);
                const float f = (ml.x == -INFINITY || ml.y <= 0.f) ? 0.f : fast_exp2(ml.x - m);
                work[rr * p.splits + s] = f;
                lsum += ml.y * f;
            }
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, o);
            const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
            __syncwarp();
            for (int s = lane; s < p.splits; s += 32) work[rr * p.splits + s] *= inv;
        }
        consumer_bar<CP_WARPS>();
        for (int i = tid; i < nrows * D; i += CP_CONSUMERS) {
            const int rr = i / D, d = i % D;
            const int r = r_lo + rr;
            float o = 0.f;
            const float *src = p.o_part + ((qrow0 + r) * p.splits) * D + d;
            for (int s = 0; s < p.splits; ++s) o = fmaf(__ldcg(src + (int64_t)s * D), work[rr * p.splits + s], o);
            if (SRC::ROTATED) {
                rows[i] = o;
            } else {
                const int hq = hk * rep + r / p.L, lq = r % p.L;
                store_out(p.out, p.out_dtype, b * p.o_sb + hq * p.o_sh + lq * p.o_sl + d, o);
            }
        }
        if (!SRC::ROTATED) return;
    }
    // TurboQuant values: rows are in the rotated basis; out = signs * H(row) / sqrt(D)
    const int nrows = r_hi - r_lo + 1;
    for (int half = 1; half < D; half <<= 1) {
        consumer_bar<CP_WARPS>();
        for (int pi = tid; pi < nrows * (D / 2); pi += CP_CONSUMERS) {
            const int rr = pi / (D / 2), j = pi % (D / 2);
            const int i0 = ((j / half) * 2 * half) + (j % half), i1 = i0 + half;
            const float xa = rows[rr * D + i0], ya = rows[rr * D + i1];
            rows[rr * D + i0] = xa + ya;
            rows[rr * D + i1] = xa - ya;
        }
    }
    consumer_bar<CP_WARPS>();
    const float fs = rsqrtf((float)D);
    for (int i = tid; i < nrows * D; i += CP_CONSUMERS) {
        const int rr = i / D, d = i % D;
        const int r = r_lo + rr;
        const int hq = hk * rep + r / p.L, lq = r % p.L;
        store_out(p.out, p.out_dtype, b * p.o_sb + hq * p.o_sh + lq * p.o_sl + d, rows[i] * fs * p.o_signs[d]);
    }
}

template <typename T, typename SRC, int NSTAGE>
void launch_chunk_packed_typed(const ChunkPackedParams &p, int ctas, cudaStream_t stream) {
    const size_t smem = (size_t)4 * CP_DQ_TILE + SRC::TABLE_BYTES + (size_t)NSTAGE * SRC::STAGE_BYTES + 16 +
                        2 * NSTAGE * sizeof(uint64_t) + 64 + 1024;
    static bool configured[64] = {false};
    const int dev = current_device();
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        KVC_CUDA(cudaFuncSetAttribute(attn_chunk_packed_kernel<T, SRC, NSTAGE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)smem));
        KVC_CUDA(cudaFuncSetAttribute(attn_chunk_packed_kernel<T, SRC, NSTAGE>,
                                      cudaFuncAttributePreferredSharedMemoryCarveout, 100));
        configured[dev] = true;
    }
    KernelTimer timer(stream);
    KVC_CUDA(launch_pdl(attn_chunk_packed_kernel<T, SRC, NSTAGE>, dim3(ctas), dim3(CP_THREADS), smem, stream, p));
    timer.stop();
    KVC_CUDA(cudaGetLastError());
    ++g_launch_count;
}

bool chunk_affine_fits(const KVSource &s, int64_t T) {
    if (s.kind != SRC_AFFINE || (s.dtype != KVC_BF16 && s.dtype != KVC_F16)) return false;
    if (s.bits != 4 && s.bits != 8) return false;
    if (s.group != 32 && s.group != 64 && s.group != 128) return false;
    const int wpr = CP_D * s.bits / 32, G = CP_D / s.group;
    if (s.st != wpr || s.gst != G) return false;
    const int64_t padded = (T + CP_TILE - 1) / CP_TILE * CP_TILE;
    if (s.sh < padded * wpr || s.gsh < padded * G) return false;
    if ((s.sh * 4) % 16 || (s.sb * 4) % 16 || (s.gsh * 2) % 16 || (s.gsb * 2) % 16) return false;
    if (((uintptr_t)s.data & 15) || ((uintptr_t)s.scales & 15) || ((uintptr_t)s.biases & 15)) return false;
    return true;
}

bool chunk_turbo_fits(const KVSource &s, int64_t T) {
    if (s.kind != SRC_TURBO || !s.data || !s.norms) return false;
    if (s.bits < 2 || s.bits > 4) return false;
    const int words = CP_D * s.bits / 32;
    if (s.words != words || s.st != words || s.gst != 1) return false;
    const int64_t padded = (T + CP_TILE - 1) / CP_TILE * CP_TILE;
    if (s.sh < padded * words || s.gsh < padded) return false;
    if ((s.sh * 4) % 16 || (s.sb * 4) % 16 || (s.gsh * 4) % 16 || (s.gsb * 4) % 16) return false;
    if (((uintptr_t)s.data & 15) || ((uintptr_t)s.norms & 15)) return false;
    return true;
}

}  // namespace

// Returns the number of kernels launched, or 0 when the call does not fit this path.
// KVC_TRACE_DISPATCH=1 prints which check sent a call to another kernel.
static int chunk_reject(int reason) {
    if (trace_dispatch()) fprintf(stderr, "[kvc] chunk_packed: not taken (check %d)\n", reason);
    return 0;
}

int launch_attention_chunk_packed(const AttnArgs &a, cudaStream_t stream) {
    if (a.q_dtype != KVC_BF16 && a.q_dtype != KVC_F16) return chunk_reject(1);
    if (a.D != CP_D) return chunk_reject(2);
    if (a.mask.mode == KVC_MASK_ARRAY) return chunk_reject(3);
    if (a.Hkv <= 0 || a.Hq % a.Hkv) return chunk_reject(4);
    if (a.T < 1 || a.T > (int64_t)1 << 30) return chunk_reject(5);
    const int rep = a.Hq / a.Hkv;
    const int64_t R = (int64_t)rep * a.L;
    if (R > (int64_t)1 << 24) return chunk_reject(6);
    const bool affine = a.k.kind == SRC_AFFINE && a.v.kind == SRC_AFFINE;
    const bool turbo = a.k.kind == SRC_TURBO && a.v.kind == SRC_TURBO;
    if (!affine && !turbo) return chunk_reject(7);
    if (affine) {
        if (a.q_signs || a.o_signs || a.q_calib) return chunk_reject(8);
        if (a.k.dtype != a.q_dtype || a.v.dtype != a.q_dtype) return chunk_reject(9);
        if (a.k.bits != a.v.bits || a.k.group != a.v.group) return chunk_reject(10);
        if (!chunk_affine_fits(a.k, a.T) || !chunk_affine_fits(a.v, a.T)) return chunk_reject(11);
    } else {
        if (!a.q_signs || !a.o_signs) return chunk_reject(12);
        if (!chunk_turbo_fits(a.k, a.T) || !chunk_turbo_fits(a.v, a.T)) return chunk_reject(13);
        const int kb = a.k.bits, vb = a.v.bits;
        const bool known = (kb == 4 && vb == 4) || (kb == 4 && vb == 2) || (kb == 3 && vb == 3) ||
                           (kb == 2 && vb == 2) || (kb == 3 && vb == 4);
        if (!known) return chunk_reject(14);
    }
    const int64_t bh = (int64_t)a.B * a.Hkv;
    const int64_t row_blocks = (R + 63) / 64;
    if (bh * row_blocks * (int64_t)sizeof(int) > CP_COUNTER_BYTES) return chunk_reject(15);
    int *status = device_status_word(a.device);
    if (!status) return chunk_reject(16);
    int *counters = counters_get(a.device, stream, CP_COUNTER_BYTES);

    const int64_t tiles = (a.T + CP_TILE - 1) / CP_TILE;
    const int slots = sm_count(a.device) * (affine ? 2 : 1);
    int64_t best_s = 1;
    double best_cost = 1e30;
    const int64_t max_s = std::min<int64_t>(tiles, 64);
    for (int64_t s = 1; s <= max_s; ++s) {
        const int64_t units = bh * row_blocks * s;
        const int64_t waves = (units + slots - 1) / slots;
        const int64_t per = (tiles + s - 1) / s;
        const double cost = (double)waves * ((double)per + 4.0);
        if (cost < best_cost - 1e-9) {
            best_cost = cost;
            best_s = s;
        }
    }
    const int64_t splits = best_s;
    const int64_t qrows = (int64_t)a.B * a.Hq * a.L;
    char *scratch = nullptr;
    size_t o_bytes = 0;
    if (splits > 1) {
        o_bytes = (size_t)qrows * splits * a.D * sizeof(float);
        const size_t ml_bytes = (size_t)qrows * splits * sizeof(float2);
        scratch = (char *)scratch_get(a.device, o_bytes + ml_bytes + 256, stream);
    }

    ChunkPackedParams p = {};
    p.q = a.q; p.out = a.out; p.out_dtype = a.q_dtype;
    p.q_sb = a.q_sb; p.q_sh = a.q_sh; p.q_sl = a.q_sl;
    p.o_sb = a.o_sb; p.o_sh = a.o_sh; p.o_sl = a.o_sl;
    p.kc = (const uint32_t *)a.k.data; p.vc = (const uint32_t *)a.v.data;
    p.ks = a.k.scales; p.kb = a.k.biases; p.vs = a.v.scales; p.vb = a.v.biases;
    p.kn = a.k.norms; p.vn = a.v.norms;
    p.kc_sb = a.k.sb; p.kc_sh = a.k.sh; p.vc_sb = a.v.sb; p.vc_sh = a.v.sh;
    p.kg_sb = a.k.gsb; p.kg_sh = a.k.gsh; p.vg_sb = a.v.gsb; p.vg_sh = a.v.gsh;
    p.q_signs = a.q_signs; p.o_signs = a.o_signs; p.q_calib = a.q_calib;
    for (int i = 0; i < 16; ++i) {
        p.kcb[i] = a.k.codebook[i];
        p.vcb[i] = a.v.codebook[i];
    }
    p.o_part = (float *)scratch;
    p.ml_part = scratch ? (float2 *)(scratch + ((o_bytes + 255) / 256) * 256) : nullptr;
    p.counters = counters; p.status = status;
    p.B = a.B; p.Hq = a.Hq; p.Hkv = a.Hkv; p.L = a.L; p.T = a.T;
    p.splits = (int)splits;
    p.row_blocks = (int)row_blocks;
    p.tiles_all = (int)tiles;
    p.causal = a.mask.mode == KVC_MASK_CAUSAL ? 1 : 0;
    p.causal_offset = a.mask.causal_offset;
    p.scale_log2 = a.scale * 1.4426950408889634f;
    const int ctas = (int)(bh * row_blocks * splits);

    if (affine) {
        const int bits = a.k.bits, group = a.k.group;
#define KVC_CPA(TT, BB, GG, NS)                                                            \
    if (bits == BB && group == GG) {                                                       \
        launch_chunk_packed_typed<TT, AffineSrc<TT, BB, GG>, NS>(p, ctas, stream);         \
        return 1;                                                                          \
    }
        if (a.q_dtype == KVC_BF16) {
            KVC_CPA(__nv_bfloat16, 4, 64, 4)
            KVC_CPA(__nv_bfloat16, 8, 64, 2)
            KVC_CPA(__nv_bfloat16, 4, 128, 4)
            KVC_CPA(__nv_bfloat16, 8, 128, 2)
            KVC_CPA(__nv_bfloat16, 4, 32, 4)
            KVC_CPA(__nv_bfloat16, 8, 32, 2)
        } else {
            KVC_CPA(__half, 4, 64, 4)
            KVC_CPA(__half, 8, 64, 2)
            KVC_CPA(__half, 4, 128, 4)
            KVC_CPA(__half, 8, 128, 2)
            KVC_CPA(__half, 4, 32, 4)
            KVC_CPA(__half, 8, 32, 2)
        }
#undef KVC_CPA
        return chunk_reject(17);
    }
    const int kb = a.k.bits, vb = a.v.bits;
#define KVC_CPT(TT, KK, VV, NS)                                                           \
    if (kb == KK && vb == VV) {                                                           \
        launch_chunk_packed_typed<TT, TurboSrc<KK, VV>, NS>(p, ctas, stream);             \
        return 1;                                                                         \
    }
    if (a.q_dtype == KVC_BF16) {
        KVC_CPT(__nv_bfloat16, 3, 4, 4)
        KVC_CPT(__nv_bfloat16, 4, 4, 4)
        KVC_CPT(__nv_bfloat16, 4, 2, 4)
        KVC_CPT(__nv_bfloat16, 3, 3, 4)
        KVC_CPT(__nv_bfloat16, 2, 2, 4)
    } else {
        KVC_CPT(__half, 3, 4, 4)
        KVC_CPT(__half, 4, 4, 4)
        KVC_CPT(__half, 4, 2, 4)
        KVC_CPT(__half, 3, 3, 4)
        KVC_CPT(__half, 2, 2, 4)
    }
#undef KVC_CPT
    return chunk_reject(18);
}

}  // namespace kvc
