// Split-K flash decoding over the TurboQuant cache (packed codebook indices plus one
// norm per row, for keys and for values) on sm_100a, for at most 8 query rows per KV
// head and head dimension 128.
//
// The math runs in the rotated basis (TurboQuantKVCache.compressedAttention,
// TurboQuantKVCache.swift:1164-1446): the query is rotated once per CTA,
//   q' = H (signs_k * q) / sqrt(D) * scale * log2(e),
// a key's score is norm_k[t] * sum_d q'[d] * centroid_k[idx_k[t, d]], the output
// accumulates sum_t (p_t * norm_v[t]) * centroid_v[idx_v[t, d]] and the merged rows go
// back through signs_v * H(.) / sqrt(D) in the epilogue shared with the other kernels.
//
// Same CTA structure as the affine kernel: a producer lane streams 64-token tiles
// (packed K, packed V, both norm vectors) through an mbarrier ring with cp.async.bulk,
// four consumer warps take 16 tokens each and keep the MMAs in the transposed
// orientation (tokens / head dims on the 16-row M side, query rows on the 8-column N
// side).
//
// Centroids are not a linear function of the index, so operands come from a lookup
// table in shared memory. One lookup turns the indices of TWO adjacent dims (2 * bits
// bits of the row) into one f16x2 operand register. The table is replicated per lane
// (entry j of lane l lives at word 32 j + l, i.e. in bank l), so a warp's 32 lookups
// never conflict whatever the indices are: 4^bits * 128 bytes per table.
//   * K side: a lane's k-slots are 32 consecutive dims of its token (= `bits` whole
//     words of the row), pairs along the head dim are exactly the A-operand pairs.
//   * V side: the A operand pairs run along TOKENS, so the looked-up (token, dim pair)
//     registers go through movmatrix (an 8x8 b16 transpose across the warp), which
//     hands every lane (dim, token pair) registers. Which head dim an accumulator row
//     stands for is a fixed permutation that the epilogue undoes.
#include "attn_common.cuh"

#include <algorithm>
#include <cstdlib>

namespace kvc {

namespace {

using namespace dev;

constexpr int TQ_WARPS = 4;
constexpr int TQ_THREADS = (TQ_WARPS + 1) * 32;
constexpr int TQ_TILE = 64;
constexpr int TQ_D = 128;
constexpr int TQ_COUNTER_BYTES = 64 * 1024;

struct TurboParams {
    const void *q;
    void *out;
    int64_t q_sb, q_sh, q_sl, o_sb, o_sh, o_sl;
    const uint32_t *kp, *vp;   // packed indices, [B, H, cap, words]
    const float *kn, *vn;      // norms, [B, H, cap]
    int64_t kp_sb, kp_sh, vp_sb, vp_sh;  // word strides (token stride = words per row)
    int64_t kn_sb, kn_sh, vn_sb, vn_sh;  // element strides (token stride = 1)
    const float *q_signs, *o_signs;      // [D] each
    const float *q_calib;                // optional [D]: key-calibration scale folded into the rotated query
    float kcb[16], vcb[16];              // centroids
    float *o_part;
    float2 *ml_part;
    int *counters;
    int *status;
    int32_t B, Hq, Hkv, L;
    int64_t T;
    int32_t splits, tiles_base, tiles_rem;
    int32_t causal;
    int32_t out_dtype;
    int32_t debug_skip;  // measurement aid: 1 = consumers release tiles without computing
    int64_t causal_offset;
    float scale_log2;
    FlatPlan flat;  // flat tile decomposition (one wave of CTAs, segments per unit)
    int32_t q_bulk; // a unit's query rows are one contiguous 16-byte aligned block
};

// Byte offset (inside a lane-replicated table) of the entry for pair j of a lane's word
// stream: ((stream >> (2 BITS j)) & (4^BITS - 1)) * 128, OR-ed with the lane's bank offset.
// A shift (a funnel shift when the field straddles two words) and one and-or.
template <int BITS, int NW>
__device__ __forceinline__ uint32_t pair_entry(const uint32_t (&w)[NW], int j, uint32_t lane_bits) {
    constexpr int B2 = 2 * BITS;
    constexpr uint32_t MASK = ((1u << B2) - 1u) << 7;
    const int bit = B2 * j, k = bit >> 5, s = bit & 31;
    uint32_t x;
    if (s + B2 <= 32) x = (s >= 7) ? (w[k] >> (s - 7)) : (w[k] << (7 - s));
    else x = __funnelshift_r(w[k], w[(k + 1 < NW) ? k + 1 : k], s - 7);
    return (x & MASK) | lane_bits;
}

__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

template <int N>
__device__ __forceinline__ void load_row_words(const uint32_t *src, uint32_t (&dst)[N]) {
    if (N == 4) {
        const uint4 x = *reinterpret_cast<const uint4 *>(src);
        dst[0] = x.x; dst[1] = x.y; dst[2] = x.z; dst[3] = x.w;
    } else if (N == 2) {
        const uint2 x = *reinterpret_cast<const uint2 *>(src);
        dst[0] = x.x; dst[1] = x.y;
    } else {
#pragma unroll
        for (int i = 0; i < N; ++i) dst[i] = src[i];
    }
}

template <typename T, int KB, int VB, int NSTAGE>
__global__ void __launch_bounds__(TQ_THREADS, 2)
attn_turbo_decode8_kernel(const __grid_constant__ TurboParams p) {
    constexpr int D = TQ_D;
    constexpr int KW = D * KB / 32, VW = D * VB / 32;   // words per row
    constexpr int KTAB = (1 << (2 * KB)) * 128, VTAB = (1 << (2 * VB)) * 128;
    constexpr int K_TILE = TQ_TILE * KW * 4, V_TILE = TQ_TILE * VW * 4, N_TILE = TQ_TILE * 4;
    constexpr int STAGE_BYTES = K_TILE + V_TILE + 2 * N_TILE;
    constexpr int RED_STRIDE = D + 8;
    static_assert(K_TILE % 16 == 0 && V_TILE % 16 == 0, "bulk copies need 16-byte multiples");

    extern __shared__ __align__(128) unsigned char smem_raw[];
    // pointer + offset (no integer round trip) so that loads through it stay ld.shared
    unsigned char *base = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
    unsigned char *ktab = base;
    unsigned char *vtab = ktab + KTAB;
    float *qrot = (float *)(vtab + VTAB);               // [8][D]
    unsigned char *stages = (unsigned char *)(qrot + 8 * D);
    constexpr int RING = NSTAGE * STAGE_BYTES;
    const FlatPlan &fp = p.flat;
    uint64_t *full = (uint64_t *)(stages + ((RING + 15) / 16) * 16);
    uint64_t *empty = full + NSTAGE;
    int *is_last = (int *)(empty + NSTAGE);
    // cross-warp buffers beside the ring (the ring stays live across segments)
    float *red_o = (float *)(is_last + 4);                               // [4][red_rows][RED_STRIDE]
    float *red_ml = red_o + TQ_WARPS * fp.red_rows * RED_STRIDE;         // [4][red_rows][2]
    float *work = red_ml + TQ_WARPS * fp.red_rows * 2;                   // [red_rows][D] (rotated output rows)
    // query rows of a segment's unit, brought in by the producer with one bulk copy (two buffers)
    uint64_t *qfull = (uint64_t *)(work + ((fp.red_rows * fp.nslots + fp.red_rows * D + 3) & ~3));  // keeps qbuf 16-byte aligned
    uint64_t *qempty = qfull + 2;
    unsigned char *qbuf = (unsigned char *)(qempty + 2);                  // [2][red_rows][D] elements

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rep = p.Hq / p.Hkv;
    const int R = rep * p.L;  // <= 8
    const int tiles = fp.tiles;
    const int64_t x_lo = flat_lo(fp, blockIdx.x), x_hi = flat_lo(fp, blockIdx.x + 1);
    const uint32_t q_bytes = (uint32_t)R * D * 2;

    if (tid == 0) {
        for (int s = 0; s < NSTAGE; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], TQ_WARPS);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&qfull[s], 1);
            mbar_init(&qempty[s], TQ_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    // ---- lookup tables, once per CTA: entry j = f16x2(centroid[j & m], centroid[j >> bits]) in every bank ----
    for (int w = tid; w < KTAB / 4; w += TQ_THREADS) {
        const int j = w >> 5;
        ((uint32_t *)ktab)[w] = pack_h2(p.kcb[j & ((1 << KB) - 1)], p.kcb[j >> KB]);
    }
    for (int w = tid; w < VTAB / 4; w += TQ_THREADS) {
        const int j = w >> 5;
        ((uint32_t *)vtab)[w] = pack_h2(p.vcb[j & ((1 << VB) - 1)], p.vcb[j >> VB]);
    }
    __syncthreads();
    pdl_wait();  // the tables came from kernel parameters; everything below reads global memory

    bool ok = true;
    const int g = lane >> 2, c = lane & 3;

    if (warp == TQ_WARPS) {
        // ---------------- producer: one stream of tiles across the segments ----------------
        if (lane == 0) {
            int it = 0, sg = 0;
            for (int64_t x = x_lo; x < x_hi && ok; ++sg) {
                const int unit = (int)(x / tiles), tb = (int)(x % tiles);
                const int n = (int)min((int64_t)(tiles - tb), x_hi - x);
                const int hk = unit % p.Hkv, b = unit / p.Hkv;
                if (p.q_bulk) {
                    const int qb = sg & 1;
                    if (sg >= 2) ok = mbar_wait(&qempty[qb], ((sg >> 1) - 1) & 1);
                    if (!ok) break;
                    mbar_expect_tx(&qfull[qb], q_bytes);
                    bulk_load(qbuf + (size_t)qb * q_bytes, (const T *)p.q + b * p.q_sb + (int64_t)hk * rep * p.q_sh, q_bytes,
                              &qfull[qb]);
                }
                const uint32_t *kp = p.kp + b * p.kp_sb + hk * p.kp_sh;
                const uint32_t *vp = p.vp + b * p.vp_sb + hk * p.vp_sh;
                const float *kn = p.kn + b * p.kn_sb + hk * p.kn_sh;
                const float *vn = p.vn + b * p.vn_sb + hk * p.vn_sh;
                for (int j = 0; j < n && ok; ++j, ++it) {
                    const int s = it % NSTAGE;
                    if (it >= NSTAGE) ok = mbar_wait(&empty[s], ((it / NSTAGE) - 1) & 1);
                    if (!ok) break;
                    unsigned char *st = stages + (size_t)s * STAGE_BYTES;
                    const int64_t t0 = (int64_t)(tb + j) * TQ_TILE;
                    mbar_expect_tx(&full[s], STAGE_BYTES);
                    bulk_load(st, kp + t0 * KW, K_TILE, &full[s]);
                    bulk_load(st + K_TILE, vp + t0 * VW, V_TILE, &full[s]);
                    bulk_load(st + K_TILE + V_TILE, kn + t0, N_TILE, &full[s]);
                    bulk_load(st + K_TILE + V_TILE + N_TILE, vn + t0, N_TILE, &full[s]);
                }
                x += n;
            }
            if (!ok) atomicExch(p.status, 7);
        }
        return;
    }

    // ---------------- consumers: one segment per unit the CTA's tile range touches ----------------
    constexpr int CT = TQ_WARPS * 32;
    int st_i = 0;          // ring stage of the next tile and its phase bit, carried across segments
    uint32_t st_ph = 0;
    int sg = 0;
    for (int64_t x = x_lo; x < x_hi; ++sg) {
        const int unit = (int)(x / tiles), tile_begin = (int)(x % tiles);
        const int ntiles = (int)min((int64_t)(tiles - tile_begin), x_hi - x);
        const int hk = unit % p.Hkv, b = unit / p.Hkv;
        // ---- rotated queries of this unit: q' = H(signs * q) / sqrt(D) * scale * log2(e), rows past R zero ----
        const T *q_stage = nullptr;
        if (p.q_bulk) {
            if (ok) {
                ok = mbar_wait(&qfull[sg & 1], (sg >> 1) & 1);
                if (!ok && lane == 0) atomicExch(p.status, 15);
            }
            q_stage = (const T *)(qbuf + (size_t)(sg & 1) * q_bytes);
        }
        for (int i = tid; i < 8 * D; i += CT) {
            const int r = i / D, d = i % D;
            float xq = 0.f;
            if (r < R && ok) {
                const int hq = hk * rep + r / p.L, l = r % p.L;
                const T qv = q_stage ? q_stage[r * D + d] : ((const T *)p.q)[b * p.q_sb + hq * p.q_sh + l * p.q_sl + d];
                xq = to_f32<T>(qv) * p.q_signs[d];
            }
            qrot[i] = xq;
        }
        if (p.q_bulk) {
            __syncwarp();
            if (ok && lane == 0) mbar_arrive(&qempty[sg & 1]);
        }
        for (int half = 1; half < D; half <<= 1) {
            consumer_bar<TQ_WARPS>();
            for (int pi = tid; pi < 8 * (D / 2); pi += CT) {
                const int r = pi / (D / 2), j = pi % (D / 2);
                const int i0 = ((j / half) * 2 * half) + (j % half), i1 = i0 + half;
                const float xa = qrot[r * D + i0], ya = qrot[r * D + i1];
                qrot[r * D + i0] = xa + ya;
                qrot[r * D + i1] = xa - ya;
            }
        }
        if (p.q_calib) {
            consumer_bar<TQ_WARPS>();
            for (int i = tid; i < 8 * D; i += CT) qrot[i] *= p.q_calib[i % D];
        }
        consumer_bar<TQ_WARPS>();
        float m_run[2], l_run[2] = {0.f, 0.f};
        float o_acc[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;

        // Q'^T fragments (B operand, column = query row g). MMA m of the K side covers, from lane
        // c, the dims 32c + 4m + {0,1} (k-slots 2c, 2c+1) and 32c + 4m + {2,3} (k-slots 2c+8, 2c+9).
        const float qf = rsqrtf((float)D) * p.scale_log2;
        uint32_t qb[8][2];
#pragma unroll
        for (int m = 0; m < 8; ++m) {
            const float *qr = qrot + g * D + 32 * c + 4 * m;
            qb[m][0] = pack_h2(qr[0] * qf, qr[1] * qf);
            qb[m][1] = pack_h2(qr[2] * qf, qr[3] * qf);
        }
        int row_limit[2];
        const int t_last = (int)(p.T - 1);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int r = 2 * c + k;
            const int l = (r < R) ? r % p.L : 0;
            row_limit[k] = p.causal ? (int)min((int64_t)t_last, p.causal_offset + l) : t_last;
        }
        const int min_limit = p.causal ? (int)min((int64_t)t_last, p.causal_offset) : t_last;
        constexpr float M_INIT = -1e30f, LAZY = 8.f;
        m_run[0] = m_run[1] = M_INIT;
        float m_thr[2] = {M_INIT, M_INIT};

        const int blk = warp;
        const int tl0 = blk * 16 + g, tl1 = tl0 + 8;  // this lane's two tokens inside a tile
        const uint32_t lane_bits = (uint32_t)lane << 2;
        const uint32_t ktab_a = smem_u32(ktab), vtab_a = smem_u32(vtab);

        for (int jt = 0; jt < ntiles; ++jt, st_i = (st_i + 1 == NSTAGE) ? 0 : st_i + 1, st_ph ^= (st_i == 0)) {
            if (!ok) continue;  // a wait ran out earlier: walk on to the segment's barriers
            const int s = st_i;
            ok = mbar_wait(&full[s], st_ph);
            if (!ok) {
                if (lane == 0) atomicExch(p.status, 8);
                continue;
            }
            if (KVC_SKIP_BITS(p) & 1) {
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
                continue;
            }
            const unsigned char *st = stages + (size_t)s * STAGE_BYTES;
            const uint32_t *kpt = (const uint32_t *)st;
            const uint32_t *vpt = (const uint32_t *)(st + K_TILE);
            const float *knt = (const float *)(st + K_TILE + V_TILE);
            const float *vnt = (const float *)(st + K_TILE + V_TILE + N_TILE);
            const int t_blk = (tile_begin + jt) * TQ_TILE + blk * 16;

            // ---- S^T = centroids[idx_k] . Q'^T, two accumulator chains ----
            float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            {
                uint32_t wa[KB], wb[KB];
                load_row_words<KB>(kpt + tl0 * KW + c * KB, wa);
                load_row_words<KB>(kpt + tl1 * KW + c * KB, wb);
#pragma unroll
                for (int m = 0; m < 8; ++m) {
                    uint32_t a[4];
                    a[0] = lds_u32(ktab_a + pair_entry<KB, KB>(wa, 2 * m, lane_bits));      // token g,   k-slots 2c, 2c+1
                    a[1] = lds_u32(ktab_a + pair_entry<KB, KB>(wb, 2 * m, lane_bits));      // token g+8
                    a[2] = lds_u32(ktab_a + pair_entry<KB, KB>(wa, 2 * m + 1, lane_bits));  // token g,   k-slots 2c+8, 2c+9
                    a[3] = lds_u32(ktab_a + pair_entry<KB, KB>(wb, 2 * m + 1, lane_bits));  // token g+8
                    mma_f16(acc[m & 1], a, qb[m][0], qb[m][1]);
                }
            }
            float sc[4];
            {
                const float n0 = knt[tl0], n1 = knt[tl1];
                sc[0] = n0 * (acc[0][0] + acc[1][0]);
                sc[1] = n0 * (acc[0][1] + acc[1][1]);
                sc[2] = n1 * (acc[0][2] + acc[1][2]);
                sc[3] = n1 * (acc[0][3] + acc[1][3]);
            }
            if (t_blk + 15 > min_limit) {  // warp-uniform: only tiles that cross a limit
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int t = t_blk + g + ((e >> 1) ? 8 : 0);
                    if (t > row_limit[e & 1]) sc[e] = -INFINITY;
                }
            }
            // ---- lazy running maximum (rescale only when a score passes the stale maximum + 8) ----
            {
                const float mx0 = fmaxf(sc[0], sc[2]), mx1 = fmaxf(sc[1], sc[3]);
                if (__any_sync(0xffffffffu, (mx0 > m_thr[0]) | (mx1 > m_thr[1]))) {
                    float mx[2] = {mx0, mx1}, alpha[2];
#pragma unroll
                    for (int k = 0; k < 2; ++k) {
                        mx[k] = fmaxf(mx[k], __shfl_xor_sync(0xffffffffu, mx[k], 4));
                        mx[k] = fmaxf(mx[k], __shfl_xor_sync(0xffffffffu, mx[k], 8));
                        mx[k] = fmaxf(mx[k], __shfl_xor_sync(0xffffffffu, mx[k], 16));
                        const float m_new = fmaxf(m_run[k], mx[k]);
                        alpha[k] = fast_exp2(m_run[k] - m_new);
                        m_run[k] = m_new;
                        m_thr[k] = (m_new > M_INIT) ? m_new + LAZY : M_INIT;
                        l_run[k] *= alpha[k];
                    }
#pragma unroll
                    for (int mt = 0; mt < 8; ++mt) {
                        o_acc[mt][0] *= alpha[0];
                        o_acc[mt][1] *= alpha[1];
                        o_acc[mt][2] *= alpha[0];
                        o_acc[mt][3] *= alpha[1];
                    }
                }
            }
            float pr[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) pr[e] = fast_exp2(sc[e] - m_run[e & 1]);
            l_run[0] += pr[0] + pr[2];
            l_run[1] += pr[1] + pr[3];
            // ---- P'^T = (p * norm_v)^T in the B-fragment layout ----
            uint32_t pb[2];
            {
                const float n0 = vnt[tl0], n1 = vnt[tl1];
                pb[0] = movmatrix_trans(pack_h2(pr[0] * n0, pr[1] * n0));  // tokens 0..7 of the block
                pb[1] = movmatrix_trans(pack_h2(pr[2] * n1, pr[3] * n1));  // tokens 8..15
            }
            // ---- O^T += centroids[idx_v]^T . P'^T ----
            // Lookup j of token g gives (token g, dims 32c + 2j, +1); the 8x8 transpose turns the
            // warp's registers into (dim row g' -> dim 32 (g' >> 1) + 2j + (g' & 1), tokens 2c, 2c+1).
            {
                uint32_t wa[VB], wb[VB];
                load_row_words<VB>(vpt + tl0 * VW + c * VB, wa);
                load_row_words<VB>(vpt + tl1 * VW + c * VB, wb);
#pragma unroll
                for (int mt = 0; mt < 8; ++mt) {
                    uint32_t a[4];
                    a[0] = movmatrix_trans(lds_u32(vtab_a + pair_entry<VB, VB>(wa, 2 * mt, lane_bits)));
                    a[1] = movmatrix_trans(lds_u32(vtab_a + pair_entry<VB, VB>(wa, 2 * mt + 1, lane_bits)));
                    a[2] = movmatrix_trans(lds_u32(vtab_a + pair_entry<VB, VB>(wb, 2 * mt, lane_bits)));
                    a[3] = movmatrix_trans(lds_u32(vtab_a + pair_entry<VB, VB>(wb, 2 * mt + 1, lane_bits)));
                    mma_f16(o_acc[mt], a, pb[0], pb[1]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }
        // a warp whose tokens were all masked reports "no maximum"
        if (m_run[0] <= M_INIT) m_run[0] = -INFINITY;
        if (m_run[1] <= M_INIT) m_run[1] = -INFINITY;

        // ---- end of the segment ----
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            l_run[k] += __shfl_xor_sync(0xffffffffu, l_run[k], 4);
            l_run[k] += __shfl_xor_sync(0xffffffffu, l_run[k], 8);
            l_run[k] += __shfl_xor_sync(0xffffffffu, l_run[k], 16);
        }
        float *wo = red_o + warp * fp.red_rows * RED_STRIDE;
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
            // accumulator rows g / g+8 of tile mt stand for lookups j = 2 mt / 2 mt + 1
            const int d0 = 32 * (g >> 1) + 2 * (2 * mt) + (g & 1), d1 = d0 + 2;
            if (2 * c < R) {
                wo[(2 * c) * RED_STRIDE + d0] = o_acc[mt][0];
                wo[(2 * c) * RED_STRIDE + d1] = o_acc[mt][2];
            }
            if (2 * c + 1 < R) {
                wo[(2 * c + 1) * RED_STRIDE + d0] = o_acc[mt][1];
                wo[(2 * c + 1) * RED_STRIDE + d1] = o_acc[mt][3];
            }
        }
        if (g == 0) {
            if (2 * c < R) {
                red_ml[(warp * fp.red_rows + 2 * c) * 2 + 0] = m_run[0];
                red_ml[(warp * fp.red_rows + 2 * c) * 2 + 1] = l_run[0];
            }
            if (2 * c + 1 < R) {
                red_ml[(warp * fp.red_rows + 2 * c + 1) * 2 + 0] = m_run[1];
                red_ml[(warp * fp.red_rows + 2 * c + 1) * 2 + 1] = l_run[1];
            }
        }
        UnitOut u;
        u.o_part = p.o_part; u.ml_part = p.ml_part; u.counters = p.counters;
        u.out = p.out; u.out_dtype = p.out_dtype;
        u.o_sb = p.o_sb; u.o_sh = p.o_sh; u.o_sl = p.o_sl;
        u.o_signs = p.o_signs;
        u.splits = 0; u.Hq = p.Hq; u.L = p.L;
        segment_epilogue<D, TQ_WARPS>(u, fp, red_o, red_ml, RED_STRIDE, work, is_last, unit, b, hk, rep, R);
        x += ntiles;
    }
}

template <int KB, int VB, int NSTAGE>
constexpr size_t turbo_fixed_smem() {
    constexpr int D = TQ_D;
    constexpr int KW = D * KB / 32, VW = D * VB / 32;
    constexpr int KTAB = (1 << (2 * KB)) * 128, VTAB = (1 << (2 * VB)) * 128;
    constexpr int STAGE_BYTES = TQ_TILE * (KW + VW) * 4 + 2 * TQ_TILE * 4;
    return (size_t)KTAB + VTAB + 8 * D * 4 + (size_t)NSTAGE * STAGE_BYTES + 16 + 2 * NSTAGE * sizeof(uint64_t) + 64 + 128;
}

inline size_t turbo_red_smem(const FlatPlan &f) {
    return (size_t)TQ_WARPS * f.red_rows * (TQ_D + 8) * 4 + (size_t)TQ_WARPS * f.red_rows * 8 +
           (size_t)f.red_rows * f.nslots * 4 + (size_t)f.red_rows * TQ_D * 4 + 4 * sizeof(uint64_t) +
           (size_t)2 * f.red_rows * TQ_D * 2 + 16;
}

template <typename T, int KB, int VB, int NSTAGE>
void launch_turbo_typed(const TurboParams &p, int ctas, cudaStream_t stream) {
    const size_t smem = turbo_fixed_smem<KB, VB, NSTAGE>() + turbo_red_smem(p.flat);
    static size_t configured[64] = {0};
    const int dev = current_device();
    if (dev >= 0 && dev < 64 && configured[dev] < smem) {
        KVC_CUDA(cudaFuncSetAttribute(attn_turbo_decode8_kernel<T, KB, VB, NSTAGE>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        KVC_CUDA(cudaFuncSetAttribute(attn_turbo_decode8_kernel<T, KB, VB, NSTAGE>,
                                      cudaFuncAttributePreferredSharedMemoryCarveout, 100));
        configured[dev] = smem;
    }
    KernelTimer timer(stream);
    KVC_CUDA(launch_pdl(attn_turbo_decode8_kernel<T, KB, VB, NSTAGE>, dim3(ctas), dim3(TQ_THREADS), smem, stream, p));
    timer.stop();
    KVC_CUDA(cudaGetLastError());
    ++g_launch_count;
}

// Rows must be contiguous, a full last tile must stay inside the (batch, head) slab (capacities
// are multiples of the tile), and every slab must keep the 16-byte alignment bulk copies need.
bool turbo_source_fits(const KVSource &s, int D, int64_t T) {
    if (s.kind != SRC_TURBO || !s.data || !s.norms) return false;
    if (s.bits < 2 || s.bits > 4) return false;
    const int words = D * s.bits / 32;
    if (s.words != words || s.st != words || s.gst != 1) return false;
    const int64_t padded = (T + TQ_TILE - 1) / TQ_TILE * TQ_TILE;
    if (s.sh < padded * words || s.gsh < padded) return false;
    if ((s.sh * 4) % 16 || (s.sb * 4) % 16 || (s.gsh * 4) % 16 || (s.gsb * 4) % 16) return false;
    if (((uintptr_t)s.data & 15) || ((uintptr_t)s.norms & 15)) return false;
    return true;
}

}  // namespace

int launch_attention_turbo_v4(const AttnArgs &a, cudaStream_t stream);
int launch_attention_verify_tc(const AttnArgs &a, cudaStream_t stream);   // attn_turbo_v4.cu: 4-bit values

// Returns the number of kernels launched, or 0 when the call does not fit this path.
int launch_attention_turbo(const AttnArgs &a, cudaStream_t stream) {
    if (a.q_dtype != KVC_BF16 && a.q_dtype != KVC_F16) return 0;
    if (a.D != TQ_D) return 0;
    if (a.mask.mode == KVC_MASK_ARRAY || !a.q_signs || !a.o_signs) return 0;
    if (a.k.kind != SRC_TURBO || a.v.kind != SRC_TURBO) return 0;
    if (a.Hkv <= 0 || a.Hq % a.Hkv) return 0;
    const int rep = a.Hq / a.Hkv;
    if (a.T < 1 || a.T > (int64_t)1 << 30) return 0;
    if (!turbo_source_fits(a.k, a.D, a.T) || !turbo_source_fits(a.v, a.D, a.T)) return 0;
    if (((uintptr_t)a.q & 1)) return 0;
    const int kb = a.k.bits, vb = a.v.bits;
    if (vb == 4 && rep * a.L > 8) {   // a verify round: the group's rows on the tensor-core kernel, keys and values decoded once
        const int n = launch_attention_verify_tc(a, stream);
        if (n > 0) return n;
    }
    if (vb == 4) {   // key bits 2..4; also takes short chunks (up to 64 query rows per kv head), eight rows at a time
        const int n = launch_attention_turbo_v4(a, stream);
        if (n > 0) return n;
    }
    const bool known = (kb == 4 && vb == 4) || (kb == 4 && vb == 2) || (kb == 3 && vb == 3) || (kb == 2 && vb == 2) ||
                       (kb == 3 && vb == 4);
    if (!known) return 0;
    if (rep * a.L > 8) return 0;
    const int64_t bh = (int64_t)a.B * a.Hkv;
    if (bh * (int64_t)sizeof(int) > TQ_COUNTER_BYTES) return 0;
    int *status = device_status_word(a.device);
    if (!status) return 0;
    int *counters = counters_get(a.device, stream, TQ_COUNTER_BYTES);

    const int64_t tiles = (a.T + TQ_TILE - 1) / TQ_TILE;
    // Flat decomposition over one wave: CTAs resident per SM by shared memory (tables + ring +
    // cross-warp buffers, +1 KB the driver reserves per CTA), at most 2 by the launch bounds.
    size_t fixed = 0;
    if (kb == 3 && vb == 4) fixed = turbo_fixed_smem<3, 4, 5>();
    else if (kb == 4 && vb == 4) fixed = turbo_fixed_smem<4, 4, 4>();
    else if (kb == 4 && vb == 2) fixed = turbo_fixed_smem<4, 2, 7>();
    else if (kb == 3 && vb == 3) fixed = turbo_fixed_smem<3, 3, 7>();
    else fixed = turbo_fixed_smem<2, 2, 10>();
    FlatPlan plan;
    plan.tiles = (int)tiles;
    plan.red_rows = rep * a.L;
    plan.nslots = 64;
    const size_t per_cta = fixed + turbo_red_smem(plan) + 1024;
    const int resident = (int)std::max<size_t>(1, std::min<size_t>(2, (size_t)227 * 1024 / per_cta));
    const int64_t work_tiles = bh * tiles;
    const int64_t ctas = std::min<int64_t>((int64_t)sm_count(a.device) * resident, work_tiles);
    plan.per = (int)(work_tiles / ctas);
    plan.rem = (int)(work_tiles % ctas);
    plan.nslots = (int)((tiles + plan.per - 1) / plan.per + 1);
    if (plan.nslots > 64) return 0;
    const int64_t splits = plan.nslots;
    const int64_t qrows = (int64_t)a.B * a.Hq * a.L;
    const size_t o_bytes = (size_t)qrows * splits * a.D * sizeof(float);
    const size_t ml_bytes = (size_t)qrows * splits * sizeof(float2);
    char *scratch = (char *)scratch_get(a.device, o_bytes + ml_bytes + 256, stream);

    TurboParams p;
    p.q = a.q; p.out = a.out; p.out_dtype = a.q_dtype;
    p.q_sb = a.q_sb; p.q_sh = a.q_sh; p.q_sl = a.q_sl;
    p.o_sb = a.o_sb; p.o_sh = a.o_sh; p.o_sl = a.o_sl;
    p.kp = (const uint32_t *)a.k.data; p.vp = (const uint32_t *)a.v.data;
    p.kn = a.k.norms; p.vn = a.v.norms;
    p.kp_sb = a.k.sb; p.kp_sh = a.k.sh; p.vp_sb = a.v.sb; p.vp_sh = a.v.sh;
    p.kn_sb = a.k.gsb; p.kn_sh = a.k.gsh; p.vn_sb = a.v.gsb; p.vn_sh = a.v.gsh;
    p.q_signs = a.q_signs; p.o_signs = a.o_signs; p.q_calib = a.q_calib;
    for (int i = 0; i < 16; ++i) {
        p.kcb[i] = a.k.codebook[i];
        p.vcb[i] = a.v.codebook[i];
    }
    p.o_part = (float *)scratch;
    p.ml_part = (float2 *)(scratch + ((o_bytes + 255) / 256) * 256);
    p.counters = counters; p.status = status;
    p.B = a.B; p.Hq = a.Hq; p.Hkv = a.Hkv; p.L = a.L; p.T = a.T;
    p.splits = (int)splits;
    p.tiles_base = (int)(tiles / splits);
    p.tiles_rem = (int)(tiles % splits);
    p.causal = a.mask.mode == KVC_MASK_CAUSAL ? 1 : 0;
    p.debug_skip = measure_skip_bits();
    p.causal_offset = a.mask.causal_offset;
    p.scale_log2 = a.scale * 1.4426950408889634f;
    p.flat = plan;
    p.q_bulk = (a.L == 1 && a.q_sh == a.D && ((uintptr_t)a.q & 15) == 0 && (a.q_sb * 2) % 16 == 0) ? 1 : 0;
    const int units = (int)ctas;

#define KVC_TQ(TT, KK, VV, NS)                                  \
    if (kb == KK && vb == VV) {                                 \
        launch_turbo_typed<TT, KK, VV, NS>(p, units, stream);   \
        return 1;                                               \
    }
    if (a.q_dtype == KVC_BF16) {
        KVC_TQ(__nv_bfloat16, 3, 4, 5)
        KVC_TQ(__nv_bfloat16, 4, 4, 4)
        KVC_TQ(__nv_bfloat16, 4, 2, 7)
        KVC_TQ(__nv_bfloat16, 3, 3, 7)
        KVC_TQ(__nv_bfloat16, 2, 2, 10)
    } else {
        KVC_TQ(__half, 3, 4, 5)
        KVC_TQ(__half, 4, 4, 4)
        KVC_TQ(__half, 4, 2, 7)
        KVC_TQ(__half, 3, 3, 7)
        KVC_TQ(__half, 2, 2, 10)
    }
#undef KVC_TQ
    return 0;
}

}  // namespace kvc
