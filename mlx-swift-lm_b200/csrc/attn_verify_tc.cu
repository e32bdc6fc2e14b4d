// Speculative verify rounds on the 5th-generation tensor cores: TurboQuant, affine and raw caches.
//
// TurboQuantKVCache.compressedAttention for a handful of query positions per head
// (TurboQuantKVCache.swift:1164-1446; the reference's kernel for this step is the causal flash pass at
// TurboQuantKernels.swift:879-1026), quantizedScaledDotProductAttention over the QuantizedKVCache
// (KVCache.swift:1045-1110) and plain scaled-dot-product attention over a KVCacheSimple for the same call
// shape: the rows of a KV head's group (rep heads x L positions, 9 ... 64 of them) all read the same keys
// and values, so the packed rows should be decoded ONCE for the group. The decode kernels cannot do that
// (their accumulators for more than eight rows do not fit the register file); here the group's rows are the
// 128-row M side of tcgen05.mma and the accumulators live in TMEM.
//
// The key tiles of all (batch, KV head) units, laid end to end, are cut into one equal range per SM; a CTA
// works through its range unit by unit. In a CTA:
//   warp 0      loads the group's queries once (TMA, 128 rows x D, rows past the group zero; rotated for
//               TurboQuant, column-permuted for the affine codec, as they are for raw caches)
//   warp 1      owns TMEM; lane 0 issues S_j = Q' K_j^T (two tiles ahead) and O_j = P_j V_j
//   warps 4, 5  softmax: thread = query row = TMEM lane 0..63 (a group has at most 64 rows here, and a warp
//               reaches the TMEM lanes 32 * (warp % 4) ...): scores to probabilities, row sums
//   warps 8, 9, 12, 13  correction: thread = (query row, half of the dims), folds O_j into the row's
//               register accumulator; warps 12, 13 also keep the running row maxima (they wait most of a
//               step for the O product anyway)
//   warps 2, 6, 10, 14 (keys) and 3, 7, 11, 15 (values)  row writers: thread = key row of the tile; the
//               row's packed codes and norm (affine: scales and biases) of the NEXT tile are prefetched
//               into registers while this one is decoded and written as the f16 row of the swizzled K / V
//               tile the tensor cores read. Raw caches: lane 0 of warps 2 and 3 issue tiled TMA loads instead.
// 16 warps leave a thread 128 registers, which is why a correction thread holds half a row.
// TurboQuant centroids come from lane-replicated tables of index PAIRS (conflict-free whatever the
// indices); affine codes become f16 by a mask and one fma. The probabilities never visit shared memory:
// the softmax warps store P_j into TMEM columns of its own, and the O product reads it there as its A operand.
// Keys past T are written as zero rows, so masked probabilities never meet a non-finite value.
//
// A unit cut by a CTA boundary: every piece writes its rows un-normalised with (max, sum); a merge kernel
// combines them. TurboQuant outputs are rows in the rotated basis (f16); the caller rotates them back.
// Every wait is bounded; a wait that runs out sets the device status word, the CTA drains and frees
// its TMEM.
#include <atomic>
#include <cstring>
#include <cstdio>
#include <cstdlib>
#include <type_traits>

#include "attn_common.cuh"
#include "common.h"
#include "tc_common.cuh"

namespace kvc {

void launch_rotate_rows_f16(const void *in, void *out, int32_t in_dtype, int32_t out_dtype, int64_t i_sb, int64_t i_sh, int64_t i_sl,
                            int64_t o_sb, int64_t o_sh, int64_t o_sl, int B, int H, int L, int D, const float *pre,
                            const float *post, cudaStream_t stream);

namespace {

using namespace dev;
using namespace tc;

constexpr int VT_D = 128;
constexpr int VT_THREADS = 512;            // 16 warps: at most 128 registers each
constexpr int VT_TILE = TC_TILE;             // 32 KB: 128 rows x 128 f16

struct VerifyParams {
    const uint32_t *kp, *vp;               // packed indices [B, H, cap, words]
    const float *kn, *vn;                  // TurboQuant: norms [B, H, cap]
    int64_t kp_sb, kp_sh, vp_sb, vp_sh, kn_sb, kn_sh, vn_sb, vn_sh;
    const uint16_t *ks, *kz, *vs, *vz;     // affine: scales and biases [B, H, cap, D / 64] (strides kn_* / vn_*, in elements)
    int32_t sz_bf16;                       // affine: scales and biases are bf16 (else f16)
    int32_t out_bf16;                      // affine: the output rows are bf16 (else f16); TurboQuant rows are f16
    int32_t permuted;                      // affine: the code bits (4 or 8); column c of a row is dim affine_dim_of(c, bits). 0: columns are dims
    float kcb[16], vcb[16];
    void *out;                             // f16 rows, rotated basis, [B, Hq, L, D] with these strides
    int64_t o_sb, o_sh, o_sl;
    int32_t B, Hq, Hkv, L, R;              // R = (Hq / Hkv) * L rows per unit
    int64_t T;
    int32_t causal;
    int64_t causal_offset;
    float scale_log2;
    int32_t tiles_per_cta, max_pieces;     // flat decomposition: CTA c owns the tiles [c, c + 1) * tiles_per_cta of all units laid end to end
    float *o_part;                         // [unit][piece][R][D]: a unit cut by a CTA boundary is merged from its pieces
    float2 *ml_part;                       // [unit][piece][R] (log2-domain max, sum)
    int *status;
    int32_t debug_skip;                    // measurement builds only (KVC_SKIP_BITS)
};

enum : int {
    VB_Q = 0,
    VB_K_FULL = 1,                     // [2] 128 arrivals: the key rows of a tile are written
    VB_K_EMPTY = VB_K_FULL + 2,        // [2] the S product has read the tile
    VB_V_FULL = VB_K_EMPTY + 2,        // [2]
    VB_V_EMPTY = VB_V_FULL + 2,        // [2]
    VB_S_FULL = VB_V_EMPTY + 2,        // [2]
    VB_S_EMPTY = VB_S_FULL + 2,        // [2]
    VB_P_FULL = VB_S_EMPTY + 2,        // [2] P_j is in TMEM
    VB_P_EMPTY = VB_P_FULL + 2,        // [2] the O product has read P_j
    VB_O_FULL = VB_P_EMPTY + 2,        // [1] the O accumulator of one tile (single: it is folded away long before the next)
    VB_O_EMPTY = VB_O_FULL + 1,        // [1]
    VB_A_FULL = VB_O_EMPTY + 1,        // [4] row statistics of a tile (taken two tiles ahead of the fold)
    VB_A_EMPTY = VB_A_FULL + 4,        // [4]
    VB_L_FULL = VB_A_EMPTY + 4,
    VB_COUNT = VB_L_FULL + 1
};

__device__ __forceinline__ uint32_t hsub2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t hfma2(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}
// One 16-bit scale or bias (bf16 or f16 bits) as an f16 pair (x, x), kept inside the f16 range.
__device__ __forceinline__ uint32_t splat_f16(uint32_t bits16, bool is_bf16) {
    float x = is_bf16 ? __uint_as_float(bits16 << 16) : __half2float(__ushort_as_half((unsigned short)bits16));
    x = fminf(fmaxf(x, -65504.f), 65504.f);
    return pack_h2(x, x);
}
// The affine codec writes the dims of every group of eight in the order 0 4 1 5 2 6 3 7 (4-bit codes: the
// nibbles i and i + 4 of a word come out of one mask as an f16 pair) or 0 2 1 3 4 6 5 7 (8-bit codes: the
// bytes i and i + 2 of a word come out of one byte permute): the queries are laid out the same way, so the
// scores do not change, and the output rows are put back in order when they are stored.
__host__ __device__ constexpr int affine_dim_of(int pos, int bits) {
    return bits == 4 ? (pos & ~7) | (((pos & 7) >> 1) + 4 * (pos & 1)) : (pos & ~3) | ((pos & 1) << 1) | ((pos >> 1) & 1);
}
// the column that holds dim `dim`
__host__ __device__ constexpr int affine_pos_of(int dim, int bits) {
    return bits == 4 ? (dim & ~7) | (2 * (dim & 3) + ((dim >> 2) & 1)) : (dim & ~3) | ((dim & 1) << 1) | ((dim >> 1) & 1);
}
constexpr bool affine_orders_invert(int bits) {
    for (int i = 0; i < 16; ++i)
        if (affine_pos_of(affine_dim_of(i, bits), bits) != i || affine_dim_of(affine_pos_of(i, bits), bits) != i) return false;
    return true;
}
static_assert(affine_orders_invert(4) && affine_orders_invert(8), "affine_pos_of must undo affine_dim_of");
static_assert(affine_dim_of(1, 4) == 4 && affine_dim_of(2, 4) == 1 && affine_dim_of(1, 8) == 2 && affine_dim_of(2, 8) == 1,
              "column order of the affine codec: nibbles (i, i + 4) and bytes (i, i + 2) come out as pairs");

__device__ __forceinline__ uint32_t hmul2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

// Index pair p (bits [2*KB*p, 2*KB*(p+1)) of the row's word stream); p is a compile-time constant
// after unrolling, so the shifts are immediates.
template <int KB, int NW>
__device__ __forceinline__ uint32_t pair_index(const uint32_t (&w)[NW], int p) {
    constexpr int B2 = 2 * KB;
    const int bit = B2 * p, k = bit >> 5, s = bit & 31;
    uint32_t x = w[k] >> s;
    if (s + B2 > 32) x |= w[k + 1] << (32 - s);
    return x & ((1u << B2) - 1u);
}

// AFFINE: the cache is the group-wise affine one (KB = 4- or 8-bit codes, groups of 64, QuantizedKVCache); the rows are
// code * scale + bias instead of norm * centroid, there are no tables, the output rows are TO.
// RAW: the cache holds plain f16 / bf16 rows (KVCacheSimple): the K / V tiles come in by tiled TMA loads (two lanes
// are the producers, the other writer warps idle), queries, tiles and probabilities are TO.
template <typename TO, int KB, bool AFFINE, bool RAW = false>
__global__ void __launch_bounds__(VT_THREADS, 1)
attn_verify_tc_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                      const __grid_constant__ CUtensorMap vmap, const __grid_constant__ VerifyParams p) {
    using TP = typename std::conditional<RAW, TO, __half>::type;      // operand type of Q', K, V and P
    constexpr int D = VT_D;
    constexpr int KW = D * KB / 32;          // key words per row
    constexpr int VW = AFFINE ? KW : D * 4 / 32;   // value words per row (TurboQuant: 4-bit; affine: as the keys)
    // 4-bit keys share the value pair table (the launcher checks that the two codebooks are the same): a second
    // 32 KB table does not fit beside the tiles
    constexpr int KTAB_ENTRIES = (AFFINE || RAW || KB == 4) ? 0 : 1 << (2 * KB);
    constexpr int VTAB_WORDS = (AFFINE || RAW) ? 0 : 256 * 32;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char *sq = base;                                  // Q' block
    unsigned char *skv = sq + VT_TILE;                         // stage s: K tile | V tile
    uint32_t *vtab = (uint32_t *)(skv + 2 * 2 * VT_TILE);      // [256 byte values][32 lanes] f16x2(c[b & 15], c[b >> 4])
    uint32_t *ktab_own = vtab + VTAB_WORDS;                    // [entries][32 lanes] f16x2
    uint32_t *ktab = KB == 4 ? vtab : ktab_own;
    uint64_t *bars = (uint64_t *)(ktab_own + KTAB_ENTRIES * 32);
    uint32_t *tmem_slot = (uint32_t *)(bars + VB_COUNT);
    float *s_alpha = (float *)(tmem_slot + 4);                 // [4][128]: rows 0..63 alpha, rows 64..127 -max
    float *s_lsum = s_alpha + 4 * TC_ROWS;                     // [128]
    float *s_mfin = s_lsum + TC_ROWS;                          // [128]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rep = p.Hq / p.Hkv;
    const int n_all = (int)((p.T + TC_KEYS - 1) / TC_KEYS);
    // The key tiles of all units laid end to end are cut into equal ranges, one per CTA (so that every SM has
    // the same work whatever the number of units): a CTA walks its range one segment (= its part of one unit)
    // after the other, the pipeline drained and the barriers set up again in between.
    const int64_t flat_end = (int64_t)p.B * p.Hkv * n_all;
    const int64_t flat_lo = (int64_t)blockIdx.x * p.tiles_per_cta, flat_hi = min(flat_end, flat_lo + (int64_t)p.tiles_per_cta);
    int *seg_stop = (int *)(s_mfin + TC_ROWS);

    auto init_barriers = [&]() {
        mbar_init(&bars[VB_Q], 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&bars[VB_K_FULL + s], RAW ? 1 : 128);
            mbar_init(&bars[VB_K_EMPTY + s], 1);
            mbar_init(&bars[VB_V_FULL + s], RAW ? 1 : 128);
            mbar_init(&bars[VB_V_EMPTY + s], 1);
            mbar_init(&bars[VB_S_FULL + s], 1);
            mbar_init(&bars[VB_S_EMPTY + s], 64);      // the two softmax warps
            mbar_init(&bars[VB_P_FULL + s], 64);
            mbar_init(&bars[VB_P_EMPTY + s], 1);
        }
        for (int s = 0; s < 4; ++s) {
            mbar_init(&bars[VB_A_FULL + s], 64);       // warps 12, 13
            mbar_init(&bars[VB_A_EMPTY + s], 192);     // the softmax and the correction threads read a tile's row statistics
        }
        mbar_init(&bars[VB_O_FULL], 1);
        mbar_init(&bars[VB_O_EMPTY], 128);             // the four correction warps
        mbar_init(&bars[VB_L_FULL], 128);              // row sums (softmax warps) and row maxima (warps 12, 13)
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    };
    if (tid == 0) init_barriers();
    // tables: key entry e of lane l = f16x2(centroid[e & m], centroid[e >> KB]); value entry i = (c, c)
    if constexpr (!AFFINE && !RAW) {
        for (int w = tid; w < KTAB_ENTRIES * 32; w += VT_THREADS) {
            const int e = w >> 5;
            ktab[w] = pack_h2(p.kcb[e & ((1 << KB) - 1)], p.kcb[e >> KB]);
        }
        for (int w = tid; w < VTAB_WORDS; w += VT_THREADS) vtab[w] = pack_h2(p.vcb[(w >> 5) & 15], p.vcb[w >> 9]);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TC_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    pdl_wait();

    int seg = 0;
    for (int64_t pos = flat_lo; pos < flat_hi; ++seg) {
    const int unit = (int)(pos / n_all), j_lo = (int)(pos % n_all);
    const int n_tiles = (int)min((int64_t)(n_all - j_lo), flat_hi - pos);
    const int hk = unit % p.Hkv, b = unit / p.Hkv;
    const bool whole = j_lo == 0 && n_tiles == n_all;                                   // this CTA has the unit to itself
    const int piece = (int)blockIdx.x - (int)(((int64_t)unit * n_all) / p.tiles_per_cta);
    if (seg > 0) {
        // everything of the segment before has completed (the MMA thread waited for its last commits): fresh
        // barriers, all phases at zero
        if (tid == 0) {
            for (int i = 0; i < VB_COUNT; ++i) asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(&bars[i])) : "memory");
            init_barriers();
        }
        __syncthreads();
    }

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(&bars[VB_Q], VT_TILE);
            tma_load_4d(sq, &qmap, &bars[VB_Q], 0, 0, unit, 0);
            tma_load_4d(sq + TC_BOX, &qmap, &bars[VB_Q], 64, 0, unit, 0);
        }
    } else if (warp == 1) {
        // ---------------- MMA issue ----------------
        if (lane == 0) {
            // operand formats at bits 7-9 (A) and 10-12 (B): 0 = f16, 1 = bf16
            constexpr uint32_t FMT = std::is_same<TP, __nv_bfloat16>::value ? 1u : 0u;
            constexpr uint32_t IDESC = (1u << 4) | (FMT << 7) | (FMT << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
            constexpr uint32_t IDESC_PV = (1u << 4) | (FMT << 7) | (FMT << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | ((128u >> 4) << 24);
            const uint64_t q_desc = umma_desc(smem_u32(sq), 16, 1024);
            const uint64_t k_desc = umma_desc(smem_u32(skv), 16, 1024);
            const uint64_t v_desc = umma_desc(smem_u32(skv) + VT_TILE, 16384, 1024);
            bool ok = mbar_wait(&bars[VB_Q], 0);
            auto issue_s = [&](int j) {
                const int s = j & 1;
                if (!mbar_wait(&bars[VB_K_FULL + s], (j >> 1) & 1)) return false;
                if (j >= 2 && !mbar_wait(&bars[VB_S_EMPTY + s], ((j >> 1) - 1) & 1)) return false;
                tc_fence_after();
                const uint64_t kd = k_desc + (uint64_t)(s * (2 * VT_TILE / 16));
                const uint32_t d_addr = tmem + (uint32_t)s * 128u;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint64_t off = (uint64_t)((ks >> 2) * (TC_BOX / 16) + (ks & 3) * 2);
                    umma_f16(d_addr, q_desc + off, kd + off, IDESC, ks > 0 ? 1u : 0u);
                }
                umma_commit(&bars[VB_S_FULL + s]);
                umma_commit(&bars[VB_K_EMPTY + s]);
                return true;
            };
            // TMEM columns: S_0, S_1 at 0, 128; O at 256; P_0, P_1 at 384, 448. The S product runs two tiles ahead
            // of the O product: S_{j+2} (which the row statistics and then the softmax of tile j + 2 wait for) is
            // issued the moment the softmax warps have read S_j, in front of O_j.
            if (ok && n_tiles > 0) ok = issue_s(0);
            if (ok && n_tiles > 1) ok = issue_s(1);
            for (int j = 0; j < n_tiles && ok; ++j) {
                if (j + 2 < n_tiles) ok = issue_s(j + 2);
                if (!ok) break;
                const int s = j & 1;
                ok = mbar_wait(&bars[VB_V_FULL + s], (j >> 1) & 1);
                if (ok) ok = mbar_wait(&bars[VB_P_FULL + s], (j >> 1) & 1);
                if (ok && j >= 1) ok = mbar_wait(&bars[VB_O_EMPTY], (j - 1) & 1);
                if (!ok) break;
                tc_fence_after();
                const uint64_t vd = v_desc + (uint64_t)(s * (2 * VT_TILE / 16));
                const uint32_t o_addr = tmem + 256u;
                // P_j is read from TMEM, where the softmax warps wrote it (16 keys = 8 columns per product)
                const uint32_t p_addr = tmem + 384u + (uint32_t)s * 64u;
#pragma unroll
                for (int ks = 0; ks < TC_KEYS / 16; ++ks)
                    umma_f16_ts(o_addr, p_addr + (uint32_t)ks * 8u, vd + (uint64_t)(ks * 128), IDESC_PV, ks > 0 ? 1u : 0u);
                umma_commit(&bars[VB_O_FULL]);
                umma_commit(&bars[VB_P_EMPTY + s]);
                umma_commit(&bars[VB_V_EMPTY + s]);
            }
            // the commits of the last two tiles nobody else waits for: they must have arrived before the barriers
            // are set up again for the next segment
            for (int back = 1; back <= 2 && ok; ++back) {
                const int jl = n_tiles - back;
                if (jl < 0) break;
                const int s = jl & 1, par = (jl >> 1) & 1;
                ok = mbar_wait(&bars[VB_K_EMPTY + s], par) && mbar_wait(&bars[VB_V_EMPTY + s], par) && mbar_wait(&bars[VB_P_EMPTY + s], par);
            }
            if (!ok) atomicExch(p.status, 26);
        }
    } else if (warp == 4 || warp == 5) {
        // ---------------- softmax: thread = row (TMEM lanes 0..63) ----------------
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        // the TMEM loads and stores below are warp-wide: a warp works on all its 32 rows (the rows past the
        // group have zero queries: finite scores, results never stored)
        const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
        const int l_pos = row % p.L;
        const int64_t limit = p.causal ? min(p.T - 1, p.causal_offset + l_pos) : p.T - 1;
        const int64_t min_limit = p.causal ? min(p.T - 1, p.causal_offset) : p.T - 1;   // the smallest limit of a live row
        float l_run = 0.f;
        bool ok = true;
        // The row maximum of a tile comes from warps 12, 13 (which read the scores first); here the scores are
        // read once more and turned into probabilities. The loop over the four 32-column blocks of a tile
        // stays rolled: unrolled over 128 columns the roles of this kernel together outgrow the instruction
        // cache, and every warp waits on fetches.
        for (int j = 0; j < n_tiles; ++j) {
            ok = mbar_wait(&bars[VB_A_FULL + (j & 3)], (j >> 2) & 1);
            if (ok) ok = mbar_wait(&bars[VB_S_FULL + (j & 1)], (j >> 1) & 1);    // complete since the statistics were taken
            if (ok && j >= 2) ok = mbar_wait(&bars[VB_P_EMPTY + (j & 1)], ((j >> 1) - 1) & 1);   // the O product of tile j - 2 has read its P
            if (!ok) break;
            const float alpha = s_alpha[(j & 3) * TC_ROWS + row], neg_m = s_alpha[(j & 3) * TC_ROWS + 64 + row];
            mbar_arrive(&bars[VB_A_EMPTY + (j & 3)]);
            tc_fence_after();
            const uint32_t s_addr = lane_addr + (uint32_t)(j & 1) * 128u;
            const int64_t key0 = (int64_t)(j_lo + j) * TC_KEYS;
            const bool edge = key0 + TC_KEYS - 1 > min_limit;        // the same for every thread
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
            for (int cb = 0; cb < 4; ++cb) {
                uint32_t raw[32];
                tmem_ld32_issue(s_addr + cb * 32, raw);
                tmem_ld_wait();
                if (edge) {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (key0 + cb * 32 + i > limit) raw[i] = 0xff800000u;
                }
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float e0 = (KVC_SKIP_BITS(p) & 16) ? 0.f : fast_exp2(fmaf(__uint_as_float(raw[2 * i]), p.scale_log2, neg_m));
                    const float e1 = (KVC_SKIP_BITS(p) & 16) ? 0.f : fast_exp2(fmaf(__uint_as_float(raw[2 * i + 1]), p.scale_log2, neg_m));
                    sum4[(2 * i) & 3] += e0;
                    sum4[(2 * i + 1) & 3] += e1;
                    pk[i] = pack_pair<TP>(e0, e1);
                }
                // P_j goes into TMEM (this thread's lane, columns of its own), where the O product reads it as its
                // A operand: the 32 scores of block cb become 16 columns
                tmem_st16_issue(lane_addr + 384u + (uint32_t)(j & 1) * 64u + cb * 16, pk);
            }
            tc_fence_before();
            mbar_arrive(&bars[VB_S_EMPTY + (j & 1)]);     // S_j has been read: the S product of tile j + 2 may overwrite it
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(&bars[VB_P_FULL + (j & 1)]);
            l_run = l_run * alpha + (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
        }
        if (ok) {
            s_lsum[row] = l_run;
            mbar_arrive(&bars[VB_L_FULL]);
        } else {
            atomicExch(p.status, 27);
        }
    } else if ((warp & 2) == 0 && warp >= 8) {
        // ---------------- correction: thread = (query row, half of the dims); TMEM lanes 0..63 ----------------
        // warps 8, 9 hold dims 0..63 of rows 0..31 / 32..63, warps 12, 13 dims 64..127
        const int quarter = warp & 3, dh = (warp >> 2) & 1;
        const int row = quarter * 32 + lane;
        const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16) + 256u + (uint32_t)dh * 64u;
        constexpr int DH = D / 2;
        float o_acc[DH];
#pragma unroll
        for (int i = 0; i < DH; ++i) o_acc[i] = 0.f;
        bool ok = true;
        // warps 12, 13 also keep the running row maximum: they read S_j as soon as it is complete (the S product
        // of tile j + 1 is issued before the O product of tile j, so this runs ahead of the fold below) and
        // publish (alpha, -max) of the tile for the softmax and the correction threads
        const int l_pos = row % p.L;
        const int64_t limit = p.causal ? min(p.T - 1, p.causal_offset + l_pos) : p.T - 1;
        const int64_t min_limit = p.causal ? min(p.T - 1, p.causal_offset) : p.T - 1;   // the smallest limit of a live row
        const uint32_t s_lane = tmem + ((uint32_t)(quarter * 32) << 16);
        float m_run = -INFINITY;
        auto stats = [&](int j) {
            if (!mbar_wait(&bars[VB_S_FULL + (j & 1)], (j >> 1) & 1)) return false;
            tc_fence_after();
            const uint32_t s_addr = s_lane + (uint32_t)(j & 1) * 128u;
            const int64_t key0 = (int64_t)(j_lo + j) * TC_KEYS;
            const bool edge = key0 + TC_KEYS - 1 > min_limit;        // the same for every thread
            float mx = -INFINITY;
#pragma unroll 1
            for (int cb = 0; cb < 4; ++cb) {
                uint32_t raw[32];
                tmem_ld32_issue(s_addr + cb * 32, raw);
                tmem_ld_wait();
                if (edge) {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (key0 + cb * 32 + i > limit) raw[i] = 0xff800000u;   // -inf
                }
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(raw[i]));
                mx = fmaxf(mx, fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])));
            }
            const float m_new = fmaxf(m_run, mx * p.scale_log2);
            const float alpha = (m_run == -INFINITY) ? 0.f : fast_exp2(m_run - m_new);
            const float neg_m = (m_new == -INFINITY) ? 0.f : -m_new;
            if (j >= 4 && !mbar_wait(&bars[VB_A_EMPTY + (j & 3)], ((j >> 2) - 1) & 1)) return false;
            s_alpha[(j & 3) * TC_ROWS + row] = alpha;
            s_alpha[(j & 3) * TC_ROWS + 64 + row] = neg_m;
            tc_fence_before();
            mbar_arrive(&bars[VB_A_FULL + (j & 3)]);
            m_run = m_new;
            return true;
        };
        auto fold = [&](int j) {      // fold O_j into the row's accumulator
            if (!mbar_wait(&bars[VB_A_FULL + (j & 3)], (j >> 2) & 1)) return false;
            const float alpha = s_alpha[(j & 3) * TC_ROWS + row];
            mbar_arrive(&bars[VB_A_EMPTY + (j & 3)]);
            if (!mbar_wait(&bars[VB_O_FULL], j & 1)) return false;
            tc_fence_after();
            if (!(KVC_SKIP_BITS(p) & 4)) {
#pragma unroll
                for (int part = 0; part < DH / 32; ++part) {
                    uint32_t raw[32];
                    tmem_ld32_issue(lane_addr + part * 32, raw);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o_acc[part * 32 + i] = fmaf(o_acc[part * 32 + i], alpha, __uint_as_float(raw[i]));
                }
            }
            tc_fence_before();
            mbar_arrive(&bars[VB_O_EMPTY]);
            return true;
        };
#pragma unroll 1
        for (int j = 0; j < n_tiles + 2 && ok; ++j) {      // the statistics run two tiles ahead of the fold
            if (dh == 1 && j < n_tiles) ok = stats(j);
            if (ok && j >= 2) ok = fold(j - 2);
        }
        if (ok && dh == 1) {
            s_mfin[row] = m_run;
            mbar_arrive(&bars[VB_L_FULL]);
        }
        if (ok) ok = mbar_wait(&bars[VB_L_FULL], 0);
        if (!ok) {
            atomicExch(p.status, 28);
        } else if (row < p.R) {
            const float l_sum = s_lsum[row];
            const int hq = hk * rep + row / p.L, lq = row % p.L;
            if (whole) {
                const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
                TO *dst = (TO *)p.out + b * p.o_sb + hq * p.o_sh + lq * p.o_sl + dh * DH;
#pragma unroll
                for (int c8 = 0; c8 < DH / 8; ++c8) {
                    // affine rows: dim 8 c + i sits in column 8 c + affine_pos_of(i)
                    constexpr int P0 = AFFINE ? affine_pos_of(0, KB) : 0, P1 = AFFINE ? affine_pos_of(1, KB) : 1;
                    constexpr int P2 = AFFINE ? affine_pos_of(2, KB) : 2, P3 = AFFINE ? affine_pos_of(3, KB) : 3;
                    constexpr int P4 = AFFINE ? affine_pos_of(4, KB) : 4, P5 = AFFINE ? affine_pos_of(5, KB) : 5;
                    constexpr int P6 = AFFINE ? affine_pos_of(6, KB) : 6, P7 = AFFINE ? affine_pos_of(7, KB) : 7;
                    uint4 w;
                    w.x = pack_pair<TO>(o_acc[c8 * 8 + P0] * inv, o_acc[c8 * 8 + P1] * inv);
                    w.y = pack_pair<TO>(o_acc[c8 * 8 + P2] * inv, o_acc[c8 * 8 + P3] * inv);
                    w.z = pack_pair<TO>(o_acc[c8 * 8 + P4] * inv, o_acc[c8 * 8 + P5] * inv);
                    w.w = pack_pair<TO>(o_acc[c8 * 8 + P6] * inv, o_acc[c8 * 8 + P7] * inv);
                    *(uint4 *)(dst + c8 * 8) = w;
                }
            } else {
                const int64_t slot = ((int64_t)unit * p.max_pieces + piece) * p.R + row;
                float4 *dst = (float4 *)(p.o_part + slot * D + dh * DH);
#pragma unroll
                for (int c4 = 0; c4 < DH / 4; ++c4) dst[c4] = make_float4(o_acc[c4 * 4], o_acc[c4 * 4 + 1], o_acc[c4 * 4 + 2], o_acc[c4 * 4 + 3]);
                if (dh == 0) p.ml_part[slot] = make_float2(s_mfin[row], l_sum);
            }
        }
    } else {
        // ---------------- row writers: thread = key row of the tile ----------------
        // warps 2, 6, 10, 14 write the key rows, warps 3, 7, 11, 15 the value rows (32 rows each), at the same time
        const bool is_v = (warp & 1) != 0;
        const int row = (warp >> 2) * 32 + lane;
        if constexpr (RAW) {
            // lane 0 of warp 2 loads the key tiles, lane 0 of warp 3 the value tiles (two boxes of 64 dims each,
            // 128-byte swizzle; rows past T come in as zeros)
            if (warp < 4 && lane == 0) {
                bool ok = true;
                const CUtensorMap *map = is_v ? &vmap : &kmap;
                const int full_bar = is_v ? VB_V_FULL : VB_K_FULL, empty_bar = is_v ? VB_V_EMPTY : VB_K_EMPTY;
                for (int j = 0; j < n_tiles && ok; ++j) {
                    const int s = j & 1;
                    if (j >= 2) ok = mbar_wait(&bars[empty_bar + s], ((j >> 1) - 1) & 1);
                    if (!ok) break;
                    unsigned char *dst = skv + (size_t)s * 2 * VT_TILE + (is_v ? VT_TILE : 0);
                    mbar_expect_tx(&bars[full_bar + s], VT_TILE);
#pragma unroll
                    for (int bx = 0; bx < D / 64; ++bx)
                        tma_load_4d(dst + bx * TC_BOX, map, &bars[full_bar + s], bx * 64, (j_lo + j) * TC_KEYS, hk, b);
                }
                if (!ok) atomicExch(p.status, 29);
            }
        } else if constexpr (AFFINE) {
            const int sw = row & 7;
            bool ok = true;
            // one code path for key and value rows (the warp's kind picks the arrays, the staging places, the tile
            // and the barriers)
            const uint32_t *cbase = is_v ? p.vp + b * p.vp_sb + hk * p.vp_sh : p.kp + b * p.kp_sb + hk * p.kp_sh;
            const uint16_t *sbase = is_v ? p.vs + b * p.vn_sb + hk * p.vn_sh : p.ks + b * p.kn_sb + hk * p.kn_sh;
            const uint16_t *zbase = is_v ? p.vz + b * p.vn_sb + hk * p.vn_sh : p.kz + b * p.kn_sb + hk * p.kn_sh;
            const int full_bar = is_v ? VB_V_FULL : VB_K_FULL, empty_bar = is_v ? VB_V_EMPTY : VB_K_EMPTY;
            const bool sz_bf16 = p.sz_bf16 != 0;
            // The packed row of the NEXT tile is loaded straight into registers while this one is decoded (a
            // thread's row is 64 or 128 contiguous bytes; a warp reads 32 rows in a row): no staging in shared
            // memory, whose data pipe is what bounds this kernel.
            uint4 nxt[KW / 4];
            uint32_t nsc = 0u, nzp = 0u;
            auto fetch = [&](int j) {      // tile j of this CTA's range
                if (j < n_tiles && !(KVC_SKIP_BITS(p) & 1)) {
                    const int64_t t = (int64_t)(j_lo + j) * TC_KEYS + row;
                    const uint4 *src = (const uint4 *)(cbase + t * KW);
#pragma unroll
                    for (int i = 0; i < KW / 4; ++i) nxt[i] = __ldg(src + i);
                    nsc = __ldg((const uint32_t *)(sbase + t * 2));
                    nzp = __ldg((const uint32_t *)(zbase + t * 2));
                }
            };
#pragma unroll
            for (int i = 0; i < KW / 4; ++i) nxt[i] = make_uint4(0u, 0u, 0u, 0u);
            fetch(0);
#pragma unroll 1
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int s = j & 1;
                uint32_t all[KW];
#pragma unroll
                for (int i = 0; i < KW / 4; ++i) {
                    all[4 * i] = nxt[i].x; all[4 * i + 1] = nxt[i].y; all[4 * i + 2] = nxt[i].z; all[4 * i + 3] = nxt[i].w;
                }
                const uint32_t sc = nsc, zp = nzp;
                fetch(j + 1);
                if (j >= 2) ok = mbar_wait(&bars[empty_bar + s], ((j >> 1) - 1) & 1);
                if (!ok) break;
                unsigned char *dst = skv + (size_t)s * 2 * VT_TILE + (is_v ? VT_TILE : 0) + row * 128;
                const bool valid = (int64_t)(j_lo + j) * TC_KEYS + row < p.T;
#pragma unroll 1
                for (int h = 0; h < D / 64; ++h) {      // half a row = one group of 64
                    const uint32_t s2 = valid ? splat_f16(h ? sc >> 16 : sc & 0xffffu, sz_bf16) : 0u;
                    const uint32_t z2 = valid ? splat_f16(h ? zp >> 16 : zp & 0xffffu, sz_bf16) : 0u;
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        uint32_t v4[4];
                        if constexpr (KB == 4) {
                            const uint32_t w = h ? all[KW / 2 + c] : all[c];      // eight 4-bit codes = dims 64 h + 8 c ...
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                // codes q and q + 4 as the f16 pair (1024 + code): minus 1024 is exact, then one fma
                                const uint32_t m = ((w >> (4 * q)) & 0x000F000Fu) | 0x64006400u;
                                v4[q] = hfma2(hsub2(m, 0x64006400u), s2, z2);
                            }
                        } else {
#pragma unroll
                            for (int q = 0; q < 2; ++q) {
                                const uint32_t w = h ? all[KW / 2 + 2 * c + q] : all[2 * c + q];   // four 8-bit codes = dims 64 h + 8 c + 4 q ...
                                // bytes 0 and 2, then 1 and 3, each under the high byte of 1024
                                v4[2 * q] = hfma2(hsub2(__byte_perm(w, 0x64646464u, 0x4240), 0x64006400u), s2, z2);
                                v4[2 * q + 1] = hfma2(hsub2(__byte_perm(w, 0x64646464u, 0x4341), 0x64006400u), s2, z2);
                            }
                        }
                        *(uint4 *)(dst + h * TC_BOX + ((c ^ sw) << 4)) = make_uint4(v4[0], v4[1], v4[2], v4[3]);
                    }
                }
                if (!(KVC_SKIP_BITS(p) & 8)) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(&bars[full_bar + s]);
            }
            if (!ok) atomicExch(p.status, 29);
        } else {
            const uint32_t *kbase = p.kp + b * p.kp_sb + hk * p.kp_sh;
            const uint32_t *vbase = p.vp + b * p.vp_sb + hk * p.vp_sh;
            const float *knb = p.kn + b * p.kn_sb + hk * p.kn_sh;
            const float *vnb = p.vn + b * p.vn_sb + hk * p.vn_sh;
            const uint32_t ktab_a = smem_u32(ktab) + (uint32_t)lane * 4u;
            const uint32_t vtab_a = smem_u32(vtab) + (uint32_t)lane * 4u;
            const int sw = row & 7;
            bool ok = true;
            // The packed row of the NEXT tile is loaded straight into registers while this one is decoded (a
            // thread's row is 32 to 64 contiguous bytes; a warp reads 32 rows in a row): no staging in shared
            // memory, whose data pipe is what bounds this kernel.
            uint4 nk[KW / 4], nv[VW / 4];
            float nkn = 0.f, nvn = 0.f;
#pragma unroll
            for (int i = 0; i < KW / 4; ++i) nk[i] = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
            for (int i = 0; i < VW / 4; ++i) nv[i] = make_uint4(0u, 0u, 0u, 0u);
            auto fetch_k = [&](int j) {      // tile j of this CTA's range
                if (j < n_tiles && !(KVC_SKIP_BITS(p) & 1)) {
                    const int64_t t = (int64_t)(j_lo + j) * TC_KEYS + row;
                    const uint4 *src = (const uint4 *)(kbase + t * KW);
#pragma unroll
                    for (int i = 0; i < KW / 4; ++i) nk[i] = __ldg(src + i);
                    nkn = __ldg(knb + t);
                }
            };
            auto fetch_v = [&](int j) {
                if (j < n_tiles && !(KVC_SKIP_BITS(p) & 1)) {
                    const int64_t t = (int64_t)(j_lo + j) * TC_KEYS + row;
                    const uint4 *src = (const uint4 *)(vbase + t * VW);
#pragma unroll
                    for (int i = 0; i < VW / 4; ++i) nv[i] = __ldg(src + i);
                    nvn = __ldg(vnb + t);
                }
            };
            // The two halves of a row are a rolled loop and each writer has one call site: unrolled, the roles of
            // this kernel together outgrow the instruction cache. Within a half the 32 lookups are issued back to
            // back, then multiplied and stored (a lookup directly before its store leaves one load in flight per
            // thread and the warp waits out every latency).
            auto write_k = [&](int j) {      // the row's copy (the group before the newest) has landed
                const int s = j & 1;
                uint32_t all[KW];
#pragma unroll
                for (int i = 0; i < KW / 4; ++i) {
                    all[4 * i] = nk[i].x; all[4 * i + 1] = nk[i].y; all[4 * i + 2] = nk[i].z; all[4 * i + 3] = nk[i].w;
                }
                const float knorm = nkn;
                fetch_k(j + 1);
                if (j >= 2 && !mbar_wait(&bars[VB_K_EMPTY + s], ((j >> 1) - 1) & 1)) return false;
                unsigned char *dst = skv + (size_t)s * 2 * VT_TILE + row * 128;
                const bool valid = (int64_t)(j_lo + j) * TC_KEYS + row < p.T;
                const float nf = fminf(knorm, 65504.f);
                const uint32_t n2 = valid ? pack_h2(nf, nf) : 0u;
#pragma unroll 1
                for (int h = 0; h < D / 64; ++h) {
                    uint32_t kw[KW / 2];         // 32 index pairs = dims 64 h ... 64 h + 63
#pragma unroll
                    for (int i = 0; i < KW / 2; ++i) kw[i] = h ? all[KW / 2 + i] : all[i];
                    uint32_t t2[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const uint32_t e = pair_index<KB, KW / 2>(kw, i);
                        if (KVC_SKIP_BITS(p) & 2) t2[i] = e;
                        else asm("ld.shared.u32 %0, [%1];" : "=r"(t2[i]) : "r"(ktab_a + (e << 7)));
                    }
#pragma unroll
                    for (int c = 0; c < 8; ++c)
                        *(uint4 *)(dst + h * TC_BOX + ((c ^ sw) << 4)) =
                            make_uint4(hmul2(t2[4 * c], n2), hmul2(t2[4 * c + 1], n2), hmul2(t2[4 * c + 2], n2), hmul2(t2[4 * c + 3], n2));
                }
                if (!(KVC_SKIP_BITS(p) & 8)) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(&bars[VB_K_FULL + s]);
                return true;
            };
            auto write_v = [&](int j) {
                const int s = j & 1;
                uint32_t all[VW];
#pragma unroll
                for (int i = 0; i < VW / 4; ++i) {
                    all[4 * i] = nv[i].x; all[4 * i + 1] = nv[i].y; all[4 * i + 2] = nv[i].z; all[4 * i + 3] = nv[i].w;
                }
                const float vnorm = nvn;
                fetch_v(j + 1);
                if (j >= 2 && !mbar_wait(&bars[VB_V_EMPTY + s], ((j >> 1) - 1) & 1)) return false;
                unsigned char *dst = skv + (size_t)s * 2 * VT_TILE + VT_TILE + row * 128;
                const bool valid = (int64_t)(j_lo + j) * TC_KEYS + row < p.T;
                const float nf = fminf(vnorm, 65504.f);
                const uint32_t n2 = valid ? pack_h2(nf, nf) : 0u;
#pragma unroll 1
                for (int h = 0; h < D / 64; ++h) {
                    uint32_t vw[VW / 2];         // word i = the eight 4-bit indices of dims 64 h + 8 i ...
#pragma unroll
                    for (int i = 0; i < VW / 2; ++i) vw[i] = h ? all[VW / 2 + i] : all[i];
                    uint32_t t2[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        // byte i % 4 of word i / 4 = the indices of two neighbouring dims: one lookup for the pair
                        const uint32_t byte = (vw[i >> 2] >> (8 * (i & 3))) & 255u;
                        if (KVC_SKIP_BITS(p) & 2) t2[i] = byte;
                        else asm("ld.shared.u32 %0, [%1];" : "=r"(t2[i]) : "r"(vtab_a + (byte << 7)));
                    }
#pragma unroll
                    for (int c = 0; c < 8; ++c)
                        *(uint4 *)(dst + h * TC_BOX + ((c ^ sw) << 4)) =
                            make_uint4(hmul2(t2[4 * c], n2), hmul2(t2[4 * c + 1], n2), hmul2(t2[4 * c + 2], n2), hmul2(t2[4 * c + 3], n2));
                }
                if (!(KVC_SKIP_BITS(p) & 8)) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(&bars[VB_V_FULL + s]);
                return true;
            };
            if (is_v) {
                fetch_v(0);
#pragma unroll 1
                for (int j = 0; j < n_tiles && ok; ++j) ok = write_v(j);
            } else {
                fetch_k(0);
#pragma unroll 1
                for (int j = 0; j < n_tiles && ok; ++j) ok = write_k(j);
            }
            if (!ok) atomicExch(p.status, 29);
        }
    }
    tc_fence_before();
    __syncthreads();
    pos += n_tiles;
    if (pos < flat_hi) {      // a wait that ran out anywhere: stop here (the status word tells the host)
        if (tid == 0) *seg_stop = *(volatile int *)p.status;
        __syncthreads();
        if (*seg_stop != 0) break;
    }
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TC_TMEM_COLS) : "memory");
    }
}

// Units cut by a CTA boundary: out[row] = sum_s o_s 2^(m_s - m) / sum_s l_s 2^(m_s - m) over the unit's pieces.
__global__ void __launch_bounds__(128) verify_merge_kernel(const __grid_constant__ VerifyParams p) {
    const int unit = blockIdx.x / p.R, row = blockIdx.x % p.R, d = threadIdx.x;
    const int hk = unit % p.Hkv, b = unit / p.Hkv, rep = p.Hq / p.Hkv;
    const int n_all = (int)((p.T + TC_KEYS - 1) / TC_KEYS);
    const int first = (int)(((int64_t)unit * n_all) / p.tiles_per_cta), last = (int)((((int64_t)unit + 1) * n_all - 1) / p.tiles_per_cta);
    const int pieces = last - first + 1;
    if (pieces == 1) return;      // written by its CTA
    float m = -INFINITY;
    for (int s = 0; s < pieces; ++s) {
        const float2 ml = p.ml_part[((int64_t)unit * p.max_pieces + s) * p.R + row];
        if (ml.y > 0.f) m = fmaxf(m, ml.x);
    }
    float o = 0.f, l = 0.f;
    for (int s = 0; s < pieces; ++s) {
        const int64_t slot = ((int64_t)unit * p.max_pieces + s) * p.R + row;
        const float2 ml = p.ml_part[slot];
        if (!(ml.y > 0.f)) continue;
        const float w = fast_exp2(ml.x - m);
        o = fmaf(p.o_part[slot * VT_D + d], w, o);
        l = fmaf(ml.y, w, l);
    }
    const int hq = hk * rep + row / p.L, lq = row % p.L;
    const int64_t at = b * p.o_sb + hq * p.o_sh + lq * p.o_sl + (p.permuted ? affine_dim_of(d, p.permuted) : d);
    const float val = l > 0.f ? o / l : 0.f;
    if (p.out_bf16) ((__nv_bfloat16 *)p.out)[at] = __float2bfloat16_rn(val);
    else ((__half *)p.out)[at] = __float2half_rn(val);
}

struct QPadParams {
    const void *q;
    __half *out;                 // [units][128][D]
    int64_t q_sb, q_sh, q_sl;
    int32_t B, Hq, Hkv, L, R;
    const float *signs, *calib;
    int32_t perm_bits;           // verify_q_plain_kernel: the code bits of the affine cache
};

// Rotated queries of every unit, padded to 128 rows: row r of unit (b, hk) is head hk*rep + r / L at
// position r % L; out = calib * H(signs * q) / sqrt(D) in f16, rows past R zero. One warp per row.
template <typename T>
__global__ void __launch_bounds__(256) verify_q_kernel(const __grid_constant__ QPadParams p) {
    constexpr int D = VT_D, E = D / 32;
    const int lane = threadIdx.x & 31;
    const int64_t gr = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t units = (int64_t)p.B * p.Hkv;
    if (gr >= units * TC_ROWS) return;
    const int unit = (int)(gr / TC_ROWS), r = (int)(gr % TC_ROWS);
    __half *dst = p.out + gr * D + E * lane;
    float x[E] = {0.f, 0.f, 0.f, 0.f};
    if (r < p.R) {
        const int hk = unit % p.Hkv, b = unit / p.Hkv, rep = p.Hq / p.Hkv;
        const int hq = hk * rep + r / p.L, l = r % p.L;
        const T *src = (const T *)p.q + b * p.q_sb + hq * p.q_sh + l * p.q_sl + E * lane;
#pragma unroll
        for (int j = 0; j < E; ++j) x[j] = to_f32<T>(src[j]) * p.signs[E * lane + j];
    }
    {
        const float a0 = x[0] + x[1], a1 = x[0] - x[1], a2 = x[2] + x[3], a3 = x[2] - x[3];
        x[0] = a0 + a2; x[2] = a0 - a2; x[1] = a1 + a3; x[3] = a1 - a3;
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
#pragma unroll
    for (int j = 0; j < E; ++j) {
        float v = x[j] * fs;
        if (p.calib) v *= p.calib[E * lane + j];
        dst[j] = __float2half_rn(fminf(fmaxf(v, -65504.f), 65504.f));
    }
}

// Queries of every unit for the affine cache, padded to 128 rows, as f16 in the column order of the key
// tiles (affine_dim_of; p.perm_bits = the code bits). One thread per eight dims.
template <typename T>
__global__ void __launch_bounds__(256) verify_q_plain_kernel(const __grid_constant__ QPadParams p) {
    constexpr int D = VT_D;
    const int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t units = (int64_t)p.B * p.Hkv;
    if (g >= units * TC_ROWS * (D / 8)) return;
    const int c8 = (int)(g % (D / 8));
    const int64_t gr = g / (D / 8);
    const int unit = (int)(gr / TC_ROWS), r = (int)(gr % TC_ROWS);
    uint4 w = make_uint4(0u, 0u, 0u, 0u);
    if (r < p.R) {
        const int hk = unit % p.Hkv, b = unit / p.Hkv, rep = p.Hq / p.Hkv;
        const int hq = hk * rep + r / p.L, l = r % p.L;
        const T *src = (const T *)p.q + b * p.q_sb + hq * p.q_sh + l * p.q_sl + c8 * 8;
        float x[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = fminf(fmaxf(to_f32<T>(src[i]), -65504.f), 65504.f);
        const int bits = p.perm_bits;
        w.x = pack_h2(x[affine_dim_of(0, bits)], x[affine_dim_of(1, bits)]);
        w.y = pack_h2(x[affine_dim_of(2, bits)], x[affine_dim_of(3, bits)]);
        w.z = pack_h2(x[affine_dim_of(4, bits)], x[affine_dim_of(5, bits)]);
        w.w = pack_h2(x[affine_dim_of(6, bits)], x[affine_dim_of(7, bits)]);
    }
    *(uint4 *)(p.out + gr * D + c8 * 8) = w;
}

template <typename TO, int KB, bool AFFINE, bool RAW = false>
bool launch_verify_typed(const CUtensorMap &qmap, const CUtensorMap &kmap, const CUtensorMap &vmap, const VerifyParams &p, int ctas,
                         cudaStream_t stream) {
    // Q' and two stages of (K tile, V tile); the two lookup tables (TurboQuant); the staged rows
    const size_t smem = (size_t)5 * VT_TILE + ((AFFINE || RAW) ? 0 : (size_t)VT_TILE + (KB == 4 ? 0 : ((size_t)1 << (2 * KB)) * 128)) +
                        VB_COUNT * sizeof(uint64_t) + 64 +
                        6 * TC_ROWS * sizeof(float) + 16 + 1024;
    static std::atomic<int> configured[64];
    const int dev = current_device();
    if (dev < 0 || dev >= 64) return false;
    int state = configured[dev].load(std::memory_order_acquire);
    if (state == 0) {
        const cudaError_t e = cudaFuncSetAttribute(attn_verify_tc_kernel<TO, KB, AFFINE, RAW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) (void)cudaGetLastError();
        state = e == cudaSuccess ? 1 : -1;
        configured[dev].store(state, std::memory_order_release);
    }
    if (state < 0) return false;
    KernelTimer timer(stream);
    KVC_CUDA(launch_pdl(attn_verify_tc_kernel<TO, KB, AFFINE, RAW>, dim3(ctas), dim3(VT_THREADS), smem, stream, qmap, kmap, vmap, p));
    timer.stop();
    ++g_launch_count;
    return true;
}

}  // namespace

// Returns the number of kernels launched, 0 when the call is left to the other kernels.
// KVC_VERIFY_TC=0 turns the path off.
int launch_attention_verify_tc(const AttnArgs &a, cudaStream_t stream) {
    static const bool off = [] {
        const char *e = std::getenv("KVC_VERIFY_TC");
        return e && e[0] == '0';
    }();
    if (off) return 0;
    if (a.D != VT_D || (a.q_dtype != KVC_BF16 && a.q_dtype != KVC_F16)) return 0;
    if (a.k.kind != SRC_TURBO || a.v.kind != SRC_TURBO || !a.q_signs || !a.o_signs || a.q_rot || a.o_rot) return 0;
    if (a.mask.mode == KVC_MASK_ARRAY || a.new_k) return 0;
    if (a.mask.mode == KVC_MASK_CAUSAL && a.mask.causal_offset < 0) return 0;
    const int kb = a.k.bits, vb = a.v.bits;
    if (vb != 4 || kb < 2 || kb > 4) return 0;
    if (kb == 4 && std::memcmp(a.k.codebook, a.v.codebook, sizeof(a.k.codebook)) != 0) return 0;   // 4-bit keys read the value pair table
    if (a.Hkv <= 0 || a.Hq % a.Hkv || a.T < 1 || a.T > (int64_t)1 << 30) return 0;
    const int rep = a.Hq / a.Hkv, R = rep * a.L;
    if (R <= 8 || R > 64) return 0;           // eight rows and fewer: the decode kernel; the row side uses TMEM lanes 0..63
    {
        // rows are read 16 bytes at a time up to the stored rows rounded to a tile of 128 keys
        const int64_t padded = (a.T + TC_KEYS - 1) / TC_KEYS * TC_KEYS;
        const int kw = a.D * kb / 32, vw = a.D * vb / 32;
        if (a.k.st != kw || a.v.st != vw || a.k.gst != 1 || a.v.gst != 1) return 0;
        if (a.k.sh < padded * kw || a.v.sh < padded * vw || a.k.gsh < padded || a.v.gsh < padded) return 0;
        if (((uintptr_t)a.k.data & 15) || ((uintptr_t)a.v.data & 15) || (a.k.sh % 4) || (a.k.sb % 4) || (a.v.sh % 4) || (a.v.sb % 4))
            return 0;
    }
    if (((uintptr_t)a.out & 15) != 0 || (a.o_sl * 2) % 16 || (a.o_sh * 2) % 16 || (a.o_sb * 2) % 16) return 0;
    int *status = device_status_word(a.device);
    if (!status) return 0;

    const int64_t units = (int64_t)a.B * a.Hkv;
    const int n_tiles = (int)((a.T + TC_KEYS - 1) / TC_KEYS);
    const int sms = sm_count(a.device);
    // the tiles of all units end to end, cut into one equal range per SM
    const int64_t flat = units * n_tiles;
    if (flat > (int64_t)1 << 40) return 0;
    const int64_t tpc64 = (flat + std::min<int64_t>(sms, flat) - 1) / std::min<int64_t>(sms, flat);
    if (tpc64 > (int64_t)1 << 30) return 0;
    const int tiles_per_cta = (int)tpc64;
    const int64_t ctas = (flat + tiles_per_cta - 1) / tiles_per_cta;
    const bool merge = tiles_per_cta % n_tiles != 0;            // some unit is cut by a CTA boundary
    const int max_pieces = (n_tiles + tiles_per_cta - 1) / tiles_per_cta + 1;

    const size_t q_bytes = (size_t)units * TC_ROWS * VT_D * sizeof(__half);
    const size_t o_bytes = merge ? (size_t)units * max_pieces * R * VT_D * sizeof(float) : 0;
    const size_t ml_bytes = merge ? (size_t)units * max_pieces * R * sizeof(float2) : 0;
    char *scratch = (char *)scratch_get(a.device, q_bytes + o_bytes + ml_bytes + 1024, stream);
    __half *qpad = (__half *)scratch;

    QPadParams qp = {};
    qp.q = a.q; qp.out = qpad;
    qp.q_sb = a.q_sb; qp.q_sh = a.q_sh; qp.q_sl = a.q_sl;
    qp.B = a.B; qp.Hq = a.Hq; qp.Hkv = a.Hkv; qp.L = a.L; qp.R = R;
    qp.signs = a.q_signs; qp.calib = a.q_calib;
    const unsigned qblocks = (unsigned)((units * TC_ROWS + 7) / 8);
    if (a.q_dtype == KVC_BF16) verify_q_kernel<__nv_bfloat16><<<qblocks, 256, 0, stream>>>(qp);
    else verify_q_kernel<__half><<<qblocks, 256, 0, stream>>>(qp);
    KVC_CUDA(cudaGetLastError());
    ++g_launch_count;
    int launches = 1;

    CUtensorMap qmap;
    if (!make_map_tc(&qmap, qpad, KVC_F16, VT_D, TC_ROWS, (int)units, 1, VT_D, (int64_t)TC_ROWS * VT_D, units * TC_ROWS * VT_D))
        fail(KVC_ERR_INTERNAL, "verify kernel: the query tensor map could not be encoded");

    VerifyParams p = {};
    p.kp = (const uint32_t *)a.k.data; p.vp = (const uint32_t *)a.v.data;
    p.kn = a.k.norms; p.vn = a.v.norms;
    p.kp_sb = a.k.sb; p.kp_sh = a.k.sh; p.vp_sb = a.v.sb; p.vp_sh = a.v.sh;
    p.kn_sb = a.k.gsb; p.kn_sh = a.k.gsh; p.vn_sb = a.v.gsb; p.vn_sh = a.v.gsh;
    for (int i = 0; i < 16; ++i) {
        p.kcb[i] = a.k.codebook[i];
        p.vcb[i] = a.v.codebook[i];
    }
    p.out = a.out;
    p.o_sb = a.o_sb; p.o_sh = a.o_sh; p.o_sl = a.o_sl;
    p.B = a.B; p.Hq = a.Hq; p.Hkv = a.Hkv; p.L = a.L; p.R = R;
    p.T = a.T;
    p.causal = a.mask.mode == KVC_MASK_CAUSAL ? 1 : 0;
    p.causal_offset = a.mask.causal_offset;
    p.scale_log2 = a.scale * 1.4426950408889634f;
    p.tiles_per_cta = tiles_per_cta; p.max_pieces = max_pieces;
    p.o_part = (float *)(scratch + ((q_bytes + 255) / 256) * 256);
    p.ml_part = (float2 *)((char *)p.o_part + ((o_bytes + 255) / 256) * 256);
    p.status = status;
    p.debug_skip = measure_skip_bits();

    bool taken = false;
    if (kb == 2) taken = launch_verify_typed<__half, 2, false>(qmap, qmap, qmap, p, (int)ctas, stream);
    else if (kb == 4) taken = launch_verify_typed<__half, 4, false>(qmap, qmap, qmap, p, (int)ctas, stream);
    else taken = launch_verify_typed<__half, 3, false>(qmap, qmap, qmap, p, (int)ctas, stream);
    if (!taken) fail(KVC_ERR_INTERNAL, "verify kernel: the device refused its shared memory");
    ++launches;
    if (merge) {
        verify_merge_kernel<<<(unsigned)(units * R), VT_D, 0, stream>>>(p);
        KVC_CUDA(cudaGetLastError());
        ++g_launch_count;
        ++launches;
    }
    // rows back from the rotated basis, in place: f16 in, the caller's dtype out
    launch_rotate_rows_f16(a.out, a.out, KVC_F16, a.q_dtype, a.o_sb, a.o_sh, a.o_sl, a.o_sb, a.o_sh, a.o_sl, a.B, a.Hq, a.L, a.D,
                           nullptr, a.o_signs, stream);
    ++launches;
    if (trace_dispatch())
        fprintf(stderr, "[kvc] verify_tc: %lld units of %d rows and %d tiles, %lld CTAs of %d tiles\n", (long long)units, R, n_tiles, (long long)ctas, tiles_per_cta);
    return launches;
}


// Queries of every unit for the raw cache, padded to 128 rows (zero rows past R), element type unchanged.
// One thread per eight dims.
template <typename T>
__global__ void __launch_bounds__(256) verify_q_raw_kernel(const QPadParams p) {
    constexpr int D = VT_D;
    const int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t units = (int64_t)p.B * p.Hkv;
    if (g >= units * TC_ROWS * (D / 8)) return;
    const int c8 = (int)(g % (D / 8));
    const int64_t gr = g / (D / 8);
    const int unit = (int)(gr / TC_ROWS), r = (int)(gr % TC_ROWS);
    uint4 w = make_uint4(0u, 0u, 0u, 0u);
    if (r < p.R) {
        const int hk = unit % p.Hkv, b = unit / p.Hkv, rep = p.Hq / p.Hkv;
        const int hq = hk * rep + r / p.L, l = r % p.L;
        const T *src = (const T *)p.q + b * p.q_sb + hq * p.q_sh + l * p.q_sl + c8 * 8;
        if (((uintptr_t)src & 15) == 0) {
            w = *(const uint4 *)src;
        } else {
            T tmp[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) tmp[i] = src[i];
            w = *(const uint4 *)tmp;
        }
    }
    *(uint4 *)((T *)p.out + gr * D + c8 * 8) = w;
}

// QuantizedKVCache verify rounds (quantizedScaledDotProductAttention over a handful of positions per head,
// KVCache.swift:1045-1110 via AttentionUtils.swift:53-71): 4- or 8-bit codes in groups of 64, head dim 128,
// 9 ... 64 rows per KV head. Returns the number of kernels launched, 0 when the call is left to the other
// kernels. KVC_VERIFY_TC=0 turns the path off.
int launch_attention_verify_tc_affine(const AttnArgs &a, cudaStream_t stream) {
    static const bool off = [] {
        const char *e = std::getenv("KVC_VERIFY_TC");
        return e && e[0] == '0';
    }();
    if (off) return 0;
    if (a.D != VT_D || (a.q_dtype != KVC_BF16 && a.q_dtype != KVC_F16)) return 0;
    if (a.k.kind != SRC_AFFINE || a.v.kind != SRC_AFFINE || a.q_signs || a.o_signs || a.q_rot || a.o_rot || a.q_calib) return 0;
    if (a.mask.mode == KVC_MASK_ARRAY || a.new_k) return 0;
    if (a.mask.mode == KVC_MASK_CAUSAL && a.mask.causal_offset < 0) return 0;
    if ((a.k.bits != 4 && a.k.bits != 8) || a.v.bits != a.k.bits || a.k.group != 64 || a.v.group != 64) return 0;
    if (a.k.dtype != a.v.dtype || (a.k.dtype != KVC_BF16 && a.k.dtype != KVC_F16)) return 0;
    if (a.Hkv <= 0 || a.Hq % a.Hkv || a.T < 1 || a.T > (int64_t)1 << 30) return 0;
    const int rep = a.Hq / a.Hkv, R = rep * a.L;
    if (R <= 16 || R > 64) return 0;          // up to 16 rows: the decode kernel streams the cache once or twice
    const int W = VT_D * a.k.bits / 32;
    constexpr int G = VT_D / 64;
    {
        // rows are read 16 bytes at a time up to the stored rows rounded to a tile of 128 keys
        const int64_t padded = (a.T + TC_KEYS - 1) / TC_KEYS * TC_KEYS;
        for (const KVSource *s : {&a.k, &a.v}) {
            if (s->st != W || s->gst != G || s->sh < padded * W || s->gsh < padded * G) return 0;
            if (((uintptr_t)s->data & 15) || (s->sh % 4) || (s->sb % 4)) return 0;
            if (((uintptr_t)s->scales & 3) || ((uintptr_t)s->biases & 3) || (s->gsh % 2) || (s->gsb % 2)) return 0;
        }
    }
    if (((uintptr_t)a.out & 15) != 0 || (a.o_sl * 2) % 16 || (a.o_sh * 2) % 16 || (a.o_sb * 2) % 16) return 0;
    int *status = device_status_word(a.device);
    if (!status) return 0;

    const int64_t units = (int64_t)a.B * a.Hkv;
    const int n_tiles = (int)((a.T + TC_KEYS - 1) / TC_KEYS);
    const int sms = sm_count(a.device);
    // the tiles of all units end to end, cut into one equal range per SM
    const int64_t flat = units * n_tiles;
    if (flat > (int64_t)1 << 40) return 0;
    const int64_t tpc64 = (flat + std::min<int64_t>(sms, flat) - 1) / std::min<int64_t>(sms, flat);
    if (tpc64 > (int64_t)1 << 30) return 0;
    const int tiles_per_cta = (int)tpc64;
    const int64_t ctas = (flat + tiles_per_cta - 1) / tiles_per_cta;
    const bool merge = tiles_per_cta % n_tiles != 0;            // some unit is cut by a CTA boundary
    const int max_pieces = (n_tiles + tiles_per_cta - 1) / tiles_per_cta + 1;

    const size_t q_bytes = (size_t)units * TC_ROWS * VT_D * sizeof(__half);
    const size_t o_bytes = merge ? (size_t)units * max_pieces * R * VT_D * sizeof(float) : 0;
    const size_t ml_bytes = merge ? (size_t)units * max_pieces * R * sizeof(float2) : 0;
    char *scratch = (char *)scratch_get(a.device, q_bytes + o_bytes + ml_bytes + 1024, stream);
    __half *qpad = (__half *)scratch;

    QPadParams qp = {};
    qp.q = a.q; qp.out = qpad;
    qp.q_sb = a.q_sb; qp.q_sh = a.q_sh; qp.q_sl = a.q_sl;
    qp.B = a.B; qp.Hq = a.Hq; qp.Hkv = a.Hkv; qp.L = a.L; qp.R = R;
    qp.perm_bits = a.k.bits;
    const unsigned qblocks = (unsigned)((units * TC_ROWS * (VT_D / 8) + 255) / 256);
    if (a.q_dtype == KVC_BF16) verify_q_plain_kernel<__nv_bfloat16><<<qblocks, 256, 0, stream>>>(qp);
    else verify_q_plain_kernel<__half><<<qblocks, 256, 0, stream>>>(qp);
    KVC_CUDA(cudaGetLastError());
    ++g_launch_count;
    int launches = 1;

    CUtensorMap qmap;
    if (!make_map_tc(&qmap, qpad, KVC_F16, VT_D, TC_ROWS, (int)units, 1, VT_D, (int64_t)TC_ROWS * VT_D, units * TC_ROWS * VT_D))
        fail(KVC_ERR_INTERNAL, "verify kernel: the query tensor map could not be encoded");

    VerifyParams p = {};
    p.kp = (const uint32_t *)a.k.data; p.vp = (const uint32_t *)a.v.data;
    p.ks = (const uint16_t *)a.k.scales; p.kz = (const uint16_t *)a.k.biases;
    p.vs = (const uint16_t *)a.v.scales; p.vz = (const uint16_t *)a.v.biases;
    p.kp_sb = a.k.sb; p.kp_sh = a.k.sh; p.vp_sb = a.v.sb; p.vp_sh = a.v.sh;
    p.kn_sb = a.k.gsb; p.kn_sh = a.k.gsh; p.vn_sb = a.v.gsb; p.vn_sh = a.v.gsh;
    p.sz_bf16 = a.k.dtype == KVC_BF16 ? 1 : 0;
    p.out_bf16 = a.q_dtype == KVC_BF16 ? 1 : 0;
    p.permuted = a.k.bits;
    p.out = a.out;
    p.o_sb = a.o_sb; p.o_sh = a.o_sh; p.o_sl = a.o_sl;
    p.B = a.B; p.Hq = a.Hq; p.Hkv = a.Hkv; p.L = a.L; p.R = R;
    p.T = a.T;
    p.causal = a.mask.mode == KVC_MASK_CAUSAL ? 1 : 0;
    p.causal_offset = a.mask.causal_offset;
    p.scale_log2 = a.scale * 1.4426950408889634f;
    p.tiles_per_cta = tiles_per_cta; p.max_pieces = max_pieces;
    p.o_part = (float *)(scratch + ((q_bytes + 255) / 256) * 256);
    p.ml_part = (float2 *)((char *)p.o_part + ((o_bytes + 255) / 256) * 256);
    p.status = status;
    p.debug_skip = measure_skip_bits();

    bool taken = false;
    if (a.k.bits == 4) {
        if (a.q_dtype == KVC_BF16) taken = launch_verify_typed<__nv_bfloat16, 4, true>(qmap, qmap, qmap, p, (int)ctas, stream);
        else taken = launch_verify_typed<__half, 4, true>(qmap, qmap, qmap, p, (int)ctas, stream);
    } else {
        if (a.q_dtype == KVC_BF16) taken = launch_verify_typed<__nv_bfloat16, 8, true>(qmap, qmap, qmap, p, (int)ctas, stream);
        else taken = launch_verify_typed<__half, 8, true>(qmap, qmap, qmap, p, (int)ctas, stream);
    }
    if (!taken) fail(KVC_ERR_INTERNAL, "verify kernel: the device refused its shared memory");
    ++launches;
    if (merge) {
        verify_merge_kernel<<<(unsigned)(units * R), VT_D, 0, stream>>>(p);
        KVC_CUDA(cudaGetLastError());
        ++g_launch_count;
        ++launches;
    }
    if (trace_dispatch())
        fprintf(stderr, "[kvc] verify_tc affine: %lld units of %d rows and %d tiles, %lld CTAs of %d tiles\n", (long long)units, R, n_tiles, (long long)ctas, tiles_per_cta);
    return launches;
}


// KVCacheSimple verify rounds (17 ... 64 rows per KV head over plain f16 / bf16 rows, head dim 128): the same
// kernel with TMA-loaded K / V tiles. Returns the number of kernels launched, 0 when the call is left to the
// other kernels. KVC_VERIFY_TC=0 turns the path off.
int launch_attention_verify_tc_raw(const AttnArgs &a, cudaStream_t stream) {
    static const bool off = [] {
        const char *e = std::getenv("KVC_VERIFY_TC");
        return e && e[0] == '0';
    }();
    if (off) return 0;
    if (a.D != VT_D || (a.q_dtype != KVC_BF16 && a.q_dtype != KVC_F16)) return 0;
    if (a.k.kind != SRC_RAW || a.v.kind != SRC_RAW || a.k.dtype != a.q_dtype || a.v.dtype != a.q_dtype) return 0;
    if (a.mask.mode == KVC_MASK_ARRAY || a.q_signs || a.o_signs || a.q_calib || a.new_k || a.q_rot || a.o_rot) return 0;
    if (a.mask.mode == KVC_MASK_CAUSAL && a.mask.causal_offset < 0) return 0;
    if (a.Hkv <= 0 || a.Hq % a.Hkv || a.T < 1 || a.T > (int64_t)1 << 30) return 0;
    const int rep = a.Hq / a.Hkv, R = rep * a.L;
    if (R <= 16 || R > 64) return 0;          // up to 16 rows: the decode kernels
    if (!strides_fit(a.k.data, a.D, a.k.st, a.k.sh, a.k.sb, a.Hkv, a.B) || !strides_fit(a.v.data, a.D, a.v.st, a.v.sh, a.v.sb, a.Hkv, a.B))
        return 0;
    if (((uintptr_t)a.out & 15) != 0 || (a.o_sl * 2) % 16 || (a.o_sh * 2) % 16 || (a.o_sb * 2) % 16) return 0;
    int *status = device_status_word(a.device);
    if (!status) return 0;

    const int64_t units = (int64_t)a.B * a.Hkv;
    const int n_tiles = (int)((a.T + TC_KEYS - 1) / TC_KEYS);
    const int sms = sm_count(a.device);
    const int64_t flat = units * n_tiles;
    if (flat > (int64_t)1 << 40) return 0;
    const int64_t tpc64 = (flat + std::min<int64_t>(sms, flat) - 1) / std::min<int64_t>(sms, flat);
    if (tpc64 > (int64_t)1 << 30) return 0;
    const int tiles_per_cta = (int)tpc64;
    const int64_t ctas = (flat + tiles_per_cta - 1) / tiles_per_cta;
    const bool merge = tiles_per_cta % n_tiles != 0;
    const int max_pieces = (n_tiles + tiles_per_cta - 1) / tiles_per_cta + 1;

    const size_t q_bytes = (size_t)units * TC_ROWS * VT_D * 2;
    const size_t o_bytes = merge ? (size_t)units * max_pieces * R * VT_D * sizeof(float) : 0;
    const size_t ml_bytes = merge ? (size_t)units * max_pieces * R * sizeof(float2) : 0;
    char *scratch = (char *)scratch_get(a.device, q_bytes + o_bytes + ml_bytes + 1024, stream);

    CUtensorMap qmap, kmap, vmap;
    if (!make_map_tc(&qmap, scratch, a.q_dtype, VT_D, TC_ROWS, (int)units, 1, VT_D, (int64_t)TC_ROWS * VT_D, units * TC_ROWS * VT_D)) return 0;
    if (!make_map_tc(&kmap, a.k.data, a.k.dtype, a.D, a.T, a.Hkv, a.B, a.k.st, a.k.sh, a.k.sb)) return 0;
    if (!make_map_tc(&vmap, a.v.data, a.v.dtype, a.D, a.T, a.Hkv, a.B, a.v.st, a.v.sh, a.v.sb)) return 0;

    QPadParams qp = {};
    qp.q = a.q; qp.out = (__half *)scratch;
    qp.q_sb = a.q_sb; qp.q_sh = a.q_sh; qp.q_sl = a.q_sl;
    qp.B = a.B; qp.Hq = a.Hq; qp.Hkv = a.Hkv; qp.L = a.L; qp.R = R;
    const unsigned qblocks = (unsigned)((units * TC_ROWS * (VT_D / 8) + 255) / 256);
    if (a.q_dtype == KVC_BF16) verify_q_raw_kernel<__nv_bfloat16><<<qblocks, 256, 0, stream>>>(qp);
    else verify_q_raw_kernel<__half><<<qblocks, 256, 0, stream>>>(qp);
    KVC_CUDA(cudaGetLastError());
    ++g_launch_count;
    int launches = 1;

    VerifyParams p = {};
    p.out_bf16 = a.q_dtype == KVC_BF16 ? 1 : 0;
    p.out = a.out;
    p.o_sb = a.o_sb; p.o_sh = a.o_sh; p.o_sl = a.o_sl;
    p.B = a.B; p.Hq = a.Hq; p.Hkv = a.Hkv; p.L = a.L; p.R = R;
    p.T = a.T;
    p.causal = a.mask.mode == KVC_MASK_CAUSAL ? 1 : 0;
    p.causal_offset = a.mask.causal_offset;
    p.scale_log2 = a.scale * 1.4426950408889634f;
    p.tiles_per_cta = tiles_per_cta; p.max_pieces = max_pieces;
    p.o_part = (float *)(scratch + ((q_bytes + 255) / 256) * 256);
    p.ml_part = (float2 *)((char *)p.o_part + ((o_bytes + 255) / 256) * 256);
    p.status = status;
    p.debug_skip = measure_skip_bits();

    bool taken = false;
    if (a.q_dtype == KVC_BF16) taken = launch_verify_typed<__nv_bfloat16, 4, false, true>(qmap, kmap, vmap, p, (int)ctas, stream);
    else taken = launch_verify_typed<__half, 4, false, true>(qmap, kmap, vmap, p, (int)ctas, stream);
    if (!taken) fail(KVC_ERR_INTERNAL, "verify kernel: the device refused its shared memory");
    ++launches;
    if (merge) {
        verify_merge_kernel<<<(unsigned)(units * R), VT_D, 0, stream>>>(p);
        KVC_CUDA(cudaGetLastError());
        ++g_launch_count;
        ++launches;
    }
    if (trace_dispatch())
        fprintf(stderr, "[kvc] verify_tc raw: %lld units of %d rows and %d tiles, %lld CTAs of %d tiles\n", (long long)units, R, n_tiles, (long long)ctas, tiles_per_cta);
    return launches;
}

}  // namespace kvc
