// Split-K flash decoding over the TurboQuant cache with 4-bit values (key bits 2, 3 or 4),
// head dimension 128, at most 8 query rows per KV head: the decode step and short verify
// chunks of TurboQuantKVCache.compressedAttention (TurboQuantKVCache.swift:1164-1446; the
// reference's kernels for this step are the flash passes at TurboQuantKernels.swift:424-542
// and :1396-1519).
//
// The math is that of attn_turbo.cu (rotated basis, query rotated once per segment, scores
// norm_k[t] * sum_d q'[d] * centroid_k[idx_k[t, d]], output sum_t (p_t * norm_v[t]) *
// centroid_v[idx_v[t, d]], inverse rotation in the epilogue). What differs is how the work is
// laid over the SM, because the step is bound by the shared-memory pipe and by instruction
// issue, not by HBM:
//
//  * ONE CTA per SM with 16 consumer warps sharing 256-token stages and four producer warps
//    (one per array of a stage: a thread's bulk copies issue one after the other, and small
//    copies are bound by issue, not by bytes), so that the lookup tables exist once per SM and
//    16 warps hide each other's table-lookup latency. A group of more than eight query rows
//    (a verify chunk) is cut into units of eight rows that stream the same tiles one after
//    the other (all but the first out of L2).
//  * Value operands without a transpose. The P V product runs as O^T = V^T P^T (head dims on
//    the 16-row side), whose A operand pairs TWO TOKENS of one head dim in a register. A lane
//    loads the same 16 dims (two words) of its four tokens, interleaves the nibbles of a token
//    pair with four logic operations per eight dims (byte = code of token A | code of token B
//    << 4) and looks the byte up in a 256-entry table of f16x2 (centroid[A], centroid[B]).
//  * Table entries are 256 bytes apart and the table starts on a 64 KB boundary of the shared
//    window: the address of a value lookup is ONE byte-permute (entry byte -> address bits
//    8..15, lane -> bits 2..6, the rest constant). The upper half of every 256-byte row holds
//    the key table (pairs of adjacent dims of one token, as in attn_turbo.cu), so both tables
//    are lane-replicated (entry j of lane l in bank l: no bank conflicts whatever the codes).
//  * The 16 warps fold their accumulators pairwise through shared memory (lane to lane: the
//    fragment layout is the same in every warp) down to four, which then go through the
//    epilogue shared with the other decode kernels.
#include "attn_common.cuh"

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstdlib>

namespace kvc {

namespace {

using namespace dev;

// 15 consumer warps and one producer warp: 16 warps, so that a thread may hold 128 registers (a
// seventeenth warp would round the CTA up to 20 in the register file's allocation and cap it at 96).
#ifndef KVC_V4_WARPS
#define KVC_V4_WARPS 15
#endif
#ifndef KVC_V4_PRODUCERS
#define KVC_V4_PRODUCERS 1
#endif
constexpr int V4_WARPS = KVC_V4_WARPS;             // consumer warps
constexpr int V4_GW = V4_WARPS;                    // warps that share a ring stage (16 tokens each)
constexpr int V4_GROUPS = 1;                       // warp groups; group i takes every V4_GROUPS-th stage
constexpr int V4_PRODUCERS = KVC_V4_PRODUCERS;     // producer warps: 4 = one per array of a stage, 1 = lanes 0..3 issue them
constexpr int V4_THREADS = (V4_WARPS + V4_PRODUCERS) * 32;
constexpr int V4_TILE = 16 * V4_GW;                // tokens per ring stage
constexpr int V4_D = 128;
constexpr int V4_VW = 16;                         // value words per row (4 bits)
constexpr int V4_MAX_STAGES = 12;                 // of 64 tokens; fewer when a stage is larger
constexpr int V4_TABLE_BYTES = 256 * 256;
constexpr int V4_SLOT_FLOATS = 36 * 32;           // one warp's accumulators: 32 outputs + 2 maxima + 2 sums per lane
constexpr int V4_COUNTER_BYTES = 64 * 1024;
constexpr int V4_MAX_CHUNKS = 8;                  // up to 64 query rows per (batch, kv head)
constexpr int V4_RED_STRIDE = V4_D + 8;

struct TurboV4Params {
    const void *q;
    void *out;
    int64_t q_sb, q_sh, q_sl, o_sb, o_sh, o_sl;
    const uint32_t *kp, *vp;   // packed indices, [B, H, cap, words]
    const float *kn, *vn;      // norms, [B, H, cap]
    int64_t kp_sb, kp_sh, vp_sb, vp_sh;  // word strides (token stride = words per row)
    int64_t kn_sb, kn_sh, vn_sb, vn_sh;  // element strides (token stride = 1)
    const float *q_signs, *o_signs;      // [D] each
    const float *q_calib;                // optional [D]
    float kcb[16], vcb[16];              // centroids
    float *o_part;
    float2 *ml_part;
    int *counters;
    int *status;
    int32_t B, Hq, Hkv, L;
    int32_t chunks;      // units per (batch, kv head): ceil(query rows of the group / 8)
    int64_t T;
    int32_t causal;
    int32_t out_dtype;
    int64_t causal_offset;
    float scale_log2;
    FlatPlan flat;
    int32_t q_bulk;      // a unit's query rows are one contiguous 16-byte aligned block
    uint32_t smem_bytes; // dynamic shared memory of the launch
    int32_t debug_skip;  // measurement builds only (KVC_SKIP_BITS): 1 = consumers release stages without computing
};

// Table lookups: the tables never change after the set-up barrier, so these loads may be scheduled
// freely (no volatile).
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

// Loads from a ring stage: ordered after the wait on the stage's barrier (volatile), explicit shared
// space (a generic load would take the slower path and 64-bit address arithmetic).
__device__ __forceinline__ float lds_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}

template <int N>
__device__ __forceinline__ void lds_words(uint32_t addr, uint32_t (&dst)[N]) {
    if constexpr (N == 4) {
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(dst[0]), "=r"(dst[1]), "=r"(dst[2]), "=r"(dst[3]) : "r"(addr));
    } else if constexpr (N == 2) {
        asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(dst[0]), "=r"(dst[1]) : "r"(addr));
    } else {
        static_assert(N == 3, "word loads are written for 2, 3 or 4 words");
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(dst[0]) : "r"(addr));
        asm volatile("ld.shared.u32 %0, [%1+4];" : "=r"(dst[1]) : "r"(addr));
        asm volatile("ld.shared.u32 %0, [%1+8];" : "=r"(dst[2]) : "r"(addr));
    }
}

// The 8x8 b16 transpose without `volatile`: every lane of the warp reaches it (it is never under a
// divergent branch here) and it has no side effect, so the compiler may schedule it among the lookups.
__device__ __forceinline__ uint32_t movmatrix_free(uint32_t x) {
    uint32_t r;
    asm("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(x));
    return r;
}

// Address of value-table entry `byte BYTE of x` for this lane: one byte permute. `lane_const`
// holds (table base | lane << 2) with the table base a multiple of 64 KB.
template <int BYTE>
__device__ __forceinline__ uint32_t value_entry(uint32_t x, uint32_t lane_const) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(x), "r"(lane_const), "n"(0x7604 | (BYTE << 4)));
    return r;
}

// Address of key-table entry for pair j of a lane's word stream (2 * BITS bits at bit 2 * BITS * j):
// the field is moved to bits 8.. and merged with (table base | 128 | lane << 2).
template <int BITS, int NW>
__device__ __forceinline__ uint32_t key_entry(const uint32_t (&w)[NW], int j, uint32_t lane_const) {
    constexpr int B2 = 2 * BITS;
    constexpr uint32_t MASK = ((1u << B2) - 1u) << 8;
    const int bit = B2 * j, k = bit >> 5, s = bit & 31;
    uint32_t x;
    if (s + B2 <= 32) x = (s >= 8) ? (w[k] >> (s - 8)) : (w[k] << (8 - s));
    else x = __funnelshift_r(w[k], w[(k + 1 < NW) ? k + 1 : k], s - 8);
    return (x & MASK) | lane_const;
}

template <typename T, int KB, bool CHUNKED>
__global__ void __launch_bounds__(V4_THREADS, 1)
attn_turbo_v4_kernel(const __grid_constant__ TurboV4Params p) {
    constexpr int D = V4_D;
    constexpr int KW = D * KB / 32;
    constexpr int K_TILE = V4_TILE * KW * 4, V_TILE = V4_TILE * V4_VW * 4, N_TILE = V4_TILE * 4;
    constexpr int STAGE_BYTES = K_TILE + V_TILE + 2 * N_TILE;
    static_assert(K_TILE % 16 == 0 && STAGE_BYTES % 128 == 0, "bulk copies need 16-byte multiples");

    extern __shared__ __align__(128) unsigned char smem_raw[];
    const FlatPlan &fp = p.flat;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // ---- shared-memory plan: the table sits on the first 64 KB boundary of the shared window at or
    // after the start of the dynamic region; the small buffers go in front of it when they fit there,
    // else behind it; the ring takes what is left (a multiple of four stages, at most twelve) ----
    const uint32_t base_a = smem_u32(smem_raw);
    const uint32_t pad = (0x10000u - (base_a & 0xFFFFu)) & 0xFFFFu;
    const uint32_t misc_bytes = 8u * V4_SLOT_FLOATS * 4u        // fold slots, later the four warps' rows
                                + 8u * D * 4u                     // rotated queries
                                + (uint32_t)(((fp.red_rows * fp.nslots + fp.red_rows * D + 3) & ~3) * 4)  // epilogue work
                                + 2u * 8u * D * 2u                // staged query rows (two buffers)
                                + (2u * V4_MAX_STAGES + 4u) * 8u + 16u + 128u;
    unsigned char *tab = smem_raw + pad;
    unsigned char *after = tab + V4_TABLE_BYTES;
    unsigned char *misc;
    if (pad >= misc_bytes) {
        misc = smem_raw + ((128u - (base_a & 127u)) & 127u);
    } else {
        misc = after;
        after += (misc_bytes + 127u) & ~127u;
    }
    const uint32_t left = p.smem_bytes - (uint32_t)(after - smem_raw);
    int nstage = min(V4_MAX_STAGES, (int)(left / STAGE_BYTES));
    nstage -= nstage % V4_GROUPS;
    if ((uint32_t)(after - smem_raw) > p.smem_bytes || nstage < 2 * V4_GROUPS || nstage < 2) {
        if (tid == 0) atomicExch(p.status, 31);   // the plan does not fit: report and leave, nothing was started
        return;
    }
    unsigned char *stages = after;
    float *slots = (float *)misc;                                        // [8][36][32]
    float *red_o = slots;                                                // [4][red_rows][RED_STRIDE] after the folds
    float *red_ml = slots + 4 * 8 * V4_RED_STRIDE;                       // [4][red_rows][2]
    float *qrot = slots + 8 * V4_SLOT_FLOATS;                            // [8][D]
    float *work = qrot + 8 * D;
    unsigned char *qbuf = (unsigned char *)(work + ((fp.red_rows * fp.nslots + fp.red_rows * D + 3) & ~3));  // [2][8][D] elements
    uint64_t *full = (uint64_t *)(qbuf + 2 * 8 * D * 2);
    uint64_t *empty = full + V4_MAX_STAGES;
    uint64_t *qfull = empty + V4_MAX_STAGES;
    uint64_t *qempty = qfull + 2;
    int *is_last = (int *)(qempty + 2);

    const int rep = p.Hq / p.Hkv;
    const int R_all = rep * p.L;   // query rows of a (batch, kv head) group, cut into p.chunks units of eight
    const int tiles = fp.tiles;
    const int64_t x_lo = flat_lo(fp, blockIdx.x), x_hi = flat_lo(fp, blockIdx.x + 1);
    const uint32_t q_bytes = (uint32_t)R_all * D * 2;   // bulk staging only runs with one chunk

    if (tid == 0) {
        for (int s = 0; s < nstage; ++s) {
            mbar_init(&full[s], 4);             // the four copies of a stage, each announced by its issuer
            mbar_init(&empty[s], V4_GW);            // the warps of the stage's group
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&qfull[s], 1);
            mbar_init(&qempty[s], V4_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    // ---- tables, once per CTA. Row e (256 bytes): words 0..31 = value entry e for lanes 0..31 =
    // f16x2(centroid_v[e & 15], centroid_v[e >> 4]); words 32..63 = key entry e for lanes 0..31 =
    // f16x2(centroid_k[e & m], centroid_k[e >> KB]) for e < 4^KB ----
    for (int w = tid; w < 256 * 32; w += V4_THREADS) {
        const int e = w >> 5;
        ((uint32_t *)tab)[e * 64 + (w & 31)] = pack_h2(p.vcb[e & 15], p.vcb[e >> 4]);
    }
    for (int w = tid; w < (1 << (2 * KB)) * 32; w += V4_THREADS) {
        const int e = w >> 5;
        ((uint32_t *)tab)[e * 64 + 32 + (w & 31)] = pack_h2(p.kcb[e & ((1 << KB) - 1)], p.kcb[e >> KB]);
    }
    if (256 % V4_TILE != 0) {
        // a cut-short last stage leaves its end as it was: start from zeros, so that what the masked
        // tokens multiply is always finite
        for (int i = tid; i < nstage * (STAGE_BYTES / 16); i += V4_THREADS) ((uint4 *)stages)[i] = make_uint4(0u, 0u, 0u, 0u);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    pdl_wait();  // the tables came from kernel parameters; everything below reads global memory

    bool ok = true;

    if (warp >= V4_WARPS) {
        // ---------------- producers: one stream of tiles across the segments ----------------
        // Four warps, one lane each: warp i issues copy i of every stage (packed keys, packed values,
        // key norms, value norms) and announces its bytes on the stage's barrier (four arrivals fill
        // it); the copies of one thread issue one after the other, those of different warps overlap.
        // The first producer also stages the query rows of each segment.
        // which of the stage's four copies this thread issues: with four producer warps lane 0 of warp i,
        // with one producer warp its lanes 0..3 (each announces its own bytes: four arrivals fill a stage)
        const int pw = V4_PRODUCERS == 4 ? warp - V4_WARPS : lane;
        const bool issuer = V4_PRODUCERS == 4 ? lane == 0 : lane < 4;
        if (issuer && !(KVC_SKIP_BITS(p) & 2)) {   // measurement bit 2: no loads at all (consumers compute on stale stages)
            int it = 0, sg = 0;
            for (int64_t x = x_lo; x < x_hi && ok; ++sg) {
                const int unit = (int)(x / tiles), tb = (int)(x % tiles);
                const int n = (int)min((int64_t)(tiles - tb), x_hi - x);
                const int bh = CHUNKED ? unit / p.chunks : unit;
                const int hk = bh % p.Hkv, b = bh / p.Hkv;
                if (p.q_bulk && pw == 0) {
                    const int qb = sg & 1;
                    if (sg >= 2) ok = mbar_wait(&qempty[qb], ((sg >> 1) - 1) & 1);
                    if (!ok) break;
                    mbar_expect_tx(&qfull[qb], q_bytes);
                    bulk_load(qbuf + (size_t)qb * (8 * D * 2), (const T *)p.q + b * p.q_sb + (int64_t)hk * rep * p.q_sh,
                              q_bytes, &qfull[qb]);
                }
                // this thread's array: source of token 0 of the unit, bytes per token, offset inside a stage
                const unsigned char *src;
                uint32_t per_token, dst_off;
                if (pw == 0) { src = (const unsigned char *)(p.kp + b * p.kp_sb + hk * p.kp_sh); per_token = KW * 4; dst_off = 0; }
                else if (pw == 1) { src = (const unsigned char *)(p.vp + b * p.vp_sb + hk * p.vp_sh); per_token = V4_VW * 4; dst_off = K_TILE; }
                else if (pw == 2) { src = (const unsigned char *)(p.kn + b * p.kn_sb + hk * p.kn_sh); per_token = 4; dst_off = K_TILE + V_TILE; }
                else { src = (const unsigned char *)(p.vn + b * p.vn_sb + hk * p.vn_sh); per_token = 4; dst_off = K_TILE + V_TILE + N_TILE; }
                // tokens the copies may touch: the stored rows rounded up to 256 (inside the slab by the
                // launch checks); a stage that would end past them is cut short
                const int64_t t_pad = (p.T + 255) / 256 * 256;
                for (int j = 0; j < n && ok; ++j, ++it) {
                    const int s = it % nstage;
                    if (it >= nstage) ok = mbar_wait(&empty[s], ((it / nstage) - 1) & 1);
                    if (!ok) break;
                    const int64_t t0 = (int64_t)(tb + j) * V4_TILE;
                    const uint32_t bytes = per_token * (uint32_t)min((int64_t)V4_TILE, t_pad - t0);
                    mbar_expect_tx(&full[s], bytes);
                    bulk_load(stages + (size_t)s * STAGE_BYTES + dst_off, src + t0 * per_token, bytes, &full[s]);
                }
                x += n;
            }
            if (!ok) atomicExch(p.status, 32);
        }
        return;
    }

    // ---------------- consumers: one segment per unit the CTA's tile range touches ----------------
    const int g = lane >> 2, c = lane & 3;
    const int grp = warp / V4_GW, wq = warp % V4_GW;
    // M row g of the score product stands for token sg = (g >> 1) + 4 (g & 1) of the warp's sixteen
    // (rows g + 8: + 8), so that after the 8x8 transpose of P the k slots (2c, 2c+1) of the value
    // product are the tokens (c, c + 4): the four lanes c then read value rows of alternating bank phase.
    const int sgm = (g >> 1) + 4 * (g & 1);
    const uint32_t tab_a = smem_u32(tab);
    const uint32_t v_const = tab_a | ((uint32_t)lane << 2);
    const uint32_t k_const = tab_a | 128u | ((uint32_t)lane << 2);
    const uint32_t stages_a = smem_u32(stages);
    int it0 = 0;   // tiles of this CTA's stream consumed by earlier segments
    int g_s = grp; // ring index and phase bit of this group's next stage (stages grp, grp + 4, ...)
    uint32_t g_ph = 0;
    int sg = 0;
    for (int64_t x = x_lo; x < x_hi; ++sg) {
        const int unit = (int)(x / tiles), tile_begin = (int)(x % tiles);
        const int ntiles = (int)min((int64_t)(tiles - tile_begin), x_hi - x);
        const int bh = CHUNKED ? unit / p.chunks : unit, row0 = CHUNKED ? (unit % p.chunks) * 8 : 0;
        const int hk = bh % p.Hkv, b = bh / p.Hkv;
        const int R = CHUNKED ? min(8, R_all - row0) : R_all;
        // ---- rotated queries of this unit: q' = H(signs * q) / sqrt(D) * scale * log2(e), rows past R zero ----
        const T *q_stage = nullptr;
        if (p.q_bulk) {
            if (ok && !(KVC_SKIP_BITS(p) & 2)) {
                ok = mbar_wait(&qfull[sg & 1], (sg >> 1) & 1);
                if (!ok && lane == 0) atomicExch(p.status, 33);
            }
            q_stage = (const T *)(qbuf + (size_t)(sg & 1) * (8 * D * 2));
        }
        // Warp r rotates row r in registers: lane l holds dims 4l .. 4l+3, the stages of the butterfly that
        // pair dims 1 and 2 apart stay inside the lane, the other five are lane exchanges. The pairs and
        // the operations ((a, b) -> (a + b, a - b), lower dim first) are those of the shared-memory
        // butterfly of the other kernels, so the rotated query is the same bit for bit.
        if (warp < 8) {
            const int r = warp;
            float x[4] = {0.f, 0.f, 0.f, 0.f};
            if (r < R && ok) {
                const int hq = hk * rep + (row0 + r) / p.L, l = (row0 + r) % p.L;
                const T *src = q_stage ? q_stage + r * D : (const T *)p.q + b * p.q_sb + hq * p.q_sh + l * p.q_sl;
#pragma unroll
                for (int j = 0; j < 4; ++j) x[j] = to_f32<T>(src[4 * lane + j]) * p.q_signs[4 * lane + j];
            }
            {
                const float a0 = x[0] + x[1], a1 = x[0] - x[1], a2 = x[2] + x[3], a3 = x[2] - x[3];
                x[0] = a0 + a2; x[2] = a0 - a2; x[1] = a1 + a3; x[3] = a1 - a3;
            }
#pragma unroll
            for (int m = 1; m < 32; m <<= 1) {
                const bool upper = (lane & m) != 0;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float y = __shfl_xor_sync(0xffffffffu, x[j], m);
                    x[j] = upper ? y - x[j] : x[j] + y;
                }
            }
            if (p.q_calib) {
#pragma unroll
                for (int j = 0; j < 4; ++j) x[j] *= p.q_calib[4 * lane + j];
            }
            *(float4 *)(qrot + r * D + 4 * lane) = make_float4(x[0], x[1], x[2], x[3]);
        }
        if (p.q_bulk) {
            __syncwarp();
            if (ok && lane == 0 && !(KVC_SKIP_BITS(p) & 2)) mbar_arrive(&qempty[sg & 1]);
        }
        consumer_bar<V4_WARPS>();
        float m_run[2], l_run[2] = {0.f, 0.f};
        float o_acc[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;

        // Q'^T fragments (B operand, column = query row g). MMA m of the key side covers, from lane
        // c, the dims 32c + 4m + {0,1} (k slots 2c, 2c+1) and 32c + 4m + {2,3} (k slots 2c+8, 2c+9).
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
            const int l = (r < R) ? (row0 + r) % p.L : 0;
            row_limit[k] = p.causal ? (int)min((int64_t)t_last, p.causal_offset + l) : t_last;
        }
        const int min_limit = p.causal ? (int)min((int64_t)t_last, p.causal_offset) : t_last;
        constexpr float M_INIT = -1e30f, LAZY = 8.f;
        m_run[0] = m_run[1] = M_INIT;
        float m_thr[2] = {M_INIT, M_INIT};

        const int tl0 = wq * 16 + sgm, tl1 = tl0 + 8;       // the two tokens of this lane's score rows
        const int tv = wq * 16 + c;                         // value tokens tv, tv + 4, tv + 8, tv + 12

        // this group's stages of the segment: every V4_GROUPS-th tile of the CTA's stream; the ring index and
        // the phase bit of the group's next stage (g_s, g_ph) are carried along instead of divided out
        for (int jt = ((grp - it0) % V4_GROUPS + V4_GROUPS) % V4_GROUPS; jt < ntiles; jt += V4_GROUPS) {
            const int s = g_s;
            const uint32_t ph = g_ph;
            g_s += V4_GROUPS;
            if (g_s >= nstage) { g_s -= nstage; g_ph ^= 1u; }
            if (!ok) continue;                              // a wait ran out earlier: walk on to the segment's barriers
            if (!(KVC_SKIP_BITS(p) & 2)) ok = mbar_wait(&full[s], ph);
            if (!ok) {
                if (lane == 0) atomicExch(p.status, 34);
                continue;
            }
            if (KVC_SKIP_BITS(p) & 1) {
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
                continue;
            }
            const uint32_t st_a = stages_a + (uint32_t)s * STAGE_BYTES;
            const uint32_t kpt_a = st_a, vpt_a = st_a + K_TILE, knt_a = st_a + K_TILE + V_TILE,
                           vnt_a = st_a + K_TILE + V_TILE + N_TILE;
            const int t_blk = (tile_begin + jt) * V4_TILE + wq * 16;

            // ---- everything this block reads from the stage, up front: the loads are the only ordered
            // (volatile) operations of the block, what follows is free to be scheduled around them ----
            uint32_t wa[KB], wb[KB];
            uint32_t va[2], vb4[2], vc[2], vd[2];
            lds_words<KB>(kpt_a + (uint32_t)(tl0 * KW + c * KB) * 4u, wa);
            lds_words<KB>(kpt_a + (uint32_t)(tl1 * KW + c * KB) * 4u, wb);
            const float kn0 = lds_f32(knt_a + 4u * tl0), kn1 = lds_f32(knt_a + 4u * tl1);
            const float vn0 = lds_f32(vnt_a + 4u * tl0), vn1 = lds_f32(vnt_a + 4u * tl1);
            {
                const uint32_t v_a = vpt_a + (uint32_t)(tv * V4_VW + 2 * g) * 4u;
                lds_words<2>(v_a, va);
                lds_words<2>(v_a + 4 * V4_VW * 4, vb4);
                lds_words<2>(v_a + 8 * V4_VW * 4, vc);
                lds_words<2>(v_a + 12 * V4_VW * 4, vd);
            }
            // ---- S^T = centroids[idx_k] . Q'^T, two accumulator chains ----
            float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#ifndef KVC_V4_MEASURE_NO_K
            {
#pragma unroll
                for (int m = 0; m < 8; ++m) {
                    uint32_t a[4];
                    a[0] = lds32(key_entry<KB, KB>(wa, 2 * m, k_const));      // row g,     k slots 2c, 2c+1
                    a[1] = lds32(key_entry<KB, KB>(wb, 2 * m, k_const));      // row g + 8
                    a[2] = lds32(key_entry<KB, KB>(wa, 2 * m + 1, k_const));  // row g,     k slots 2c+8, 2c+9
                    a[3] = lds32(key_entry<KB, KB>(wb, 2 * m + 1, k_const));  // row g + 8
                    mma_f16(acc[m & 1], a, qb[m][0], qb[m][1]);
                }
            }
#endif
            float sc[4];
            {
                const float n0 = kn0, n1 = kn1;
                sc[0] = n0 * (acc[0][0] + acc[1][0]);
                sc[1] = n0 * (acc[0][1] + acc[1][1]);
                sc[2] = n1 * (acc[0][2] + acc[1][2]);
                sc[3] = n1 * (acc[0][3] + acc[1][3]);
            }
            if (t_blk + 15 > min_limit) {  // warp-uniform: only tiles that cross a limit
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int t = t_blk + sgm + ((e >> 1) ? 8 : 0);
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
            // ---- P'^T = (p * norm_v)^T in the B-fragment layout: after the transpose lane (g, c) holds
            // query row g and the k slots (2c, 2c+1), i.e. the tokens (c, c + 4) [+ 8 in the second register] ----
            uint32_t pb[2];
            {
                pb[0] = movmatrix_free(pack_h2(pr[0] * vn0, pr[1] * vn0));
                pb[1] = movmatrix_free(pack_h2(pr[2] * vn1, pr[3] * vn1));
            }
#ifndef KVC_V4_MEASURE_NO_V
            // ---- O^T += centroids[idx_v]^T . P'^T ----
            // The lane owns dims 16g .. 16g+15 of its four tokens. For word w and byte b of the
            // interleaved registers, output tile mt = 4w + b has row g = dim 16g + 2mt (even nibbles)
            // and row g + 8 = dim 16g + 2mt + 1 (odd nibbles).
            {
#pragma unroll
                for (int w = 0; w < 2; ++w) {
                    const uint32_t lo_ab = (va[w] & 0x0F0F0F0Fu) | ((vb4[w] << 4) & 0xF0F0F0F0u);
                    const uint32_t hi_ab = ((va[w] >> 4) & 0x0F0F0F0Fu) | (vb4[w] & 0xF0F0F0F0u);
                    const uint32_t lo_cd = (vc[w] & 0x0F0F0F0Fu) | ((vd[w] << 4) & 0xF0F0F0F0u);
                    const uint32_t hi_cd = ((vc[w] >> 4) & 0x0F0F0F0Fu) | (vd[w] & 0xF0F0F0F0u);
                    uint32_t a[4];
#define KVC_V4_TILE(BYTE)                                                  \
    a[0] = lds32(value_entry<BYTE>(lo_ab, v_const));                       \
    a[1] = lds32(value_entry<BYTE>(hi_ab, v_const));                       \
    a[2] = lds32(value_entry<BYTE>(lo_cd, v_const));                       \
    a[3] = lds32(value_entry<BYTE>(hi_cd, v_const));                       \
    mma_f16(o_acc[4 * w + BYTE], a, pb[0], pb[1]);
                    KVC_V4_TILE(0)
                    KVC_V4_TILE(1)
                    KVC_V4_TILE(2)
                    KVC_V4_TILE(3)
#undef KVC_V4_TILE
                }
            }
#else
            o_acc[0][0] += __uint_as_float(pb[0]) + __uint_as_float(pb[1]);
#endif
            __syncwarp();
            if (lane == 0 && !(KVC_SKIP_BITS(p) & 2)) mbar_arrive(&empty[s]);
        }
        it0 += ntiles;
        // a warp whose tokens were all masked (or that had no stage in this segment) reports "no maximum"
        if (m_run[0] <= M_INIT) m_run[0] = -INFINITY;
        if (m_run[1] <= M_INIT) m_run[1] = -INFINITY;

        // ---- fold the 16 warps down to 4, lane to lane ----
#pragma unroll 1
        for (int half = 8; half >= 4; half >>= 1) {   // warp w + half folds into warp w (a missing sixteenth warp folds nothing)
            consumer_bar<V4_WARPS>();   // the slots are free (first pass: the query fragments are in registers)
            if (warp >= half && warp < 2 * half) {
                float *sl = slots + (warp - half) * V4_SLOT_FLOATS + lane;
#pragma unroll
                for (int mt = 0; mt < 8; ++mt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) sl[(mt * 4 + e) * 32] = o_acc[mt][e];
                sl[32 * 32] = m_run[0]; sl[33 * 32] = m_run[1];
                sl[34 * 32] = l_run[0]; sl[35 * 32] = l_run[1];
            }
            consumer_bar<V4_WARPS>();
            if (warp < half && warp + half < V4_WARPS) {
                const float *sl = slots + warp * V4_SLOT_FLOATS + lane;
                float fa[2], fb[2];
#pragma unroll
                for (int k = 0; k < 2; ++k) {
                    const float mb = sl[(32 + k) * 32], lb = sl[(34 + k) * 32];
                    const float mn = fmaxf(m_run[k], mb);
                    fa[k] = (m_run[k] == -INFINITY) ? 0.f : fast_exp2(m_run[k] - mn);
                    fb[k] = (mb == -INFINITY) ? 0.f : fast_exp2(mb - mn);
                    l_run[k] = l_run[k] * fa[k] + lb * fb[k];
                    m_run[k] = mn;
                }
#pragma unroll
                for (int mt = 0; mt < 8; ++mt)
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        o_acc[mt][e] = o_acc[mt][e] * fa[e & 1] + sl[(mt * 4 + e) * 32] * fb[e & 1];
            }
        }
        consumer_bar<V4_WARPS>();   // the last reads of the slots are done: they become the four warps' rows
        if (warp < 4) {
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                l_run[k] += __shfl_xor_sync(0xffffffffu, l_run[k], 4);
                l_run[k] += __shfl_xor_sync(0xffffffffu, l_run[k], 8);
                l_run[k] += __shfl_xor_sync(0xffffffffu, l_run[k], 16);
            }
            float *wo = red_o + warp * fp.red_rows * V4_RED_STRIDE;
#pragma unroll
            for (int mt = 0; mt < 8; ++mt) {
                const int d0 = 16 * g + 2 * mt, d1 = d0 + 1;
                if (2 * c < R) {
                    wo[(2 * c) * V4_RED_STRIDE + d0] = o_acc[mt][0];
                    wo[(2 * c) * V4_RED_STRIDE + d1] = o_acc[mt][2];
                }
                if (2 * c + 1 < R) {
                    wo[(2 * c + 1) * V4_RED_STRIDE + d0] = o_acc[mt][1];
                    wo[(2 * c + 1) * V4_RED_STRIDE + d1] = o_acc[mt][3];
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
        }
        UnitOut u;
        u.o_part = p.o_part; u.ml_part = p.ml_part; u.counters = p.counters;
        u.out = p.out; u.out_dtype = p.out_dtype;
        u.o_sb = p.o_sb; u.o_sh = p.o_sh; u.o_sl = p.o_sl;
        u.o_signs = p.o_signs;
        u.splits = 0; u.Hq = p.Hq; u.L = p.L;
        segment_epilogue<D, V4_WARPS, 4>(u, fp, red_o, red_ml, V4_RED_STRIDE, work, is_last, unit, b, hk, rep, R, -1, 0, row0);
        x += ntiles;
    }
}

template <typename T, int KB, bool CHUNKED>
bool launch_v4_typed(const TurboV4Params &p, int ctas, size_t smem, cudaStream_t stream) {
    // 0 = not yet, 1 = ready, -1 = the device refused the shared memory
    static std::atomic<int> configured[64];
    const int dev = current_device();
    if (dev < 0 || dev >= 64) return false;
    int state = configured[dev].load(std::memory_order_acquire);
    if (state == 0) {
        cudaError_t e = cudaFuncSetAttribute(attn_turbo_v4_kernel<T, KB, CHUNKED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(attn_turbo_v4_kernel<T, KB, CHUNKED>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        if (e != cudaSuccess) (void)cudaGetLastError();
        state = e == cudaSuccess ? 1 : -1;
        configured[dev].store(state, std::memory_order_release);
    }
    if (state < 0) return false;
    KernelTimer timer(stream);
    KVC_CUDA(launch_pdl(attn_turbo_v4_kernel<T, KB, CHUNKED>, dim3(ctas), dim3(V4_THREADS), smem, stream, p));
    timer.stop();
    KVC_CUDA(cudaGetLastError());
    ++g_launch_count;
    return true;
}

}  // namespace

// The caller (launch_attention_turbo) has checked dtype, head dim, masks, sources and alignment;
// this path adds: 4-bit values, key bits 2..4, and the whole opt-in shared memory of an SM.
// Returns the number of kernels launched, 0 when the call is left to the other kernel.
int launch_attention_turbo_v4(const AttnArgs &a, cudaStream_t stream) {
    static const bool off = [] {
        const char *e = std::getenv("KVC_TURBO_V4");
        return e && e[0] == '0';
    }();
    if (off) return 0;
    const int kb = a.k.bits, vb = a.v.bits;
    if (vb != 4 || kb < 2 || kb > 4) return 0;
    const int rep = a.Hq / a.Hkv;
    // a group of more than eight query rows (a verify chunk) is cut into units of eight rows; the
    // units of one (batch, kv head) are neighbours in the flat order, so they stream the same tiles
    // at about the same time and all but the first find them in L2
    const int chunks = (rep * a.L + 7) / 8;
    if (chunks > V4_MAX_CHUNKS) return 0;
    const int64_t bh = (int64_t)a.B * a.Hkv * chunks;
    if (bh * (int64_t)sizeof(int) > V4_COUNTER_BYTES) return 0;
    {
        // a full last stage must stay inside the (batch, head) slab
        const int64_t padded = (a.T + 255) / 256 * 256;
        if (a.k.sh < padded * a.k.words || a.v.sh < padded * a.v.words || a.k.gsh < padded || a.v.gsh < padded) return 0;
    }
    int *status = device_status_word(a.device);
    if (!status) return 0;
    int *counters = counters_get(a.device, stream, V4_COUNTER_BYTES);

    const int64_t tiles = (a.T + V4_TILE - 1) / V4_TILE;
    FlatPlan plan;
    plan.tiles = (int)tiles;
    plan.red_rows = std::min(8, rep * a.L);
    const int64_t work_tiles = bh * tiles;
    const int64_t ctas = std::min<int64_t>((int64_t)sm_count(a.device), work_tiles);
    plan.per = (int)(work_tiles / ctas);
    plan.rem = (int)(work_tiles % ctas);
    plan.nslots = (int)((tiles + plan.per - 1) / plan.per + 1);
    if (plan.nslots > 64) return 0;
    const int64_t qrows = (int64_t)a.B * a.Hq * a.L;
    const size_t o_bytes = (size_t)qrows * plan.nslots * a.D * sizeof(float);
    const size_t ml_bytes = (size_t)qrows * plan.nslots * sizeof(float2);
    char *scratch = (char *)scratch_get(a.device, o_bytes + ml_bytes + 256, stream);

    TurboV4Params p;
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
    p.B = a.B; p.Hq = a.Hq; p.Hkv = a.Hkv; p.L = a.L; p.T = a.T; p.chunks = chunks;
    p.causal = a.mask.mode == KVC_MASK_CAUSAL ? 1 : 0;
    p.causal_offset = a.mask.causal_offset;
    p.scale_log2 = a.scale * 1.4426950408889634f;
    p.flat = plan;
    p.q_bulk = (chunks == 1 && a.L == 1 && a.q_sh == a.D && ((uintptr_t)a.q & 15) == 0 && (a.q_sb * 2) % 16 == 0) ? 1 : 0;
    // everything an SM offers a CTA: 227 KB opt-in maximum
    const size_t smem = (size_t)227 * 1024;
    p.smem_bytes = (uint32_t)smem;
    p.debug_skip = measure_skip_bits();

    bool taken = false;
#define KVC_V4(TT, KK) \
    if (kb == KK) taken = chunks > 1 ? launch_v4_typed<TT, KK, true>(p, (int)ctas, smem, stream) \
                                     : launch_v4_typed<TT, KK, false>(p, (int)ctas, smem, stream);
    if (a.q_dtype == KVC_BF16) {
        KVC_V4(__nv_bfloat16, 2) KVC_V4(__nv_bfloat16, 3) KVC_V4(__nv_bfloat16, 4)
    } else {
        KVC_V4(__half, 2) KVC_V4(__half, 3) KVC_V4(__half, 4)
    }
#undef KVC_V4
    if (taken && chunks > 1 && trace_dispatch()) fprintf(stderr, "[kvc] turbo_v4: %d units of eight query rows per kv head\n", chunks);
    return taken ? 1 : 0;
}

}  // namespace kvc
