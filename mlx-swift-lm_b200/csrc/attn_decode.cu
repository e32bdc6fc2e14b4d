// Split-K flash decoding for raw f16/bf16 caches on sm_100a.
//
// Work unit = (batch, KV head, token split). A CTA of one producer warp and
// four consumer warps streams its token range through a ring of shared-memory
// stages: the producer issues tiled TMA loads (cp.async.bulk.tensor, 128-byte
// swizzle) of K and V tiles straight from the cache arrays and signals an
// mbarrier per stage; each consumer warp owns 16 of a tile's 64 tokens, scores
// all query rows of the GQA group against them with m16n8k16 tensor-core MMAs
// (queries are the 16-row A operand, so every K/V byte is read from HBM and
// from shared memory exactly once for the whole group), keeps an online
// softmax in registers and accumulates P.V with a second MMA. The four warps'
// states are merged in shared memory into one un-normalised partial per unit.
// The last unit of a (batch, head) to finish - found with a ticket counter -
// merges the partials of all splits with a log-sum-exp reduction and writes
// the output row, so no second kernel is needed.
//
// Shared-memory layout of a tile: boxes of [64 tokens][64 elements] (128 bytes
// per row), 16-byte chunk c of row r stored at chunk c ^ (r & 7).
//   * K operand (B fragment, "col-major"): a lane reads whole 16-byte chunks of
//     its token's row; the k-slot <-> head-dim assignment of the MMAs is a
//     permutation (shared with the Q fragments) chosen so that a quarter-warp
//     touches all eight chunk columns: no bank conflicts, no shuffles.
//   * V operand: ldmatrix.trans over eight consecutive token rows, which the
//     swizzle spreads over all eight chunk columns as well.
//
// Every wait on an mbarrier is bounded; a wait that runs out records an error
// code in a device status word and the CTA leaves its loops.
#include "attn_common.cuh"

#include <algorithm>
#include <cstdlib>
#include <mutex>

namespace kvc {

namespace {

using namespace dev;

constexpr int CONSUMER_WARPS = 4;
constexpr int DEC_THREADS = (CONSUMER_WARPS + 1) * 32;
constexpr int TILE_T = 64;  // tokens per tile: one 16-token block per consumer warp
constexpr int BOX_BYTES = TILE_T * 128;
constexpr int COUNTER_BYTES = 64 * 1024;  // ticket counters at the start of the scratch arena

struct DecodeParams {
    const void *q;
    void *out;
    int64_t q_sb, q_sh, q_sl, o_sb, o_sh, o_sl;
    float *o_part;
    float2 *ml_part;
    int *counters;
    int *status;
    int32_t B, Hq, Hkv, L;
    int64_t T;
    int32_t splits;       // units per (batch, head)
    int32_t tiles_base;   // tiles per unit; the first tiles_rem units take one more
    int32_t tiles_rem;
    int32_t causal;
    int32_t out_dtype;
    int32_t debug_skip;  // measurement aid: 1 = consumers release tiles without computing
    int32_t row_blocks;  // chunk kernel: 64-row blocks per (batch, head)
    int32_t tiles_all;   // chunk kernel: tiles covering all T tokens
    FlatPlan flat;       // flat kernel
    int32_t q_bulk;      // flat kernel: the unit's query rows are one contiguous 16-byte aligned block
    // cache arrays as plain pointers (byte strides): fused append target, and the measurement aid
    // debug_skip & 2 (linear bulk copies of the same bytes instead of the tiled TMA loads)
    unsigned char *k_base, *v_base;
    int64_t kv_sb, kv_sh, kv_st;
    // fused append: the new rows [B, Hkv, D] of this step (null = the cache already holds them)
    const void *new_k, *new_v;
    int32_t early_tiles;  // flat kernel: the stored rows may be streamed before the preceding kernel has finished
    int64_t new_slot;     // flat kernel, fused append: token index the new row is stored at (T - 1, or a ring slot)
    int64_t nk_sb, nk_sh, nv_sb, nv_sh;  // element strides
    int64_t causal_offset;
    float scale_log2;  // scale * log2(e)
};

template <typename T, int D, int NSTAGE>
__global__ void __launch_bounds__(DEC_THREADS, (D <= 128 ? 2 : 1))
attn_decode_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                   const DecodeParams p) {
    constexpr int TILE_BYTES = TILE_T * D * 2;     // one K (or V) tile
    constexpr int BOXES = D / 64;                  // [64 tokens][64 elements] boxes per tile
    constexpr int KSTEPS = D / 16;
    constexpr int NT_O = D / 8;                    // output n-tiles (8 head dims each)
    constexpr int RED_STRIDE = D + 8;              // padded row of the cross-warp merge buffer
    static_assert(TILE_T == 16 * CONSUMER_WARPS, "one 16-token block per consumer warp");
    static_assert(CONSUMER_WARPS * 16 * RED_STRIDE * 4 + 512 + 16 * 64 * 4 <= NSTAGE * 2 * TILE_BYTES, "merge buffers must fit");

    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // pointer + offset (no integer round trip) so that loads through it stay ld.shared
    unsigned char *stages = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint64_t *full = (uint64_t *)(stages + (size_t)NSTAGE * 2 * TILE_BYTES);
    uint64_t *empty = full + NSTAGE;
    int *is_last = (int *)(empty + NSTAGE);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x % p.splits;
    const int bh = blockIdx.x / p.splits;
    const int hk = bh % p.Hkv, b = bh / p.Hkv;
    const int rep = p.Hq / p.Hkv;
    const int R = rep * p.L;

    // balanced split of the tile range
    const int tile_begin = split * p.tiles_base + min(split, p.tiles_rem);
    const int ntiles = p.tiles_base + (split < p.tiles_rem ? 1 : 0);

    if (tid == 0) {
        for (int s = 0; s < NSTAGE; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], CONSUMER_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    pdl_wait();  // everything below reads what earlier kernels on the stream wrote

    bool ok = true;
    const int g = lane >> 2, c = lane & 3;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o_acc[NT_O][4];
#pragma unroll
    for (int i = 0; i < NT_O; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;

    if (warp == CONSUMER_WARPS) {
        // ---------------- producer ----------------
        if (lane == 0) {
            for (int it = 0; it < ntiles && ok; ++it) {
                const int s = it % NSTAGE;
                if (it >= NSTAGE) ok = mbar_wait(&empty[s], ((it / NSTAGE) - 1) & 1);
                if (!ok) break;
                unsigned char *kt = stages + (size_t)s * 2 * TILE_BYTES;
                unsigned char *vt = kt + TILE_BYTES;
                mbar_expect_tx(&full[s], 2 * TILE_BYTES);
                const int t0 = (tile_begin + it) * TILE_T;
#pragma unroll
                for (int bx = 0; bx < BOXES; ++bx) {
                    tma_load_4d(kt + bx * BOX_BYTES, &kmap, &full[s], bx * 64, t0, hk, b);
                    tma_load_4d(vt + bx * BOX_BYTES, &vmap, &full[s], bx * 64, t0, hk, b);
                }
            }
            if (!ok) atomicExch(p.status, 1);
        }
    } else {
        // ---------------- consumers ----------------
        // Query fragments: rows r < R of this KV head's group; row r <-> (rep index r / L, position r % L).
        // k-step ks = (box bx, pass ps, half h): lane c covers chunk 2c + ps of the box, elements 4h..4h+3.
        uint32_t qa[KSTEPS][4];
        int64_t row_limit[2];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = g + 8 * half;
            const int l = r % p.L;
            row_limit[half] = (r < R) ? (p.causal ? min(p.T - 1, p.causal_offset + l) : p.T - 1) : -1;
        }
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            const int bx = ks / 4, ps = (ks >> 1) & 1, h = ks & 1;
            const int d0 = bx * 64 + (2 * c + ps) * 8 + 4 * h;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int r = g + 8 * half;
                uint32_t w0 = 0, w1 = 0;
                if (r < R) {
                    const int hq = hk * rep + r / p.L, l = r % p.L;
                    const T *qp = (const T *)p.q + b * p.q_sb + hq * p.q_sh + l * p.q_sl + d0;
                    w0 = *(const uint32_t *)qp;
                    w1 = *(const uint32_t *)(qp + 2);
                }
                qa[ks][half] = w0;      // a0 / a1: k-slots 2c, 2c+1
                qa[ks][2 + half] = w1;  // a2 / a3: k-slots 2c+8, 2c+9
            }
        }
        // Lane-constant byte offsets inside a box.
        //   K: token row (16*warp + 8*j + g), chunk (2c + ps) ^ g
        //   V (ldmatrix): lane supplies the row of matrix i = lane / 8: token 16*warp + 8*(i & 1) + (lane & 7),
        //                 chunk (2*cp + (i >> 1)) ^ (lane & 7) for chunk pair cp
        const int blk = warp;
        uint32_t k_off[2];
#pragma unroll
        for (int ps = 0; ps < 2; ++ps) k_off[ps] = (uint32_t)((blk * 16 + g) * 128 + (((2 * c + ps) ^ g) << 4));
        uint32_t v_off[4];
        {
            const int mi = lane >> 3, rr = lane & 7;
#pragma unroll
            for (int cp = 0; cp < 4; ++cp)
                v_off[cp] = (uint32_t)((blk * 16 + (mi & 1) * 8 + rr) * 128 + (((2 * cp + (mi >> 1)) ^ rr) << 4));
        }

        for (int it = 0; it < ntiles && ok; ++it) {
            const int s = it % NSTAGE;
            ok = mbar_wait(&full[s], (it / NSTAGE) & 1);
            if (!ok) break;
            if (KVC_SKIP_BITS(p)) {
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
                continue;
            }
            const unsigned char *kt = stages + (size_t)s * 2 * TILE_BYTES;
            const uint32_t vt_addr = smem_u32(kt + TILE_BYTES);
            const int64_t t_blk = (int64_t)(tile_begin + it) * TILE_T + blk * 16;

            // ---- S = Q K^T for 16 tokens (two n-tiles of 8), the two accumulator chains interleaved ----
            float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int bx = 0; bx < BOXES; ++bx) {
#pragma unroll
                for (int ps = 0; ps < 2; ++ps) {
                    const uint4 k0 = *(const uint4 *)(kt + bx * BOX_BYTES + k_off[ps]);
                    const uint4 k1 = *(const uint4 *)(kt + bx * BOX_BYTES + k_off[ps] + 8 * 128);
                    const int ks = bx * 4 + ps * 2;
                    MmaType<T>::mma(sc[0], qa[ks], k0.x, k0.y);
                    MmaType<T>::mma(sc[1], qa[ks], k1.x, k1.y);
                    MmaType<T>::mma(sc[0], qa[ks + 1], k0.z, k0.w);
                    MmaType<T>::mma(sc[1], qa[ks + 1], k1.z, k1.w);
                }
            }
            // ---- online softmax (log2 domain) ----
            float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < 2; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int half = e >> 1;
                    const int64_t t = t_blk + j * 8 + 2 * c + (e & 1);
                    float v = sc[j][e] * p.scale_log2;
                    v = (t <= row_limit[half]) ? v : -INFINITY;
                    sc[j][e] = v;
                    tmax[half] = fmaxf(tmax[half], v);
                }
            }
            float alpha[2];
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                tmax[half] = fmaxf(tmax[half], __shfl_xor_sync(0xffffffffu, tmax[half], 1));
                tmax[half] = fmaxf(tmax[half], __shfl_xor_sync(0xffffffffu, tmax[half], 2));
                const float m_new = fmaxf(m_run[half], tmax[half]);
                alpha[half] = (m_new == -INFINITY) ? 1.f : fast_exp2(m_run[half] - m_new);
                m_run[half] = m_new;
            }
            uint32_t pa[4];
            {
                float pr[2][4];
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int half = e >> 1;
                        pr[j][e] = (m_run[half] == -INFINITY) ? 0.f : fast_exp2(sc[j][e] - m_run[half]);
                    }
#pragma unroll
                for (int half = 0; half < 2; ++half)
                    l_run[half] = l_run[half] * alpha[half] + pr[0][2 * half] + pr[0][2 * half + 1] +
                                  pr[1][2 * half] + pr[1][2 * half + 1];
                pa[0] = MmaType<T>::pack(pr[0][0], pr[0][1]);  // row g,   k-slots 2c, 2c+1   (tokens 0..7)
                pa[1] = MmaType<T>::pack(pr[0][2], pr[0][3]);  // row g+8
                pa[2] = MmaType<T>::pack(pr[1][0], pr[1][1]);  // row g,   k-slots 2c+8, 2c+9 (tokens 8..15)
                pa[3] = MmaType<T>::pack(pr[1][2], pr[1][3]);  // row g+8
            }
            // ---- O = O * alpha + P V (rescale only when some row's maximum moved) ----
            if (__any_sync(0xffffffffu, (alpha[0] != 1.f) | (alpha[1] != 1.f))) {
#pragma unroll
                for (int nt = 0; nt < NT_O; ++nt) {
                    o_acc[nt][0] *= alpha[0];
                    o_acc[nt][1] *= alpha[0];
                    o_acc[nt][2] *= alpha[1];
                    o_acc[nt][3] *= alpha[1];
                }
            }
#pragma unroll
            for (int bx = 0; bx < BOXES; ++bx) {
#pragma unroll
                for (int cp = 0; cp < 4; ++cp) {
                    // four 8x8 matrices: (tokens 0..7 | 8..15) x (chunk 2cp | 2cp+1) of this box
                    uint32_t vf[4];
                    ldmatrix_x4_trans(vf, vt_addr + bx * BOX_BYTES + v_off[cp]);
                    MmaType<T>::mma(o_acc[bx * 8 + 2 * cp], pa, vf[0], vf[1]);
                    MmaType<T>::mma(o_acc[bx * 8 + 2 * cp + 1], pa, vf[2], vf[3]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }
        if (!ok && lane == 0) atomicExch(p.status, 2);
    }

    // ---------------- merge the four consumer warps ----------------
    __syncthreads();
    float *red_o = (float *)stages;                                  // [4][16][RED_STRIDE]
    float *red_ml = red_o + CONSUMER_WARPS * 16 * RED_STRIDE;        // [4][16][2]
    if (warp < CONSUMER_WARPS) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            l_run[half] += __shfl_xor_sync(0xffffffffu, l_run[half], 1);
            l_run[half] += __shfl_xor_sync(0xffffffffu, l_run[half], 2);
        }
        float *wo = red_o + warp * 16 * RED_STRIDE;
#pragma unroll
        for (int nt = 0; nt < NT_O; ++nt) {
            // n-tile nt: C columns 2c, 2c+1 <-> head dims 8*nt + 2c, 8*nt + 2c + 1
            *(float2 *)&wo[g * RED_STRIDE + 8 * nt + 2 * c] = make_float2(o_acc[nt][0], o_acc[nt][1]);
            *(float2 *)&wo[(g + 8) * RED_STRIDE + 8 * nt + 2 * c] = make_float2(o_acc[nt][2], o_acc[nt][3]);
        }
        if (c == 0) {
            red_ml[(warp * 16 + g) * 2 + 0] = m_run[0];
            red_ml[(warp * 16 + g) * 2 + 1] = l_run[0];
            red_ml[(warp * 16 + g + 8) * 2 + 0] = m_run[1];
            red_ml[(warp * 16 + g + 8) * 2 + 1] = l_run[1];
        }
    }
    __syncthreads();
    UnitOut u;
    u.o_part = p.o_part; u.ml_part = p.ml_part; u.counters = p.counters;
    u.out = p.out; u.out_dtype = p.out_dtype;
    u.o_sb = p.o_sb; u.o_sh = p.o_sh; u.o_sl = p.o_sl;
    u.o_signs = nullptr;
    u.splits = p.splits; u.Hq = p.Hq; u.L = p.L;
    // work area behind the cross-warp buffers (the stage ring is idle by now)
    float *work = red_ml + CONSUMER_WARPS * 16 * 2;
    unit_epilogue<D, CONSUMER_WARPS>(u, red_o, red_ml, RED_STRIDE, work, is_last, b, hk, rep, R, split, bh);
}

// ---------------------------------------------------------------------
// Flat tile decomposition of the same decode computation. All (batch, head) units have
// the same number of tiles, so the launch is one wave of resident CTAs and CTA c simply
// owns the flat tile range [c W / G, (c + 1) W / G) of the W = units x tiles tiles. A
// range that crosses a unit boundary is processed as consecutive segments: the producer
// keeps streaming through the boundary, the consumers finish a segment (cross-warp
// merge, partial to scratch, ticket) and start the next with fresh state. Every CTA does
// the same amount of streaming whatever the shape, and the ramp at both ends of the
// launch is paid once. The cross-warp buffer sits beside the ring (the ring stays live),
// and the consumer warps synchronise among themselves with a named barrier that every
// warp reaches whether or not one of its bounded waits has run out.
// ---------------------------------------------------------------------
template <typename T, int D, int NSTAGE>
__global__ void __launch_bounds__(DEC_THREADS, (D <= 128 ? 2 : 1))
attn_decode_flat_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                        const DecodeParams p) {
    constexpr int TILE_BYTES = TILE_T * D * 2;
    constexpr int BOXES = D / 64;
    constexpr int KSTEPS = D / 16;
    constexpr int NT_O = D / 8;
    constexpr int RED_STRIDE = D + 8;

    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *stages = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint64_t *full = (uint64_t *)(stages + (size_t)NSTAGE * 2 * TILE_BYTES);
    uint64_t *empty = full + NSTAGE;
    int *is_last = (int *)(empty + NSTAGE);
    const FlatPlan &fp = p.flat;
    float *red_o = (float *)(is_last + 4);                                   // [4][red_rows][RED_STRIDE]
    float *red_ml = red_o + CONSUMER_WARPS * fp.red_rows * RED_STRIDE;       // [4][red_rows][2]
    float *work = red_ml + CONSUMER_WARPS * fp.red_rows * 2;                 // [red_rows][nslots]
    // Query rows of a segment's unit, brought in by the producer with one bulk copy (two buffers):
    // plain loads issued by the consumers while the tile stream saturates the memory system cost
    // several microseconds per segment.
    uint64_t *qfull = (uint64_t *)(work + ((fp.red_rows * fp.nslots + 3) & ~3));   // keeps qbuf 16-byte aligned
    uint64_t *qempty = qfull + 2;
    unsigned char *qbuf = (unsigned char *)(qempty + 2);                      // [2][red_rows][D] elements

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rep = p.Hq / p.Hkv;
    const int R = rep * p.L;
    const int tiles = fp.tiles;
    const int64_t x_lo = flat_lo(fp, blockIdx.x), x_hi = flat_lo(fp, blockIdx.x + 1);
    const uint32_t q_bytes = (uint32_t)R * D * 2;

    if (tid == 0) {
        for (int s = 0; s < NSTAGE; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], CONSUMER_WARPS);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&qfull[s], 1);
            mbar_init(&qempty[s], CONSUMER_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    // Everything read below was written by earlier kernels on the stream, so it comes after the wait
    // on the preceding kernel. One exception, early_tiles: the producer streams its first tiles of
    // stored rows before that wait. The host vouches that the preceding kernel does not write them (it
    // is a layer of the same batched call, working on another cache), and every kernel before that one
    // has completed, because kernels release their successor only after their own wait.
    const bool early = p.early_tiles != 0 && warp == CONSUMER_WARPS;
    if (!early) {
        pdl_wait();
        pdl_trigger();
    }

    bool ok = true;
    if (warp == CONSUMER_WARPS) {
        // ---------------- producer: one stream of tiles across the segments ----------------
        if (lane == 0) {
            int it = 0, sg = 0;
            bool waited = !early;
            for (int64_t x = x_lo; x < x_hi && ok; ++sg) {
                const int unit = (int)(x / tiles), t0 = (int)(x % tiles);
                const int n = (int)min((int64_t)(tiles - t0), x_hi - x);
                const int hk = unit % p.Hkv, b = unit / p.Hkv;
                int j_first = 0;
                if (!waited) {
                    // the ring is empty: up to NSTAGE tiles go out before the wait
                    for (; j_first < n && j_first < NSTAGE; ++j_first, ++it) {
                        unsigned char *kt = stages + (size_t)it * 2 * TILE_BYTES;
                        unsigned char *vt = kt + TILE_BYTES;
                        mbar_expect_tx(&full[it], 2 * TILE_BYTES);
                        const int tok = (t0 + j_first) * TILE_T;
#pragma unroll
                        for (int bx = 0; bx < BOXES; ++bx) {
                            tma_load_4d(kt + bx * BOX_BYTES, &kmap, &full[it], bx * 64, tok, hk, b);
                            tma_load_4d(vt + bx * BOX_BYTES, &vmap, &full[it], bx * 64, tok, hk, b);
                        }
                    }
                    pdl_wait();
                    pdl_trigger();
                    waited = true;
                }
                if (p.q_bulk) {
                    const int qb = sg & 1;
                    if (sg >= 2) ok = mbar_wait(&qempty[qb], ((sg >> 1) - 1) & 1);
                    if (!ok) break;
                    mbar_expect_tx(&qfull[qb], q_bytes);
                    bulk_load(qbuf + (size_t)qb * q_bytes, (const T *)p.q + b * p.q_sb + (int64_t)hk * rep * p.q_sh, q_bytes,
                              &qfull[qb]);
                }
                for (int j = j_first; j < n && ok; ++j, ++it) {
                    const int s = it % NSTAGE;
                    if (it >= NSTAGE) {
                        // measurement aid (debug_skip & 4): the producer alone recycles the ring
                        if (KVC_SKIP_BITS(p) & 4) ok = mbar_wait(&full[s], ((it / NSTAGE) - 1) & 1);
                        else ok = mbar_wait(&empty[s], ((it / NSTAGE) - 1) & 1);
                    }
                    if (!ok) break;
                    unsigned char *kt = stages + (size_t)s * 2 * TILE_BYTES;
                    unsigned char *vt = kt + TILE_BYTES;
                    mbar_expect_tx(&full[s], 2 * TILE_BYTES);
                    const int tok = (t0 + j) * TILE_T;
                    if (KVC_SKIP_BITS(p) & 2) {
                        const int64_t off = b * p.kv_sb + hk * p.kv_sh + (int64_t)tok * p.kv_st;
                        bulk_load(kt, p.k_base + off, TILE_BYTES, &full[s]);
                        bulk_load(vt, p.v_base + off, TILE_BYTES, &full[s]);
                        continue;
                    }
#pragma unroll
                    for (int bx = 0; bx < BOXES; ++bx) {
                        tma_load_4d(kt + bx * BOX_BYTES, &kmap, &full[s], bx * 64, tok, hk, b);
                        tma_load_4d(vt + bx * BOX_BYTES, &vmap, &full[s], bx * 64, tok, hk, b);
                    }
                }
                x += n;
            }
            if (!ok) atomicExch(p.status, 9);
        }
        return;
    }

    // ---------------- consumers ----------------
    if (KVC_SKIP_BITS(p) & 8) return;  // measurement aid: no consumer work at all (with 4: producer-only streaming)
    const int g = lane >> 2, c = lane & 3;
    // Fused append: token T - 1 is not in the cache yet; the tiles are masked up to T - 2 and the
    // new row is scored from its source by warp 0 of the CTA that owns the unit's last tile.
    const bool fused = p.new_k != nullptr;
    // Appending at the end: the tiles are simply cut one token short. Replacing a row inside a
    // wrapped ring: every token is visible except that slot, which still holds the row it loses.
    const bool ring = fused && p.new_slot != p.T - 1;
    const int64_t t_cached = p.T - ((fused && !ring) ? 2 : 1);
    const int64_t hole = ring ? p.new_slot : -1;
    int64_t row_limit[2];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = g + 8 * half;
        const int l = r % p.L;
        row_limit[half] = (r < R) ? (p.causal ? min(t_cached, p.causal_offset + l) : t_cached) : -1;
    }
    const int blk = warp;
    uint32_t k_off[2];
#pragma unroll
    for (int ps = 0; ps < 2; ++ps) k_off[ps] = (uint32_t)((blk * 16 + g) * 128 + (((2 * c + ps) ^ g) << 4));
    uint32_t v_off[4];
    {
        const int mi = lane >> 3, rr = lane & 7;
#pragma unroll
        for (int cp = 0; cp < 4; ++cp)
            v_off[cp] = (uint32_t)((blk * 16 + (mi & 1) * 8 + rr) * 128 + (((2 * cp + (mi >> 1)) ^ rr) << 4));
    }

    int it = 0, sg = 0;
    for (int64_t x = x_lo; x < x_hi; ++sg) {
        const int unit = (int)(x / tiles), t0 = (int)(x % tiles);
        const int n = (int)min((int64_t)(tiles - t0), x_hi - x);
        const int hk = unit % p.Hkv, b = unit / p.Hkv;

        if (fused && warp == 0 && t0 + n == tiles && lane < 4) {
            // the new rows are consumed at the end of the segment: pull them towards L2 now
            const char *kn = (const char *)((const T *)p.new_k + b * p.nk_sb + hk * p.nk_sh);
            const char *vn = (const char *)((const T *)p.new_v + b * p.nv_sb + hk * p.nv_sh);
            const char *line = ((lane & 1) ? vn : kn) + (lane >> 1) * 128;
            if ((lane >> 1) * 128 < D * 2) asm volatile("prefetch.global.L2 [%0];" ::"l"(line));
        }
        uint32_t qa[KSTEPS][4];
        if (p.q_bulk) {
            const int qb = sg & 1;
            if (ok) {
                ok = mbar_wait(&qfull[qb], (sg >> 1) & 1);
                if (!ok && lane == 0) atomicExch(p.status, 13);
            }
            const unsigned char *qs = qbuf + (size_t)qb * q_bytes;
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
                const int bx = ks / 4, ps = (ks >> 1) & 1, h = ks & 1;
                const int d0 = bx * 64 + (2 * c + ps) * 8 + 4 * h;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int r = g + 8 * half;
                    uint2 w = make_uint2(0u, 0u);
                    if (r < R && ok) w = *(const uint2 *)(qs + ((size_t)r * D + d0) * 2);
                    qa[ks][half] = w.x;
                    qa[ks][2 + half] = w.y;
                }
            }
            __syncwarp();
            if (ok && lane == 0) mbar_arrive(&qempty[qb]);
        } else
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            const int bx = ks / 4, ps = (ks >> 1) & 1, h = ks & 1;
            const int d0 = bx * 64 + (2 * c + ps) * 8 + 4 * h;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int r = g + 8 * half;
                uint32_t w0 = 0, w1 = 0;
                if (r < R && !(KVC_SKIP_BITS(p) & 32)) {
                    const int hq = hk * rep + r / p.L, l = r % p.L;
                    const T *qp = (const T *)p.q + b * p.q_sb + hq * p.q_sh + l * p.q_sl + d0;
                    w0 = *(const uint32_t *)qp;
                    w1 = *(const uint32_t *)(qp + 2);
                }
                qa[ks][half] = w0;
                qa[ks][2 + half] = w1;
            }
        }
        float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
        float o_acc[NT_O][4];
#pragma unroll
        for (int i = 0; i < NT_O; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;

        for (int j = 0; j < n; ++j, ++it) {
            if (!ok || (KVC_SKIP_BITS(p) & 4)) continue;  // a wait ran out earlier: walk on to the barriers below
            const int s = it % NSTAGE;
            ok = mbar_wait(&full[s], (it / NSTAGE) & 1);
            if (!ok) {
                if (lane == 0) atomicExch(p.status, 10);
                continue;
            }
            if (KVC_SKIP_BITS(p) & 1) {
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
                continue;
            }
            const unsigned char *kt = stages + (size_t)s * 2 * TILE_BYTES;
            const uint32_t vt_addr = smem_u32(kt + TILE_BYTES);
            const int64_t t_blk = (int64_t)(t0 + j) * TILE_T + blk * 16;

            float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int bx = 0; bx < BOXES; ++bx) {
#pragma unroll
                for (int ps = 0; ps < 2; ++ps) {
                    const uint4 k0 = *(const uint4 *)(kt + bx * BOX_BYTES + k_off[ps]);
                    const uint4 k1 = *(const uint4 *)(kt + bx * BOX_BYTES + k_off[ps] + 8 * 128);
                    const int ks = bx * 4 + ps * 2;
                    MmaType<T>::mma(sc[0], qa[ks], k0.x, k0.y);
                    MmaType<T>::mma(sc[1], qa[ks], k1.x, k1.y);
                    MmaType<T>::mma(sc[0], qa[ks + 1], k0.z, k0.w);
                    MmaType<T>::mma(sc[1], qa[ks + 1], k1.z, k1.w);
                }
            }
            float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int half = e >> 1;
                    const int64_t t = t_blk + jj * 8 + 2 * c + (e & 1);
                    float v = sc[jj][e] * p.scale_log2;
                    v = (t <= row_limit[half] && t != hole) ? v : -INFINITY;
                    sc[jj][e] = v;
                    tmax[half] = fmaxf(tmax[half], v);
                }
            }
            float alpha[2];
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                tmax[half] = fmaxf(tmax[half], __shfl_xor_sync(0xffffffffu, tmax[half], 1));
                tmax[half] = fmaxf(tmax[half], __shfl_xor_sync(0xffffffffu, tmax[half], 2));
                const float m_new = fmaxf(m_run[half], tmax[half]);
                alpha[half] = (m_new == -INFINITY) ? 1.f : fast_exp2(m_run[half] - m_new);
                m_run[half] = m_new;
            }
            uint32_t pa[4];
            {
                float pr[2][4];
#pragma unroll
                for (int jj = 0; jj < 2; ++jj)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int half = e >> 1;
                        pr[jj][e] = (m_run[half] == -INFINITY) ? 0.f : fast_exp2(sc[jj][e] - m_run[half]);
                    }
#pragma unroll
                for (int half = 0; half < 2; ++half)
                    l_run[half] = l_run[half] * alpha[half] + pr[0][2 * half] + pr[0][2 * half + 1] +
                                  pr[1][2 * half] + pr[1][2 * half + 1];
                pa[0] = MmaType<T>::pack(pr[0][0], pr[0][1]);
                pa[1] = MmaType<T>::pack(pr[0][2], pr[0][3]);
                pa[2] = MmaType<T>::pack(pr[1][0], pr[1][1]);
                pa[3] = MmaType<T>::pack(pr[1][2], pr[1][3]);
            }
            if (__any_sync(0xffffffffu, (alpha[0] != 1.f) | (alpha[1] != 1.f))) {
#pragma unroll
                for (int nt = 0; nt < NT_O; ++nt) {
                    o_acc[nt][0] *= alpha[0];
                    o_acc[nt][1] *= alpha[0];
                    o_acc[nt][2] *= alpha[1];
                    o_acc[nt][3] *= alpha[1];
                }
            }
#pragma unroll
            for (int bx = 0; bx < BOXES; ++bx) {
#pragma unroll
                for (int cp = 0; cp < 4; ++cp) {
                    uint32_t vf[4];
                    ldmatrix_x4_trans(vf, vt_addr + bx * BOX_BYTES + v_off[cp]);
                    MmaType<T>::mma(o_acc[bx * 8 + 2 * cp], pa, vf[0], vf[1]);
                    MmaType<T>::mma(o_acc[bx * 8 + 2 * cp + 1], pa, vf[2], vf[3]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }

        if (fused && warp == 0 && t0 + n == tiles && !(KVC_SKIP_BITS(p) & 32)) {
            // ---- the step's new token: score q . k_new, fold it into this warp's state, store the rows ----
            const T *kn = (const T *)p.new_k + b * p.nk_sb + hk * p.nk_sh;
            const T *vn = (const T *)p.new_v + b * p.nv_sb + hk * p.nv_sh;
            float dot[2] = {0.f, 0.f};
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
                const int bx = ks / 4, ps = (ks >> 1) & 1, h = ks & 1;
                const int d0 = bx * 64 + (2 * c + ps) * 8 + 4 * h;
                const uint2 kw = *(const uint2 *)(kn + d0);
                const float2 k01 = MmaType<T>::unpack(kw.x), k23 = MmaType<T>::unpack(kw.y);
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const float2 q01 = MmaType<T>::unpack(qa[ks][half]), q23 = MmaType<T>::unpack(qa[ks][2 + half]);
                    dot[half] += q01.x * k01.x + q01.y * k01.y + q23.x * k23.x + q23.y * k23.y;
                }
            }
            float pn[2], alpha[2];
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                dot[half] += __shfl_xor_sync(0xffffffffu, dot[half], 1);
                dot[half] += __shfl_xor_sync(0xffffffffu, dot[half], 2);
                const float sc_new = (g + 8 * half < R) ? dot[half] * p.scale_log2 : -INFINITY;
                const float m_new = fmaxf(m_run[half], sc_new);
                alpha[half] = (m_new == -INFINITY) ? 1.f : fast_exp2(m_run[half] - m_new);
                pn[half] = (m_new == -INFINITY) ? 0.f : fast_exp2(sc_new - m_new);
                m_run[half] = m_new;
                l_run[half] = l_run[half] * alpha[half] + (c == 0 ? pn[half] : 0.f);  // once per row
            }
#pragma unroll
            for (int nt = 0; nt < NT_O; ++nt) {
                const float2 vv = MmaType<T>::unpack(*(const uint32_t *)(vn + 8 * nt + 2 * c));
                o_acc[nt][0] = o_acc[nt][0] * alpha[0] + pn[0] * vv.x;
                o_acc[nt][1] = o_acc[nt][1] * alpha[0] + pn[0] * vv.y;
                o_acc[nt][2] = o_acc[nt][2] * alpha[1] + pn[1] * vv.x;
                o_acc[nt][3] = o_acc[nt][3] * alpha[1] + pn[1] * vv.y;
            }
            // the append itself: rows of D elements, 16 bytes per lane
            const int64_t row_off = b * p.kv_sb + hk * p.kv_sh + p.new_slot * p.kv_st;
            constexpr int CHUNKS = D * 2 / 16;
            for (int i = lane; i < 2 * CHUNKS; i += 32) {
                const bool is_v = i >= CHUNKS;
                const int ch = is_v ? i - CHUNKS : i;
                const uint4 x = *(const uint4 *)((const unsigned char *)(is_v ? vn : kn) + ch * 16);
                *(uint4 *)((is_v ? p.v_base : p.k_base) + row_off + ch * 16) = x;
            }
        }

        // ---- end of the segment: merge the four warps, publish the partial, maybe merge the unit ----
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            l_run[half] += __shfl_xor_sync(0xffffffffu, l_run[half], 1);
            l_run[half] += __shfl_xor_sync(0xffffffffu, l_run[half], 2);
        }
        {
            float *wo = red_o + warp * fp.red_rows * RED_STRIDE;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int r = g + 8 * half;
                if (r >= R) continue;
#pragma unroll
                for (int nt = 0; nt < NT_O; ++nt)
                    *(float2 *)&wo[r * RED_STRIDE + 8 * nt + 2 * c] = make_float2(o_acc[nt][2 * half], o_acc[nt][2 * half + 1]);
                if (c == 0) {
                    red_ml[(warp * fp.red_rows + r) * 2 + 0] = m_run[half];
                    red_ml[(warp * fp.red_rows + r) * 2 + 1] = l_run[half];
                }
            }
        }
        UnitOut u;
        u.o_part = p.o_part; u.ml_part = p.ml_part; u.counters = p.counters;
        u.out = p.out; u.out_dtype = p.out_dtype;
        u.o_sb = p.o_sb; u.o_sh = p.o_sh; u.o_sl = p.o_sl;
        u.o_signs = nullptr;
        u.splits = 0; u.Hq = p.Hq; u.L = p.L;
        if (!(KVC_SKIP_BITS(p) & 16))
            segment_epilogue<D, CONSUMER_WARPS>(u, fp, red_o, red_ml, RED_STRIDE, work, is_last, unit, b, hk, rep, R);
        x += n;
    }
}

// ---------------------------------------------------------------------
// Multi-token chunks (prefill chunks, speculative verify rounds): more than 16 query
// rows per KV head. Same ring, tiles and fragment layouts as above, but the consumer
// warps split the QUERY ROWS instead of the tokens: a CTA owns a block of 64 rows of one
// (batch, KV head) group (row r <-> head r / L of the group, position r % L), warp w owns
// rows 16w .. 16w+15 with their own softmax state and output accumulators, and every
// warp walks all four 16-token blocks of each tile. Under a causal mask a CTA only
// streams the tiles some row of its block can see. With one split per block the rows are
// normalised and written straight to the output; otherwise partials go to scratch and the
// last CTA of the block merges them.
// ---------------------------------------------------------------------
template <typename T, int D, int NSTAGE>
__global__ void __launch_bounds__(DEC_THREADS, (D <= 128 ? 2 : 1))
attn_chunk_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                  const DecodeParams p) {
    constexpr int TILE_BYTES = TILE_T * D * 2;
    constexpr int BOXES = D / 64;
    constexpr int KSTEPS = D / 16;
    constexpr int NT_O = D / 8;

    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *stages = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint64_t *full = (uint64_t *)(stages + (size_t)NSTAGE * 2 * TILE_BYTES);
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

    // tiles some row of the block can see, then this split's share of them
    int tiles_needed = p.tiles_all;
    if (p.causal) {
        const int max_l = (r_lo / p.L == r_hi / p.L) ? (r_hi % p.L) : (p.L - 1);
        const int64_t lim = min(p.T - 1, p.causal_offset + max_l);
        tiles_needed = (int)min((int64_t)p.tiles_all, lim / TILE_T + 1);
    }
    const int t_base = tiles_needed / p.splits, t_rem = tiles_needed % p.splits;
    const int tile_begin = split * t_base + min(split, t_rem);
    const int ntiles = t_base + (split < t_rem ? 1 : 0);

    if (tid == 0) {
        for (int s = 0; s < NSTAGE; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], CONSUMER_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    pdl_wait();  // everything below reads what earlier kernels on the stream wrote

    bool ok = true;
    const int g = lane >> 2, c = lane & 3;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o_acc[NT_O][4];
#pragma unroll
    for (int i = 0; i < NT_O; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;

    if (warp == CONSUMER_WARPS) {
        if (lane == 0) {
            for (int it = 0; it < ntiles && ok; ++it) {
                const int s = it % NSTAGE;
                if (it >= NSTAGE) ok = mbar_wait(&empty[s], ((it / NSTAGE) - 1) & 1);
                if (!ok) break;
                unsigned char *kt = stages + (size_t)s * 2 * TILE_BYTES;
                unsigned char *vt = kt + TILE_BYTES;
                mbar_expect_tx(&full[s], 2 * TILE_BYTES);
                const int t0 = (tile_begin + it) * TILE_T;
#pragma unroll
                for (int bx = 0; bx < BOXES; ++bx) {
                    tma_load_4d(kt + bx * BOX_BYTES, &kmap, &full[s], bx * 64, t0, hk, b);
                    tma_load_4d(vt + bx * BOX_BYTES, &vmap, &full[s], bx * 64, t0, hk, b);
                }
            }
            if (!ok) atomicExch(p.status, 3);
        }
    } else {
        const int r_warp = r_lo + 16 * warp;
        uint32_t qa[KSTEPS][4];
        int row_limit[2];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = r_warp + g + 8 * half;
            const int l = r % p.L;
            row_limit[half] = (r < R) ? (int)(p.causal ? min(p.T - 1, p.causal_offset + l) : p.T - 1) : -1;
        }
        // the warp's widest and narrowest limits (rows past R excluded from the narrowest)
        int lim_max = max(row_limit[0], row_limit[1]);
        int lim_min = min(row_limit[0] < 0 ? 0x7fffffff : row_limit[0], row_limit[1] < 0 ? 0x7fffffff : row_limit[1]);
#pragma unroll
        for (int o = 4; o <= 16; o <<= 1) {
            lim_max = max(lim_max, __shfl_xor_sync(0xffffffffu, lim_max, o));
            lim_min = min(lim_min, __shfl_xor_sync(0xffffffffu, lim_min, o));
        }
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            const int bx = ks / 4, ps = (ks >> 1) & 1, h = ks & 1;
            const int d0 = bx * 64 + (2 * c + ps) * 8 + 4 * h;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int r = r_warp + g + 8 * half;
                uint32_t w0 = 0, w1 = 0;
                if (r < R) {
                    const int hq = hk * rep + r / p.L, l = r % p.L;
                    const T *qp = (const T *)p.q + b * p.q_sb + hq * p.q_sh + l * p.q_sl + d0;
                    w0 = *(const uint32_t *)qp;
                    w1 = *(const uint32_t *)(qp + 2);
                }
                qa[ks][half] = w0;
                qa[ks][2 + half] = w1;
            }
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

        for (int it = 0; it < ntiles && ok; ++it) {
            const int s = it % NSTAGE;
            ok = mbar_wait(&full[s], (it / NSTAGE) & 1);
            if (!ok) break;
            const unsigned char *kt = stages + (size_t)s * 2 * TILE_BYTES;
            const uint32_t vt_addr = smem_u32(kt + TILE_BYTES);
#pragma unroll 1
            for (int blk = 0; blk < 4; ++blk) {
                const int t_blk = (tile_begin + it) * TILE_T + blk * 16;
                if (t_blk > lim_max) break;  // warp-uniform: nothing further in this tile is visible
                const uint32_t boff = blk * 16 * 128;
                float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
                for (int bx = 0; bx < BOXES; ++bx) {
#pragma unroll
                    for (int ps = 0; ps < 2; ++ps) {
                        const uint4 k0 = *(const uint4 *)(kt + bx * BOX_BYTES + boff + k_off[ps]);
                        const uint4 k1 = *(const uint4 *)(kt + bx * BOX_BYTES + boff + k_off[ps] + 8 * 128);
                        const int ks = bx * 4 + ps * 2;
                        MmaType<T>::mma(sc[0], qa[ks], k0.x, k0.y);
                        MmaType<T>::mma(sc[1], qa[ks], k1.x, k1.y);
                        MmaType<T>::mma(sc[0], qa[ks + 1], k0.z, k0.w);
                        MmaType<T>::mma(sc[1], qa[ks + 1], k1.z, k1.w);
                    }
                }
                const bool edge = t_blk + 15 > lim_min;  // warp-uniform
                float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int j = 0; j < 2; ++j) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int half = e >> 1;
                        float v = sc[j][e] * p.scale_log2;
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
                    const float m_new = fmaxf(m_run[half], tmax[half]);
                    alpha[half] = (m_new == -INFINITY) ? 1.f : fast_exp2(m_run[half] - m_new);
                    m_run[half] = m_new;
                }
                uint32_t pa[4];
                {
                    float pr[2][4];
#pragma unroll
                    for (int j = 0; j < 2; ++j)
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int half = e >> 1;
                            pr[j][e] = (m_run[half] == -INFINITY) ? 0.f : fast_exp2(sc[j][e] - m_run[half]);
                        }
#pragma unroll
                    for (int half = 0; half < 2; ++half)
                        l_run[half] = l_run[half] * alpha[half] + pr[0][2 * half] + pr[0][2 * half + 1] +
                                      pr[1][2 * half] + pr[1][2 * half + 1];
                    pa[0] = MmaType<T>::pack(pr[0][0], pr[0][1]);
                    pa[1] = MmaType<T>::pack(pr[0][2], pr[0][3]);
                    pa[2] = MmaType<T>::pack(pr[1][0], pr[1][1]);
                    pa[3] = MmaType<T>::pack(pr[1][2], pr[1][3]);
                }
                if (__any_sync(0xffffffffu, (alpha[0] != 1.f) | (alpha[1] != 1.f))) {
#pragma unroll
                    for (int nt = 0; nt < NT_O; ++nt) {
                        o_acc[nt][0] *= alpha[0];
                        o_acc[nt][1] *= alpha[0];
                        o_acc[nt][2] *= alpha[1];
                        o_acc[nt][3] *= alpha[1];
                    }
                }
#pragma unroll
                for (int bx = 0; bx < BOXES; ++bx) {
#pragma unroll
                    for (int cp = 0; cp < 4; ++cp) {
                        uint32_t vf[4];
                        ldmatrix_x4_trans(vf, vt_addr + bx * BOX_BYTES + boff + v_off[cp]);
                        MmaType<T>::mma(o_acc[bx * 8 + 2 * cp], pa, vf[0], vf[1]);
                        MmaType<T>::mma(o_acc[bx * 8 + 2 * cp + 1], pa, vf[2], vf[3]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }
        if (!ok && lane == 0) atomicExch(p.status, 4);

        // ---- the warp's 16 rows: straight to the output, or partials for the merge ----
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            l_run[half] += __shfl_xor_sync(0xffffffffu, l_run[half], 1);
            l_run[half] += __shfl_xor_sync(0xffffffffu, l_run[half], 2);
        }
        const int64_t qrow0 = ((int64_t)b * p.Hq + hk * rep) * p.L;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = r_warp + g + 8 * half;
            if (r >= R) continue;
            if (p.splits == 1) {
                const float inv = l_run[half] > 0.f ? 1.f / l_run[half] : 0.f;
                const int hq = hk * rep + r / p.L, lq = r % p.L;
                const int64_t base = b * p.o_sb + hq * p.o_sh + lq * p.o_sl;
#pragma unroll
                for (int nt = 0; nt < NT_O; ++nt) {
                    store_out(p.out, p.out_dtype, base + 8 * nt + 2 * c, o_acc[nt][2 * half] * inv);
                    store_out(p.out, p.out_dtype, base + 8 * nt + 2 * c + 1, o_acc[nt][2 * half + 1] * inv);
                }
            } else {
                const int64_t pbase = (qrow0 + r) * p.splits + split;
#pragma unroll
                for (int nt = 0; nt < NT_O; ++nt)
                    __stcg((float2 *)&p.o_part[pbase * D + 8 * nt + 2 * c],
                           make_float2(o_acc[nt][2 * half], o_acc[nt][2 * half + 1]));
                if (c == 0) __stcg(&p.ml_part[pbase], make_float2(m_run[half], l_run[half]));
            }
        }
    }
    if (p.splits == 1) return;

    // ---- split merge by the last CTA of this row block ----
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const int ticket = atomicAdd(&p.counters[unit], 1);
        const int last = (ticket == p.splits - 1) ? 1 : 0;
        if (last) p.counters[unit] = 0;
        *is_last = last;
    }
    __syncthreads();
    if (!*is_last) return;
    __threadfence();
    float *work = (float *)stages;  // [rows of the block][splits] merge weights (the ring is idle)
    const int64_t qrow0 = ((int64_t)b * p.Hq + hk * rep) * p.L;
    const int nrows = r_hi - r_lo + 1;
    for (int rr = warp; rr < nrows; rr += DEC_THREADS / 32) {
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
    __syncthreads();
    for (int i = tid; i < nrows * D; i += DEC_THREADS) {
        const int rr = i / D, d = i % D;
        const int r = r_lo + rr;
        float o = 0.f;
        const float *src = p.o_part + ((qrow0 + r) * p.splits) * D + d;
        for (int s = 0; s < p.splits; ++s) o = fmaf(__ldcg(src + (int64_t)s * D), work[rr * p.splits + s], o);
        const int hq = hk * rep + r / p.L, lq = r % p.L;
        store_out(p.out, p.out_dtype, b * p.o_sb + hq * p.o_sh + lq * p.o_sl + d, o);
    }
}

// ---------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
        if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) fn = (EncodeTiledFn)p;
        else (void)cudaGetLastError();
    });
    return fn;
}

bool make_map(CUtensorMap *map, const KVSource &s, int D, int64_t T, int Hkv, int B) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return false;
    const cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)T, (cuuint64_t)Hkv, (cuuint64_t)B};
    const cuuint64_t strides[3] = {(cuuint64_t)s.st * 2, (cuuint64_t)(Hkv > 1 ? s.sh : s.st * T) * 2,
                                   (cuuint64_t)(B > 1 ? s.sb : (Hkv > 1 ? s.sh * Hkv : s.st * T)) * 2};
    const cuuint32_t box[4] = {64, (cuuint32_t)TILE_T, 1, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUtensorMapDataType dt = s.dtype == KVC_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUresult r = fn(map, dt, 4, const_cast<void *>(s.data), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

bool source_fits(const KVSource &s, int D, int Hkv, int B) {
    if (s.kind != SRC_RAW || (s.dtype != KVC_BF16 && s.dtype != KVC_F16)) return false;
    if (((uintptr_t)s.data & 15) != 0) return false;
    auto ok = [](int64_t st) { return st > 0 && (st * 2) % 16 == 0; };
    if (!ok(s.st) || s.st < D) return false;
    if (Hkv > 1 && !ok(s.sh)) return false;
    if (B > 1 && !ok(s.sb)) return false;
    return true;
}

template <typename T, int D, int NSTAGE>
void launch_typed(const CUtensorMap &kmap, const CUtensorMap &vmap, const DecodeParams &p, int units,
                  cudaStream_t stream) {
    const size_t smem = (size_t)NSTAGE * 2 * (TILE_T * D * 2) + 2 * NSTAGE * sizeof(uint64_t) + 64 + 1024;
    static bool configured[64] = {false};
    const int dev = current_device();
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        KVC_CUDA(cudaFuncSetAttribute(attn_decode_kernel<T, D, NSTAGE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)smem));
        KVC_CUDA(cudaFuncSetAttribute(attn_decode_kernel<T, D, NSTAGE>,
                                      cudaFuncAttributePreferredSharedMemoryCarveout, 100));
        configured[dev] = true;
    }
    KernelTimer timer(stream);
    KVC_CUDA(launch_pdl(attn_decode_kernel<T, D, NSTAGE>, dim3(units), dim3(DEC_THREADS), smem, stream, kmap, vmap, p));
    timer.stop();
    KVC_CUDA(cudaGetLastError());
    ++g_launch_count;
}

template <typename T, int D, int NSTAGE>
void launch_flat_typed(const CUtensorMap &kmap, const CUtensorMap &vmap, const DecodeParams &p, int ctas, size_t smem,
                       cudaStream_t stream) {
    static size_t configured[64] = {0};
    const int dev = current_device();
    if (dev >= 0 && dev < 64 && configured[dev] < smem) {
        KVC_CUDA(cudaFuncSetAttribute(attn_decode_flat_kernel<T, D, NSTAGE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)smem));
        KVC_CUDA(cudaFuncSetAttribute(attn_decode_flat_kernel<T, D, NSTAGE>,
                                      cudaFuncAttributePreferredSharedMemoryCarveout, 100));
        configured[dev] = smem;
    }
    KernelTimer timer(stream);
    KVC_CUDA(launch_pdl(attn_decode_flat_kernel<T, D, NSTAGE>, dim3(ctas), dim3(DEC_THREADS), smem, stream, kmap, vmap, p));
    timer.stop();
    KVC_CUDA(cudaGetLastError());
    ++g_launch_count;
}

template <typename T, int D, int NSTAGE>
void launch_chunk_typed(const CUtensorMap &kmap, const CUtensorMap &vmap, const DecodeParams &p, int ctas,
                        cudaStream_t stream) {
    const size_t smem = (size_t)NSTAGE * 2 * (TILE_T * D * 2) + 2 * NSTAGE * sizeof(uint64_t) + 64 + 1024;
    static bool configured[64] = {false};
    const int dev = current_device();
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        KVC_CUDA(cudaFuncSetAttribute(attn_chunk_kernel<T, D, NSTAGE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)smem));
        KVC_CUDA(cudaFuncSetAttribute(attn_chunk_kernel<T, D, NSTAGE>,
                                      cudaFuncAttributePreferredSharedMemoryCarveout, 100));
        configured[dev] = true;
    }
    KernelTimer timer(stream);
    KVC_CUDA(launch_pdl(attn_chunk_kernel<T, D, NSTAGE>, dim3(ctas), dim3(DEC_THREADS), smem, stream, kmap, vmap, p));
    timer.stop();
    KVC_CUDA(cudaGetLastError());
    ++g_launch_count;
}

}  // namespace

// Returns the number of kernels launched, or 0 when the call does not fit this path.
int launch_attention_decode(const AttnArgs &a, cudaStream_t stream) {
    if (a.q_dtype != KVC_BF16 && a.q_dtype != KVC_F16) return 0;
    if (a.D != 64 && a.D != 128 && a.D != 256) return 0;
    if (a.k.dtype != a.q_dtype || a.v.dtype != a.q_dtype) return 0;
    if (a.mask.mode == KVC_MASK_ARRAY) return 0;
    if (a.q_signs || a.o_signs || a.q_calib) return 0;
    if (a.Hkv <= 0 || a.Hq % a.Hkv) return 0;
    const int rep = a.Hq / a.Hkv;
    if (a.T < 1 || a.T > (int64_t)1 << 30) return 0;
    if (!source_fits(a.k, a.D, a.Hkv, a.B) || !source_fits(a.v, a.D, a.Hkv, a.B)) return 0;
    if (((uintptr_t)a.q & 3) || (a.q_sb & 1) || (a.q_sh & 1) || (a.q_sl & 1)) return 0;
    const int64_t bh = (int64_t)a.B * a.Hkv;
    const bool chunk = rep * a.L > 16;  // more rows than one MMA row block: rows split across warps
    const int64_t row_blocks = chunk ? ((int64_t)rep * a.L + 63) / 64 : 1;
    if (bh * row_blocks * (int64_t)sizeof(int) > COUNTER_BYTES) return 0;
    if (chunk && (int64_t)rep * a.L > (int64_t)1 << 24) return 0;

    CUtensorMap kmap, vmap;
    if (!make_map(&kmap, a.k, a.D, a.T, a.Hkv, a.B) || !make_map(&vmap, a.v, a.D, a.T, a.Hkv, a.B)) return 0;
    int *status = device_status_word(a.device);
    int *counters = counters_get(a.device, stream, COUNTER_BYTES);
    if (!status || !counters) return 0;

    const int64_t tiles = (a.T + TILE_T - 1) / TILE_T;
    const int slots = sm_count(a.device) * (a.D <= 128 ? 2 : 1);

    // Decode (one MMA row block): flat decomposition over one wave of CTAs when its cross-warp
    // buffer fits beside the ring; KVC_DECODE_FLAT=0 keeps the per-unit split kernel.
    if (!chunk) {
        static const bool flat_off = [] {
            const char *e = std::getenv("KVC_DECODE_FLAT");
            return e && e[0] == '0';
        }();
        const int R = rep * a.L;
        const int64_t work = bh * tiles;
        const int64_t ctas = std::min<int64_t>(slots, work);
        const int64_t per = work / ctas, rem = work % ctas;
        const int64_t nslots = (tiles + per - 1) / per + 1;
        const int nstage = a.D == 64 ? 6 : 3;
        const size_t ring = (size_t)nstage * 2 * (TILE_T * a.D * 2);
        const size_t red = (size_t)CONSUMER_WARPS * R * (a.D + 8) * 4 + (size_t)CONSUMER_WARPS * R * 8 + (size_t)R * nslots * 4 +
                           16 + 4 * sizeof(uint64_t) + (size_t)2 * R * a.D * 2;
        const size_t smem = ring + 2 * nstage * sizeof(uint64_t) + 64 + red + 1024;
        const size_t budget = (a.D <= 128 ? 112 : 224) * 1024;
        const bool fused_ok = !a.new_k || (a.L == 1 && a.mask.mode != KVC_MASK_CAUSAL && !((uintptr_t)a.new_k & 15) &&
                                           !((uintptr_t)a.new_v & 15) && (a.nk_sb * 2) % 16 == 0 && (a.nk_sh * 2) % 16 == 0 &&
                                           (a.nv_sb * 2) % 16 == 0 && (a.nv_sh * 2) % 16 == 0);
        if (!flat_off && smem <= budget && nslots <= 64 && fused_ok) {
            const int64_t qrows_f = (int64_t)a.B * a.Hq * a.L;
            const size_t o_bytes_f = (size_t)qrows_f * nslots * a.D * sizeof(float);
            const size_t ml_bytes_f = (size_t)qrows_f * nslots * sizeof(float2);
            char *scratch_f = (char *)scratch_get(a.device, o_bytes_f + ml_bytes_f + 256, stream);
            DecodeParams p = {};
            p.q = a.q; p.out = a.out; p.out_dtype = a.q_dtype;
            p.q_sb = a.q_sb; p.q_sh = a.q_sh; p.q_sl = a.q_sl;
            p.o_sb = a.o_sb; p.o_sh = a.o_sh; p.o_sl = a.o_sl;
            p.o_part = (float *)scratch_f;
            p.ml_part = (float2 *)(scratch_f + ((o_bytes_f + 255) / 256) * 256);
            p.counters = counters; p.status = status;
            p.B = a.B; p.Hq = a.Hq; p.Hkv = a.Hkv; p.L = a.L; p.T = a.T;
            p.splits = 1; p.tiles_base = 0; p.tiles_rem = 0; p.row_blocks = 1;
            p.causal = a.mask.mode == KVC_MASK_CAUSAL ? 1 : 0;
            p.debug_skip = measure_skip_bits();
            p.k_base = (unsigned char *)a.k.data; p.v_base = (unsigned char *)a.v.data;
            p.kv_sb = a.k.sb * 2; p.kv_sh = a.k.sh * 2; p.kv_st = a.k.st * 2;
            p.new_k = a.new_k; p.new_v = a.new_v;
            p.new_slot = (a.new_slot >= 0 && a.new_slot < a.T) ? a.new_slot : a.T - 1;
            {
                // early tiles: fused append only (the kernel's tiles end before the row it writes), the
                // caller's word on the preceding launch, and that launch being a kernel that released
                // this one only after its own wait. KVC_EARLY_TILES=0 turns it off.
                static const bool early_off = [] {
                    const char *e = std::getenv("KVC_EARLY_TILES");
                    return e && e[0] == '0';
                }();
                p.early_tiles = (!early_off && a.new_k && a.stored_rows_settled && g_last_chained_launch == g_launch_count &&
                                 KVC_SKIP_BITS(p) == 0) ? 1 : 0;
            }
            p.nk_sb = a.nk_sb; p.nk_sh = a.nk_sh; p.nv_sb = a.nv_sb; p.nv_sh = a.nv_sh;
            p.causal_offset = a.mask.causal_offset;
            p.scale_log2 = a.scale * 1.4426950408889634f;
            p.tiles_all = (int)tiles;
            p.flat.tiles = (int)tiles;
            p.flat.per = (int)per; p.flat.rem = (int)rem;
            p.flat.nslots = (int)nslots; p.flat.red_rows = R;
            p.q_bulk = (a.L == 1 && a.q_sh == a.D && ((uintptr_t)a.q & 15) == 0 && (a.q_sb * 2) % 16 == 0) ? 1 : 0;
#define KVC_FLAT(TT, DD, NS) launch_flat_typed<TT, DD, NS>(kmap, vmap, p, (int)ctas, smem, stream)
            if (a.q_dtype == KVC_BF16) {
                if (a.D == 64) KVC_FLAT(__nv_bfloat16, 64, 6);
                else if (a.D == 128) KVC_FLAT(__nv_bfloat16, 128, 3);
                else KVC_FLAT(__nv_bfloat16, 256, 3);
            } else {
                if (a.D == 64) KVC_FLAT(__half, 64, 6);
                else if (a.D == 128) KVC_FLAT(__half, 128, 3);
                else KVC_FLAT(__half, 256, 3);
            }
#undef KVC_FLAT
            g_last_chained_launch = g_launch_count;
            return 1;
        }
    }

    if (a.new_k) return 0;  // only the flat decode kernel appends by itself; the caller appends and comes back

    // Units per (batch, head): minimise waves x (tiles per unit + fixed cost), with
    // `slots` CTAs resident at once; ties go to fewer splits.
    int64_t best_s = 1;
    double best_cost = 1e30;
    const int64_t max_s = std::min<int64_t>(tiles, 64);
    for (int64_t s = 1; s <= max_s; ++s) {
        const int64_t units = bh * row_blocks * s;
        const int64_t waves = (units + slots - 1) / slots;
        const int64_t per = (tiles + s - 1) / s;
        const double cost = (double)waves * ((double)per + 2.5);
        if (cost < best_cost - 1e-9) {
            best_cost = cost;
            best_s = s;
        }
    }
    const int64_t splits = best_s;

    const int64_t qrows = (int64_t)a.B * a.Hq * a.L;
    const size_t o_bytes = (size_t)qrows * splits * a.D * sizeof(float);
    const size_t ml_bytes = (size_t)qrows * splits * sizeof(float2);
    char *scratch = (char *)scratch_get(a.device, o_bytes + ml_bytes + 256, stream);
    float *o_part = (float *)scratch;
    float2 *ml_part = (float2 *)(scratch + ((o_bytes + 255) / 256) * 256);

    DecodeParams p = {};
    p.q = a.q; p.out = a.out; p.out_dtype = a.q_dtype;
    p.q_sb = a.q_sb; p.q_sh = a.q_sh; p.q_sl = a.q_sl;
    p.o_sb = a.o_sb; p.o_sh = a.o_sh; p.o_sl = a.o_sl;
    p.o_part = o_part; p.ml_part = ml_part; p.counters = counters; p.status = status;
    p.B = a.B; p.Hq = a.Hq; p.Hkv = a.Hkv; p.L = a.L; p.T = a.T;
    p.splits = (int)splits;
    p.tiles_base = (int)(tiles / splits);
    p.tiles_rem = (int)(tiles % splits);
    p.causal = a.mask.mode == KVC_MASK_CAUSAL ? 1 : 0;
    p.debug_skip = measure_skip_bits();
    p.causal_offset = a.mask.causal_offset;
    p.scale_log2 = a.scale * 1.4426950408889634f;
    p.row_blocks = (int)row_blocks;
    p.tiles_all = (int)tiles;
    const int units = (int)(bh * splits);

    if (chunk) {
        const int ctas = (int)(bh * row_blocks * splits);
#define KVC_CHK(TT, DD, NS) launch_chunk_typed<TT, DD, NS>(kmap, vmap, p, ctas, stream)
        if (a.q_dtype == KVC_BF16) {
            if (a.D == 64) KVC_CHK(__nv_bfloat16, 64, 6);
            else if (a.D == 128) KVC_CHK(__nv_bfloat16, 128, 3);
            else KVC_CHK(__nv_bfloat16, 256, 3);
        } else {
            if (a.D == 64) KVC_CHK(__half, 64, 6);
            else if (a.D == 128) KVC_CHK(__half, 128, 3);
            else KVC_CHK(__half, 256, 3);
        }
#undef KVC_CHK
        return 1;
    }

#define KVC_DEC(TT, DD, NS) launch_typed<TT, DD, NS>(kmap, vmap, p, units, stream)
    if (a.q_dtype == KVC_BF16) {
        if (a.D == 64) KVC_DEC(__nv_bfloat16, 64, 6);
        else if (a.D == 128) KVC_DEC(__nv_bfloat16, 128, 3);
        else KVC_DEC(__nv_bfloat16, 256, 3);
    } else {
        if (a.D == 64) KVC_DEC(__half, 64, 6);
        else if (a.D == 128) KVC_DEC(__half, 128, 3);
        else KVC_DEC(__half, 256, 3);
    }
#undef KVC_DEC
    return 1;
}

}  // namespace kvc
