// Prefill / long verify chunks over raw K/V on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// attentionWithCacheUpdate's scaledDotProductAttention call (AttentionUtils.swift:87-93) for a chunk
// of L query positions per head: one CTA takes 128 consecutive positions of one query head and walks
// the 128-key tiles it can see.
//
//   warp 0      TMA producer: the Q block once, then K and V tiles into two slots each (K one tile ahead)
//   warp 1      owns the TMEM allocation; lane 0 issues the MMAs:
//                 S_j = Q K_j^T          (A = Q, B = K_j, both K-major)      -> TMEM S buffer j % 2
//                 O_j = P_j V_j          (A = P_j from shared memory, B = V_j MN-major) -> TMEM O buffer j % 2
//   warps 2..5  softmax: thread = query row = TMEM lane. S_j comes out of TMEM in one round trip (128
//               registers), row maximum, exponentials, P_j written as the next MMA's A operand in
//               shared memory (two P tiles, so that tile j + 1 never waits for O_j to have read
//               P_j); the rescale factor of the tile goes to the correction warps
//   warps 6..9  correction: thread = query row. O_j comes out of TMEM and is folded into the row's
//               register accumulator, o = o * alpha_j + O_j; normalisation and the store at the end
//
// Every O_j is a fresh product (no accumulation in TMEM), so the running-maximum rescale never has to
// touch TMEM. S_{j+1} is issued before O_j: the tensor cores work on the next scores while the
// softmax warps are busy with the current ones, and the correction warps trail by one product.
//
// Shared-memory operand layout (what TMA's 128-byte swizzle writes): a box is 128 rows x 128 bytes
// (64 elements), 16-byte chunk c of row r at chunk c ^ (r & 7); a 128 x 128 tile is two boxes (Q, K and
// V tiles at head dim 64 are one box, the O product then has 64 columns).
// Matrix descriptors: K-major operands advance 32 bytes per 16-element k-step inside the row, 8-row
// groups are 1024 bytes apart; the MN-major V tile advances 2048 bytes per 16 keys, its two 64-dim
// halves are 16384 bytes apart (leading offset) and its 8-key groups 1024 bytes (stride offset).
//
// Every wait is bounded; a wait that runs out sets the device status word, the CTA drains and frees
// its TMEM.
#include <atomic>
#include <cuda.h>

#include <cstdlib>
#include <mutex>
#include <type_traits>

#include "attn_common.cuh"
#include "common.h"
#include "tc_common.cuh"

namespace kvc {
namespace {

using namespace dev;

using namespace tc;


struct ChunkTcParams {
    void *out;
    int64_t o_sb, o_sh, o_sl;
    int32_t B, Hq, Hkv, L;
    int64_t T;
    int32_t row_blocks;
    int32_t causal;
    int64_t causal_offset;
    float scale_log2;
    int *status;
};

enum : int {
    BAR_Q = 0,
    BAR_K_FULL = 1,                         // [TC_STAGES]
    BAR_K_EMPTY = BAR_K_FULL + TC_STAGES,   // [TC_STAGES] free once the S product has read the tile
    BAR_V_FULL = BAR_K_EMPTY + TC_STAGES,   // [TC_STAGES]
    BAR_V_EMPTY = BAR_V_FULL + TC_STAGES,   // [TC_STAGES] free once the O product has read the tile
    BAR_S_FULL = BAR_V_EMPTY + TC_STAGES,   // [2]
    BAR_S_EMPTY = BAR_S_FULL + 2,           // [2]
    BAR_P_FULL = BAR_S_EMPTY + 2,           // [2]
    BAR_P_EMPTY = BAR_P_FULL + 2,           // [2]
    BAR_O_FULL = BAR_P_EMPTY + 2,           // [2]
    BAR_O_EMPTY = BAR_O_FULL + 2,           // [2]
    BAR_A_FULL = BAR_O_EMPTY + 2,           // [2] rescale factors of a tile written
    BAR_A_EMPTY = BAR_A_FULL + 2,           // [2] ... and read
    BAR_L_FULL = BAR_A_EMPTY + 2,           // row sums written
    BAR_COUNT = BAR_L_FULL + 1
};

template <typename T, int D>
__global__ void __launch_bounds__(TC_THREADS, 1)
attn_chunk_tc_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                     const __grid_constant__ CUtensorMap vmap, const ChunkTcParams p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    constexpr int NBOX = D / 64;                               // boxes of 64 head dims per Q / K / V tile
    constexpr int QKV_TILE = NBOX * TC_BOX;                    // bytes of a 128-row tile of D head dims
    unsigned char *sq = base;                                  // Q block
    unsigned char *skv = sq + QKV_TILE;                        // ring: stage s = K tile | V tile
    uint64_t *bars = (uint64_t *)(skv + TC_STAGES * 2 * QKV_TILE);
    uint32_t *tmem_slot = (uint32_t *)(bars + BAR_COUNT);
    float *s_alpha = (float *)(tmem_slot + 4);                 // [2][128] rescale factor of tile j for each row
    float *s_lsum = s_alpha + 2 * TC_ROWS;                     // [128] final row sums

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // unit = (batch, KV head, row block, query head of the group): the CTAs that share K/V are neighbours
    const int rep = p.Hq / p.Hkv;
    int u = blockIdx.x;
    const int hr = u % rep; u /= rep;
    // with a causal mask the late row blocks see the most keys: they go first, the short ones fill the tail
    const int rb = p.row_blocks - 1 - (u % p.row_blocks); u /= p.row_blocks;
    const int hk = u % p.Hkv;
    const int b = u / p.Hkv;
    const int hq = hk * rep + hr;
    const int l0 = rb * TC_ROWS;
    // keys this block can see: up to the last row's limit
    const int64_t last_l = min((int64_t)p.L - 1, (int64_t)l0 + TC_ROWS - 1);
    const int64_t keys = p.causal ? min(p.T, p.causal_offset + last_l + 1) : p.T;
    const int n_tiles = (int)((keys + TC_KEYS - 1) / TC_KEYS);

    if (tid == 0) {
        mbar_init(&bars[BAR_Q], 1);
        for (int s = 0; s < TC_STAGES; ++s) {
            mbar_init(&bars[BAR_K_FULL + s], 1);
            mbar_init(&bars[BAR_K_EMPTY + s], 1);
            mbar_init(&bars[BAR_V_FULL + s], 1);
            mbar_init(&bars[BAR_V_EMPTY + s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&bars[BAR_S_FULL + s], 1);
            mbar_init(&bars[BAR_S_EMPTY + s], 128);
            mbar_init(&bars[BAR_O_FULL + s], 1);
            mbar_init(&bars[BAR_O_EMPTY + s], 128);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&bars[BAR_A_FULL + s], 128);
            mbar_init(&bars[BAR_A_EMPTY + s], 128);
        }
        mbar_init(&bars[BAR_L_FULL], 128);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&bars[BAR_P_FULL + s], 128);
            mbar_init(&bars[BAR_P_EMPTY + s], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
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
    pdl_wait();  // everything below reads what earlier kernels on the stream wrote

    if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0) {
            bool ok = true;
            mbar_expect_tx(&bars[BAR_Q], QKV_TILE);
#pragma unroll
            for (int bx = 0; bx < NBOX; ++bx) tma_load_4d(sq + bx * TC_BOX, &qmap, &bars[BAR_Q], bx * 64, l0, hq, b);
            // A K slot is free as soon as its score product is done, a V slot only after the output
            // product one tile later: K runs one tile ahead of V so that neither waits for the other.
            auto load_k = [&](int j) {
                const int s = j % TC_STAGES;
                if (j >= TC_STAGES && !mbar_wait(&bars[BAR_K_EMPTY + s], ((j / TC_STAGES) - 1) & 1)) return false;
                unsigned char *kt = skv + (size_t)s * 2 * QKV_TILE;
                mbar_expect_tx(&bars[BAR_K_FULL + s], QKV_TILE);
#pragma unroll
                for (int bx = 0; bx < NBOX; ++bx) tma_load_4d(kt + bx * TC_BOX, &kmap, &bars[BAR_K_FULL + s], bx * 64, j * TC_KEYS, hk, b);
                return true;
            };
            auto load_v = [&](int j) {
                const int s = j % TC_STAGES;
                if (j >= TC_STAGES && !mbar_wait(&bars[BAR_V_EMPTY + s], ((j / TC_STAGES) - 1) & 1)) return false;
                unsigned char *vt = skv + (size_t)s * 2 * QKV_TILE + QKV_TILE;
                mbar_expect_tx(&bars[BAR_V_FULL + s], QKV_TILE);
#pragma unroll
                for (int bx = 0; bx < NBOX; ++bx) tma_load_4d(vt + bx * TC_BOX, &vmap, &bars[BAR_V_FULL + s], bx * 64, j * TC_KEYS, hk, b);
                return true;
            };
            if (n_tiles > 0) ok = load_k(0);
            for (int j = 0; j < n_tiles && ok; ++j) {
                if (j + 1 < n_tiles) ok = load_k(j + 1);
                if (ok) ok = load_v(j);
            }
            if (!ok) atomicExch(p.status, 21);
        }
    } else if (warp == 1) {
        // ---------------- MMA issue ----------------
        if (lane == 0) {
            // instruction descriptor: f32 accumulator (bits 4-5 = 1), A and B formats (bits 7-9 and 10-12:
            // 0 = f16, 1 = bf16), B major at bit 16 (1 = MN-major), N / 8 at bits 17-22, M / 16 at 24-28
            constexpr uint32_t FMT = sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
            constexpr uint32_t IDESC = (1u << 4) | (FMT << 7) | (FMT << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
            // the O product has N = D columns
            constexpr uint32_t IDESC_PV = (1u << 4) | (FMT << 7) | (FMT << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | ((128u >> 4) << 24);
            // Descriptors differ only in the start-address field (16-byte units): a box is 1024 units, a
            // k-step inside a box row 2, 16 keys of the MN-major V tile 128.
            const uint64_t q_desc = umma_desc(smem_u32(sq), 16, 1024);
            const uint64_t k_desc = umma_desc(smem_u32(skv), 16, 1024);
            const uint64_t v_desc = umma_desc(smem_u32(skv) + QKV_TILE, 16384, 1024);
            bool ok = mbar_wait(&bars[BAR_Q], 0);
            auto issue_s = [&](int j) {
                const int s = j % TC_STAGES;
                if (!mbar_wait(&bars[BAR_K_FULL + s], (j / TC_STAGES) & 1)) return false;
                if (j >= 2 && !mbar_wait(&bars[BAR_S_EMPTY + (j & 1)], ((j >> 1) - 1) & 1)) return false;
                tc_fence_after();
                const uint64_t kd = k_desc + (uint64_t)(s * (2 * QKV_TILE / 16));
                const uint32_t d_addr = tmem + (uint32_t)(j & 1) * 128u;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint64_t off = (uint64_t)((ks >> 2) * (TC_BOX / 16) + (ks & 3) * 2);
                    umma_f16(d_addr, q_desc + off, kd + off, IDESC, ks > 0 ? 1u : 0u);
                }
                umma_commit(&bars[BAR_S_FULL + (j & 1)]);
                umma_commit(&bars[BAR_K_EMPTY + s]);
                return true;
            };
            if (ok) ok = issue_s(0);
            for (int j = 0; j < n_tiles && ok; ++j) {
                if (j + 1 < n_tiles) ok = issue_s(j + 1);
                if (!ok) break;
                const int s = j % TC_STAGES;
                ok = mbar_wait(&bars[BAR_V_FULL + s], (j / TC_STAGES) & 1);
                if (ok) ok = mbar_wait(&bars[BAR_P_FULL + (j & 1)], (j >> 1) & 1);
                if (ok && j >= 1) ok = mbar_wait(&bars[BAR_O_EMPTY], (j - 1) & 1);
                if (!ok) break;
                tc_fence_after();
                const uint64_t vd = v_desc + (uint64_t)(s * (2 * QKV_TILE / 16));
                // TMEM columns: S_0, S_1 at 0, 128; O at 256 (one accumulator: it is folded away long before the
                // next O product is due); P_0, P_1 at 384, 448, written there by the softmax warps and read as
                // the A operand (16 keys = 8 columns per product)
                const uint32_t o_addr = tmem + 256u;
                const uint32_t p_addr = tmem + 384u + (uint32_t)(j & 1) * 64u;
#pragma unroll
                for (int ks = 0; ks < TC_KEYS / 16; ++ks)
                    umma_f16_ts(o_addr, p_addr + (uint32_t)ks * 8u, vd + (uint64_t)(ks * 128), IDESC_PV, ks > 0 ? 1u : 0u);
                umma_commit(&bars[BAR_O_FULL]);
                umma_commit(&bars[BAR_P_EMPTY + (j & 1)]);
                umma_commit(&bars[BAR_V_EMPTY + s]);
            }
            if (!ok) atomicExch(p.status, 22);
        }
    } else if (warp < 6) {
        // ---------------- softmax: thread = row ----------------
        const int quarter = warp & 3;                       // the TMEM lanes this warp may touch
        const int row = quarter * 32 + lane;
        const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
        const int64_t l = (int64_t)l0 + row;
        const int64_t limit = p.causal ? min(p.T - 1, p.causal_offset + l) : p.T - 1;   // last visible key
        const int64_t block_min_limit = p.causal ? min(p.T - 1, p.causal_offset + l0) : p.T - 1;
        float m_run = -INFINITY, l_run = 0.f;
        bool ok = true;
        for (int j = 0; j < n_tiles; ++j) {
            ok = mbar_wait(&bars[BAR_S_FULL + (j & 1)], (j >> 1) & 1);
            if (!ok) break;
            tc_fence_after();
            const uint32_t s_addr = lane_addr + (uint32_t)(j & 1) * 128u;
            uint32_t raw[TC_KEYS];
#pragma unroll
            for (int cb = 0; cb < 4; ++cb) tmem_ld32_issue(s_addr + cb * 32, raw + cb * 32);
            tmem_ld_wait();
            // the scores are in registers: the S buffer is free for tile j + 2
            tc_fence_before();
            mbar_arrive(&bars[BAR_S_EMPTY + (j & 1)]);
            const int64_t key0 = (int64_t)j * TC_KEYS;
            if (key0 + TC_KEYS - 1 > block_min_limit) {   // some row of the block loses keys in this tile
#pragma unroll
                for (int i = 0; i < TC_KEYS; ++i)
                    if (key0 + i > limit) raw[i] = 0xff800000u;   // -inf
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < TC_KEYS; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(raw[i]));
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            const float m_new = fmaxf(m_run, mx * p.scale_log2);
            const float alpha = (m_run == -INFINITY) ? 0.f : fast_exp2(m_run - m_new);
            const float neg_m = (m_new == -INFINITY) ? 0.f : -m_new;
            // hand the tile's rescale factor to the correction warps
            if (j >= 2) ok = mbar_wait(&bars[BAR_A_EMPTY + (j & 1)], ((j >> 1) - 1) & 1);
            if (!ok) break;
            s_alpha[(j & 1) * TC_ROWS + row] = alpha;
            mbar_arrive(&bars[BAR_A_FULL + (j & 1)]);
            // this P tile is free once the O product of two tiles ago has read it
            if (j >= 2) ok = mbar_wait(&bars[BAR_P_EMPTY + (j & 1)], ((j >> 1) - 1) & 1);
            if (!ok) break;
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int kc = 0; kc < TC_KEYS / 8; ++kc) {   // 16-byte chunk (8 keys) of the row
                float e[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    e[i] = fast_exp2(fmaf(__uint_as_float(raw[kc * 8 + i]), p.scale_log2, neg_m));   // exp2(-inf) = 0
                    sum4[i & 3] += e[i];
                }
                // the probabilities as pairs, kept in the registers the scores came in (entry 4 kc + q of the
                // packed row: always behind the scores still to be read)
#pragma unroll
                for (int q = 0; q < 4; ++q) raw[kc * 4 + q] = pack_pair<T>(e[2 * q], e[2 * q + 1]);
                // P_j goes into TMEM (this thread's lane), where the O product reads it as its A operand
                if (kc == 7) tmem_st32_issue(lane_addr + 384u + (uint32_t)(j & 1) * 64u, raw);
            }
            tmem_st32_issue(lane_addr + 384u + (uint32_t)(j & 1) * 64u + 32u, raw + 32);
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(&bars[BAR_P_FULL + (j & 1)]);
            l_run = l_run * alpha + (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            m_run = m_new;
        }
        if (ok) {
            s_lsum[row] = l_run;
            mbar_arrive(&bars[BAR_L_FULL]);
        } else {
            atomicExch(p.status, 23);
        }
    } else {
        // ---------------- correction: thread = row ----------------
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16) + 256u;
        const int64_t l = (int64_t)l0 + row;
        float o_acc[D];
#pragma unroll
        for (int i = 0; i < D; ++i) o_acc[i] = 0.f;
        bool ok = true;
        for (int j = 0; j < n_tiles; ++j) {
            ok = mbar_wait(&bars[BAR_A_FULL + (j & 1)], (j >> 1) & 1);
            if (!ok) break;
            const float alpha = s_alpha[(j & 1) * TC_ROWS + row];
            mbar_arrive(&bars[BAR_A_EMPTY + (j & 1)]);
            ok = mbar_wait(&bars[BAR_O_FULL], j & 1);
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int half = 0; half < D / 64; ++half) {
                uint32_t raw[64];
                tmem_ld32_issue(lane_addr + half * 64, raw);
                tmem_ld32_issue(lane_addr + half * 64 + 32, raw + 32);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 64; ++i) o_acc[half * 64 + i] = fmaf(o_acc[half * 64 + i], alpha, __uint_as_float(raw[i]));
            }
            tc_fence_before();
            mbar_arrive(&bars[BAR_O_EMPTY]);
        }
        if (ok) ok = mbar_wait(&bars[BAR_L_FULL], 0);
        if (!ok) {
            atomicExch(p.status, 24);
        } else if (l < p.L) {
            const float l_sum = s_lsum[row];
            const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
            T *dst = (T *)p.out + b * p.o_sb + hq * p.o_sh + l * p.o_sl;
#pragma unroll
            for (int c8 = 0; c8 < D / 8; ++c8) {
                uint4 w;
                w.x = pack_pair<T>(o_acc[c8 * 8 + 0] * inv, o_acc[c8 * 8 + 1] * inv);
                w.y = pack_pair<T>(o_acc[c8 * 8 + 2] * inv, o_acc[c8 * 8 + 3] * inv);
                w.z = pack_pair<T>(o_acc[c8 * 8 + 4] * inv, o_acc[c8 * 8 + 5] * inv);
                w.w = pack_pair<T>(o_acc[c8 * 8 + 6] * inv, o_acc[c8 * 8 + 7] * inv);
                *(uint4 *)(dst + c8 * 8) = w;
            }
        }
    }
    // all roles meet here; TMEM goes back whatever happened
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TC_TMEM_COLS) : "memory");
    }
}

template <typename T, int D>
bool launch_tc_typed(const CUtensorMap &qmap, const CUtensorMap &kmap, const CUtensorMap &vmap, const ChunkTcParams &p, int ctas,
                     cudaStream_t stream) {
    const size_t smem = (size_t)(D / 64) * TC_BOX * (1 + 2 * TC_STAGES) + BAR_COUNT * sizeof(uint64_t) + 64 +
                        3 * TC_ROWS * sizeof(float) + 1024;
    // 0 = not yet, 1 = ready, -1 = refused; distinct handles may call from distinct host threads
    static std::atomic<int> configured[64];
    const int dev = current_device();
    if (dev < 0 || dev >= 64) return false;
    int state = configured[dev].load(std::memory_order_acquire);
    if (state == 0) {
        // setting the attribute twice from two racing threads is harmless; the result is the same
        const cudaError_t e = cudaFuncSetAttribute(attn_chunk_tc_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) (void)cudaGetLastError();
        state = e == cudaSuccess ? 1 : -1;
        configured[dev].store(state, std::memory_order_release);
    }
    if (state < 0) return false;
    KernelTimer timer(stream);
    KVC_CUDA(launch_pdl(attn_chunk_tc_kernel<T, D>, dim3(ctas), dim3(TC_THREADS), smem, stream, qmap, kmap, vmap, p));
    timer.stop();
    ++g_launch_count;
    return true;
}

}  // namespace

// Returns 1 when the call was taken (head dim 64 or 128, f16 / bf16 raw K and V, no array mask, enough
// 128-row blocks to fill the part), 0 otherwise. KVC_CHUNK_TC=0 turns the path off.
bool attention_chunk_tc_accepts(const AttnArgs &a) {
    static const bool off = [] {
        const char *e = std::getenv("KVC_CHUNK_TC");
        return e && e[0] == '0';
    }();
    if (off) return false;
    if ((a.D != 128 && a.D != 64) || (a.q_dtype != KVC_BF16 && a.q_dtype != KVC_F16)) return false;
    if (a.k.kind != SRC_RAW || a.v.kind != SRC_RAW || a.k.dtype != a.q_dtype || a.v.dtype != a.q_dtype) return false;
    if (a.mask.mode == KVC_MASK_ARRAY || a.q_signs || a.o_signs || a.q_calib || a.new_k || a.q_rot || a.o_rot) return false;
    if (a.Hkv <= 0 || a.Hq % a.Hkv || a.T < 1 || a.T > (int64_t)1 << 30 || a.L < 64) return false;
    if (a.mask.mode == KVC_MASK_CAUSAL && a.mask.causal_offset < 0) return false;
    const int64_t row_blocks = ((int64_t)a.L + TC_ROWS - 1) / TC_ROWS;
    const int64_t ctas = (int64_t)a.B * a.Hq * row_blocks;
    // a CTA owns an SM (its TMEM and 193 KB of shared memory): fewer blocks than half the part run
    // better on the split-K kernel
    if (ctas < sm_count(a.device) / 2 || ctas > (int64_t)1 << 30) return false;
    if (!strides_fit(a.q, a.D, a.q_sl, a.q_sh, a.q_sb, a.Hq, a.B)) return false;
    if (!strides_fit(a.k.data, a.D, a.k.st, a.k.sh, a.k.sb, a.Hkv, a.B) || !strides_fit(a.v.data, a.D, a.v.st, a.v.sh, a.v.sb, a.Hkv, a.B))
        return false;
    if (((uintptr_t)a.out & 15) != 0 || (a.o_sl * 2) % 16 || (a.o_sh * 2) % 16 || (a.o_sb * 2) % 16) return false;
    return true;
}

int launch_attention_chunk_tc(const AttnArgs &a, cudaStream_t stream) {
    if (!attention_chunk_tc_accepts(a)) return 0;
    const int64_t row_blocks = ((int64_t)a.L + TC_ROWS - 1) / TC_ROWS;
    const int64_t ctas = (int64_t)a.B * a.Hq * row_blocks;
    int *status = device_status_word(a.device);
    if (!status) return 0;
    CUtensorMap qmap, kmap, vmap;
    if (!make_map_tc(&qmap, a.q, a.q_dtype, a.D, a.L, a.Hq, a.B, a.q_sl, a.q_sh, a.q_sb)) return 0;
    if (!make_map_tc(&kmap, a.k.data, a.k.dtype, a.D, a.T, a.Hkv, a.B, a.k.st, a.k.sh, a.k.sb)) return 0;
    if (!make_map_tc(&vmap, a.v.data, a.v.dtype, a.D, a.T, a.Hkv, a.B, a.v.st, a.v.sh, a.v.sb)) return 0;
    ChunkTcParams p = {};
    p.out = a.out;
    p.o_sb = a.o_sb; p.o_sh = a.o_sh; p.o_sl = a.o_sl;
    p.B = a.B; p.Hq = a.Hq; p.Hkv = a.Hkv; p.L = a.L; p.T = a.T;
    p.row_blocks = (int)row_blocks;
    p.causal = a.mask.mode == KVC_MASK_CAUSAL ? 1 : 0;
    p.causal_offset = a.mask.causal_offset;
    p.scale_log2 = a.scale * 1.4426950408889634f;
    p.status = status;
    bool taken;
    if (a.D == 128)
        taken = a.q_dtype == KVC_BF16 ? launch_tc_typed<__nv_bfloat16, 128>(qmap, kmap, vmap, p, (int)ctas, stream)
                                      : launch_tc_typed<__half, 128>(qmap, kmap, vmap, p, (int)ctas, stream);
    else
        taken = a.q_dtype == KVC_BF16 ? launch_tc_typed<__nv_bfloat16, 64>(qmap, kmap, vmap, p, (int)ctas, stream)
                                      : launch_tc_typed<__half, 64>(qmap, kmap, vmap, p, (int)ctas, stream);
    if (taken && trace_dispatch()) fprintf(stderr, "[kvc] chunk_tc: %lld CTAs of 128 rows\n", (long long)ctas);
    return taken ? 1 : 0;
}

}  // namespace kvc
