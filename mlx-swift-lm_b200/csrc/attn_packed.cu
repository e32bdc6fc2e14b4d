// Split-K flash decoding over the group-wise affine-quantised cache
// (QuantizedKVCache, 4- or 8-bit codes) on sm_100a.
//
// Same CTA structure as the raw-cache decode kernel: a producer warp streams
// tiles of 64 tokens through an mbarrier ring, here with untiled TMA bulk copies
// (cp.async.bulk) because every array of the packed cache is contiguous per
// (batch, head): codes [64 x D*bits/8 bytes], scales and biases [64 x D/group]
// for K and for V. Four consumer warps take 16 tokens each.
//
// Dequantisation happens in registers and is folded around the tensor-core MMAs:
//   scores:  q . (s*c + b) = s * (q . c) + b * sum(q)      per group of the row
//            -> the MMA runs on the raw integer codes (exact in f16) with one
//               accumulator per group; scale and bias are applied to the 16x8
//               score fragment afterwards;
//   values:  sum_t p_t (s_t c_t + b_t) = sum_t (p_t s_t) c_t + sum_t p_t b_t
//            -> the probabilities are pre-multiplied by the token's scale (one A
//               fragment per group), the bias term is a per-row scalar sum.
// Codes become f16 operands with the exponent trick: (x & 0x000F000F) | 0x64006400
// is the f16 pair (1024 + n_lo, 1024 + n_hi), one subtraction removes the 1024.
// K codes are read as whole words of the token's row (the k-slot <-> head-dim
// assignment is a permutation shared with the query fragments, kept inside one
// quantisation group per MMA); V codes go through ldmatrix.trans, which hands
// each lane the 16-bit units of two consecutive tokens in one register, exactly
// the token-pair layout the P.V operand needs.
#include "attn_common.cuh"

#include <algorithm>
#include <cstdlib>

namespace kvc {

namespace {

using namespace dev;

constexpr int PK_WARPS = 4;
constexpr int PK_THREADS = (PK_WARPS + 1) * 32;
constexpr int PK_TILE = 64;
// The 8-row decode kernel takes its consumer-warp count as a template parameter (16 tokens per warp and
// stage): 4 warps x 3 CTAs per SM, or 15 warps x 1 CTA (16 warps with the producer: 128 registers each).
// Uniform batches of 4-bit codes at head dim 128 take the 15-warp form (77.8 against 85.4 us per launch on
// the Qwen2-7B shape); ragged lists of caches keep 64-token tiles (their units end at any length and the
// 240-token tiles measured 4 % slower there).
constexpr int affine8_warps(int D, int bits, bool varlen) { return (D == 128 && bits == 4 && !varlen) ? 15 : 4; }
constexpr int affine8_ctas(int D, int bits, bool varlen) { return affine8_warps(D, bits, varlen) == 15 ? 1 : 3; }
constexpr int PK_COUNTER_BYTES = 64 * 1024;

struct AffineParams {
    const void *q;
    void *out;
    int64_t q_sb, q_sh, q_sl, o_sb, o_sh, o_sl;
    const uint32_t *kc, *vc;           // codes
    const void *ks, *kb, *vs, *vb;     // scales / biases (dtype T)
    int64_t kc_sb, kc_sh, vc_sb, vc_sh;  // word strides (token stride = words per row)
    int64_t kg_sb, kg_sh, vg_sb, vg_sh;  // element strides of scales/biases (token stride = groups)
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
    FlatPlan flat;  // decode8 kernel: flat tile decomposition
    int32_t q_bulk; // decode8 kernel: a unit's query rows are one contiguous 16-byte aligned block
    int32_t chunks; // decode8 kernel: units per (batch, kv head) = ceil(query rows of the group / 8); 1 for decode
};

// One decode step for a list of independent caches (one sequence each, its own length) in one
// launch: units are (sequence, KV head), sequence i has tiles[i] tiles per head and its units
// start at flat tile Hkv * tile_prefix[i].
struct VarlenAttnSeq {
    const void *q;
    void *out;
    const uint32_t *kc, *vc;
    const void *ks, *kb, *vs, *vb;
    int64_t c_sh, g_sh;  // head strides (words / elements) of this cache's arrays
    int32_t T, tile_prefix;
};
struct VarlenAttnTable {
    int32_t n;
    VarlenAttnSeq seq[KVC_VARLEN_MAX];
};

__device__ __forceinline__ uint32_t hsub2_1024(uint32_t x) {
    uint32_t r;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(x), "r"(0x64006400u));
    return r;
}

// Operand pair (b0, b1) number `which` of a packed code word, as f16 pairs minus nothing
// (the caller subtracts 1024). 4-bit: word = nibbles n0..n7, pair 0 = {(n0,n4),(n1,n5)},
// pair 1 = {(n2,n6),(n3,n7)}. 8-bit: word = bytes b0..b3, single pair {(b0,b1),(b2,b3)}.
template <int BITS>
__device__ __forceinline__ void code_pair(uint32_t w, int which, uint32_t &b0, uint32_t &b1) {
    if (BITS == 4) {
        const uint32_t x = w >> (8 * which);
        b0 = hsub2_1024((x & 0x000F000Fu) | 0x64006400u);
        b1 = hsub2_1024(((x >> 4) & 0x000F000Fu) | 0x64006400u);
    } else {
        b0 = hsub2_1024(__byte_perm(w, 0x64646464u, 0x4140));
        b1 = hsub2_1024(__byte_perm(w, 0x64646464u, 0x4342));
    }
}

// Head dims that the four k-slot pairs of MMA `m` (within a lane's word `wl` of a
// group) stand for; used once to lay the query fragments out to match.
template <int BITS>
__device__ __forceinline__ void kslot_dims(int word_in_row, int which, int (&d)[4]) {
    if (BITS == 4) {
        const int base = word_in_row * 8 + 2 * which;
        d[0] = base;       // k-slot 2c
        d[1] = base + 4;   // k-slot 2c+1
        d[2] = base + 1;   // k-slot 2c+8
        d[3] = base + 5;   // k-slot 2c+9
    } else {
        const int base = word_in_row * 4;
        d[0] = base; d[1] = base + 1; d[2] = base + 2; d[3] = base + 3;
    }
}

template <typename T, int D, int BITS, int GROUP, int NSTAGE>
__global__ void __launch_bounds__(PK_THREADS, 2)
attn_affine_kernel(const AffineParams p) {
    constexpr int G = D / GROUP;                  // groups per row
    constexpr int RB = D * BITS / 8;              // code bytes per row
    constexpr int WPR = RB / 4;                   // words per row
    constexpr int WPG = GROUP * BITS / 32;        // words per group
    constexpr int WPL = WPG / 4;                  // words per lane per group
    constexpr int MPW = (BITS == 4) ? 2 : 1;      // MMAs per word
    constexpr int MPG = WPL * MPW;                // MMAs (k-steps) per group
    constexpr int SB = G * 2;                     // scale (or bias) bytes per token
    constexpr int CODE_TILE = PK_TILE * RB;
    constexpr int SC_TILE = PK_TILE * SB;
    constexpr int STAGE_BYTES = 2 * CODE_TILE + 4 * SC_TILE;
    constexpr int EPU = 16 / BITS;                // elements per 16-bit unit
    constexpr int CH = RB / 16;                   // 16-byte chunks per row
    constexpr int NT_O = D / 8;
    constexpr int RED_STRIDE = D + 8;
    static_assert(WPL >= 1 && G >= 1 && G <= 4, "unsupported group layout");
    static_assert(CH % 2 == 0, "rows must hold an even number of 16-byte chunks");
    static_assert(STAGE_BYTES % 16 == 0 && SC_TILE % 16 == 0, "bulk copies need 16-byte multiples");

    extern __shared__ __align__(128) unsigned char smem_raw[];
    // pointer + offset (no integer round trip) so that loads through it stay ld.shared
    unsigned char *stages = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
    constexpr int RING = NSTAGE * STAGE_BYTES;
    constexpr int RED_BYTES = PK_WARPS * 16 * RED_STRIDE * 4 + PK_WARPS * 16 * 2 * 4 + 16 * 64 * 4;
    constexpr int BODY = RING > RED_BYTES ? RING : RED_BYTES;
    uint64_t *full = (uint64_t *)(stages + ((BODY + 15) / 16) * 16);
    uint64_t *empty = full + NSTAGE;
    int *is_last = (int *)(empty + NSTAGE);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x % p.splits;
    const int bh = blockIdx.x / p.splits;
    const int hk = bh % p.Hkv, b = bh / p.Hkv;
    const int rep = p.Hq / p.Hkv;
    const int R = rep * p.L;
    const int tile_begin = split * p.tiles_base + min(split, p.tiles_rem);
    const int ntiles = p.tiles_base + (split < p.tiles_rem ? 1 : 0);

    if (tid == 0) {
        for (int s = 0; s < NSTAGE; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], PK_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    pdl_wait();  // everything below reads what earlier kernels on the stream wrote

    bool ok = true;
    const int g = lane >> 2, c = lane & 3;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float bsum[2][G];  // sum_t p_t * bias_t per row half and value group
    float o_acc[NT_O][4];
#pragma unroll
    for (int i = 0; i < NT_O; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int gr = 0; gr < G; ++gr) bsum[h][gr] = 0.f;

    if (warp == PK_WARPS) {
        // ---------------- producer ----------------
        if (lane == 0) {
            const uint32_t *kc = p.kc + b * p.kc_sb + hk * p.kc_sh;
            const uint32_t *vc = p.vc + b * p.vc_sb + hk * p.vc_sh;
            const T *ks = (const T *)p.ks + b * p.kg_sb + hk * p.kg_sh;
            const T *kb = (const T *)p.kb + b * p.kg_sb + hk * p.kg_sh;
            const T *vs = (const T *)p.vs + b * p.vg_sb + hk * p.vg_sh;
            const T *vb = (const T *)p.vb + b * p.vg_sb + hk * p.vg_sh;
            for (int it = 0; it < ntiles && ok; ++it) {
                const int s = it % NSTAGE;
                if (it >= NSTAGE) ok = mbar_wait(&empty[s], ((it / NSTAGE) - 1) & 1);
                if (!ok) break;
                unsigned char *st = stages + (size_t)s * STAGE_BYTES;
                const int64_t t0 = (int64_t)(tile_begin + it) * PK_TILE;
                mbar_expect_tx(&full[s], STAGE_BYTES);
                bulk_load(st, kc + t0 * WPR, CODE_TILE, &full[s]);
                bulk_load(st + CODE_TILE, vc + t0 * WPR, CODE_TILE, &full[s]);
                bulk_load(st + 2 * CODE_TILE, ks + t0 * G, SC_TILE, &full[s]);
                bulk_load(st + 2 * CODE_TILE + SC_TILE, kb + t0 * G, SC_TILE, &full[s]);
                bulk_load(st + 2 * CODE_TILE + 2 * SC_TILE, vs + t0 * G, SC_TILE, &full[s]);
                bulk_load(st + 2 * CODE_TILE + 3 * SC_TILE, vb + t0 * G, SC_TILE, &full[s]);
            }
            if (!ok) atomicExch(p.status, 3);
        }
    } else {
        // ---------------- consumers ----------------
        // Query fragments (f16), laid out to match the code words each lane reads, and
        // sum(q) per row half and key group for the bias term.
        uint32_t qa[G][MPG][4];
        float qsum[2][G];
        int64_t row_limit[2];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = g + 8 * half;
            const int l = r % p.L;
            row_limit[half] = (r < R) ? (p.causal ? min(p.T - 1, p.causal_offset + l) : p.T - 1) : -1;
#pragma unroll
            for (int gr = 0; gr < G; ++gr) qsum[half][gr] = 0.f;
        }
#pragma unroll
        for (int gr = 0; gr < G; ++gr) {
#pragma unroll
            for (int m = 0; m < MPG; ++m) {
                const int wl = m / MPW, which = m % MPW;
                int dd[4];
                kslot_dims<BITS>(gr * WPG + c * WPL + wl, which, dd);
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int r = g + 8 * half;
                    float x[4] = {0.f, 0.f, 0.f, 0.f};
                    if (r < R) {
                        const int hq = hk * rep + r / p.L, l = r % p.L;
                        const T *qp = (const T *)p.q + b * p.q_sb + hq * p.q_sh + l * p.q_sl;
#pragma unroll
                        for (int k = 0; k < 4; ++k) x[k] = __half2float(__float2half_rn(to_f32<T>(qp[dd[k]])));
                    }
                    qa[gr][m][half] = pack_h2(x[0], x[1]);      // a0 / a1
                    qa[gr][m][2 + half] = pack_h2(x[2], x[3]);  // a2 / a3
                    qsum[half][gr] += x[0] + x[1] + x[2] + x[3];
                }
            }
        }
#pragma unroll
        for (int half = 0; half < 2; ++half)
#pragma unroll
            for (int gr = 0; gr < G; ++gr) {
                qsum[half][gr] += __shfl_xor_sync(0xffffffffu, qsum[half][gr], 1);
                qsum[half][gr] += __shfl_xor_sync(0xffffffffu, qsum[half][gr], 2);
            }

        const int blk = warp;
        // ldmatrix row address of this lane inside a V code tile: matrix mi = lane / 8
        const int v_tok = blk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
        const int v_chunk_off = (lane >> 4);  // 0 or 1: second chunk of the pair

        for (int it = 0; it < ntiles && ok; ++it) {
            const int s = it % NSTAGE;
            ok = mbar_wait(&full[s], (it / NSTAGE) & 1);
            if (!ok) break;
            const unsigned char *st = stages + (size_t)s * STAGE_BYTES;
            const unsigned char *kct = st;
            const unsigned char *vct = st + CODE_TILE;
            const T *kst = (const T *)(st + 2 * CODE_TILE);
            const T *kbt = (const T *)(st + 2 * CODE_TILE + SC_TILE);
            const T *vst = (const T *)(st + 2 * CODE_TILE + 2 * SC_TILE);
            const T *vbt = (const T *)(st + 2 * CODE_TILE + 3 * SC_TILE);
            const int64_t t_blk = (int64_t)(tile_begin + it) * PK_TILE + blk * 16;

            // ---- integer dot products q . c per group, two n-tiles of 8 tokens ----
            float acc[2][G][4];
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int gr = 0; gr < G; ++gr) acc[j][gr][0] = acc[j][gr][1] = acc[j][gr][2] = acc[j][gr][3] = 0.f;
#pragma unroll
            for (int gr = 0; gr < G; ++gr) {
                uint32_t w[2][WPL];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const uint32_t *wp = (const uint32_t *)(kct + (blk * 16 + j * 8 + g) * RB) + gr * WPG + c * WPL;
#pragma unroll
                    for (int k = 0; k < WPL; ++k) w[j][k] = wp[k];
                }
#pragma unroll
                for (int m = 0; m < MPG; ++m) {
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        uint32_t b0, b1;
                        code_pair<BITS>(w[j][m / MPW], m % MPW, b0, b1);
                        mma_f16(acc[j][gr], qa[gr][m], b0, b1);
                    }
                }
            }
            // ---- scores = s * acc + b * sum(q), masked, in the log2 domain ----
            float sc[2][4];
            float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < 2; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int half = e >> 1;
                    const int tl = blk * 16 + j * 8 + 2 * c + (e & 1);  // token inside the tile
                    float v = 0.f;
#pragma unroll
                    for (int gr = 0; gr < G; ++gr)
                        v += to_f32<T>(kst[tl * G + gr]) * acc[j][gr][e] + to_f32<T>(kbt[tl * G + gr]) * qsum[half][gr];
                    v *= p.scale_log2;
                    const int64_t t = t_blk + j * 8 + 2 * c + (e & 1);
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
            float pr[2][4];
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int half = e >> 1;
                    pr[j][e] = (m_run[half] == -INFINITY) ? 0.f : fast_exp2(sc[j][e] - m_run[half]);
                }
            const bool rescale = __any_sync(0xffffffffu, (alpha[0] != 1.f) | (alpha[1] != 1.f));
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                l_run[half] = l_run[half] * alpha[half] + pr[0][2 * half] + pr[0][2 * half + 1] + pr[1][2 * half] +
                              pr[1][2 * half + 1];
            }
            if (rescale) {
#pragma unroll
                for (int nt = 0; nt < NT_O; ++nt) {
                    o_acc[nt][0] *= alpha[0];
                    o_acc[nt][1] *= alpha[0];
                    o_acc[nt][2] *= alpha[1];
                    o_acc[nt][3] *= alpha[1];
                }
#pragma unroll
                for (int gr = 0; gr < G; ++gr) {
                    bsum[0][gr] *= alpha[0];
                    bsum[1][gr] *= alpha[1];
                }
            }
            // ---- per-group A fragments p * s_v, and the bias sums ----
            uint32_t pa[G][4];
#pragma unroll
            for (int gr = 0; gr < G; ++gr) {
                float sv[2][2], bv[2][2];  // [n-tile j][token 2c + 0/1]
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int k = 0; k < 2; ++k) {
                        const int tl = blk * 16 + j * 8 + 2 * c + k;
                        sv[j][k] = to_f32<T>(vst[tl * G + gr]);
                        bv[j][k] = to_f32<T>(vbt[tl * G + gr]);
                    }
                pa[gr][0] = pack_h2(pr[0][0] * sv[0][0], pr[0][1] * sv[0][1]);
                pa[gr][1] = pack_h2(pr[0][2] * sv[0][0], pr[0][3] * sv[0][1]);
                pa[gr][2] = pack_h2(pr[1][0] * sv[1][0], pr[1][1] * sv[1][1]);
                pa[gr][3] = pack_h2(pr[1][2] * sv[1][0], pr[1][3] * sv[1][1]);
                bsum[0][gr] += pr[0][0] * bv[0][0] + pr[0][1] * bv[0][1] + pr[1][0] * bv[1][0] + pr[1][1] * bv[1][1];
                bsum[1][gr] += pr[0][2] * bv[0][0] + pr[0][3] * bv[0][1] + pr[1][2] * bv[1][0] + pr[1][3] * bv[1][1];
            }
            // ---- O += (p s) . codes: ldmatrix.trans hands out token pairs per 16-bit unit ----
            const uint32_t v_row = smem_u32(vct + v_tok * RB);
#pragma unroll
            for (int cp = 0; cp < CH / 2; ++cp) {
                uint32_t vf[4];
                ldmatrix_x4_trans(vf, v_row + (2 * cp + v_chunk_off) * 16);
#pragma unroll
                for (int q2 = 0; q2 < 2; ++q2) {
                    const int chunk = 2 * cp + q2;
                    constexpr int dims_per_chunk = 8 * EPU;
                    const int gr = (chunk * dims_per_chunk) / GROUP;
#pragma unroll
                    for (int i = 0; i < EPU; ++i) {
                        uint32_t b0, b1;
                        if (BITS == 4) {
                            b0 = hsub2_1024(((vf[2 * q2] >> (4 * i)) & 0x000F000Fu) | 0x64006400u);
                            b1 = hsub2_1024(((vf[2 * q2 + 1] >> (4 * i)) & 0x000F000Fu) | 0x64006400u);
                        } else {
                            const uint32_t sel = i ? 0x4341u : 0x4240u;
                            b0 = hsub2_1024(__byte_perm(vf[2 * q2], 0x64646464u, sel));
                            b1 = hsub2_1024(__byte_perm(vf[2 * q2 + 1], 0x64646464u, sel));
                        }
                        mma_f16(o_acc[chunk * EPU + i], pa[gr], b0, b1);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }
        if (!ok && lane == 0) atomicExch(p.status, 4);
    }

    // ---------------- merge the consumer warps, then the splits ----------------
    __syncthreads();
    float *red_o = (float *)stages;
    float *red_ml = red_o + PK_WARPS * 16 * RED_STRIDE;
    if (warp < PK_WARPS) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            l_run[half] += __shfl_xor_sync(0xffffffffu, l_run[half], 1);
            l_run[half] += __shfl_xor_sync(0xffffffffu, l_run[half], 2);
#pragma unroll
            for (int gr = 0; gr < G; ++gr) {
                bsum[half][gr] += __shfl_xor_sync(0xffffffffu, bsum[half][gr], 1);
                bsum[half][gr] += __shfl_xor_sync(0xffffffffu, bsum[half][gr], 2);
            }
        }
        float *wo = red_o + warp * 16 * RED_STRIDE;
#pragma unroll
        for (int nt = 0; nt < NT_O; ++nt) {
            // n-tile nt = chunk * EPU + i: columns 2c, 2c+1 <-> dims chunk*8*EPU + EPU*col + i
            const int chunk = nt / EPU, i = nt % EPU;
            const int d0 = chunk * 8 * EPU + EPU * (2 * c) + i, d1 = d0 + EPU;
            const int gr = d0 / GROUP;
            wo[g * RED_STRIDE + d0] = o_acc[nt][0] + bsum[0][gr];
            wo[g * RED_STRIDE + d1] = o_acc[nt][1] + bsum[0][gr];
            wo[(g + 8) * RED_STRIDE + d0] = o_acc[nt][2] + bsum[1][gr];
            wo[(g + 8) * RED_STRIDE + d1] = o_acc[nt][3] + bsum[1][gr];
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
    float *work = red_ml + PK_WARPS * 16 * 2;
    unit_epilogue<D, PK_WARPS>(u, red_o, red_ml, RED_STRIDE, work, is_last, b, hk, rep, R, split, bh);
}

// ---------------------------------------------------------------------
// Decode orientation (at most 8 query rows per KV head, i.e. GQA ratio <= 8
// with one new token): the MMAs are transposed so that tokens (for Q.K^T) and
// head dims (for P.V) fill the 16-row M side and the query rows the 8-column N
// side. Compared with the kernel above this halves the MMA count and the
// accumulator registers (three or four CTAs per SM instead of two), which is what the
// latency-bound conversion chain needs.
//   S^T[16 tok x 8 rows]  = K[16 tok x 16 d] . Q^T[16 d x 8 rows]      (A = codes)
//   O^T[16 d  x 8 rows]  += V^T[16 d x 16 tok] . P'^T[16 tok x 8 rows]  (A = codes via ldmatrix.trans)
// P'^T reaches its B-fragment layout with movmatrix (an 8x8 transpose across
// the warp).
//
// The loop is bound by instruction issue (integer pipe first), not by the tensor
// pipe, so every step is written for instruction count:
//   * codes become f16 operands with one mask-or per operand register and one
//     shift per word (CodeWord / UnitPair below);
//   * the masked bits are used as they are, as f16 SUBNORMALS (n * 2^-24 or n * 2^-20):
//     exact, no offset to cancel and no second instruction; the power of two is folded
//     into the query fragments / the exponential (K side) and the epilogue (V side);
//   * the query is pre-multiplied by scale * log2(e), scores come out of the MMA in
//     the exp2 domain;
//   * the running maximum is lazy: a tile only takes the shuffle-reduce / rescale
//     path when one of its scores exceeds the running maximum by more than 2^8,
//     otherwise probabilities are exp2(score - stale max) <= 256, well inside f16;
//   * the causal / length mask is only evaluated on the tiles that cross a limit.
// ---------------------------------------------------------------------
// ---- code words -> f16 operand pairs without per-element shifts ----
// 4-bit: a word holds nibbles n0..n7. Masking a nibble in place under the exponent of
// 64.0 (0x5400, ulp 1/16) gives  64 + n/16  for the nibbles at bits 0..3 of a half
// ("low" pairs) and  64 + n  for those at bits 4..7 ("high" pairs); one shift by 8
// brings the other two nibbles of each half into reach. Pair k of a word:
//   k = 0: (n0, n4) low    k = 1: (n1, n5) high    k = 2: (n2, n6) low    k = 3: (n3, n7) high
// 8-bit: bytes under the exponent of 1024.0 (0x6400, ulp 1): 1024 + n, pairs (b0,b1), (b2,b3).
template <int BITS>
struct CodeWord {
    uint32_t w, w8;
    __device__ __forceinline__ explicit CodeWord(uint32_t word) : w(word), w8(BITS == 4 ? (word >> 8) : 0u) {}
    // pair k of the word, still carrying its offset (and the 1/16 factor of low pairs)
    __device__ __forceinline__ uint32_t raw(int k) const {
        if (BITS == 4) {
            const uint32_t x = (k & 2) ? w8 : w;
            return (k & 1) ? ((x & 0x00F000F0u) | 0x54005400u) : ((x & 0x000F000Fu) | 0x54005400u);
        }
        return __byte_perm(w, 0x64646464u, k ? 0x4342 : 0x4140);
    }
    // pair k as f16 SUBNORMALS: the masked bits alone are n * 2^-24 (nibbles at bits 0..3 of a
    // half, bytes) or n * 2^-20 (nibbles at bits 4..7): exact, no offset, one instruction.
    // The tensor core takes subnormal f16 inputs at full precision; the power-of-two factor
    // is constant per k-slot (K side) or per output tile (V side) and is applied elsewhere.
    __device__ __forceinline__ uint32_t sub(int k) const {
        if (BITS == 4) {
            const uint32_t x = (k & 2) ? w8 : w;
            return (k & 1) ? (x & 0x00F000F0u) : (x & 0x000F000Fu);
        }
        return __byte_perm(w, 0u, k ? 0x4342 : 0x4140);
    }
    // pair k as exact integer codes in f16
    __device__ __forceinline__ uint32_t exact(int k) const {
        const uint32_t x = raw(k);
        uint32_t r;
        if (BITS == 4) {
            if (k & 1) asm("add.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(x), "r"(0xD400D400u));             // - 64
            else asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(x), "r"(0x4C004C00u), "r"(0xE400E400u));  // * 16 - 1024
        } else {
            asm("add.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(x), "r"(0xE400E400u));                       // - 1024
        }
        return r;
    }
};

// The register ldmatrix.trans returns from a V code tile holds two 16-bit units (token 2c in
// the low half, token 2c+1 in the high half); element i of both units as exact f16 codes.
// 4-bit units hold 4 elements (same nibble positions as above), 8-bit units 2.
template <int BITS>
struct UnitPair {
    uint32_t v, v8;
    __device__ __forceinline__ explicit UnitPair(uint32_t reg) : v(reg), v8(BITS == 4 ? (reg >> 8) : 0u) {}
    // element i of both units as f16 subnormals (see CodeWord::sub): n * 2^-24, or n * 2^-20
    // for the odd elements of 4-bit units
    __device__ __forceinline__ uint32_t sub(int i) const {
        if (BITS == 4) {
            const uint32_t src = (i & 2) ? v8 : v;
            return (i & 1) ? (src & 0x00F000F0u) : (src & 0x000F000Fu);
        }
        return __byte_perm(v, 0u, i ? 0x4341 : 0x4240);
    }
    __device__ __forceinline__ uint32_t exact(int i) const {
        uint32_t x, r;
        if (BITS == 4) {
            const uint32_t src = (i & 2) ? v8 : v;
            if (i & 1) {
                x = (src & 0x00F000F0u) | 0x54005400u;
                asm("add.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(x), "r"(0xD400D400u));
            } else {
                x = (src & 0x000F000Fu) | 0x54005400u;
                asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(x), "r"(0x4C004C00u), "r"(0xE400E400u));
            }
        } else {
            x = __byte_perm(v, 0x64646464u, i ? 0x4341 : 0x4240);
            asm("add.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(x), "r"(0xE400E400u));
        }
        return r;
    }
};

// Two consecutive scale / bias elements (storage dtype T) as floats.
template <typename T> __device__ __forceinline__ float2 unpack_pair(uint32_t w);
template <> __device__ __forceinline__ float2 unpack_pair<__nv_bfloat16>(uint32_t w) {
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
}
template <> __device__ __forceinline__ float2 unpack_pair<__half>(uint32_t w) {
    return __half22float2(*reinterpret_cast<const __half2 *>(&w));
}

// The G group values of token `tok` from a [tokens][G] tile in shared memory.
template <typename T, int G>
__device__ __forceinline__ void load_groups(const T *tile, int tok, float (&out)[G]) {
    if (G == 1) {
        out[0] = to_f32<T>(tile[tok]);
    } else {
        const uint32_t *p32 = reinterpret_cast<const uint32_t *>(tile + tok * G);
#pragma unroll
        for (int i = 0; i < G / 2; ++i) {
            const float2 f = unpack_pair<T>(p32[i]);
            out[2 * i] = f.x;
            out[2 * i + 1] = f.y;
        }
    }
}

// N consecutive 32-bit words from shared memory with the widest loads the count allows.
template <int N>
__device__ __forceinline__ void load_words(const uint32_t *src, uint32_t (&dst)[N]) {
    if (N % 4 == 0) {
#pragma unroll
        for (int i = 0; i < N / 4; ++i) {
            const uint4 x = reinterpret_cast<const uint4 *>(src)[i];
            dst[4 * i] = x.x; dst[4 * i + 1] = x.y; dst[4 * i + 2] = x.z; dst[4 * i + 3] = x.w;
        }
    } else if (N % 2 == 0) {
#pragma unroll
        for (int i = 0; i < N / 2; ++i) {
            const uint2 x = reinterpret_cast<const uint2 *>(src)[i];
            dst[2 * i] = x.x; dst[2 * i + 1] = x.y;
        }
    } else {
#pragma unroll
        for (int i = 0; i < N; ++i) dst[i] = src[i];
    }
}

// Flat tile x -> the unit (batch or sequence `b`, KV head `hk`) it belongs to, the tile index inside
// the unit and the unit's tile count.
template <bool VARLEN, int TILE>
__device__ __forceinline__ void resolve_unit(const AffineParams &p, const VarlenAttnTable &vt, int64_t x, int tiles,
                                             int &unit, int &tile, int &utiles, int &hk, int &b) {
    if (!VARLEN) {
        unit = (int)(x / tiles);
        tile = (int)(x % tiles);
        utiles = tiles;
        const int bh = unit / p.chunks;   // a group of more than eight query rows is cut into units of eight
        hk = bh % p.Hkv;
        b = bh / p.Hkv;
        return;
    }
    int i = 0;
    for (int step = 16; step >= 1; step >>= 1)   // largest i with Hkv * tile_prefix[i] <= x
        if (i + step < vt.n && (int64_t)p.Hkv * vt.seq[i + step].tile_prefix <= x) i += step;
    const int64_t base = (int64_t)p.Hkv * vt.seq[i].tile_prefix;
    utiles = (vt.seq[i].T + TILE - 1) / TILE;
    hk = (int)((x - base) / utiles);
    tile = (int)((x - base) % utiles);
    b = i;
    unit = i * p.Hkv + hk;
}

template <typename T, int D, int BITS, int GROUP, int NSTAGE, int MINB, bool VARLEN, int NW>
__global__ void __launch_bounds__((NW + 1) * 32, MINB)
attn_affine_decode8_kernel(const AffineParams p, const __grid_constant__ VarlenAttnTable vt) {
    constexpr int P8_WARPS = NW, P8_TILE = NW * 16;
    constexpr int G = D / GROUP;
    constexpr int RB = D * BITS / 8;
    constexpr int WPR = RB / 4;
    constexpr int WPG = GROUP * BITS / 32;
    constexpr int WPL = WPG / 4;
    constexpr int MPW = (BITS == 4) ? 2 : 1;
    constexpr int MPG = WPL * MPW;
    constexpr int SB = G * 2;
    constexpr int CODE_TILE = P8_TILE * RB;
    constexpr int SC_TILE = P8_TILE * SB;
    constexpr int STAGE_BYTES = 2 * CODE_TILE + 4 * SC_TILE;
    constexpr int EPU = 16 / BITS;
    constexpr int CH = RB / 16;
    constexpr int MT_O = D / 16;                  // output m-tiles (16 head dims each)
    constexpr int RED_STRIDE = D + 8;
    static_assert(WPL >= 1 && G >= 1 && G <= 4, "unsupported group layout");
    static_assert((2 * 8 * EPU) <= GROUP, "a pair of 16-byte chunks must stay inside one group");
    static_assert(STAGE_BYTES % 16 == 0 && SC_TILE % 16 == 0, "bulk copies need 16-byte multiples");

    extern __shared__ __align__(128) unsigned char smem_raw[];
    // pointer + offset (no integer round trip) so that loads through it stay ld.shared
    unsigned char *stages = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
    constexpr int RING = NSTAGE * STAGE_BYTES;
    const FlatPlan &fp = p.flat;
    uint64_t *full = (uint64_t *)(stages + ((RING + 15) / 16) * 16);
    uint64_t *empty = full + NSTAGE;
    int *is_last = (int *)(empty + NSTAGE);
    // cross-warp buffers beside the ring (the ring stays live across segments)
    float *red_o = (float *)(is_last + 4);                               // [4][red_rows][RED_STRIDE]
    float *red_ml = red_o + P8_WARPS * fp.red_rows * RED_STRIDE;         // [4][red_rows][2]
    // the buffers behind keep 16-byte alignment (the staged query rows are a bulk-copy destination)
    float *work = red_ml + ((P8_WARPS * fp.red_rows * 2 + 3) & ~3);      // [red_rows][nslots]
    // query rows of a segment's unit, brought in by the producer with one bulk copy (two buffers)
    uint64_t *qfull = (uint64_t *)(work + ((fp.red_rows * fp.nslots + 3) & ~3));
    uint64_t *qempty = qfull + 2;
    unsigned char *qbuf = (unsigned char *)(qempty + 2);                  // [2][red_rows][D] elements

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rep = p.Hq / p.Hkv;
    const int R_all = rep * p.L;   // query rows of a (batch, kv head) group; a unit carries up to eight of them
    const int tiles = fp.tiles;
    const int64_t x_lo = flat_lo(fp, blockIdx.x), x_hi = flat_lo(fp, blockIdx.x + 1);
    const uint32_t q_bytes = (uint32_t)R_all * D * 2;   // bulk staging only runs with one unit per group

    if (tid == 0) {
        for (int s = 0; s < NSTAGE; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], P8_WARPS);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&qfull[s], 1);
            mbar_init(&qempty[s], P8_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (256 % P8_TILE != 0) {
        // a cut-short last tile leaves the end of its stage as it was: start from zeros, so that what the
        // masked tokens multiply is always finite
        for (int i = tid; i < RING / 16; i += (NW + 1) * 32) ((uint4 *)stages)[i] = make_uint4(0u, 0u, 0u, 0u);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    pdl_wait();  // everything below reads what earlier kernels on the stream wrote

    bool ok = true;
    const int g = lane >> 2, c = lane & 3;

    if (warp == P8_WARPS) {
        // ---------------- producer: one stream of tiles across the segments ----------------
        if (lane == 0) {
            int it = 0, sg = 0;
            for (int64_t x = x_lo; x < x_hi && ok; ++sg) {
                int unit, tb, utiles, hk, b;
                resolve_unit<VARLEN, P8_TILE>(p, vt, x, tiles, unit, tb, utiles, hk, b);
                const int n = (int)min((int64_t)(utiles - tb), x_hi - x);
                if (p.q_bulk) {
                    const int qb = sg & 1;
                    if (sg >= 2) ok = mbar_wait(&qempty[qb], ((sg >> 1) - 1) & 1);
                    if (!ok) break;
                    const T *qsrc = VARLEN ? (const T *)vt.seq[b].q + (int64_t)hk * rep * p.q_sh
                                           : (const T *)p.q + b * p.q_sb + (int64_t)hk * rep * p.q_sh;
                    mbar_expect_tx(&qfull[qb], q_bytes);
                    bulk_load(qbuf + (size_t)qb * q_bytes, qsrc, q_bytes, &qfull[qb]);
                }
                const uint32_t *kc, *vc;
                const T *ks, *kb, *vs, *vb;
                if (VARLEN) {
                    const VarlenAttnSeq &sq = vt.seq[b];
                    kc = sq.kc + hk * sq.c_sh; vc = sq.vc + hk * sq.c_sh;
                    ks = (const T *)sq.ks + hk * sq.g_sh; kb = (const T *)sq.kb + hk * sq.g_sh;
                    vs = (const T *)sq.vs + hk * sq.g_sh; vb = (const T *)sq.vb + hk * sq.g_sh;
                } else {
                    kc = p.kc + b * p.kc_sb + hk * p.kc_sh;
                    vc = p.vc + b * p.vc_sb + hk * p.vc_sh;
                    ks = (const T *)p.ks + b * p.kg_sb + hk * p.kg_sh;
                    kb = (const T *)p.kb + b * p.kg_sb + hk * p.kg_sh;
                    vs = (const T *)p.vs + b * p.vg_sb + hk * p.vg_sh;
                    vb = (const T *)p.vb + b * p.vg_sb + hk * p.vg_sh;
                }
                // tokens of this unit that copies may touch: the stored rows rounded up to 256 (inside the
                // slab by the launch checks); a tile of 240 tokens may end past them and is then cut short
                const int64_t t_pad = ((VARLEN ? (int64_t)vt.seq[b].T : p.T) + 255) / 256 * 256;
                for (int j = 0; j < n && ok; ++j, ++it) {
                    const int s = it % NSTAGE;
                    if (it >= NSTAGE) ok = mbar_wait(&empty[s], ((it / NSTAGE) - 1) & 1);
                    if (!ok) break;
                    unsigned char *st = stages + (size_t)s * STAGE_BYTES;
                    const int64_t t0 = (int64_t)(tb + j) * P8_TILE;
                    const uint32_t rows = (uint32_t)min((int64_t)P8_TILE, t_pad - t0);
                    mbar_expect_tx(&full[s], rows * (2 * RB + 4 * SB));
                    bulk_load(st, kc + t0 * WPR, rows * RB, &full[s]);
                    bulk_load(st + CODE_TILE, vc + t0 * WPR, rows * RB, &full[s]);
                    bulk_load(st + 2 * CODE_TILE, ks + t0 * G, rows * SB, &full[s]);
                    bulk_load(st + 2 * CODE_TILE + SC_TILE, kb + t0 * G, rows * SB, &full[s]);
                    bulk_load(st + 2 * CODE_TILE + 2 * SC_TILE, vs + t0 * G, rows * SB, &full[s]);
                    bulk_load(st + 2 * CODE_TILE + 3 * SC_TILE, vb + t0 * G, rows * SB, &full[s]);
                }
                x += n;
            }
            if (!ok) atomicExch(p.status, 5);
        }
        return;
    }

    // ---------------- consumers: one segment per unit the CTA's tile range touches ----------------
    int st_i = 0;          // ring stage of the next tile and its phase bit, carried across segments
    uint32_t st_ph = 0;
    int sg = 0;
    for (int64_t x = x_lo; x < x_hi; ++sg) {
        int unit, tile_begin, utiles, hk, b;
        resolve_unit<VARLEN, P8_TILE>(p, vt, x, tiles, unit, tile_begin, utiles, hk, b);
        const int ntiles = (int)min((int64_t)(utiles - tile_begin), x_hi - x);
        const int64_t T_seq = VARLEN ? (int64_t)vt.seq[b].T : p.T;   // tokens of this unit's sequence
        const int row0 = VARLEN ? 0 : (unit % p.chunks) * 8;         // first query row of the group this unit carries
        const int R = min(8, R_all - row0);
        // per-lane state for query rows 2c and 2c+1
        float m_run[2], l_run[2] = {0.f, 0.f};
        float bsum[2][G];
        float o_acc[MT_O][4];
#pragma unroll
        for (int i = 0; i < MT_O; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int gr = 0; gr < G; ++gr) bsum[h][gr] = 0.f;
        // Q^T fragments: B operand column = query row g; k-slots follow the code words.
        // q' = f16(q * scale * log2 e). The code operands are f16 subnormals n * 2^-24 (or
        // n * 2^-20 for the nibbles at bits 4..7): the k-slots fed by the smaller form carry
        // 16 q', so every product is n q' 2^-20 (4-bit) or n q' 2^-24 (8-bit) = n q' / KSCALE.
        constexpr float LOWMUL = (BITS == 4) ? 16.f : 1.f;
        constexpr float KSCALE = (BITS == 4) ? 1048576.f : 16777216.f;
        const T *q_stage = nullptr;   // the unit's rows [R][D] in shared memory when the producer staged them
        if (p.q_bulk) {
            const int qslot = sg & 1;
            if (ok) {
                ok = mbar_wait(&qfull[qslot], (sg >> 1) & 1);
                if (!ok && lane == 0) atomicExch(p.status, 14);
            }
            q_stage = (const T *)(qbuf + (size_t)qslot * q_bytes);
        }
        uint32_t qb[G][MPG][2];
        float qsum_own[G];
#pragma unroll
        for (int gr = 0; gr < G; ++gr) qsum_own[gr] = 0.f;
#pragma unroll
        for (int gr = 0; gr < G; ++gr) {
#pragma unroll
            for (int m = 0; m < MPG; ++m) {
                int dd[4];
                kslot_dims<BITS>(gr * WPG + c * WPL + m / MPW, m % MPW, dd);
                float x[4] = {0.f, 0.f, 0.f, 0.f};
                if (g < R && ok) {
                    const int hq = hk * rep + (row0 + g) / p.L, l = (row0 + g) % p.L;
                    const T *qp = q_stage ? q_stage + g * D
                                  : VARLEN ? (const T *)vt.seq[b].q + hq * p.q_sh + l * p.q_sl
                                           : (const T *)p.q + b * p.q_sb + hq * p.q_sh + l * p.q_sl;
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        x[k] = __half2float(__float2half_rn(to_f32<T>(qp[dd[k]]) * p.scale_log2));
                }
                qb[gr][m][0] = pack_h2(x[0] * LOWMUL, x[1] * LOWMUL);   // k-slots 2c, 2c+1
                qb[gr][m][1] = pack_h2(x[2], x[3]);                     // k-slots 2c+8, 2c+9
                qsum_own[gr] += x[0] + x[1] + x[2] + x[3];
            }
        }
        // sum(q') / KSCALE of rows 2c, 2c+1: multiplies the bias; scores stay in units of
        // 1 / KSCALE until the exponential.
        float qsum[2][G];
#pragma unroll
        for (int gr = 0; gr < G; ++gr) {
            float v = qsum_own[gr];
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            v *= (1.f / KSCALE);
            qsum[0][gr] = __shfl_sync(0xffffffffu, v, (2 * c) * 4);
            qsum[1][gr] = __shfl_sync(0xffffffffu, v, (2 * c + 1) * 4);
        }
        if (p.q_bulk) {
            __syncwarp();
            if (ok && lane == 0) mbar_arrive(&qempty[sg & 1]);
        }
        // Last visible token per row. Rows past R hold zero queries and are never written
        // out; they take the limit of a real row so that they do not force the mask path.
        int row_limit[2];
        const int t_last = (int)(T_seq - 1);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int r = 2 * c + k;
            const int l = (r < R) ? (row0 + r) % p.L : 0;
            row_limit[k] = p.causal ? (int)min((int64_t)t_last, p.causal_offset + l) : t_last;
        }
        const int min_limit = p.causal ? (int)min((int64_t)t_last, p.causal_offset) : t_last;
        constexpr float M_INIT = -1e30f, LAZY = 8.f;
        m_run[0] = m_run[1] = M_INIT;
        float m_thr[2] = {M_INIT, M_INIT};  // (m_run + LAZY) / KSCALE once a maximum exists

        const int blk = warp;
        // ldmatrix rows: matrix mi = lane / 8 -> tokens (mi >> 1) * 8 + lane % 8, chunk parity mi & 1
        const int v_tok = blk * 16 + ((lane >> 4) & 1) * 8 + (lane & 7);
        const int v_chunk_off = (lane >> 3) & 1;
        const int tl0 = blk * 16 + g, tl1 = tl0 + 8;  // this lane's two tokens inside a tile
        const uint32_t k_off0 = tl0 * RB + c * WPL * 4, k_off1 = tl1 * RB + c * WPL * 4;
        const uint32_t v_off = v_tok * RB + v_chunk_off * 16;

        for (int jt = 0; jt < ntiles; ++jt, st_i = (st_i + 1 == NSTAGE) ? 0 : st_i + 1, st_ph ^= (st_i == 0)) {
            if (!ok) continue;  // a wait ran out earlier: walk on to the segment's barriers
            const int s = st_i;
            ok = mbar_wait(&full[s], st_ph);
            if (!ok) {
                if (lane == 0) atomicExch(p.status, 6);
                continue;
            }
            if (KVC_SKIP_BITS(p) & 1) {
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
                continue;
            }
            const unsigned char *st = stages + (size_t)s * STAGE_BYTES;
            const unsigned char *kct = st;
            const unsigned char *vct = st + CODE_TILE;
            const T *kst = (const T *)(st + 2 * CODE_TILE);
            const T *kbt = (const T *)(st + 2 * CODE_TILE + SC_TILE);
            const T *vst = (const T *)(st + 2 * CODE_TILE + 2 * SC_TILE);
            const T *vbt = (const T *)(st + 2 * CODE_TILE + 3 * SC_TILE);
            const int t_blk = (tile_begin + jt) * P8_TILE + blk * 16;
            if (KVC_SKIP_BITS(p) & 6) {
                // measurement aid (results are meaningless): 2 = only the K half, 4 = only the V half
                if (KVC_SKIP_BITS(p) & 2) {
#pragma unroll
                    for (int gr = 0; gr < G; ++gr) {
                        uint32_t wa[WPL], wb[WPL];
                        load_words<WPL>((const uint32_t *)(kct + k_off0) + gr * WPG, wa);
                        load_words<WPL>((const uint32_t *)(kct + k_off1) + gr * WPG, wb);
#pragma unroll
                        for (int wi = 0; wi < WPL; ++wi) {
                            const CodeWord<BITS> ca(wa[wi]), cb(wb[wi]);
#pragma unroll
                            for (int which = 0; which < MPW; ++which) {
                                uint32_t a[4] = {ca.exact(2 * which), cb.exact(2 * which), ca.exact(2 * which + 1),
                                                 cb.exact(2 * which + 1)};
                                mma_f16(o_acc[gr], a, qb[gr][wi * MPW + which][0], qb[gr][wi * MPW + which][1]);
                            }
                        }
                    }
                }
                if (KVC_SKIP_BITS(p) & 4) {
                    const uint32_t v_row = smem_u32(vct + v_off);
#pragma unroll
                    for (int cp = 0; cp < CH / 2; ++cp) {
                        uint32_t vf[4];
                        ldmatrix_x4_trans(vf, v_row + cp * 32);
                        const UnitPair<BITS> u0(vf[0]), u1(vf[1]), u2(vf[2]), u3(vf[3]);
#pragma unroll
                        for (int i = 0; i < EPU; ++i) {
                            uint32_t a[4] = {u0.exact(i), u1.exact(i), u2.exact(i), u3.exact(i)};
                            mma_f16(o_acc[cp * EPU + i], a, qb[0][0][0], qb[0][0][1]);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
                continue;
            }

            // ---- S^T = codes . Q'^T per group ----
            float acc[G][4];
#pragma unroll
            for (int gr = 0; gr < G; ++gr) {
                acc[gr][0] = acc[gr][1] = acc[gr][2] = acc[gr][3] = 0.f;
                uint32_t wa[WPL], wb[WPL];
                load_words<WPL>((const uint32_t *)(kct + k_off0) + gr * WPG, wa);
                load_words<WPL>((const uint32_t *)(kct + k_off1) + gr * WPG, wb);
#pragma unroll
                for (int wi = 0; wi < WPL; ++wi) {
                    const CodeWord<BITS> ca(wa[wi]), cb(wb[wi]);
#pragma unroll
                    for (int which = 0; which < MPW; ++which) {
                        uint32_t a[4];
                        a[0] = ca.sub(2 * which);       // token g,   k-slots 2c, 2c+1
                        a[1] = cb.sub(2 * which);       // token g+8
                        a[2] = ca.sub(2 * which + 1);   // token g,   k-slots 2c+8, 2c+9
                        a[3] = cb.sub(2 * which + 1);   // token g+8
                        mma_f16(acc[gr], a, qb[gr][wi * MPW + which][0], qb[gr][wi * MPW + which][1]);
                    }
                }
            }
            // ---- scores in the exp2 domain, in units of 1 / KSCALE: s * acc + b * sum(q') / KSCALE ----
            float sc[4] = {0.f, 0.f, 0.f, 0.f};
            {
                float s0[G], s1[G], b0[G], b1[G];
                load_groups<T, G>(kst, tl0, s0);
                load_groups<T, G>(kst, tl1, s1);
                load_groups<T, G>(kbt, tl0, b0);
                load_groups<T, G>(kbt, tl1, b1);
#pragma unroll
                for (int gr = 0; gr < G; ++gr) {
                    sc[0] = fmaf(s0[gr], acc[gr][0], fmaf(b0[gr], qsum[0][gr], sc[0]));
                    sc[1] = fmaf(s0[gr], acc[gr][1], fmaf(b0[gr], qsum[1][gr], sc[1]));
                    sc[2] = fmaf(s1[gr], acc[gr][2], fmaf(b1[gr], qsum[0][gr], sc[2]));
                    sc[3] = fmaf(s1[gr], acc[gr][3], fmaf(b1[gr], qsum[1][gr], sc[3]));
                }
            }
            if (t_blk + 15 > min_limit) {  // warp-uniform: only tiles that cross a limit
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int t = t_blk + g + ((e >> 1) ? 8 : 0);
                    if (t > row_limit[e & 1]) sc[e] = -INFINITY;
                }
            }
            // ---- lazy running maximum ----
            {
                const float mx0 = fmaxf(sc[0], sc[2]), mx1 = fmaxf(sc[1], sc[3]);
                if (__any_sync(0xffffffffu, (mx0 > m_thr[0]) | (mx1 > m_thr[1]))) {
                    float mx[2] = {mx0, mx1}, alpha[2];
#pragma unroll
                    for (int k = 0; k < 2; ++k) {
                        mx[k] = fmaxf(mx[k], __shfl_xor_sync(0xffffffffu, mx[k], 4));
                        mx[k] = fmaxf(mx[k], __shfl_xor_sync(0xffffffffu, mx[k], 8));
                        mx[k] = fmaxf(mx[k], __shfl_xor_sync(0xffffffffu, mx[k], 16));
                        const float m_new = fmaxf(m_run[k], mx[k] * KSCALE);
                        alpha[k] = fast_exp2(m_run[k] - m_new);
                        m_run[k] = m_new;
                        m_thr[k] = (m_new > M_INIT) ? (m_new + LAZY) * (1.f / KSCALE) : M_INIT;
                        l_run[k] *= alpha[k];
                    }
#pragma unroll
                    for (int mt = 0; mt < MT_O; ++mt) {
                        o_acc[mt][0] *= alpha[0];
                        o_acc[mt][1] *= alpha[1];
                        o_acc[mt][2] *= alpha[0];
                        o_acc[mt][3] *= alpha[1];
                    }
#pragma unroll
                    for (int gr = 0; gr < G; ++gr) {
                        bsum[0][gr] *= alpha[0];
                        bsum[1][gr] *= alpha[1];
                    }
                }
            }
            float pr[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) pr[e] = fast_exp2(fmaf(sc[e], KSCALE, -m_run[e & 1]));
            l_run[0] += pr[0] + pr[2];
            l_run[1] += pr[1] + pr[3];
            // ---- P'^T = (p * s_v)^T per group, moved to the B-fragment layout ----
            uint32_t pb[G][2];
            {
                float s0[G], s1[G], b0[G], b1[G];
                load_groups<T, G>(vst, tl0, s0);
                load_groups<T, G>(vst, tl1, s1);
                load_groups<T, G>(vbt, tl0, b0);
                load_groups<T, G>(vbt, tl1, b1);
#pragma unroll
                for (int gr = 0; gr < G; ++gr) {
                    pb[gr][0] = movmatrix_trans(pack_h2(pr[0] * s0[gr], pr[1] * s0[gr]));  // tokens 0..7 of the block
                    pb[gr][1] = movmatrix_trans(pack_h2(pr[2] * s1[gr], pr[3] * s1[gr]));  // tokens 8..15
                    bsum[0][gr] = fmaf(pr[0], b0[gr], fmaf(pr[2], b1[gr], bsum[0][gr]));
                    bsum[1][gr] = fmaf(pr[1], b0[gr], fmaf(pr[3], b1[gr], bsum[1][gr]));
                }
            }
            // ---- O^T += codes^T . P'^T (subnormal operands; the 2^24 / 2^20 leaves in the epilogue) ----
            const uint32_t v_row = smem_u32(vct + v_off);
#pragma unroll
            for (int cp = 0; cp < CH / 2; ++cp) {
                uint32_t vf[4];
                ldmatrix_x4_trans(vf, v_row + cp * 32);
                constexpr int dims_per_pair = 2 * 8 * EPU;
                const int gr = (cp * dims_per_pair) / GROUP;
                const UnitPair<BITS> u0(vf[0]), u1(vf[1]), u2(vf[2]), u3(vf[3]);
#pragma unroll
                for (int i = 0; i < EPU; ++i) {
                    uint32_t a[4];
                    a[0] = u0.sub(i);
                    a[1] = u1.sub(i);
                    a[2] = u2.sub(i);
                    a[3] = u3.sub(i);
                    mma_f16(o_acc[cp * EPU + i], a, pb[gr][0], pb[gr][1]);
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
#pragma unroll
            for (int gr = 0; gr < G; ++gr) {
                bsum[k][gr] += __shfl_xor_sync(0xffffffffu, bsum[k][gr], 4);
                bsum[k][gr] += __shfl_xor_sync(0xffffffffu, bsum[k][gr], 8);
                bsum[k][gr] += __shfl_xor_sync(0xffffffffu, bsum[k][gr], 16);
            }
        }
        float *wo = red_o + warp * fp.red_rows * RED_STRIDE;
#pragma unroll
        for (int mt = 0; mt < MT_O; ++mt) {
            // m-tile mt = cp * EPU + i: d-row g <-> dim (2cp)*8*EPU + EPU*g + i, d-row g+8 <-> next chunk
            const int cp = mt / EPU, i = mt % EPU;
            const int d0 = (2 * cp) * 8 * EPU + EPU * g + i, d1 = d0 + 8 * EPU;
            const int gr = d0 / GROUP;
            const float vs = (BITS == 4 && (i & 1)) ? 1048576.f : 16777216.f;  // undo the subnormal factor
            if (2 * c < R) {
                wo[(2 * c) * RED_STRIDE + d0] = fmaf(o_acc[mt][0], vs, bsum[0][gr]);
                wo[(2 * c) * RED_STRIDE + d1] = fmaf(o_acc[mt][2], vs, bsum[0][gr]);
            }
            if (2 * c + 1 < R) {
                wo[(2 * c + 1) * RED_STRIDE + d0] = fmaf(o_acc[mt][1], vs, bsum[1][gr]);
                wo[(2 * c + 1) * RED_STRIDE + d1] = fmaf(o_acc[mt][3], vs, bsum[1][gr]);
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
        u.out = VARLEN ? vt.seq[b].out : p.out;
        u.out_dtype = p.out_dtype;
        u.o_sb = VARLEN ? 0 : p.o_sb;   // var-len: `b` is the sequence, every sequence has its own output
        u.o_sh = p.o_sh; u.o_sl = p.o_sl;
        u.o_signs = nullptr;
        u.splits = 0; u.Hq = p.Hq; u.L = p.L;
        segment_epilogue<D, P8_WARPS>(u, fp, red_o, red_ml, RED_STRIDE, work, is_last, unit, b, hk, rep, R,
                                      x - tile_begin, utiles, row0);
        x += ntiles;
    }
}

template <typename T, int D, int BITS, int GROUP, int NSTAGE>
void launch_affine_typed(const AffineParams &p, int units, cudaStream_t stream) {
    constexpr int G = D / GROUP;
    constexpr int RB = D * BITS / 8;
    constexpr int STAGE_BYTES = 2 * PK_TILE * RB + 4 * PK_TILE * G * 2;
    constexpr int RED_BYTES = PK_WARPS * 16 * (D + 8) * 4 + PK_WARPS * 16 * 2 * 4 + 16 * 64 * 4;
    constexpr int BODY = NSTAGE * STAGE_BYTES > RED_BYTES ? NSTAGE * STAGE_BYTES : RED_BYTES;
    const size_t smem = (size_t)BODY + 16 + 2 * NSTAGE * sizeof(uint64_t) + 64 + 128;
    static bool configured[64] = {false};
    const int dev = current_device();
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        KVC_CUDA(cudaFuncSetAttribute(attn_affine_kernel<T, D, BITS, GROUP, NSTAGE>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        KVC_CUDA(cudaFuncSetAttribute(attn_affine_kernel<T, D, BITS, GROUP, NSTAGE>,
                                      cudaFuncAttributePreferredSharedMemoryCarveout, 100));
        configured[dev] = true;
    }
    KernelTimer timer(stream);
    KVC_CUDA(launch_pdl(attn_affine_kernel<T, D, BITS, GROUP, NSTAGE>, dim3(units), dim3(PK_THREADS), smem, stream, p));
    timer.stop();
    KVC_CUDA(cudaGetLastError());
    ++g_launch_count;
}

template <typename T, int D, int BITS, int GROUP, int NSTAGE, int MINB, bool VARLEN, int NW>
void launch_affine8_typed(const AffineParams &p, const VarlenAttnTable &vt, int ctas, cudaStream_t stream) {
    constexpr int P8_WARPS = NW, P8_TILE = NW * 16, P8_THREADS = (NW + 1) * 32;
    constexpr int G = D / GROUP;
    constexpr int RB = D * BITS / 8;
    constexpr int STAGE_BYTES = 2 * P8_TILE * RB + 4 * P8_TILE * G * 2;
    const size_t red = (size_t)P8_WARPS * p.flat.red_rows * (D + 8) * 4 + (size_t)P8_WARPS * p.flat.red_rows * 8 + 32 +
                       (size_t)p.flat.red_rows * p.flat.nslots * 4 + 16 + 4 * sizeof(uint64_t) +
                       (size_t)2 * p.flat.red_rows * D * 2;
    const size_t smem = (size_t)NSTAGE * STAGE_BYTES + 16 + 2 * NSTAGE * sizeof(uint64_t) + 64 + red + 128;
    static size_t configured[64] = {0};
    const int dev = current_device();
    if (dev >= 0 && dev < 64 && configured[dev] < smem) {
        KVC_CUDA(cudaFuncSetAttribute(attn_affine_decode8_kernel<T, D, BITS, GROUP, NSTAGE, MINB, VARLEN, NW>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        KVC_CUDA(cudaFuncSetAttribute(attn_affine_decode8_kernel<T, D, BITS, GROUP, NSTAGE, MINB, VARLEN, NW>,
                                      cudaFuncAttributePreferredSharedMemoryCarveout, 100));
        configured[dev] = smem;
    }
    KernelTimer timer(stream);
    KVC_CUDA(launch_pdl(attn_affine_decode8_kernel<T, D, BITS, GROUP, NSTAGE, MINB, VARLEN, NW>, dim3(ctas), dim3(P8_THREADS),
                        smem, stream, p, vt));
    timer.stop();
    KVC_CUDA(cudaGetLastError());
    ++g_launch_count;
}

bool affine_source_fits(const KVSource &s, int D, int64_t T) {
    if (s.kind != SRC_AFFINE || (s.dtype != KVC_BF16 && s.dtype != KVC_F16)) return false;
    if (s.bits != 4 && s.bits != 8) return false;
    if (s.group != 32 && s.group != 64 && s.group != 128) return false;
    if (D % s.group) return false;
    const int wpr = D * s.bits / 32, G = D / s.group;
    if (s.st != wpr || s.gst != G) return false;  // rows must be contiguous
    const int64_t padded = (T + 255) / 256 * 256;   // the largest stage any of these kernels streams
    // a full last tile must stay inside the (batch, head) slab, and slabs must keep 16-byte alignment
    if (s.sh < padded * wpr || s.gsh < padded * G) return false;
    if ((s.sh * 4) % 16 || (s.sb * 4) % 16 || (s.gsh * 2) % 16 || (s.gsb * 2) % 16) return false;
    if (((uintptr_t)s.data & 15) || ((uintptr_t)s.scales & 15) || ((uintptr_t)s.biases & 15)) return false;
    return true;
}

}  // namespace

namespace {
const VarlenAttnTable kNoVarlen = {};

constexpr int affine8_stages(int D, int bits, bool varlen) {
    if (affine8_warps(D, bits, varlen) == 15) return 4;
    return bits == 4 ? (D == 128 ? 5 : 8) : (D == 128 ? 4 : 6);
}

int affine_resident_ctas(int D, int bits, int group, int rows, bool varlen) {
    // CTAs that fit an SM by shared memory: ring + cross-warp buffers (+1 KB the driver reserves)
    const int ns = affine8_stages(D, bits, varlen), nw = affine8_warps(D, bits, varlen), tile = nw * 16;
    const size_t stage = (size_t)2 * tile * (D * bits / 8) + (size_t)4 * tile * (D / group) * 2;
    const size_t red = (size_t)nw * rows * (D + 8) * 4 + (size_t)nw * rows * 8 + 32 + (size_t)rows * 64 * 4 +
                       64 + (size_t)2 * rows * D * 2;
    const size_t per_cta = ns * stage + red + 512 + 1024;
    return (int)std::max<size_t>(1, std::min<size_t>(affine8_ctas(D, bits, varlen), (size_t)227 * 1024 / per_cta));
}
}  // namespace

// One decode step over n independent affine caches (B = 1, L = 1 each, same head layout and
// quantisation) in one launch. Returns launches made, 0 when the calls do not fit.
int launch_attention_affine_varlen(const AttnArgs *args, int n, cudaStream_t stream) {
    if (n < 1 || n > KVC_VARLEN_MAX) return 0;
    const AttnArgs &a0 = args[0];
    if (a0.q_dtype != KVC_BF16 && a0.q_dtype != KVC_F16) return 0;
    if (a0.D != 64 && a0.D != 128) return 0;
    if (a0.Hkv <= 0 || a0.Hq % a0.Hkv) return 0;
    const int rep = a0.Hq / a0.Hkv;
    if (rep > 8 || (2 * 8 * (16 / std::max(a0.k.bits, 1))) > a0.k.group) return 0;
    VarlenAttnTable vt = {};
    vt.n = n;
    int64_t prefix = 0, max_tiles = 0;
    for (int i = 0; i < n; ++i) {
        const AttnArgs &a = args[i];
        if (a.B != 1 || a.L != 1 || a.mask.mode != KVC_MASK_NONE || a.q_signs || a.o_signs || a.q_calib) return 0;
        if (a.q_dtype != a0.q_dtype || a.D != a0.D || a.Hq != a0.Hq || a.Hkv != a0.Hkv || a.scale != a0.scale) return 0;
        if (a.q_sh != a0.q_sh || a.q_sl != a0.q_sl || a.o_sh != a0.o_sh || a.o_sl != a0.o_sl) return 0;
        if (a.k.kind != SRC_AFFINE || a.v.kind != SRC_AFFINE) return 0;
        if (a.k.dtype != a.q_dtype || a.v.dtype != a.q_dtype) return 0;
        if (a.k.bits != a0.k.bits || a.v.bits != a0.k.bits || a.k.group != a0.k.group || a.v.group != a0.k.group) return 0;
        if (a.k.bits != 4 && a.k.bits != 8) return 0;
        if (a.T < 1 || a.T > (int64_t)1 << 30) return 0;
        if (!affine_source_fits(a.k, a.D, a.T) || !affine_source_fits(a.v, a.D, a.T)) return 0;
        if (a.k.sh != a.v.sh || a.k.gsh != a.v.gsh) return 0;
        if (((uintptr_t)a.q & 1)) return 0;
        VarlenAttnSeq &sq = vt.seq[i];
        sq.q = a.q; sq.out = a.out;
        sq.kc = (const uint32_t *)a.k.data; sq.vc = (const uint32_t *)a.v.data;
        sq.ks = a.k.scales; sq.kb = a.k.biases; sq.vs = a.v.scales; sq.vb = a.v.biases;
        sq.c_sh = a.k.sh; sq.g_sh = a.k.gsh;
        sq.T = (int32_t)a.T;
        sq.tile_prefix = (int32_t)prefix;
        const int64_t tile8 = affine8_warps(a0.D, a0.k.bits, true) * 16;
        const int64_t tl = (a.T + tile8 - 1) / tile8;
        prefix += tl;
        max_tiles = std::max(max_tiles, tl);
    }
    if (a0.D / a0.k.group > 4 || (a0.k.group * a0.k.bits) / 32 < 4) return 0;
    const int64_t units = (int64_t)n * a0.Hkv;
    if (units * (int64_t)sizeof(int) > PK_COUNTER_BYTES) return 0;
    int *status = device_status_word(a0.device);
    if (!status) return 0;
    int *counters = counters_get(a0.device, stream, PK_COUNTER_BYTES);

    const int64_t work_tiles = prefix * a0.Hkv;
    const int resident = affine_resident_ctas(a0.D, a0.k.bits, a0.k.group, rep, true);
    const int64_t ctas = std::min<int64_t>((int64_t)sm_count(a0.device) * resident, work_tiles);
    AffineParams p = {};
    p.flat.tiles = (int)max_tiles;
    p.flat.per = (int)(work_tiles / ctas);
    p.flat.rem = (int)(work_tiles % ctas);
    p.flat.nslots = (int)((max_tiles + p.flat.per - 1) / p.flat.per + 1);
    p.flat.red_rows = rep;
    if (p.flat.nslots > 64) return 0;
    p.q_bulk = a0.q_sh == a0.D ? 1 : 0;
    for (int i = 0; i < n; ++i)
        if ((uintptr_t)args[i].q & 15) p.q_bulk = 0;
    const int64_t qrows = (int64_t)n * a0.Hq;
    const size_t o_bytes = (size_t)qrows * p.flat.nslots * a0.D * sizeof(float);
    const size_t ml_bytes = (size_t)qrows * p.flat.nslots * sizeof(float2);
    char *scratch = (char *)scratch_get(a0.device, o_bytes + ml_bytes + 256, stream);
    p.out_dtype = a0.q_dtype;
    p.q_sh = a0.q_sh; p.q_sl = a0.q_sl; p.o_sh = a0.o_sh; p.o_sl = a0.o_sl;
    p.o_part = (float *)scratch;
    p.ml_part = (float2 *)(scratch + ((o_bytes + 255) / 256) * 256);
    p.counters = counters; p.status = status;
    p.B = n; p.Hq = a0.Hq; p.Hkv = a0.Hkv; p.L = 1; p.T = 0;
    p.splits = p.flat.nslots;
    p.chunks = 1;
    p.causal = 0;
    p.causal_offset = 0;
    p.scale_log2 = a0.scale * 1.4426950408889634f;
    const int bits = a0.k.bits, group = a0.k.group;
#define KVC_AFFV(TT, DD, BB, GG, NS)                                                        \
    if (a0.D == DD && bits == BB && group == GG) {                                           \
        launch_affine8_typed<TT, DD, BB, GG, affine8_stages(DD, BB, true), affine8_ctas(DD, BB, true), true, affine8_warps(DD, BB, true)>(p, vt, (int)ctas, stream);         \
        return 1;                                                                            \
    }
    if (a0.q_dtype == KVC_BF16) {
        KVC_AFFV(__nv_bfloat16, 128, 4, 64, 5)
        KVC_AFFV(__nv_bfloat16, 128, 8, 64, 4)
    } else {
        KVC_AFFV(__half, 128, 4, 64, 5)
        KVC_AFFV(__half, 128, 8, 64, 4)
    }
#undef KVC_AFFV
    return 0;
}

int launch_attention_verify_tc_affine(const AttnArgs &a, cudaStream_t stream);   // attn_verify_tc.cu

int launch_attention_affine(const AttnArgs &a, cudaStream_t stream) {
    if (a.q_dtype != KVC_BF16 && a.q_dtype != KVC_F16) return 0;
    if (a.D != 64 && a.D != 128) return 0;
    if (a.mask.mode == KVC_MASK_ARRAY || a.q_signs || a.o_signs || a.q_calib) return 0;
    if (a.k.kind != SRC_AFFINE || a.v.kind != SRC_AFFINE) return 0;
    if (a.k.dtype != a.q_dtype || a.v.dtype != a.q_dtype) return 0;
    if (a.k.bits != a.v.bits || a.k.group != a.v.group) return 0;
    if (a.Hkv <= 0 || a.Hq % a.Hkv) return 0;
    const int rep = a.Hq / a.Hkv;
    if (rep * a.L > 64 || a.T < 1 || a.T > (int64_t)1 << 30) return 0;
    if (!affine_source_fits(a.k, a.D, a.T) || !affine_source_fits(a.v, a.D, a.T)) return 0;
    if (a.D / a.k.group > 4 || (a.k.group * a.k.bits) / 32 < 4) return 0;
    if (((uintptr_t)a.q & 1)) return 0;
    if (rep * a.L > 16) {      // a verify round of a wide head group: the rows decoded once, on the tensor cores
        const int n = launch_attention_verify_tc_affine(a, stream);
        if (n) return n;
    }
    // Up to 8 query rows per kv head: the transposed decode kernel. 9..16 rows: the 16-row kernel.
    // 17..64 rows where the tensor-core verify kernel does not apply: the decode kernel again, the group cut into
    // units of eight rows that stream the same tiles one after the other (all but the first out of L2).
    const bool pairs_fit = (2 * 8 * (16 / a.k.bits)) <= a.k.group;
    const int chunks = rep * a.L > 16 ? (rep * a.L + 7) / 8 : 1;
    if (chunks > 1 && !pairs_fit) return 0;
    const int64_t bh = (int64_t)a.B * a.Hkv * chunks;
    if (bh * (int64_t)sizeof(int) > PK_COUNTER_BYTES) return 0;
    int *status = device_status_word(a.device);
    if (!status) return 0;
    int *counters = counters_get(a.device, stream, PK_COUNTER_BYTES);

    // at most 8 query rows and chunk pairs inside one group: transposed decode kernel (its own tile size)
    const bool decode8 = (rep * a.L <= 8 || chunks > 1) && pairs_fit;
    const int64_t tile8 = affine8_warps(a.D, a.k.bits, false) * 16;
    const int64_t tiles = decode8 ? (a.T + tile8 - 1) / tile8 : (a.T + PK_TILE - 1) / PK_TILE;
    // resident CTAs per SM (a fourth CTA fits the 4-bit kernels at 94 registers but measured slower)
    const int slots = sm_count(a.device) * (decode8 ? 3 : 2);
    int64_t best_s = 1;
    double best_cost = 1e30;
    const int64_t max_s = std::min<int64_t>(tiles, 64);
    // One wave of resident CTAs measures best (cfg4 shape: 384 CTAs on 444 slots, 90 us, against
    // 97-102 us for 4..10 splits): a second wave pays the prologue / merge again and runs
    // against a half-empty machine at its end.
    for (int64_t s = 1; s <= max_s; ++s) {
        const int64_t units = bh * s;
        const int64_t waves = (units + slots - 1) / slots;
        const int64_t per = (tiles + s - 1) / s;
        const double cost = (double)waves * ((double)per + 6.0);
        if (cost < best_cost - 1e-9) {
            best_cost = cost;
            best_s = s;
        }
    }
    // decode8: flat decomposition over one wave of resident CTAs (every CTA streams the same number
    // of tiles); the partial slots per unit take the place of the splits
    const int64_t work_tiles = bh * tiles;
    const int flat_resident = affine_resident_ctas(a.D, a.k.bits, a.k.group, std::min(8, rep * a.L), false);
    const int64_t flat_ctas = std::min<int64_t>((int64_t)sm_count(a.device) * flat_resident, work_tiles);
    const int64_t flat_per = work_tiles / flat_ctas, flat_rem = work_tiles % flat_ctas;
    const int64_t flat_slots = (tiles + flat_per - 1) / flat_per + 1;
    if (decode8 && flat_slots > 64) return 0;
    const int64_t splits = decode8 ? flat_slots : best_s;
    const int64_t qrows = (int64_t)a.B * a.Hq * a.L;
    const size_t o_bytes = (size_t)qrows * splits * a.D * sizeof(float);
    const size_t ml_bytes = (size_t)qrows * splits * sizeof(float2);
    char *scratch = (char *)scratch_get(a.device, o_bytes + ml_bytes + 256, stream);

    AffineParams p;
    p.q = a.q; p.out = a.out; p.out_dtype = a.q_dtype;
    p.q_sb = a.q_sb; p.q_sh = a.q_sh; p.q_sl = a.q_sl;
    p.o_sb = a.o_sb; p.o_sh = a.o_sh; p.o_sl = a.o_sl;
    p.kc = (const uint32_t *)a.k.data; p.vc = (const uint32_t *)a.v.data;
    p.ks = a.k.scales; p.kb = a.k.biases; p.vs = a.v.scales; p.vb = a.v.biases;
    p.kc_sb = a.k.sb; p.kc_sh = a.k.sh; p.vc_sb = a.v.sb; p.vc_sh = a.v.sh;
    p.kg_sb = a.k.gsb; p.kg_sh = a.k.gsh; p.vg_sb = a.v.gsb; p.vg_sh = a.v.gsh;
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
    p.flat.tiles = (int)tiles;
    p.flat.per = (int)flat_per; p.flat.rem = (int)flat_rem;
    p.flat.nslots = (int)flat_slots; p.flat.red_rows = decode8 ? std::min(8, rep * a.L) : rep * a.L;
    p.chunks = chunks;
    p.q_bulk = (chunks == 1 && a.L == 1 && a.q_sh == a.D && ((uintptr_t)a.q & 15) == 0 && (a.q_sb * 2) % 16 == 0) ? 1 : 0;
    const int units = decode8 ? (int)flat_ctas : (int)(bh * splits);

    const int bits = a.k.bits, group = a.k.group;
#define KVC_AFF8(TT, DD, BB, GG, NS)                                         \
    if (a.D == DD && bits == BB && group == GG) {                            \
        launch_affine8_typed<TT, DD, BB, GG, affine8_stages(DD, BB, false), affine8_ctas(DD, BB, false), false, affine8_warps(DD, BB, false)>(p, kNoVarlen, units, stream); \
        return 1;                                                            \
    }
    if (decode8) {
        if (a.q_dtype == KVC_BF16) {
            KVC_AFF8(__nv_bfloat16, 128, 4, 64, 5)
            KVC_AFF8(__nv_bfloat16, 128, 8, 64, 4)
            KVC_AFF8(__nv_bfloat16, 128, 4, 128, 5)
            KVC_AFF8(__nv_bfloat16, 128, 8, 128, 4)
            KVC_AFF8(__nv_bfloat16, 128, 8, 32, 4)
            KVC_AFF8(__nv_bfloat16, 64, 4, 64, 8)
            KVC_AFF8(__nv_bfloat16, 64, 8, 64, 6)
        } else {
            KVC_AFF8(__half, 128, 4, 64, 5)
            KVC_AFF8(__half, 128, 8, 64, 4)
            KVC_AFF8(__half, 128, 4, 128, 5)
            KVC_AFF8(__half, 128, 8, 128, 4)
            KVC_AFF8(__half, 128, 8, 32, 4)
            KVC_AFF8(__half, 64, 4, 64, 8)
            KVC_AFF8(__half, 64, 8, 64, 6)
        }
    }
#undef KVC_AFF8
#define KVC_AFF(TT, DD, BB, GG, NS)                                          \
    if (a.D == DD && bits == BB && group == GG) {                            \
        launch_affine_typed<TT, DD, BB, GG, NS>(p, units, stream);           \
        return 1;                                                            \
    }
    if (a.q_dtype == KVC_BF16) {
        KVC_AFF(__nv_bfloat16, 128, 4, 64, 8)
        KVC_AFF(__nv_bfloat16, 128, 8, 64, 5)
        KVC_AFF(__nv_bfloat16, 128, 4, 32, 8)
        KVC_AFF(__nv_bfloat16, 128, 4, 128, 8)
        KVC_AFF(__nv_bfloat16, 128, 8, 128, 5)
        KVC_AFF(__nv_bfloat16, 64, 4, 64, 8)
        KVC_AFF(__nv_bfloat16, 64, 8, 64, 8)
    } else {
        KVC_AFF(__half, 128, 4, 64, 8)
        KVC_AFF(__half, 128, 8, 64, 5)
        KVC_AFF(__half, 128, 4, 32, 8)
        KVC_AFF(__half, 128, 4, 128, 8)
        KVC_AFF(__half, 128, 8, 128, 5)
        KVC_AFF(__half, 64, 4, 64, 8)
        KVC_AFF(__half, 64, 8, 64, 8)
    }
#undef KVC_AFF
    return 0;
}

}  // namespace kvc
