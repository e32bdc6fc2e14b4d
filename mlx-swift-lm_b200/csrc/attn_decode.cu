// Split-K flash decoding for raw f16/bf16 caches on sm_100a.
//
// Work unit = (batch, KV head, token split). A CTA of one producer warp and
// four consumer warps streams its token range through a ring of shared-memory
// stages: the producer issues tiled TMA loads (cp.async.bulk.tensor, 128-byte
// swizzle) of K and V tiles straight from the cache arrays and signals an
// mbarrier per stage; each consumer warp owns 16 of a tile's 64 tokens, scores all
// query rows of the GQA group against them with m16n8k16 tensor-core MMAs
// (queries are the 16-row A operand, so every K/V byte is read from HBM and
// from shared memory exactly once for the whole group), keeps an online
// softmax in registers and accumulates P.V with a second MMA. The four warps'
// states are merged in shared memory and written as one un-normalised partial
// per unit; the log-sum-exp merge kernel combines the splits.
//
// Shared-memory layout of a tile: boxes of [tokens][64 elements] (128 bytes
// per row), 16-byte chunk c of row r stored at chunk c ^ (r & 7). The operand
// fragments are built from whole 16-byte chunks: the k-slot <-> head-dim
// assignment of the Q.K^T MMAs and the column <-> head-dim assignment of the
// P.V MMAs are permutations chosen so that every lane reads full chunks and
// every quarter-warp touches all eight chunk columns (no bank conflicts).
//
// Every wait on an mbarrier is bounded; a wait that runs out records an error
// code in a device status word and the CTA leaves its loops.
#include "common.h"

#include <cuda.h>

#include <algorithm>
#include <mutex>

namespace kvc {

void launch_merge(const float *o_part, const float2 *ml_part, int splits, const AttnArgs &a,
                  cudaStream_t stream);

namespace {

constexpr int CONSUMER_WARPS = 4;
constexpr int DEC_THREADS = (CONSUMER_WARPS + 1) * 32;
constexpr int TILE_T = 64;  // tokens per tile: one 16-token block per consumer warp
constexpr uint32_t SPIN_LIMIT = 1u << 24;

struct DecodeParams {
    const void *q;
    int64_t q_sb, q_sh, q_sl;
    float *o_part;
    float2 *ml_part;
    int *status;
    int32_t B, Hq, Hkv, L;
    int64_t T;
    int32_t splits;
    int32_t tiles_per_split;
    int32_t causal;  // 0 / 1
    int64_t causal_offset;
    float scale_log2;  // scale * log2(e)
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Bounded wait; returns false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
        uint32_t done;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}

__device__ __forceinline__ void tma_load_4d(void *dst, const CUtensorMap *map, uint64_t *bar, int x, int y,
                                            int z, int w) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
        : "memory");
}

template <typename T> struct MmaType;
template <> struct MmaType<__nv_bfloat16> {
    static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
            "{%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        uint32_t r;
        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
        return r;
    }
};
template <> struct MmaType<__half> {
    static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
            "{%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        uint32_t r;
        asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
        return r;
    }
};

// Address of 16-byte chunk `chunk` of row `row` inside a [rows][128 B] box with the 128-byte swizzle.
__device__ __forceinline__ const uint4 *box_chunk(const char *box, int row, int chunk) {
    return (const uint4 *)(box + row * 128 + ((chunk ^ (row & 7)) << 4));
}

template <typename T, int D, int NSTAGE>
__global__ void __launch_bounds__(DEC_THREADS, (D <= 128 ? 2 : 1))
attn_decode_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                   const DecodeParams p) {
    constexpr int TILE_BYTES = TILE_T * D * 2;     // one K (or V) tile
    constexpr int BOXES = D / 64;                  // 64-element boxes per row
    constexpr int BOX_BYTES = TILE_T * 128;
    constexpr int KSTEPS = D / 16;
    constexpr int NT_O = D / 8;                    // output n-tiles
    static_assert(TILE_T == 16 * CONSUMER_WARPS, "one 16-token block per consumer warp");

    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // [NSTAGE][K tile | V tile], then barriers
    unsigned char *stages = (unsigned char *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t *full = (uint64_t *)(stages + (size_t)NSTAGE * 2 * TILE_BYTES);
    uint64_t *empty = full + NSTAGE;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x % p.splits;
    const int bh = blockIdx.x / p.splits;
    const int hk = bh % p.Hkv, b = bh / p.Hkv;
    const int rep = p.Hq / p.Hkv;
    const int R = rep * p.L;

    const int64_t total_tiles = (p.T + TILE_T - 1) / TILE_T;
    const int64_t tile_begin = (int64_t)split * p.tiles_per_split;
    const int ntiles = (int)max((int64_t)0, min((int64_t)p.tiles_per_split, total_tiles - tile_begin));

    if (tid == 0) {
        for (int s = 0; s < NSTAGE; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], CONSUMER_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    bool ok = true;
    // Per-lane state of the consumer warps (rows g and g+8 of the 16-row tile).
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
                const int t0 = (int)((tile_begin + it) * TILE_T);
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
            // k-step ks = (box bx, pass ps, half h): lane c covers chunk y = 2c + ps of the box,
            // elements 4h..4h+3 of that chunk.
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

        for (int it = 0; it < ntiles && ok; ++it) {
            const int s = it % NSTAGE;
            ok = mbar_wait(&full[s], (it / NSTAGE) & 1);
            if (!ok) break;
            const char *kt = (const char *)stages + (size_t)s * 2 * TILE_BYTES;
            const char *vt = kt + TILE_BYTES;
            const int64_t t_tile = (tile_begin + it) * TILE_T;

            {
                const int blk = warp;  // this warp's 16 tokens of the tile
                // ---- S = Q K^T for 16 tokens (two n-tiles of 8) ----
                float sc[2][4];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
                    const int row = blk * 16 + j * 8 + g;  // this lane's token (B-fragment column g)
#pragma unroll
                    for (int bx = 0; bx < BOXES; ++bx) {
#pragma unroll
                        for (int ps = 0; ps < 2; ++ps) {
                            const uint4 kv = *box_chunk(kt + bx * BOX_BYTES, row, 2 * c + ps);
                            const int ks = bx * 4 + ps * 2;
                            MmaType<T>::mma(sc[j], qa[ks], kv.x, kv.y);
                            MmaType<T>::mma(sc[j], qa[ks + 1], kv.z, kv.w);
                        }
                    }
                }
                // ---- online softmax (log2 domain) ----
                float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int j = 0; j < 2; ++j) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int half = e >> 1;
                        const int64_t t = t_tile + blk * 16 + j * 8 + 2 * c + (e & 1);
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
                    alpha[half] = (m_new == -INFINITY) ? 1.f : exp2f(m_run[half] - m_new);
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
                            pr[j][e] = (m_run[half] == -INFINITY) ? 0.f : exp2f(sc[j][e] - m_run[half]);
                        }
#pragma unroll
                    for (int half = 0; half < 2; ++half)
                        l_run[half] = l_run[half] * alpha[half] + pr[0][2 * half] + pr[0][2 * half + 1] +
                                      pr[1][2 * half] + pr[1][2 * half + 1];
                    pa[0] = MmaType<T>::pack(pr[0][0], pr[0][1]);  // row g,   k-slots 2c, 2c+1   (n-tile 0)
                    pa[1] = MmaType<T>::pack(pr[0][2], pr[0][3]);  // row g+8
                    pa[2] = MmaType<T>::pack(pr[1][0], pr[1][1]);  // row g,   k-slots 2c+8, 2c+9 (n-tile 1)
                    pa[3] = MmaType<T>::pack(pr[1][2], pr[1][3]);  // row g+8
                }
                // ---- O = O * alpha + P V ----
#pragma unroll
                for (int nt = 0; nt < NT_O; ++nt) {
                    o_acc[nt][0] *= alpha[0];
                    o_acc[nt][1] *= alpha[0];
                    o_acc[nt][2] *= alpha[1];
                    o_acc[nt][3] *= alpha[1];
                }
                const int r0 = blk * 16 + 2 * c;  // tokens of k-slots 2c, 2c+1; +8 for 2c+8, 2c+9
#pragma unroll
                for (int bx = 0; bx < BOXES; ++bx) {
                    const char *box = vt + bx * BOX_BYTES;
                    // chunk g of four token rows: 8 head dims x 4 tokens
                    const uint4 v0 = *box_chunk(box, r0, g);
                    const uint4 v1 = *box_chunk(box, r0 + 1, g);
                    const uint4 v2 = *box_chunk(box, r0 + 8, g);
                    const uint4 v3 = *box_chunk(box, r0 + 9, g);
                    const uint32_t w0[4] = {v0.x, v0.y, v0.z, v0.w};
                    const uint32_t w1[4] = {v1.x, v1.y, v1.z, v1.w};
                    const uint32_t w2[4] = {v2.x, v2.y, v2.z, v2.w};
                    const uint32_t w3[4] = {v3.x, v3.y, v3.z, v3.w};
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        // MMA column g <-> head dim 64*bx + 8*g + e
                        const uint32_t sel = (e & 1) ? 0x7632u : 0x5410u;
                        const uint32_t b0 = __byte_perm(w0[e >> 1], w1[e >> 1], sel);
                        const uint32_t b1 = __byte_perm(w2[e >> 1], w3[e >> 1], sel);
                        MmaType<T>::mma(o_acc[bx * 8 + e], pa, b0, b1);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }
        if (!ok && lane == 0) atomicExch(p.status, 2);
    }

    // ---------------- merge the four consumer warps ----------------
    __syncthreads();
    float *red_o = (float *)stages;                         // [4][16][D]
    float *red_ml = red_o + CONSUMER_WARPS * 16 * D;        // [4][16][2]
    if (warp < CONSUMER_WARPS) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            l_run[half] += __shfl_xor_sync(0xffffffffu, l_run[half], 1);
            l_run[half] += __shfl_xor_sync(0xffffffffu, l_run[half], 2);
        }
        float *wo = red_o + warp * 16 * D;
#pragma unroll
        for (int nt = 0; nt < NT_O; ++nt) {
            // n-tile (bx, e): C columns 2c, 2c+1 <-> head dims 64*bx + 8*(2c) + e, 64*bx + 8*(2c+1) + e
            const int bx = nt / 8, e = nt % 8;
            const int d_a = bx * 64 + 16 * c + e, d_b = d_a + 8;
            wo[g * D + d_a] = o_acc[nt][0];
            wo[g * D + d_b] = o_acc[nt][1];
            wo[(g + 8) * D + d_a] = o_acc[nt][2];
            wo[(g + 8) * D + d_b] = o_acc[nt][3];
        }
        if (c == 0) {
            red_ml[(warp * 16 + g) * 2 + 0] = m_run[0];
            red_ml[(warp * 16 + g) * 2 + 1] = l_run[0];
            red_ml[(warp * 16 + g + 8) * 2 + 0] = m_run[1];
            red_ml[(warp * 16 + g + 8) * 2 + 1] = l_run[1];
        }
    }
    __syncthreads();
    constexpr float LN2 = 0.6931471805599453f;
    for (int i = tid; i < R * D; i += DEC_THREADS) {
        const int r = i / D, d = i % D;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < CONSUMER_WARPS; ++w) m = fmaxf(m, red_ml[(w * 16 + r) * 2]);
        float o = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < CONSUMER_WARPS; ++w) {
            const float mw = red_ml[(w * 16 + r) * 2];
            const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - m);
            o += red_o[(w * 16 + r) * D + d] * f;
            l += red_ml[(w * 16 + r) * 2 + 1] * f;
        }
        const int hq = hk * rep + r / p.L, lq = r % p.L;
        const int64_t qrow = ((int64_t)b * p.Hq + hq) * p.L + lq;
        const int64_t base = qrow * p.splits + split;
        p.o_part[base * D + d] = o;
        if (d == 0) p.ml_part[base] = make_float2(m == -INFINITY ? -INFINITY : m * LN2, l);
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

bool make_map(CUtensorMap *map, const KVSource &s, int D, int64_t T, int Hkv, int B, int tile_t) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return false;
    const cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)T, (cuuint64_t)Hkv, (cuuint64_t)B};
    const cuuint64_t strides[3] = {(cuuint64_t)s.st * 2, (cuuint64_t)(Hkv > 1 ? s.sh : s.st * T) * 2,
                                   (cuuint64_t)(B > 1 ? s.sb : (Hkv > 1 ? s.sh * Hkv : s.st * T)) * 2};
    const cuuint32_t box[4] = {64, (cuuint32_t)tile_t, 1, 1};
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

int *status_word(int device) {
    static int *words[64] = {nullptr};
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (device < 0 || device >= 64) return nullptr;
    if (!words[device]) {
        int *p = nullptr;
        if (cudaMalloc(&p, sizeof(int)) != cudaSuccess) {
            (void)cudaGetLastError();
            return nullptr;
        }
        (void)cudaMemset(p, 0, sizeof(int));
        words[device] = p;
    }
    return words[device];
}

template <typename T, int D, int NSTAGE>
void launch_typed(const CUtensorMap &kmap, const CUtensorMap &vmap, const DecodeParams &p, int units,
                  cudaStream_t stream) {
    const size_t smem = (size_t)NSTAGE * 2 * (TILE_T * D * 2) + 2 * NSTAGE * sizeof(uint64_t) + 1024;
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
    attn_decode_kernel<T, D, NSTAGE><<<units, DEC_THREADS, smem, stream>>>(kmap, vmap, p);
    timer.stop();
    KVC_CUDA(cudaGetLastError());
    ++g_launch_count;
}

}  // namespace

int decode_status(int device) {
    int *w = status_word(device);
    if (!w) return 0;
    int v = 0;
    if (cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) {
        (void)cudaGetLastError();
        return -1;
    }
    return v;
}

// Returns the number of kernels launched, or 0 when the call does not fit this path.
int launch_attention_decode(const AttnArgs &a, cudaStream_t stream) {
    if (a.q_dtype != KVC_BF16 && a.q_dtype != KVC_F16) return 0;
    if (a.D != 64 && a.D != 128 && a.D != 256) return 0;
    if (a.k.dtype != a.q_dtype || a.v.dtype != a.q_dtype) return 0;
    if (a.mask.mode == KVC_MASK_ARRAY) return 0;
    if (a.q_signs || a.o_signs || a.q_calib) return 0;
    if (a.Hkv <= 0 || a.Hq % a.Hkv) return 0;
    const int rep = a.Hq / a.Hkv;
    if (rep * a.L > 16 || a.T < 1 || a.T > (int64_t)1 << 30) return 0;
    if (!source_fits(a.k, a.D, a.Hkv, a.B) || !source_fits(a.v, a.D, a.Hkv, a.B)) return 0;
    if (((uintptr_t)a.q & 3) || (a.q_sb & 1) || (a.q_sh & 1) || (a.q_sl & 1)) return 0;
    if ((int64_t)a.B * a.Hkv > 65535 * 16) return 0;

    const int tile_t = TILE_T;
    CUtensorMap kmap, vmap;
    if (!make_map(&kmap, a.k, a.D, a.T, a.Hkv, a.B, tile_t) || !make_map(&vmap, a.v, a.D, a.T, a.Hkv, a.B, tile_t))
        return 0;
    int *status = status_word(a.device);
    if (!status) return 0;

    const int64_t tiles = (a.T + tile_t - 1) / tile_t;
    const int64_t bh = (int64_t)a.B * a.Hkv;
    const int sms = sm_count(a.device);
    // aim for ~6 units per SM so the hardware scheduler balances the tail, but
    // keep at least 4 tiles (one per consumer warp) in a unit
    int64_t want_units = (int64_t)sms * 6;
    int64_t splits = std::max<int64_t>(1, std::min<int64_t>((want_units + bh - 1) / bh, (tiles + 3) / 4));
    splits = std::min<int64_t>(splits, 256);
    int64_t tiles_per_split = (tiles + splits - 1) / splits;
    splits = (tiles + tiles_per_split - 1) / tiles_per_split;

    const int64_t qrows = (int64_t)a.B * a.Hq * a.L;
    const size_t o_bytes = (size_t)qrows * splits * a.D * sizeof(float);
    const size_t ml_bytes = (size_t)qrows * splits * sizeof(float2);
    char *scratch = (char *)scratch_get(a.device, o_bytes + ml_bytes + 256, stream);
    float *o_part = (float *)scratch;
    float2 *ml_part = (float2 *)(scratch + ((o_bytes + 255) / 256) * 256);

    DecodeParams p;
    p.q = a.q; p.q_sb = a.q_sb; p.q_sh = a.q_sh; p.q_sl = a.q_sl;
    p.o_part = o_part; p.ml_part = ml_part; p.status = status;
    p.B = a.B; p.Hq = a.Hq; p.Hkv = a.Hkv; p.L = a.L; p.T = a.T;
    p.splits = (int)splits; p.tiles_per_split = (int)tiles_per_split;
    p.causal = a.mask.mode == KVC_MASK_CAUSAL ? 1 : 0;
    p.causal_offset = a.mask.causal_offset;
    p.scale_log2 = a.scale * 1.4426950408889634f;
    const int units = (int)(bh * splits);

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
    launch_merge(o_part, ml_part, (int)splits, a, stream);
    return 2;
}

}  // namespace kvc
