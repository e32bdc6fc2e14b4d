// Device primitives shared by the TMA-staged attention kernels: mbarrier
// (bounded waits), TMA tile and bulk loads, ldmatrix, fast exp2 and the
// m16n8k16 tensor-core MMA for f16 / bf16 operands.
#pragma once

#include "common.h"

#include <cstdlib>
#include <utility>

#include <cuda.h>

// Measurement aids (switching consumer work off piece by piece to time the producer alone) exist
// only in a build made with -DKVC_MEASURE_AIDS, which the shipped build never sets: without the
// flag the skip bits are the constant 0, the branches on them compile away and no environment
// variable is read.
#ifdef KVC_MEASURE_AIDS
#define KVC_SKIP_BITS(p) ((p).debug_skip)
#else
#define KVC_SKIP_BITS(p) 0
#endif

namespace kvc {

inline int measure_skip_bits() {
#ifdef KVC_MEASURE_AIDS
    static const int bits = [] {
        const char *e = std::getenv("KVC_DECODE_DEBUG_SKIP");
        return e ? std::atoi(e) : 0;
    }();
    return bits;
#else
    return 0;
#endif
}

// KVC_TRACE_DISPATCH=1 makes the chunk paths say on stderr which kernel took a call. Read at each
// use (tests switch it on inside a running process); only chunk launches consult it, never decode.
inline bool trace_dispatch() {
    const char *e = std::getenv("KVC_TRACE_DISPATCH");
    return e && e[0] == '1';
}

namespace dev {

constexpr uint32_t SPIN_LIMIT = 1u << 24;

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

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr)
                 : "memory");
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Programmatic dependent launch: a kernel launched with launch_pdl() may start while the
// kernel before it on the stream is still running; everything it reads from global memory
// must come after pdl_wait(), which returns once that kernel has completed and flushed.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Lets the next kernel on the stream (if it was launched with launch_pdl) be scheduled as soon as
// every CTA of this one has issued it or exited. Issued only AFTER pdl_wait(): a kernel that starts
// early then knows that everything up to the kernel before its predecessor has completed.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 8x8 transpose of b16 elements across the warp: lane (g, c) gives row g, columns 2c, 2c+1
// and receives row g of the transpose.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
    uint32_t r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(x));
    return r;
}

template <typename T> struct MmaType;
template <> struct MmaType<__nv_bfloat16> {
    static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
            "{%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        uint32_t r;
        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
        return r;
    }
    static __device__ __forceinline__ void store(void *p, int64_t i, float v) {
        ((__nv_bfloat16 *)p)[i] = __float2bfloat16_rn(v);
    }
    static __device__ __forceinline__ float2 unpack(uint32_t w) {
        return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
    }
};
template <> struct MmaType<__half> {
    static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
            "{%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        uint32_t r;
        asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
        return r;
    }
    static __device__ __forceinline__ void store(void *p, int64_t i, float v) {
        ((__half *)p)[i] = __float2half_rn(v);
    }
    static __device__ __forceinline__ float2 unpack(uint32_t w) {
        return __half22float2(*reinterpret_cast<const __half2 *>(&w));
    }
};


// Untiled bulk copy global -> shared (both 16-byte aligned, size a multiple of 16).
__device__ __forceinline__ void bulk_load(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst)), "l"((uint64_t)src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// ---------------------------------------------------------------------
// End of a work unit: merge the consumer warps of the CTA into one partial,
// publish it, and let the last unit of the (batch, head) merge all splits.
// ---------------------------------------------------------------------
struct UnitOut {
    float *o_part;      // [query row][split][D]
    float2 *ml_part;    // [query row][split] (log2-domain max, sum)
    int *counters;      // one ticket per (batch, head), self-resetting
    void *out;
    int32_t out_dtype;
    int64_t o_sb, o_sh, o_sl;
    const float *o_signs;  // optional: rotate merged rows back (TurboQuant values)
    int32_t splits, Hq, L;
};

__device__ __forceinline__ void store_out(void *p, int32_t dtype, int64_t i, float v) {
    switch (dtype) {
        case KVC_F32: ((float *)p)[i] = v; break;
        case KVC_F16: ((__half *)p)[i] = __float2half_rn(v); break;
        default: ((__nv_bfloat16 *)p)[i] = __float2bfloat16_rn(v); break;
    }
}

// Preconditions: every consumer warp w < NWARPS has written its un-normalised
// rows to red_o[(w*16 + r) * red_stride + d] and (max, sum) to red_ml[(w*16 + r)*2],
// followed by a __syncthreads(). `work` is shared memory that does not overlap
// red_o / red_ml, at least R * max(splits, D) floats; `flag` one int of shared memory.
template <int D, int NWARPS>
__device__ void unit_epilogue(const UnitOut &u, const float *red_o, const float *red_ml, int red_stride,
                              float *work, int *flag, int b, int hk, int rep, int R, int split, int bh) {
    const int tid = threadIdx.x, nthreads = blockDim.x, warp = tid >> 5, lane = tid & 31;
    constexpr int row0 = 0;  // a unit of this epilogue always carries the whole group
    const int64_t qrow0 = ((int64_t)b * u.Hq + hk * rep) * u.L + row0;  // the group's rows are consecutive query rows
    for (int i = tid; i < R * D; i += nthreads) {
        const int r = i / D, d = i % D;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < NWARPS; ++w) m = fmaxf(m, red_ml[(w * 16 + r) * 2]);
        float o = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < NWARPS; ++w) {
            const float mw = red_ml[(w * 16 + r) * 2];
            const float f = (mw == -INFINITY) ? 0.f : fast_exp2(mw - m);
            o += red_o[(w * 16 + r) * red_stride + d] * f;
            l += red_ml[(w * 16 + r) * 2 + 1] * f;
        }
        const int64_t base = (qrow0 + r) * u.splits + split;
        __stcg(&u.o_part[base * D + d], o);
        if (d == 0) __stcg(&u.ml_part[base], make_float2(m, l));
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const int ticket = atomicAdd(&u.counters[bh], 1);
        const int last = (ticket == u.splits - 1) ? 1 : 0;
        if (last) u.counters[bh] = 0;
        *flag = last;
    }
    __syncthreads();
    if (!*flag) return;
    __threadfence();
    // merge weights per (row, split)
    for (int r = warp; r < R; r += nthreads / 32) {
        float m = -INFINITY;
        for (int s = lane; s < u.splits; s += 32) m = fmaxf(m, __ldcg(&u.ml_part[(qrow0 + r) * u.splits + s]).x);
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        float lsum = 0.f;
        for (int s = lane; s < u.splits; s += 32) {
            const float2 ml = __ldcg(&u.ml_part[(qrow0 + r) * u.splits + s]);
            const float f = (ml.x == -INFINITY || ml.y <= 0.f) ? 0.f : fast_exp2(ml.x - m);
            work[r * u.splits + s] = f;
            lsum += ml.y * f;
        }
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, o);
        const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
        __syncwarp();
        for (int s = lane; s < u.splits; s += 32) work[r * u.splits + s] *= inv;
    }
    __syncthreads();
    if (!u.o_signs) {
        for (int i = tid; i < R * D; i += nthreads) {
            const int r = i / D, d = i % D;
            float o = 0.f;
            const float *src = u.o_part + ((qrow0 + r) * u.splits) * D + d;
            for (int s = 0; s < u.splits; ++s) o = fmaf(__ldcg(src + (int64_t)s * D), work[r * u.splits + s], o);
            const int hq = hk * rep + (row0 + r) / u.L, lq = (row0 + r) % u.L;
            store_out(u.out, u.out_dtype, b * u.o_sb + hq * u.o_sh + lq * u.o_sl + d, o);
        }
        return;
    }
    // TurboQuant values: the merged rows are in the rotated basis; out = signs * H(o) / sqrt(D).
    float *rows = work + R * u.splits;  // [R][D]
    for (int i = tid; i < R * D; i += nthreads) {
        const int r = i / D, d = i % D;
        float o = 0.f;
        const float *src = u.o_part + ((qrow0 + r) * u.splits) * D + d;
        for (int s = 0; s < u.splits; ++s) o = fmaf(__ldcg(src + (int64_t)s * D), work[r * u.splits + s], o);
        rows[i] = o;
    }
    for (int half = 1; half < D; half <<= 1) {
        __syncthreads();
        for (int pidx = tid; pidx < R * (D / 2); pidx += nthreads) {
            const int r = pidx / (D / 2), j = pidx % (D / 2);
            const int i0 = ((j / half) * 2 * half) + (j % half), i1 = i0 + half;
            const float x = rows[r * D + i0], y = rows[r * D + i1];
            rows[r * D + i0] = x + y;
            rows[r * D + i1] = x - y;
        }
    }
    __syncthreads();
    const float f = rsqrtf((float)D);
    for (int i = tid; i < R * D; i += nthreads) {
        const int r = i / D, d = i % D;
        const int hq = hk * rep + (row0 + r) / u.L, lq = (row0 + r) % u.L;
        store_out(u.out, u.out_dtype, b * u.o_sb + hq * u.o_sh + lq * u.o_sl + d, rows[i] * f * u.o_signs[d]);
    }
}

// ---------------------------------------------------------------------
// Flat tile decomposition shared by the decode kernels. All (batch, head) units have
// `tiles` tiles; CTA c owns the consecutive flat tiles [flat_lo(c), flat_lo(c + 1)) of the
// units * tiles in the launch and walks them as segments (one per unit it touches). The
// partial of a segment goes to slot (c - first CTA of the unit) of the unit's partials.
// ---------------------------------------------------------------------
struct FlatPlan {
    int32_t tiles;     // tiles per unit
    int32_t per, rem;  // CTA c owns per + (c < rem) tiles
    int32_t nslots;    // partial slots per unit
    int32_t red_rows;  // rows of the cross-warp buffers (>= query rows per unit)
};

__device__ __forceinline__ int64_t flat_lo(const FlatPlan &f, int c) { return (int64_t)c * f.per + min(c, f.rem); }

__device__ __forceinline__ int flat_cta_of(const FlatPlan &f, int64_t x) {
    const int64_t big = (int64_t)f.rem * (f.per + 1);
    return x < big ? (int)(x / (f.per + 1)) : f.rem + (int)((x - big) / f.per);
}

// Barrier among the NW consumer warps only (the producer warp never joins it). Every consumer
// warp reaches every one of these whether or not one of its bounded waits has run out.
template <int NW>
__device__ __forceinline__ void consumer_bar() {
    asm volatile("bar.sync 1, %0;" ::"n"(NW * 32) : "memory");
}

// End of a segment, called by all NW consumer warps (tid = 0 .. 32 NW - 1) after each has
// written its un-normalised rows to red_o[(warp * red_rows + r) * red_stride + d] and
// red_ml[(warp * red_rows + r) * 2 + {0, 1}] = (max, sum): merges the warps, writes the
// segment's partial, takes a ticket and, in the CTA that completes the unit, merges all
// partials (log-sum-exp) and writes the output rows (through signs * H(.) / sqrt(D) when
// o_signs is set). `work` holds red_rows * D floats when o_signs is set and is unused otherwise.
// NBUF (default NW) is the number of warps that wrote cross-warp buffers: a kernel that has already
// folded its NW warps down to NBUF of them passes the smaller count, all NW warps still take part.
template <int D, int NW, int NBUF = NW>
__device__ void segment_epilogue(const UnitOut &u, const FlatPlan &f, const float *red_o, const float *red_ml,
                                 int red_stride, float *work, int *flag, int unit, int b, int hk, int rep, int R,
                                 int64_t x_unit = -1, int unit_tiles = 0, int row0 = 0) {
    // row0: the unit covers the query rows row0 .. row0 + R - 1 of its (batch, kv head) group (a group
    // of more rows than one unit carries is cut into several units)
    const int tid = threadIdx.x;
    constexpr int NT = NW * 32;
    consumer_bar<NW>();
    // the unit's flat tile range: uniform units unless the caller passes a var-len range
    if (x_unit < 0) {
        x_unit = (int64_t)unit * f.tiles;
        unit_tiles = f.tiles;
    }
    const int first_cta = flat_cta_of(f, x_unit);
    const int expected = flat_cta_of(f, x_unit + unit_tiles - 1) - first_cta + 1;
    const int slot = (int)blockIdx.x - first_cta;
    const int64_t qrow0 = ((int64_t)b * u.Hq + hk * rep) * u.L + row0;
    for (int i = tid; i < R * D; i += NT) {
        const int r = i / D, d = i % D;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < NBUF; ++w) m = fmaxf(m, red_ml[(w * f.red_rows + r) * 2]);
        float o = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < NBUF; ++w) {
            const float mw = red_ml[(w * f.red_rows + r) * 2];
            const float fw = (mw == -INFINITY) ? 0.f : fast_exp2(mw - m);
            o += red_o[(w * f.red_rows + r) * red_stride + d] * fw;
            l += red_ml[(w * f.red_rows + r) * 2 + 1] * fw;
        }
        const int64_t base = (qrow0 + r) * f.nslots + slot;
        __stcg(&u.o_part[base * D + d], o);
        if (d == 0) __stcg(&u.ml_part[base], make_float2(m, l));
    }
    __threadfence();
    consumer_bar<NW>();
    if (tid == 0) {
        const int ticket = atomicAdd(&u.counters[unit], 1);
        const int last = (ticket == expected - 1) ? 1 : 0;
        if (last) u.counters[unit] = 0;
        *flag = last;
    }
    consumer_bar<NW>();
    if (*flag) {
        __threadfence();
        // Every thread merges its own (row, dim) elements: the (max, sum) pairs and the partial
        // values of all slots are loaded together (one round trip), the weights are recomputed per
        // element (a unit has a handful of slots).
        float *rows = work;  // [R][D], only for the rotated (TurboQuant) output
        for (int i = tid; i < R * D; i += NT) {
            const int r = i / D, d = i % D;
            const float2 *mlp = u.ml_part + (qrow0 + r) * f.nslots;
            const float *src = u.o_part + ((qrow0 + r) * f.nslots) * D + d;
            float m = -INFINITY, o = 0.f, lsum = 0.f;
            for (int s0 = 0; s0 < expected; s0 += 8) {   // all loads of a batch of 8 slots are issued together
                float2 ml[8];
                float ov[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const bool in = s0 + j < expected;
                    ml[j] = in ? __ldcg(&mlp[s0 + j]) : make_float2(-INFINITY, 0.f);
                    ov[j] = in ? __ldcg(src + (int64_t)(s0 + j) * D) : 0.f;
                }
                float mb = m;
#pragma unroll
                for (int j = 0; j < 8; ++j) mb = fmaxf(mb, (ml[j].y > 0.f) ? ml[j].x : -INFINITY);
                const float keep = (m == -INFINITY) ? 0.f : fast_exp2(m - mb);   // rescale what earlier batches gave
                o *= keep;
                lsum *= keep;
                m = mb;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float fw = (ml[j].x == -INFINITY || ml[j].y <= 0.f) ? 0.f : fast_exp2(ml[j].x - m);
                    lsum = fmaf(ml[j].y, fw, lsum);
                    o = fmaf(ov[j], fw, o);
                }
            }
            o = lsum > 0.f ? o / lsum : 0.f;
            if (!u.o_signs) {
                const int hq = hk * rep + (row0 + r) / u.L, lq = (row0 + r) % u.L;
                store_out(u.out, u.out_dtype, b * u.o_sb + hq * u.o_sh + lq * u.o_sl + d, o);
            } else {
                rows[i] = o;
            }
        }
        if (u.o_signs) {
            // TurboQuant values: the merged rows are in the rotated basis; out = signs * H(o) / sqrt(D).
            // A warp takes a row: lane l holds dims E*l .. E*l + E - 1, the stages that pair dims less
            // than E apart stay inside the lane, the other five are lane exchanges. Pairs and operations
            // ((a, b) -> (a + b, a - b), lower dim first) are those of the stage-by-stage butterfly.
            static_assert(D % 32 == 0 && D / 32 >= 1 && D / 32 <= 16, "one warp spans a row");
            constexpr int E = D / 32;
            const int warp = tid >> 5, lane = tid & 31;
            consumer_bar<NW>();
            const float fs = rsqrtf((float)D);
            for (int r = warp; r < R; r += NW) {
                float x[E];
#pragma unroll
                for (int j = 0; j < E; ++j) x[j] = rows[r * D + E * lane + j];
#pragma unroll
                for (int h = 1; h < E; h <<= 1)
#pragma unroll
                    for (int i = 0; i < E; ++i)
                        if ((i & h) == 0) {
                            const float xa = x[i], ya = x[i + h];
                            x[i] = xa + ya;
                            x[i + h] = xa - ya;
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
                const int hq = hk * rep + (row0 + r) / u.L, lq = (row0 + r) % u.L;
#pragma unroll
                for (int j = 0; j < E; ++j) {
                    const int d = E * lane + j;
                    store_out(u.out, u.out_dtype, b * u.o_sb + hq * u.o_sh + lq * u.o_sl + d, x[j] * fs * u.o_signs[d]);
                }
            }
        }
    }
    consumer_bar<NW>();  // buffers and flag are reused by the next segment
}

}  // namespace dev

// Launch with programmatic stream serialization (see dev::pdl_wait). KVC_NO_PDL=1 falls
// back to a plain launch.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args &&...args) {
    static const bool off = [] {
        const char *e = std::getenv("KVC_NO_PDL");
        return e && e[0] == '1';
    }();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = off ? 0 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

}  // namespace kvc
