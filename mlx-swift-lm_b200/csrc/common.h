// Internal declarations shared by the host-side cache logic and the CUDA
// kernels of the B200 KV-cache library.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>
#include <cstdio>
#include <stdexcept>
#include <string>

#include "../../include/kvcache_b200.h"

namespace kvc {

// ---------------------------------------------------------------------
// errors: internal code throws kvc::Error, the C-ABI layer turns it into a
// status code plus a thread-local message.
// ---------------------------------------------------------------------
struct Error : std::runtime_error {
    kvc_status code;
    Error(kvc_status c, const std::string &m) : std::runtime_error(m), code(c) {}
};

[[noreturn]] inline void fail(kvc_status code, const std::string &msg) { throw Error(code, msg); }

#define KVC_CUDA(expr)                                                                    \
    do {                                                                                  \
        cudaError_t _e = (expr);                                                          \
        if (_e != cudaSuccess) {                                                          \
            cudaError_t _sticky = cudaGetLastError();                                     \
            (void)_sticky;                                                                \
            ::kvc::fail(_e == cudaErrorMemoryAllocation ? KVC_ERR_OUT_OF_MEMORY           \
                                                        : KVC_ERR_CUDA,                   \
                        std::string(#expr) + ": " + cudaGetErrorString(_e));              \
        }                                                                                 \
    } while (0)

#define KVC_REQUIRE(cond, msg)                                  \
    do {                                                        \
        if (!(cond)) ::kvc::fail(KVC_ERR_INVALID_ARG, (msg));   \
    } while (0)

inline size_t dtype_size(int32_t dt) {
    switch (dt) {
        case KVC_F32: return 4;
        case KVC_F16: return 2;
        case KVC_BF16: return 2;
        case KVC_U32: return 4;
        case KVC_BOOL: return 1;
        default: fail(KVC_ERR_INVALID_ARG, "unknown dtype");
    }
}

inline bool is_float_dtype(int32_t dt) { return dt == KVC_F32 || dt == KVC_F16 || dt == KVC_BF16; }

// ---------------------------------------------------------------------
// device memory: stream-ordered allocations from the device's default pool.
// ---------------------------------------------------------------------
void *dev_alloc(size_t bytes, cudaStream_t stream);
void dev_free(void *ptr, cudaStream_t stream);
// Scratch that grows on demand, one arena per (device, stream), reused by every
// attention call enqueued on that stream (split-K partials).
void *scratch_get(int device, size_t bytes, cudaStream_t stream);
// Zero-initialised ticket counters of the same (device, stream) arena; fixed size.
int *counters_get(int device, cudaStream_t stream, size_t bytes);
int current_device();
int sm_count(int device);
int *device_status_word(int device);  // shared by all kernels with bounded waits
int device_status(int device);        // reads it (0 = no wait ever ran out)
bool device_status_reset(int device);  // clears it
void device_wait_probe(int device, uint32_t iterations, cudaStream_t stream);  // a wait that runs out on purpose

// ---------------------------------------------------------------------
// kernel launch descriptors
// ---------------------------------------------------------------------

// Source of K or V rows for the attention kernels.
enum SourceKind : int32_t {
    SRC_RAW = 0,     // rows of `dtype` elements
    SRC_AFFINE = 1,  // packed affine codes + per-group scale/bias
    SRC_TURBO = 2    // packed codebook indices + per-row norm
};

struct KVSource {
    int32_t kind = SRC_RAW;
    int32_t dtype = KVC_BF16;      // RAW: element type; AFFINE: scale/bias type
    const void *data = nullptr;    // RAW rows / packed words
    const void *scales = nullptr;  // AFFINE
    const void *biases = nullptr;  // AFFINE
    const float *norms = nullptr;  // TURBO
    int64_t sb = 0, sh = 0, st = 0;     // element (or word) strides of `data` over batch, head, token
    int64_t gsb = 0, gsh = 0, gst = 0;  // strides of scales/biases (elements) or norms
    int32_t bits = 0;
    int32_t group = 0;
    int32_t words = 0;             // packed words per row
    float codebook[16] = {0};      // TURBO centroids
};

struct MaskDesc {
    int32_t mode = KVC_MASK_NONE;
    int32_t dtype = KVC_BOOL;  // KVC_BOOL or a float dtype (additive)
    const void *data = nullptr;
    int64_t sb = 0, sh = 0, sl = 0, st = 0;  // broadcast strides over [B, Hq, L, T]
    int64_t causal_offset = 0;               // row l sees t <= causal_offset + l
};

struct AttnArgs {
    // queries / output: [B, Hq, L, D]
    const void *q = nullptr;
    void *out = nullptr;
    int32_t q_dtype = KVC_BF16;
    int64_t q_sb = 0, q_sh = 0, q_sl = 0;  // inner stride must be 1
    int64_t o_sb = 0, o_sh = 0, o_sl = 0;
    int32_t B = 0, Hq = 0, Hkv = 0, L = 0, D = 0;
    int64_t T = 0;
    float scale = 1.f;
    KVSource k, v;
    MaskDesc mask;
    // TurboQuant: rotate queries by the key signs before scoring and un-rotate
    // the merged output by the value signs (device pointers to [D] floats).
    // Fused append (decode, raw caches): the step's new key / value rows [B, Hkv, 1, D] have NOT been
    // written to the cache yet; the kernel scores them from here and stores them at token T - 1 itself.
    const void *new_k = nullptr, *new_v = nullptr;
    int64_t nk_sb = 0, nk_sh = 0, nv_sb = 0, nv_sh = 0;  // element strides (inner stride 1)
    // Token index the new row is stored at: T - 1 (append at the end) unless the cache is a wrapped
    // ring, where it replaces the oldest row somewhere in the middle; that row is not attended.
    int64_t new_slot = -1;
    // The caller vouches that the launch right before this one on the stream (a layer of the same
    // batched call) does not write the rows of this cache that are already stored, so the kernel may
    // stream them before that launch has finished.
    bool stored_rows_settled = false;
    const float *q_signs = nullptr;
    const float *q_calib = nullptr;  // optional per-dim key-calibration scale
    // Dense rotations for head dims that are not powers of two (row-major [D, D] device matrices Pi):
    // queries go through q' = Pi_k q, merged outputs through out = o' Pi_v (TurboQuantKVCache.swift:601-603,
    // :1335-1338). Set instead of q_signs / o_signs.
    const float *q_rot = nullptr;
    const float *o_rot = nullptr;
    const float *o_signs = nullptr;
    int device = 0;
};

// Append S new rows per (batch, head) into a [B, H, cap, W] cache array at
// token position `pos` (K and V in one launch).
struct AppendArgs {
    const void *k_src = nullptr, *v_src = nullptr;
    int64_t ks_sb = 0, ks_sh = 0, ks_ss = 0, ks_sd = 1;  // source element strides
    int64_t vs_sb = 0, vs_sh = 0, vs_ss = 0, vs_sd = 1;
    void *k_dst = nullptr, *v_dst = nullptr;
    int64_t kd_sb = 0, kd_sh = 0, kd_st = 0;  // destination element strides (inner 1)
    int64_t vd_sb = 0, vd_sh = 0, vd_st = 0;
    int32_t B = 0, H = 0, S = 0, Dk = 0, Dv = 0;
    int64_t pos = 0;
    int32_t esize = 2;
};

// Row gather used by the rotating cache (temporal re-order, front trim,
// logical views) and by growth copies: destination token j of every
// (batch, head) takes source token seg-mapped(j).
struct GatherSeg { int64_t src_start; int64_t count; };
struct GatherArgs {
    const void *src = nullptr;
    void *dst = nullptr;
    int64_t s_sb = 0, s_sh = 0, s_st = 0;  // element strides
    int64_t d_sb = 0, d_sh = 0, d_st = 0;
    int32_t B = 0, H = 0, W = 0;           // W elements per row
    int32_t esize = 2;
    int32_t nseg = 0;
    GatherSeg seg[4];
    int64_t dst_start = 0;                 // first destination token
};

// Rotary positions for a query tensor and a key tensor [B, H, L, D] in one launch (either may be absent).
struct RopeTensor {
    const void *src = nullptr;
    void *dst = nullptr;
    int64_t s_sb = 0, s_sh = 0, s_sl = 0;   // element strides (inner stride 1)
    int64_t d_sb = 0, d_sh = 0, d_sl = 0;
    int32_t B = 0, H = 0, L = 0;
};
struct RopeArgs {
    RopeTensor q, k;
    int32_t dtype = KVC_BF16;
    int32_t D = 0, dims = 0, traditional = 0;
    double log2_base_over_half = 0.0;  // log2(base) / (dims / 2)
    float scale = 1.f;
    int64_t offset = 0;
};
void launch_rope(const RopeArgs &a, cudaStream_t stream);

void launch_append(const AppendArgs &a, cudaStream_t stream);
void launch_gather(const GatherArgs &a, cudaStream_t stream);

// Affine group quantisation of [B, H, S, D] rows written straight into cache
// arrays at token `pos`.
struct QuantAppendArgs {
    const void *src = nullptr;
    int32_t dtype = KVC_BF16;
    int64_t s_sb = 0, s_sh = 0, s_ss = 0, s_sd = 1;
    uint32_t *codes = nullptr;
    void *scales = nullptr, *biases = nullptr;
    int64_t c_sb = 0, c_sh = 0, c_st = 0;  // word strides
    int64_t g_sb = 0, g_sh = 0, g_st = 0;  // scale/bias element strides
    int32_t B = 0, H = 0, S = 0, D = 0;
    int32_t group = 64, bits = 8;
    int64_t pos = 0;
};
void launch_affine_quantize(const QuantAppendArgs &a, cudaStream_t stream);
// K and V rows in one launch (v may be null).
void launch_affine_quantize2(const QuantAppendArgs &k, const QuantAppendArgs *v, cudaStream_t stream);

// Quantise-append of ONE new token for a list of independent caches in one launch.
constexpr int KVC_VARLEN_MAX = 32;
struct VarlenQuantSeq {
    const void *ksrc, *vsrc;              // [H, D] rows of the new token
    uint32_t *kcodes, *vcodes;            // head 0 at the append position
    void *kscales, *kbiases, *vscales, *vbiases;
    int64_t c_sh, g_sh;                   // head strides (words / elements) of this cache
};
struct VarlenQuantArgs {
    int32_t n, H, D, group, bits, dtype;
    int64_t src_sh;                       // head stride of the new rows (elements)
    VarlenQuantSeq seq[KVC_VARLEN_MAX];
};
// false when the shape is outside the warp kernel's domain (the caller then loops over the caches)
bool launch_affine_quantize_varlen(const VarlenQuantArgs &a, cudaStream_t stream);

struct DequantArgs {
    const uint32_t *codes = nullptr;
    const void *scales = nullptr, *biases = nullptr;
    void *out = nullptr;
    int32_t dtype = KVC_BF16;
    int64_t rows = 0;
    int64_t c_srow = 0, g_srow = 0, o_srow = 0;
    int32_t D = 0, group = 64, bits = 8;
};
void launch_affine_dequantize(const DequantArgs &a, cudaStream_t stream);

// TurboQuant fused encode: unit-normalise, sign flip, Walsh-Hadamard
// butterfly, boundary quantise, pack; raw norm stored per row.
struct TurboEncodeArgs {
    const void *src = nullptr;
    int32_t dtype = KVC_BF16;
    int64_t s_sb = 0, s_sh = 0, s_ss = 0, s_sd = 1;
    uint32_t *packed = nullptr;
    float *norms = nullptr;
    int64_t p_sb = 0, p_sh = 0, p_st = 0;  // word strides
    int64_t n_sb = 0, n_sh = 0, n_st = 1;  // norm strides
    int32_t B = 0, H = 0, S = 0, D = 0, bits = 4;
    int64_t pos = 0;
    const float *signs = nullptr;       // device [D]
    float boundaries[15] = {0};         // 2^bits - 1 used
    // Key calibration (TurboQuantKVCache.swift:867-886): when `calib` (device [D]) is set, the rotated
    // row is divided by it before the boundary search and the stored norm becomes
    // norm / ||centroids[idx] * calib|| (fusedQuantizePackScaled, TurboQuantKernels.swift:354-411).
    const float *calib = nullptr;
    float centroids[16] = {0};          // 2^bits used, read with `calib` and on the dense path
    // Dense rotation (head dims that are not powers of two, fusedEncodeSource, TurboQuantKernels.swift:103-204):
    // row-major [D, D] device matrix Pi, rotated = Pi * unit; the stored norm is norm / ||centroids[idx]||.
    const float *rotation = nullptr;
};
void launch_turbo_encode(const TurboEncodeArgs &a, cudaStream_t stream);
// Per-dimension fixed-point sums of the rotated unit rows of `a.src` for the calibration scale:
// sums[d] += rint(r * 2^30), sums[D + d] += rint(r * r * 2^36) with r the value the encode kernel
// quantises; integer accumulation makes the result independent of the order of the rows.
// `sums` is a device array of 2 * D int64, zeroed by the caller.
void launch_turbo_calib_stats(const TurboEncodeArgs &a, long long *sums, cudaStream_t stream);
void launch_turbo_encode2(const TurboEncodeArgs &k, const TurboEncodeArgs *v, cudaStream_t stream);

// Attention: returns the number of kernels launched.
int launch_attention(const AttnArgs &a, cudaStream_t stream);

// Boolean causal/window mask [n, offset + n] (createCausalMask) and the
// rolled single-token window mask of a wrapped rotating cache.
void launch_causal_mask(uint8_t *out, int64_t n, int64_t offset, int64_t window, cudaStream_t s);
void launch_rolled_mask(uint8_t *out, int64_t size, int64_t window, int64_t shift, cudaStream_t s);
void launch_causal_mask_lengths(uint8_t *out, int64_t n, int64_t offset, int64_t window, const int32_t *lengths,
                                int64_t batch, cudaStream_t s);

// Count of kernels launched by this library on the calling thread since the
// last reset (benchmarks report it).
extern thread_local int64_t g_launch_count;
// Value of g_launch_count right after the last launch of a kernel that releases its successor only
// after its own wait on its predecessor (-1: none yet).
extern thread_local int64_t g_last_chained_launch;

// Event timing of the dominant attention kernel (off unless a benchmark enables it).
bool timing_enabled();
void timing_set(bool on);
void timing_begin(cudaStream_t s, cudaEvent_t *start, cudaEvent_t *stop);
void timing_end(cudaStream_t s, cudaEvent_t start, cudaEvent_t stop);
void timing_read(double *total_ms, int64_t *launches, bool reset);

struct KernelTimer {
    cudaStream_t s;
    cudaEvent_t a = nullptr, b = nullptr;
    bool on;
    explicit KernelTimer(cudaStream_t stream) : s(stream), on(timing_enabled()) {
        if (on) timing_begin(s, &a, &b);
    }
    void stop() {
        if (on) timing_end(s, a, b);
        on = false;
    }
};

}  // namespace kvc
