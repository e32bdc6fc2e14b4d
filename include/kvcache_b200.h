/*
 * kvcache_b200.h -- C interface of the B200 (sm_100a) KV-cache library.
 *
 * The library re-implements, as hand-written CUDA behind a plain C ABI, the
 * KV-cache hot path of mlx-swift-lm (Libraries/MLXLMCommon): KVCacheSimple,
 * RotatingKVCache, QuantizedKVCache, TurboQuantKVCache, the staged rotating
 * round used by speculative decoding, quantizedScaledDotProductAttention,
 * TurboQuantKVCache.compressedAttention and the attentionWithCacheUpdate
 * dispatcher. A SwiftPM target imports this header through the
 * module.modulemap beside it, the same way MLXCXGrammar imports
 * xgrammar_c.h; nothing else of the library is visible to Swift.
 *
 * Conventions
 *   - Every fallible function returns kvc_status: 0 on success, a negative
 *     discriminated code on failure. kvc_last_error_message() gives the text
 *     recorded on the calling thread. Nothing aborts the process: what the
 *     reference treats as a fatalError/precondition is KVC_ERR_INVALID_ARG or
 *     KVC_ERR_INVALID_STATE here, and the Swift wrapper decides whether to trap.
 *   - Handles (kvc_cache, kvc_round, kvc_comm) are opaque and owned by the
 *     caller; *_free is safe on NULL. A handle owns its device buffers.
 *   - Tensors cross the boundary as kvc_tensor: a raw device pointer, a dtype,
 *     up to 5 dims and element strides. Inputs are borrowed for the duration
 *     of the enqueue. Output views alias handle memory and stay valid until
 *     the next mutating call on that handle.
 *   - Every call that touches device memory takes a CUDA stream (cudaStream_t
 *     passed as void*, NULL = legacy default stream) and only enqueues work;
 *     the *_host entry points and kvc_state_export are the only ones that
 *     synchronise.
 *   - A handle is not thread-safe; like the reference's cache objects it is
 *     owned by one generation at a time. Distinct handles may be driven from
 *     distinct threads and streams.
 *   - There is no CPU fallback: on a machine without a CUDA device every
 *     device call fails with KVC_ERR_CUDA.
 */

#ifndef KVCACHE_B200_H
#define KVCACHE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ */
/* status, version                                                     */
/* ------------------------------------------------------------------ */

typedef int32_t kvc_status;
#define KVC_OK                   ((int32_t)0)
#define KVC_ERR_INTERNAL         ((int32_t)-1)
#define KVC_ERR_INVALID_ARG      ((int32_t)-2)  /* shape/dtype/handle rejected before any work       */
#define KVC_ERR_INVALID_STATE    ((int32_t)-3)  /* call not valid in the cache's current state       */
#define KVC_ERR_UNSUPPORTED      ((int32_t)-4)  /* valid in the reference, not built here (documented)*/
#define KVC_ERR_CUDA             ((int32_t)-5)  /* CUDA runtime error; message carries the string    */
#define KVC_ERR_OUT_OF_MEMORY    ((int32_t)-6)
#define KVC_ERR_NOT_TRIMMABLE    ((int32_t)-7)  /* staged round / rewind refused (fail-closed)       */
#define KVC_ERR_TIMEOUT          ((int32_t)-8)  /* a bounded device-side wait ran out                */
#define KVC_ERR_COMM             ((int32_t)-9)  /* NCCL error                                        */

/* Library version string, static storage. */
const char *kvc_version(void);

/* Message of the last failure on the calling thread (thread-local storage,
 * valid until the next kvc_* call on this thread); NULL if none. */
const char *kvc_last_error_message(void);

/* 1 when the library was built for and sees an sm_100 device, else 0. */
int32_t kvc_device_available(void);

/* ------------------------------------------------------------------ */
/* tensors                                                             */
/* ------------------------------------------------------------------ */

typedef enum {
    KVC_F32 = 0,
    KVC_F16 = 1,
    KVC_BF16 = 2,
    KVC_U32 = 3,
    KVC_BOOL = 4   /* one byte per element, mask arrays only */
} kvc_dtype;

#define KVC_MAX_DIMS 5

/* A strided view of device (or, for *_host calls, host) memory.
 * stride[] is in elements. */
typedef struct kvc_tensor {
    void   *data;
    int32_t dtype;                 /* kvc_dtype */
    int32_t ndim;
    int64_t shape[KVC_MAX_DIMS];
    int64_t stride[KVC_MAX_DIMS];
} kvc_tensor;

/* Attention mask modes; mirrors MLXFast.ScaledDotProductAttentionMaskMode as
 * used by attentionWithCacheUpdate (AttentionUtils.swift:37-95). */
typedef enum {
    KVC_MASK_NONE = 0,
    KVC_MASK_CAUSAL = 1,   /* query row l may see key t when t <= (T - L) + l */
    KVC_MASK_ARRAY = 2     /* explicit array: bool (keep where true) or additive,
                              broadcastable to [B, Hq, L, T]                     */
} kvc_mask_mode;

/* ------------------------------------------------------------------ */
/* cache objects                                                       */
/* ------------------------------------------------------------------ */

typedef struct kvc_cache kvc_cache;

typedef enum {
    KVC_KIND_SIMPLE = 0,     /* KVCacheSimple        KVCache.swift:391-538  */
    KVC_KIND_ROTATING = 1,   /* RotatingKVCache      KVCache.swift:541-900  */
    KVC_KIND_QUANTIZED = 2,  /* QuantizedKVCache     KVCache.swift:923-1210 */
    KVC_KIND_TURBO = 3,      /* TurboQuantKVCache    TurboQuantKVCache.swift:633-1604 */
    KVC_KIND_CHUNKED = 4,    /* ChunkedKVCache       KVCache.swift:1213-1304 (chunkSize travels in max_size, <= 0 = nil) */
    KVC_KIND_LIST = 5        /* CacheList            KVCache.swift:1556-1726 (made by kvc_list_create) */
} kvc_kind;

/* Construction parameters; one struct for the four initialisers
 *   KVCacheSimple()                      + var step = 256      (KVCache.swift:394-398)
 *   RotatingKVCache(maxSize:keep:step:)                         (KVCache.swift:565-570)
 *   QuantizedKVCache(groupSize:bits:mode:)   64 / 8 / affine    (KVCache.swift:931-937)
 *   TurboQuantKVCache(bits:keyBits:valueBits:seed:keyGroupSize:) (TurboQuantKVCache.swift:695-707)
 * Fields that do not apply to `kind` are ignored. Zero-initialise, then call
 * kvc_config_default() to get the reference's defaults. */
typedef struct kvc_config {
    int32_t  kind;            /* kvc_kind                                            */
    int32_t  device;          /* CUDA device ordinal; -1 = current device            */
    int32_t  step;            /* growth quantum in tokens (256)                      */
    int32_t  max_size;        /* rotating: window capacity                           */
    int32_t  keep;            /* rotating: pinned prefix                             */
    int32_t  group_size;      /* quantized: requested group size (64)                */
    int32_t  bits;            /* quantized: 2, 4 or 8; turbo: bits for keys and values */
    int32_t  key_bits;        /* turbo: -1 = bits; 0 = raw keys; 8 = affine keys     */
    int32_t  value_bits;      /* turbo: -1 = bits                                    */
    int32_t  key_group_size;  /* turbo affine-K group size (64)                      */
    uint64_t seed;            /* turbo: rotation seed (42); values use seed + 1      */
    int64_t  reserve_tokens;  /* capacity hint: tokens to reserve up front, 0 = none.
                                 Invisible to the protocol surface (state exports
                                 only ever expose [..<offset]).                      */
    int32_t  turbo_affine_values; /* turbo: 1 = store values as group-wise affine codes
                                 (value_bits, key_group_size) instead of rotated
                                 codebook indices. Not a mode of the reference's
                                 TurboQuantKVCache; it is the "keys 3-bit codebook,
                                 values 4-bit affine" layout of the 70B benchmark
                                 configuration.                                      */
} kvc_config;

void       kvc_config_default(kvc_config *cfg, int32_t kind);
kvc_status kvc_create(const kvc_config *cfg, kvc_cache **out);
/* Buffers the handle still holds are released in the order of the stream its last
 * update / attention / state call ran on (kernels queued there may still read them), on
 * the handle's own device. A handle driven from several streams must be quiescent on the
 * others. */
void       kvc_free(kvc_cache *cache);

/* CacheList(caches...)  KVCache.swift:1556-1568. The list takes ownership of the
 * children (freeing the list frees them; do not free them yourself). Children
 * may be lists. update / attention on the list itself are refused like the
 * reference's fatalError (:1576-1578): work goes through kvc_list_child. */
kvc_status kvc_list_create(kvc_cache *const *children, int32_t count, kvc_cache **out);
int32_t    kvc_list_count(const kvc_cache *list);
/* subscript(index:) :1572-1574: borrowed handle, valid while the list lives. */
kvc_cache *kvc_list_child(const kvc_cache *list, int32_t index);

/* ChunkedKVCache.maybeTrimFront()  KVCache.swift:1222-1232: once the buffer holds
 * chunkSize rows or more, drops everything but its last chunkSize rows and advances
 * startPosition. kvc_start_position returns that counter (0 for other kinds). */
kvc_status kvc_maybe_trim_front(kvc_cache *cache, void *stream);
int64_t    kvc_start_position(const kvc_cache *cache);

/* prepare(lengths:) / finalize()  KVCache.swift:97-103. For every cache kind of this
 * library they are the reference's empty defaults (BaseKVCache :229-233; only the
 * state-space ArraysCache keeps the lengths); a CacheList forwards to its children
 * (:1633-1643). Provided so that callers written against the protocol link. */
kvc_status kvc_prepare(kvc_cache *cache, const int32_t *lengths, int32_t count);
kvc_status kvc_finalize(kvc_cache *cache);

/* createCausalMask(n:offset:windowSize:lengths:)  KVCache.swift:253-275. Writes the boolean
 * mask (one byte per element) for `n` query rows at `offset`: [n, offset + n] without
 * lengths, [batch, 1, n, offset + n] with `lengths` (device int32 [batch]: row b also
 * requires key index < lengths[b]). window_size < 0 means nil. */
kvc_status kvc_create_causal_mask(int32_t n, int64_t offset, int64_t window_size, const int32_t *lengths_dev,
                                  int32_t batch, void *out_mask, void *stream);

/* KVCache.offset / maxSize (-1 when nil) / kind. `offset` is a settable
 * property in the reference (BaseKVCache.offset, KVCache.swift:185); setting
 * it moves no data. */
int64_t    kvc_offset(const kvc_cache *cache);
kvc_status kvc_set_offset(kvc_cache *cache, int64_t offset);
int64_t    kvc_max_size(const kvc_cache *cache);
int32_t    kvc_kind_of(const kvc_cache *cache);
/* RotatingKVCache.idx (ring write cursor); -1 for other kinds. */
int64_t    kvc_ring_index(const kvc_cache *cache);
/* QuantizedKVCache.groupSize (after first-use resolution) and bits. */
int32_t    kvc_group_size(const kvc_cache *cache);
int32_t    kvc_bits(const kvc_cache *cache);
/* TurboQuantKVCache.isCompressed. */
int32_t    kvc_is_compressed(const kvc_cache *cache);
/* Bytes of device memory the handle currently holds (TurboQuantKVCache.memoryBytes
 * counts logical rows; this counts reserved capacity as well). */
int64_t    kvc_memory_bytes(const kvc_cache *cache);

/* Reserve capacity for `tokens` cached positions without changing any
 * observable state. Has no counterpart in the reference, which re-allocates
 * and copies every `step` tokens (KVCache.swift:413-436). */
kvc_status kvc_reserve(kvc_cache *cache, int64_t tokens, int32_t batch, int32_t kv_heads,
                       int32_t head_dim, int32_t dtype, void *stream);

/* update(keys:values:) -> (keys, values)
 *   KVCacheSimple.update      KVCache.swift:404-447
 *   RotatingKVCache.update    KVCache.swift:742-750 (updateInPlace :684-740, updateConcat :660-682)
 *   TurboQuantKVCache.update  TurboQuantKVCache.swift:802-846 (raw prefill phase)
 * keys/values: [B, Hkv, S, D]. out_k/out_v receive views of the cached K/V
 * exactly as the reference returns them (length `offset`, or the physical ring
 * for a full rotating cache). QuantizedKVCache rejects this call like the
 * reference does (KVCache.swift:1106-1110). */
kvc_status kvc_update(kvc_cache *cache, const kvc_tensor *keys, const kvc_tensor *values,
                      void *stream, kvc_tensor *out_k, kvc_tensor *out_v);

/* updateQuantized(keys:values:) -> ((w, scales, biases), (w, scales, biases))
 *   QuantizedKVCache.updateQuantized  KVCache.swift:1011-1102
 * out_k[3]/out_v[3]: views [B,Hkv,offset,D*bits/32] u32, [B,Hkv,offset,D/g]
 * scales and biases in the input dtype. */
kvc_status kvc_update_quantized(kvc_cache *cache, const kvc_tensor *keys, const kvc_tensor *values,
                                void *stream, kvc_tensor out_k[3], kvc_tensor out_v[3]);

/* getQuantizedState()  KVCache.swift:993-1002. Returns KVC_ERR_INVALID_STATE
 * when the cache is empty (the reference returns nil). */
kvc_status kvc_quantized_state(kvc_cache *cache, kvc_tensor out_k[3], kvc_tensor out_v[3]);

/* attentionWithCacheUpdate(queries:keys:values:cache:scale:mask:)  AttentionUtils.swift:37-95
 * The fused fast path: appends (or quantizes / encodes) the new K/V into the
 * cache and runs attention over the cache, dispatching on the cache kind as
 * the reference does:
 *   turbo, L>1 and not yet compressed -> raw update + SDPA      (:56-63)
 *   turbo otherwise                   -> compressedAttention     (:68-71, TurboQuantKVCache.swift:1164-1446)
 *   quantized                         -> updateQuantized + quantizedScaledDotProductAttention (:72-84)
 *   simple / rotating                 -> update + scaledDotProductAttention (:86-93)
 * queries [B,Hq,L,D], keys/values [B,Hkv,L,D], out [B,Hq,L,D] in the query
 * dtype. mask may be NULL unless mask_mode == KVC_MASK_ARRAY. */
kvc_status kvc_attention(kvc_cache *cache, const kvc_tensor *queries, const kvc_tensor *keys,
                         const kvc_tensor *values, float scale, int32_t mask_mode,
                         const kvc_tensor *mask, const kvc_tensor *out, void *stream);

/* Same call with every tensor in HOST memory (contiguous; pinned memory keeps
 * the copies asynchronous): enqueues the host-to-device copies of the step's
 * inputs, kvc_attention, and the device-to-host copy of the result on `stream`.
 * With synchronize != 0 the call returns after the result has landed in
 * `out`; with 0 the caller synchronises the stream itself (e.g. once per
 * decode step). */
kvc_status kvc_attention_host(kvc_cache *cache, const kvc_tensor *queries, const kvc_tensor *keys,
                              const kvc_tensor *values, float scale, int32_t mask_mode,
                              const kvc_tensor *mask, const kvc_tensor *out, void *stream,
                              int32_t synchronize);

/* MLXFast.scaledDotProductAttention as called at AttentionUtils.swift:46-52,
 * :59-62, :87-93, for callers that use update() and then attend themselves.
 * q [B,Hq,L,D], k/v [B,Hkv,T,D] (any strides), out [B,Hq,L,D]. */
kvc_status kvc_sdpa(const kvc_tensor *queries, const kvc_tensor *keys, const kvc_tensor *values,
                    float scale, int32_t mask_mode, const kvc_tensor *mask,
                    const kvc_tensor *out, void *stream);

/* kvc_sdpa without any allocation. No counterpart in the reference.
 * For hosts that must keep the CUDA allocator off the request path: a server
 * whose own pool owns the device's memory budget, or a decoder that cannot
 * tolerate the device-wide synchronisation of cudaMalloc/cudaFree. The
 * regular entry points keep split-K partials in an arena that grows on demand;
 * this one keeps them in a fixed 4 MiB array inside the library's device image
 * (present on every GPU that loads the library, until the process exits), and
 * it calls no cudaMalloc, cudaFree or other allocating routine.
 * Limits: raw f32/f16/bf16 K/V contiguous along the head dim, D <= 256, mask
 * none or causal, and B*Hq*L*(4*D+8) + 256 bytes must fit the array; larger
 * calls are rejected with KVC_ERR_INVALID_ARG (use kvc_sdpa for those).
 * The first call on a device looks up the array's device address
 * (cudaGetSymbolAddress) with that device current; make that call before any
 * stream capture. All calls share the array: calls whose kernels can overlap
 * on the GPU race on it, so keep them on one stream or order them. */
kvc_status kvc_sdpa_noalloc(const kvc_tensor *queries, const kvc_tensor *keys,
                            const kvc_tensor *values, float scale, int32_t mask_mode,
                            const kvc_tensor *out, void *stream);

/* quantizedScaledDotProductAttention(queries:quantizedKeys:quantizedValues:scale:mask:groupSize:bits:mode:)
 *   KVCache.swift:2351-2447.  qk/qv: (codes u32, scales, biases). */
kvc_status kvc_quantized_sdpa(const kvc_tensor *queries, const kvc_tensor qk[3],
                              const kvc_tensor qv[3], float scale, int32_t mask_mode,
                              const kvc_tensor *mask, int32_t group_size, int32_t bits,
                              const kvc_tensor *out, void *stream);

/* quantized(_:groupSize:bits:) / dequantized(...) as used at KVCache.swift:506-509,
 * :1069-1070, :1197-1202 (MLX affine mode). x [..., D] -> codes u32
 * [..., D*bits/32], scales/biases [..., D/g] in x's dtype. Tensors contiguous. */
kvc_status kvc_affine_quantize(const kvc_tensor *x, int32_t group_size, int32_t bits,
                               const kvc_tensor *codes, const kvc_tensor *scales,
                               const kvc_tensor *biases, void *stream);
kvc_status kvc_affine_dequantize(const kvc_tensor *codes, const kvc_tensor *scales,
                                 const kvc_tensor *biases, int32_t group_size, int32_t bits,
                                 const kvc_tensor *out, void *stream);

/* trim(_:) -> tokens trimmed.
 *   KVCacheSimple :474-478, RotatingKVCache :826-831, QuantizedKVCache :1171-1175,
 *   TurboQuantKVCache.swift:1583-1603 */
kvc_status kvc_trim(kvc_cache *cache, int64_t n, int64_t *out_trimmed);
/* isTrimmable / isTrimmable(after:)  KVCache.swift:817-823 (others: always 1). */
int32_t    kvc_is_trimmable(const kvc_cache *cache);
int32_t    kvc_is_trimmable_after(const kvc_cache *cache, int64_t positions);

/* trimPromptCache / canTrimPromptCache over a list of caches (KVCache.swift:2293-2306):
 * all-or-nothing; returns 0 trimmed when any cache is not trimmable. */
int32_t    kvc_can_trim_prompt_cache(kvc_cache *const *caches, int32_t count);
kvc_status kvc_trim_prompt_cache(kvc_cache *const *caches, int32_t count, int64_t n,
                                 int64_t *out_trimmed);

/* makeMask(n:windowSize:returnArray:)
 *   BaseKVCache.makeMask :236-250, RotatingKVCache.makeMask :834-871,
 *   createCausalMask :253-275.
 * window_size < 0 means nil. On return *out_mode is a kvc_mask_mode; when it
 * is KVC_MASK_ARRAY, out_mask (caller-allocated KVC_BOOL device tensor of at
 * least out_rows*out_cols bytes, may be NULL to query the shape only) is
 * filled on `stream` and out_rows/out_cols give its shape ([n, offset+n] for
 * multi-token masks, [1, maskSize] for the rolled single-token mask). */
kvc_status kvc_make_mask(const kvc_cache *cache, int32_t n, int64_t window_size,
                         int32_t return_array, int32_t *out_mode, int64_t *out_rows,
                         int64_t *out_cols, void *out_mask, void *stream);

/* state / metaState (the serialisation surface).
 * kvc_state_count: number of arrays `state` would return (0 when empty).
 * kvc_state_get:   view i of the state, exactly the reference's arrays
 *                  (shape, dtype, order; for a rotating cache the PHYSICAL ring).
 * kvc_state_set:   adopt `count` device arrays (copied) as the new state.
 * kvc_meta_state:  writes the metaState strings joined by '\n' into buf
 *                  (returns the needed size incl. NUL in *out_len).
 * kvc_set_meta_state: parse the same format. */
int32_t    kvc_state_count(const kvc_cache *cache);
kvc_status kvc_state_get(kvc_cache *cache, int32_t index, kvc_tensor *out);
kvc_status kvc_state_set(kvc_cache *cache, const kvc_tensor *arrays, int32_t count, void *stream);
kvc_status kvc_state_export(kvc_cache *cache, int32_t index, void *host_dst, size_t host_bytes,
                            kvc_tensor *out_desc, void *stream);
kvc_status kvc_meta_state(const kvc_cache *cache, char *buf, size_t buf_len, size_t *out_len);
kvc_status kvc_set_meta_state(kvc_cache *cache, const char *joined);

/* copy()  KVCache.swift:525-533, :877-885, :1177-1185. Deep copy on `stream`. */
kvc_status kvc_copy(const kvc_cache *cache, void *stream, kvc_cache **out);

/* KVCacheSimple.toQuantized(groupSize:bits:) :486-523 and
 * QuantizedKVCache.toUnquantized() :1188-1209. The source is left untouched. */
kvc_status kvc_to_quantized(const kvc_cache *simple, int32_t group_size, int32_t bits,
                            void *stream, kvc_cache **out);
kvc_status kvc_to_unquantized(const kvc_cache *quantized, void *stream, kvc_cache **out);
/* maybeTurboQuantizeKVCache's per-layer conversion (TurboQuantKVCache.swift:1748-1759):
 * new turbo cache holding the simple cache's rows as its raw prefill phase. */
kvc_status kvc_to_turbo(const kvc_cache *simple, int32_t key_bits, int32_t value_bits,
                        int32_t key_group_size, void *stream, kvc_cache **out);

/* RotatingKVCache.logicalView(tail:)  KVCache.swift:631-658: the trailing
 * `tail` entries in chronological order, without mutating the ring. The
 * views alias a scratch buffer owned by the handle (valid until the next call
 * on it). KVC_ERR_INVALID_STATE before the first write (reference: nil). */
kvc_status kvc_logical_view(kvc_cache *cache, int64_t tail, void *stream,
                            kvc_tensor *out_k, kvc_tensor *out_v);

/* ------------------------------------------------------------------ */
/* staged speculative round over a rotating cache                      */
/*   RotatingStagedKVCache.swift:12-130, KVCacheRound.swift:87-206,    */
/*   KVCacheStorage.beginRound/commit/rollback/rewindLastRound         */
/*   KVCachePlan.swift:219-347                                         */
/* ------------------------------------------------------------------ */

typedef struct kvc_round kvc_round;

/* Begin a round of at most `max_positions` staged tokens over `cache`
 * (rotating: rows are staged beside the ring; other kinds: written through
 * and trimmed on commit). Fail-closed: refuses (KVC_ERR_NOT_TRIMMABLE) before
 * touching anything if the cache cannot honour a later rollback. */
kvc_status kvc_round_begin(kvc_cache *cache, int32_t max_positions, kvc_round **out);
/* update() during the round: returns logicalView(tail: min(offset, maxSize-1)) ++ staged. */
kvc_status kvc_round_update(kvc_round *round, const kvc_tensor *keys, const kvc_tensor *values,
                            void *stream, kvc_tensor *out_k, kvc_tensor *out_v);
/* attention over the same presentation (update + SDPA). */
kvc_status kvc_round_attention(kvc_round *round, const kvc_tensor *queries,
                               const kvc_tensor *keys, const kvc_tensor *values, float scale,
                               int32_t mask_mode, const kvc_tensor *mask, const kvc_tensor *out,
                               void *stream);
/* Offset the round presents to the model (cache offset + staged rows). */
int64_t    kvc_round_offset(const kvc_round *round);
/* Keep the first `retain` staged rows (written through the cache's normal
 * update path), drop the rest; ends the round. */
kvc_status kvc_round_commit(kvc_round *round, int32_t retain, void *stream);
/* Drop every staged row; ends the round. */
kvc_status kvc_round_rollback(kvc_round *round, void *stream);
/* rewindLastRound(count): take back up to `count` of the positions the last
 * committed round kept. Uses the restore point recorded at commit when the
 * ring had wrapped (restore, then replay the surviving prefix); without one it
 * is a plain trim, which a non-trimmable cache refuses (0 rewound). Any other
 * write to the cache drops the restore point. */
kvc_status kvc_rewind_last_round(kvc_cache *cache, int64_t count, void *stream,
                                 int64_t *out_rewound);
void       kvc_round_free(kvc_round *round);

/* ------------------------------------------------------------------ */
/* the caller's step around the cache: rotary positions at the cache     */
/* offset, speculative rounds over a layer list                          */
/* ------------------------------------------------------------------ */

/* Parameters of the rotary embedding the models construct (MLXNN.RoPE as used at
 * MLXLLM/Models/Llama.swift:36-41): the first `dims` features of every head are rotated,
 * pairs (i, i + dims/2) or, when `traditional`, (2i, 2i+1); angle of pair i at position p is
 * p * scale * base^(-2i/dims). */
typedef struct kvc_rope_config {
    int32_t dims;         /* rotated features per head (even, <= head dim) */
    int32_t traditional;  /* 1 = interleaved pairs */
    float   base;         /* 10000 */
    float   scale;        /* 1 */
} kvc_rope_config;

/* applyRotaryPosition(rope, to: x, offset:)  MLXLMCommon/RoPEApplication.swift:58-69.
 * x, out: [B, H, L, D] (inner stride 1; out may alias x). Row l gets position offset + l. */
kvc_status kvc_rope(const kvc_tensor *x, int64_t offset, const kvc_rope_config *rope,
                    const kvc_tensor *out, void *stream);

/* The attention block's cache step as the models write it (MLXLLM/Models/Llama.swift:58-69):
 *   offset  = cache.ropeOffset            (the cache offset; 0 without a cache)
 *   queries = applyRotaryPosition(rope, to: queries, offset: offset)
 *   keys    = applyRotaryPosition(rope, to: keys,    offset: offset)
 *   out     = attentionWithCacheUpdate(queries, keys, values, cache, scale, mask)
 * Queries and keys are rotated by ONE launch into buffers the handle keeps, then the
 * fused update + attention runs on them; the inputs are not modified. */
kvc_status kvc_attention_rope(kvc_cache *cache, const kvc_tensor *queries, const kvc_tensor *keys,
                              const kvc_tensor *values, const kvc_rope_config *rope, float scale,
                              int32_t mask_mode, const kvc_tensor *mask, const kvc_tensor *out,
                              void *stream);

/* A speculative round over the layer list of a model (KVCacheStorage.beginRound / commit,
 * KVCachePlan.swift:219-300, as driven by the speculative iterators, Evaluate.swift:1179-1286).
 * kvc_storage_begin_round opens one staged round per cache, all or nothing: when any
 * cache refuses (it could not be rewound after `max_positions` more tokens) nothing is
 * opened and KVC_ERR_NOT_TRIMMABLE comes back, so the caller can fall back to unstaged
 * decoding like the reference does (:219-228). out_rounds receives `count` handles.
 * kvc_storage_round_attention runs the verify pass of every layer (queries[i] etc. belong
 * to caches[i]'s round) on `stream`. kvc_storage_commit keeps the first `retaining`
 * positions the round wrote in every cache, drops the rest and frees the rounds
 * (retaining 0 = rollback). */
kvc_status kvc_storage_begin_round(kvc_cache *const *caches, int32_t count, int32_t max_positions,
                                   kvc_round **out_rounds);
kvc_status kvc_storage_round_attention(kvc_round *const *rounds, int32_t count, const kvc_tensor *queries,
                                       const kvc_tensor *keys, const kvc_tensor *values, float scale,
                                       int32_t mask_mode, const kvc_tensor *outs, void *stream);
kvc_status kvc_storage_commit(kvc_round **rounds, int32_t count, int32_t retaining, void *stream);

/* The rewind at the end of speculateRound without staged rounds (Evaluate.swift:1262-1264):
 * the main model's caches give back num_draft - accepted positions, the draft model's
 * max(num_draft - accepted - 1, 0); both through trimPromptCache (all or nothing).
 * is_draft selects the rule; *out_trimmed receives the positions actually trimmed. */
kvc_status kvc_speculate_rewind(kvc_cache *const *caches, int32_t count, int32_t num_draft,
                                int32_t accepted, int32_t is_draft, int64_t *out_trimmed);

/* ------------------------------------------------------------------ */
/* TurboQuant codec pieces (TurboQuantKVCache.swift:47-621,            */
/* TurboQuantKernels.swift:224-342, :354-411)                          */
/* ------------------------------------------------------------------ */

/* PW(count,bits) = ceil(count*bits/32)  TurboQuantPacking.packedWidth :354-356 */
int32_t    kvc_turbo_packed_width(int32_t count, int32_t bits);
/* Lloyd-Max centroids (2^bits, ascending) and boundaries (2^bits-1 midpoints)
 * for the Beta coordinate distribution; host arrays. */
kvc_status kvc_turbo_codebook(int32_t dim, int32_t bits, float *centroids, float *boundaries);
/* The seeded +-1 sign vector of the randomised Hadamard rotation; host array [dim]. */
kvc_status kvc_turbo_signs(int32_t dim, uint64_t seed, float *signs);
/* Override a turbo cache's codebooks / sign vectors (e.g. with the tables the
 * Swift side already holds) before its first encode. NULL keeps the default. */
kvc_status kvc_turbo_set_codec(kvc_cache *cache, const float *key_centroids,
                               const float *value_centroids, const float *key_signs,
                               const float *value_signs, int32_t dim);
/* The dense random rotation the codec uses for head dims that are not powers of two
 * (TurboQuantRotation.rotationMatrix, TurboQuantKVCache.swift:246-259): QR of a seeded Gaussian
 * matrix, sign-corrected; host array, row-major [dim, dim]. The reference draws it from MLXRandom
 * and factors it with MLX's QR (not reproducible outside MLX); this library's generator is its own
 * (splitmix64 + Box-Muller, Householder QR in double precision). kvc_turbo_set_rotation hands a
 * cache the matrices a host already holds (before the first encode); NULL keeps the default. */
kvc_status kvc_turbo_rotation(int32_t dim, uint64_t seed, float *rotation);
kvc_status kvc_turbo_set_rotation(kvc_cache *cache, const float *key_rotation,
                                  const float *value_rotation, int32_t dim);
/* Fused WHT encode of rows [rows, D] -> packed [rows, PW] u32 + raw norms f32
 * (fusedEncodeWHT, TurboQuantKernels.swift:224-342 / :1672-1719). signs_dev is
 * a device array [D]; boundaries_host a host array [2^bits - 1]. */
kvc_status kvc_turbo_encode(const kvc_tensor *rows, const float *signs_dev,
                            const float *boundaries_host, int32_t bits,
                            const kvc_tensor *packed, const kvc_tensor *norms, void *stream);

/* ------------------------------------------------------------------ */
/* prompt-cache files (safetensors, shared with Python mlx-lm)          */
/* ------------------------------------------------------------------ */

/* savePromptCache(url:cache:metadata:) (KVCache.swift:1797-1846): tensors "i.j" = array j of cache
 * i's state, metadata "0.i.j" = its metaState strings, "1.<key>" = user metadata, "2.i" = class
 * name ("KVCache", "RotatingKVCache", "QuantizedKVCache", "TurboQuantKVCache"). Synchronises the
 * stream (the arrays are copied to the host). */
kvc_status kvc_save_prompt_cache(const char *path, kvc_cache *const *caches, int32_t count,
                                 const char *const *meta_keys, const char *const *meta_values,
                                 int32_t meta_count, void *stream);

/* loadPromptCache(url:) (KVCache.swift:1859-1987, restoreCacheFromMetaState :2031-2138): rebuilds
 * the caches of a file on `device` (-1 = current). Writes up to `capacity` handles (owned by the
 * caller) and the count; the user metadata into meta_buf as NUL-terminated strings, key then value,
 * closed by an empty key (*meta_needed = bytes needed; a smaller buffer is zero-filled). Call once
 * with out_caches = NULL to size both. Corrupt files (wrong array / metadata counts, unknown
 * class, sizes that do not match shapes) and files carrying model state are rejected. */
kvc_status kvc_load_prompt_cache(const char *path, int32_t device, kvc_cache **out_caches, int32_t capacity,
                                 int32_t *out_count, char *meta_buf, size_t meta_len, size_t *meta_needed,
                                 void *stream);

/* ------------------------------------------------------------------ */
/* list-level dynamic conversion (generation loop: maybeQuantizeKVCache) */
/* ------------------------------------------------------------------ */

/* resolveTurboScheme (TurboQuantKVCache.swift:1611-1635) / resolveAffineScheme (KVCache.swift:2455-2461):
 * return 1 and fill the outputs for a known scheme name, 0 otherwise. key_bits 0 = raw keys,
 * 8 = 8-bit affine keys. */
int32_t kvc_resolve_turbo_scheme(const char *scheme, int32_t *key_bits, int32_t *value_bits);
int32_t kvc_resolve_affine_scheme(const char *scheme, int32_t *bits, int32_t *group_size);

/* KVCacheTree.turboQuantProtectedPaths (KVCacheTree.swift:118-134) on a flat list of layers: writes
 * flags[i] = 1 for the layers that get 8-bit affine protection instead of a fragile TurboQuant scheme
 * (0 < key_bits < 8, or value_bits <= 2): the first and last min(2, eligible / 2) layers among those
 * whose kind is SIMPLE, QUANTIZED or TURBO. Pure host logic; kinds are KVC_KIND_* values. */
kvc_status kvc_turbo_protected_layers(const int32_t *kinds, int32_t count, int32_t key_bits,
                                      int32_t value_bits, int32_t *flags);

/* maybeAffineQuantizeKVCache (KVCache.swift:2500-2520): every KVCacheSimple of the list whose offset
 * exceeds compression_start is replaced by its toQuantized conversion (the old handle is freed, the
 * slot receives the new one); layers whose shape cannot be quantised stay as they are. *complete = 0
 * when some simple layer is still waiting for compression_start. */
kvc_status kvc_maybe_affine_quantize(kvc_cache **caches, int32_t count, int32_t bits, int32_t group_size,
                                     int64_t compression_start, void *stream, int32_t *complete);

/* maybeTurboQuantizeKVCache (TurboQuantKVCache.swift:1690-1762): the same walk with a TurboQuant
 * scheme; protected boundary layers become 8-bit affine (group 64) caches, the others
 * TurboQuantKVCache(bits = max(key_bits, value_bits), key_bits, value_bits) holding the live rows in
 * their raw phase; rotating layers are left alone. */
kvc_status kvc_maybe_turbo_quantize(kvc_cache **caches, int32_t count, int32_t key_bits, int32_t value_bits,
                                    int64_t quantized_kv_start, void *stream, int32_t *complete);

/* attentionWithCacheUpdate for `count` INDEPENDENT caches in one call: cache i appends keys[i] /
 * values[i] (one new token, [1, Hkv, 1, D]) and attends queries[i] ([1, Hq, 1, D]) over its own
 * length into outs[i]. This is a ragged decode batch the way the reference holds it (one cache
 * object per sequence, `BaseKVCache.offset` per cache, KVCache.swift:185; AttentionUtils.swift:37-95
 * called once per sequence), executed as ONE quantise-append launch and ONE attention launch when
 * all caches are QuantizedKVCache of one layout (up to 32 per launch); any other mix is executed
 * cache by cache with identical results. */
kvc_status kvc_attention_varlen(kvc_cache *const *caches, int32_t count, const kvc_tensor *queries,
                                const kvc_tensor *keys, const kvc_tensor *values, float scale,
                                const kvc_tensor *outs, void *stream);

/* Compressed-domain append without attention: compresses a raw prefix if the
 * cache still holds one, then encodes keys/values [B, H, S, D] and appends them
 * (the cache-side half of compressedAttention, TurboQuantKVCache.swift:1176-1200:
 * compressRawCache :895 + encodeNewToken :1010-1147). Chunked prefill into the
 * compressed representation uses this so that the raw prefix never has to exist
 * in full. */
kvc_status kvc_turbo_encode_new_token(kvc_cache *cache, const kvc_tensor *keys,
                                      const kvc_tensor *values, void *stream);

/* ------------------------------------------------------------------ */
/* multi-GPU: KV-head (or batch) sharded attention + all-gather        */
/* ------------------------------------------------------------------ */

typedef struct kvc_comm kvc_comm;
#define KVC_UNIQUE_ID_BYTES 128
/* Rank 0 creates the id, every rank passes the same bytes to kvc_comm_init. */
kvc_status kvc_comm_unique_id(uint8_t id[KVC_UNIQUE_ID_BYTES]);
kvc_status kvc_comm_init(int32_t rank, int32_t world, const uint8_t id[KVC_UNIQUE_ID_BYTES],
                         kvc_comm **out);
void       kvc_comm_free(kvc_comm *comm);
int32_t    kvc_comm_rank(const kvc_comm *comm);
int32_t    kvc_comm_world(const kvc_comm *comm);
/* Symmetric memory for the gathered attention outputs. Collective over the
 * communicator (every rank calls it with the same size, in the same order):
 * allocates `bytes` on this rank, maps every peer's allocation of the same
 * call through CUDA IPC and returns this rank's pointer. When the `out_full`
 * of kvc_attention_sharded lies inside such memory, the per-layer exchange is
 * done with peer stores instead of ncclAllGather: every rank's attention
 * kernel writes its slice into its own copy in the final layout, one kernel
 * pushes the slice into every peer's copy with plain 16-byte stores over
 * NVLink, releases an arrival counter in the peer's memory and waits until
 * every peer's slice has arrived (bounded: a wait that runs out stores code
 * 41 in the status word read by kvc_device_status and the kernel returns).
 * A gathered buffer may be written again only after at least one other
 * exchange on the same communicator has completed in between (consecutive
 * layers of a model satisfy this). Freed with the communicator.
 * No counterpart in the reference (it has no multi-device path). */
kvc_status kvc_comm_symm_alloc(kvc_comm *comm, size_t bytes, void *stream, void **out_ptr);
/* Iterations of the bounded arrival wait (default 2^26, each at least 64 ns). */
kvc_status kvc_comm_set_wait_limit(kvc_comm *comm, uint32_t iterations);

/* This rank attends over its own shard (cache holds Hkv/world heads, queries
 * carry the matching Hq/world heads) and the per-layer outputs are
 * all-gathered along the head axis into out_full [B, Hq, L, D] on every rank.
 * shard_axis: 1 = heads, 0 = batch (when Hkv < world). */
kvc_status kvc_attention_sharded(kvc_comm *comm, kvc_cache *cache, const kvc_tensor *queries,
                                 const kvc_tensor *keys, const kvc_tensor *values, float scale,
                                 int32_t mask_mode, const kvc_tensor *mask,
                                 const kvc_tensor *out_full, int32_t shard_axis, void *stream);

/* kvc_attention_sharded on caches[i] for i in [0, count): the layers of one
 * decode step, each followed by its all-gather, issued back to back. */
kvc_status kvc_attention_sharded_batch(kvc_comm *comm, kvc_cache *const *caches, int32_t count,
                                       const kvc_tensor *queries, const kvc_tensor *keys,
                                       const kvc_tensor *values, float scale, int32_t mask_mode,
                                       const kvc_tensor *outs_full, int32_t shard_axis, void *stream);

/* ------------------------------------------------------------------ */
/* instrumentation                                                     */
/* ------------------------------------------------------------------ */

/* Number of kernels this library launched from the calling thread since the
 * last reset; pass reset != 0 to zero the counter after reading it. */
int64_t    kvc_launch_count(int32_t reset);

/* The calls one decode step makes, issued back to back: kvc_attention (or,
 * with host != 0, kvc_attention_host) on caches[i] with q[i], k[i], v[i],
 * outs[i] for i in [0, count). This is the loop over layers of
 * TokenIterator.step (Evaluate.swift:905-916) as a native caller would run it;
 * mask arrays are not supported here. synchronize != 0 waits for the stream
 * once at the end. */
kvc_status kvc_attention_batch(kvc_cache *const *caches, int32_t count, const kvc_tensor *queries,
                               const kvc_tensor *keys, const kvc_tensor *values, float scale,
                               int32_t mask_mode, const kvc_tensor *outs, void *stream,
                               int32_t host, int32_t synchronize);

/* Device-side waits in the attention kernels (on shared-memory barriers fed
 * by TMA) are bounded. A wait that runs out stores a non-zero code in a
 * per-device status word instead of spinning forever; this call copies the
 * word of the current device back (synchronising with it). 0 = no wait ever
 * ran out; -1 = the word could not be read. The affected call's output is
 * undefined when the status is non-zero (KVC_ERR_TIMEOUT territory). */
int32_t    kvc_device_status(void);
/* Clears the status word of the current device (after the caller has dealt
 * with a reported timeout). */
kvc_status kvc_device_status_reset(void);
/* Launches a one-thread kernel whose bounded wait can never be satisfied: it
 * polls a word that stays zero `iterations` times (<= 2^24, each at least 32 ns),
 * then stores code 40 in the status word and returns. Lets a host check the
 * timeout reporting path without any fault or hang on the device. No
 * counterpart in the reference. */
kvc_status kvc_device_wait_probe(uint32_t iterations, void *stream);

/* Event timing of the dominant attention kernel. While enabled, every
 * attention call brackets its main kernel (not the merge or append kernels)
 * with CUDA events on the launching stream; kvc_timing_read waits for the
 * recorded events and returns the accumulated milliseconds and launch count.
 * Off by default; meant for a dedicated measurement pass. */
void       kvc_timing_enable(int32_t on);
kvc_status kvc_timing_read(double *total_ms, int64_t *launches, int32_t reset);

#ifdef __cplusplus
}
#endif

#endif /* KVCACHE_B200_H */
