// Swift face of libkvcache_b200: classes with the member names of
// MLXLMCommon's KVCache protocol (Libraries/MLXLMCommon/KVCache.swift:46-104)
// that forward to the C ABI in kvcache_b200.h. In the mlx-swift-lm tree these
// classes adopt `KVCache` / `QuantizedKVCacheProtocol` directly; here the
// array type is abstracted as `DeviceArray` so the file compiles without MLX.
//
// Not compiled in this repository's build image (no Swift toolchain); the C ABI
// underneath is what the test-suite exercises.
import CKVCacheB200
import Foundation

/// What the wrapper needs from an array type: a device pointer, a dtype, a shape
/// and element strides. `MLXArray` on a CUDA backend provides all four.
public protocol DeviceArray {
    var devicePointer: UnsafeMutableRawPointer? { get }
    var kvcDType: Int32 { get }
    var shape: [Int] { get }
    var elementStrides: [Int] { get }
    /// Wrap library-owned memory (a view into the cache) without copying.
    static func view(_ t: kvc_tensor) -> Self
    static func empty(shape: [Int], kvcDType: Int32) -> Self
}

public struct KVCacheB200Error: Error, CustomStringConvertible {
    public let status: Int32
    public let description: String
}

@inline(__always)
func check(_ status: kvc_status) throws {
    if status != 0 {
        let msg = kvc_last_error_message().map { String(cString: $0) } ?? "unknown error"
        throw KVCacheB200Error(status: status, description: msg)
    }
}

/// The reference traps on programmer errors (fatalError / precondition); the
/// wrapper keeps that convention for the non-throwing protocol members.
@inline(__always)
func must(_ status: kvc_status) {
    do { try check(status) } catch { fatalError("\(error)") }
}

func describe<A: DeviceArray>(_ a: A) -> kvc_tensor {
    var t = kvc_tensor()
    t.data = a.devicePointer
    t.dtype = a.kvcDType
    t.ndim = Int32(a.shape.count)
    withUnsafeMutablePointer(to: &t.shape) { p in
        p.withMemoryRebound(to: Int64.self, capacity: 5) { s in
            for (i, d) in a.shape.enumerated() { s[i] = Int64(d) }
        }
    }
    withUnsafeMutablePointer(to: &t.stride) { p in
        p.withMemoryRebound(to: Int64.self, capacity: 5) { s in
            for (i, d) in a.elementStrides.enumerated() { s[i] = Int64(d) }
        }
    }
    return t
}

public enum MaskMode<A: DeviceArray> {
    case none, causal
    case array(A)
}

/// Base class: owns one kvc_cache handle. Mirrors BaseKVCache (KVCache.swift:184-251).
open class B200KVCache<A: DeviceArray> {
    private(set) var handle: OpaquePointer
    private var ownsHandle = true
    public var stream: UnsafeMutableRawPointer? = nil

    /// The library replaced (and freed) this wrapper's handle during a list-level conversion.
    func forgetHandle() { ownsHandle = false }

    /// Wrapper of the class that matches the handle's kind.
    static func wrap(adopting h: OpaquePointer) -> B200KVCache<A> {
        switch kvc_kind_of(h) {
        case KVC_KIND_ROTATING: return RotatingKVCacheB200<A>(adopting: h)
        case KVC_KIND_QUANTIZED: return QuantizedKVCacheB200<A>(adopting: h)
        case KVC_KIND_TURBO: return TurboQuantKVCacheB200<A>(adopting: h)
        case KVC_KIND_CHUNKED: return ChunkedKVCacheB200<A>(adopting: h)
        case KVC_KIND_LIST: return CacheListB200<A>(adopting: h)
        default: return KVCacheSimpleB200<A>(adopting: h)
        }
    }

    init(config: kvc_config) {
        var cfg = config
        var h: OpaquePointer? = nil
        must(kvc_create(&cfg, &h))
        handle = h!
    }

    init(adopting h: OpaquePointer) { handle = h }

    deinit { if ownsHandle { kvc_free(handle) } }

    public var offset: Int {
        get { Int(kvc_offset(handle)) }
        set { must(kvc_set_offset(handle, Int64(newValue))) }
    }

    public var maxSize: Int? {
        let m = kvc_max_size(handle)
        return m < 0 ? nil : Int(m)
    }

    /// update(keys:values:) -> (keys, values): views of the cached arrays.
    public func update(keys: A, values: A) -> (A, A) {
        var k = describe(keys), v = describe(values)
        var ok = kvc_tensor(), ov = kvc_tensor()
        must(kvc_update(handle, &k, &v, stream, &ok, &ov))
        return (A.view(ok), A.view(ov))
    }

    public var state: [A] {
        get {
            (0 ..< Int(kvc_state_count(handle))).map { i in
                var t = kvc_tensor()
                must(kvc_state_get(handle, Int32(i), &t))
                return A.view(t)
            }
        }
        set {
            var arrays = newValue.map(describe)
            must(kvc_state_set(handle, &arrays, Int32(arrays.count), stream))
        }
    }

    public var metaState: [String] {
        get {
            var n = 0
            must(kvc_meta_state(handle, nil, 0, &n))
            var buf = [CChar](repeating: 0, count: n)
            must(kvc_meta_state(handle, &buf, n, &n))
            return String(cString: buf).split(separator: "\n", omittingEmptySubsequences: false).map(String.init)
        }
        set { must(kvc_set_meta_state(handle, newValue.joined(separator: "\n"))) }
    }

    public var isTrimmable: Bool { kvc_is_trimmable(handle) != 0 }
    public func isTrimmable(after positions: Int) -> Bool { kvc_is_trimmable_after(handle, Int64(positions)) != 0 }

    @discardableResult
    public func trim(_ n: Int) -> Int {
        var t: Int64 = 0
        must(kvc_trim(handle, Int64(n), &t))
        return Int(t)
    }

    public func copy() -> B200KVCache<A> {
        var h: OpaquePointer? = nil
        must(kvc_copy(handle, stream, &h))
        return B200KVCache<A>(adopting: h!)
    }

    /// prepare(lengths:rightPadding:) / finalize() (KVCache.swift:86-104): no-ops for the caches of this path.
    public func prepare(lengths: [Int32]) {
        var l = lengths
        must(kvc_prepare(handle, &l, Int32(l.count)))
    }
    public func finalize() { must(kvc_finalize(handle)) }

    /// The cache step of an attention block (Llama.swift:58-100): rotary positions at this cache's offset
    /// for queries and keys, then attentionWithCacheUpdate.
    public func attention(queries: A, keys: A, values: A, rope: RoPEB200, scale: Float, mask: MaskMode<A> = .none) -> A {
        let out = A.empty(shape: queries.shape, kvcDType: queries.kvcDType)
        var q = describe(queries), k = describe(keys), v = describe(values), o = describe(out)
        var cfg = rope.config
        switch mask {
        case .none: must(kvc_attention_rope(handle, &q, &k, &v, &cfg, scale, Int32(KVC_MASK_NONE.rawValue), nil, &o, stream))
        case .causal: must(kvc_attention_rope(handle, &q, &k, &v, &cfg, scale, Int32(KVC_MASK_CAUSAL.rawValue), nil, &o, stream))
        case .array(let m):
            var mt = describe(m)
            must(kvc_attention_rope(handle, &q, &k, &v, &cfg, scale, Int32(KVC_MASK_ARRAY.rawValue), &mt, &o, stream))
        }
        return out
    }

    /// attentionWithCacheUpdate for this cache (AttentionUtils.swift:37-95).
    public func attention(queries: A, keys: A, values: A, scale: Float, mask: MaskMode<A> = .none) -> A {
        let out = A.empty(shape: queries.shape, kvcDType: queries.kvcDType)
        var q = describe(queries), k = describe(keys), v = describe(values), o = describe(out)
        switch mask {
        case .none: must(kvc_attention(handle, &q, &k, &v, scale, Int32(KVC_MASK_NONE.rawValue), nil, &o, stream))
        case .causal: must(kvc_attention(handle, &q, &k, &v, scale, Int32(KVC_MASK_CAUSAL.rawValue), nil, &o, stream))
        case .array(let m):
            var mt = describe(m)
            must(kvc_attention(handle, &q, &k, &v, scale, Int32(KVC_MASK_ARRAY.rawValue), &mt, &o, stream))
        }
        return out
    }
}

func defaults(_ kind: kvc_kind) -> kvc_config {
    var cfg = kvc_config()
    kvc_config_default(&cfg, Int32(kind.rawValue))
    return cfg
}

/// RoPE(dimensions:traditional:base:scale:) as the attention blocks hold it.
public struct RoPEB200 {
    public var dimensions: Int
    public var traditional = false
    public var base: Float = 10000
    public var scale: Float = 1
    public init(dimensions: Int, traditional: Bool = false, base: Float = 10000, scale: Float = 1) {
        self.dimensions = dimensions; self.traditional = traditional; self.base = base; self.scale = scale
    }
    var config: kvc_rope_config {
        kvc_rope_config(dims: Int32(dimensions), traditional: traditional ? 1 : 0, base: base, scale: scale)
    }
    /// applyRotaryPosition(rope, to: x, offset:) (RoPEApplication.swift:58-69)
    public func callAsFunction<A: DeviceArray>(_ x: A, offset: Int, stream: UnsafeMutableRawPointer? = nil) -> A {
        let out = A.empty(shape: x.shape, kvcDType: x.kvcDType)
        var xi = describe(x), o = describe(out), cfg = config
        must(kvc_rope(&xi, Int64(offset), &cfg, &o, stream))
        return out
    }
}

/// ChunkedKVCache (KVCache.swift:1213-1312).
public final class ChunkedKVCacheB200<A: DeviceArray>: B200KVCache<A> {
    override init(adopting h: OpaquePointer) { super.init(adopting: h) }

    public init(chunkSize: Int? = nil, step: Int = 256) {
        var cfg = defaults(KVC_KIND_CHUNKED)
        cfg.max_size = Int32(chunkSize ?? -1)     // the chunk size travels in max_size; -1 = nil
        cfg.step = Int32(step)
        super.init(config: cfg)
    }

    public func maybeTrimFront() { must(kvc_maybe_trim_front(handle, stream)) }
    public var startPosition: Int { Int(kvc_start_position(handle)) }
}

/// CacheList (KVCache.swift:1645-1790): a composite entry of the layer array. The children are handed
/// over to the list; `subscript` gives a borrowed wrapper of one of them.
public final class CacheListB200<A: DeviceArray>: B200KVCache<A> {
    override init(adopting h: OpaquePointer) { super.init(adopting: h) }

    public init(_ caches: B200KVCache<A>...) {
        var handles: [OpaquePointer?] = caches.map { $0.handle }
        var h: OpaquePointer? = nil
        must(kvc_list_create(&handles, Int32(handles.count), &h))
        for c in caches { c.forgetHandle() }      // the list owns them now
        super.init(adopting: h!)
    }

    public var count: Int { Int(kvc_list_count(handle)) }
    public subscript(index: Int) -> B200KVCache<A> {
        let w = B200KVCache<A>.wrap(adopting: kvc_list_child(handle, Int32(index))!)
        w.forgetHandle()                          // borrowed: the list frees it
        return w
    }
}

public final class KVCacheSimpleB200<A: DeviceArray>: B200KVCache<A> {
    override init(adopting h: OpaquePointer) { super.init(adopting: h) }

    public init(step: Int = 256) {
        var cfg = defaults(KVC_KIND_SIMPLE)
        cfg.step = Int32(step)
        super.init(config: cfg)
    }

    public func toQuantized(groupSize: Int = 64, bits: Int = 4) throws -> QuantizedKVCacheB200<A> {
        var h: OpaquePointer? = nil
        try check(kvc_to_quantized(handle, Int32(groupSize), Int32(bits), stream, &h))
        return QuantizedKVCacheB200<A>(adopting: h!)
    }
}

public final class RotatingKVCacheB200<A: DeviceArray>: B200KVCache<A> {
    override init(adopting h: OpaquePointer) { super.init(adopting: h) }

    public init(maxSize: Int, keep: Int = 0, step: Int = 256) {
        var cfg = defaults(KVC_KIND_ROTATING)
        cfg.max_size = Int32(maxSize)
        cfg.keep = Int32(keep)
        cfg.step = Int32(step)
        super.init(config: cfg)
    }

    /// logicalView(tail:) (KVCache.swift:631-658); nil before the first write.
    public func logicalView(tail: Int) -> (A, A)? {
        var k = kvc_tensor(), v = kvc_tensor()
        let st = kvc_logical_view(handle, Int64(tail), stream, &k, &v)
        if st == KVC_ERR_INVALID_STATE { return nil }
        must(st)
        return (A.view(k), A.view(v))
    }
}

public final class QuantizedKVCacheB200<A: DeviceArray>: B200KVCache<A> {
    public init(groupSize: Int = 64, bits: Int = 8) {
        var cfg = defaults(KVC_KIND_QUANTIZED)
        cfg.group_size = Int32(groupSize)
        cfg.bits = Int32(bits)
        super.init(config: cfg)
    }

    override init(adopting h: OpaquePointer) { super.init(adopting: h) }

    public var groupSize: Int { Int(kvc_group_size(handle)) }
    public var bits: Int { Int(kvc_bits(handle)) }

    /// updateQuantized(keys:values:) (KVCache.swift:1011-1102).
    public func updateQuantized(keys: A, values: A) -> ((A, A, A?), (A, A, A?)) {
        var k = describe(keys), v = describe(values)
        var ok = [kvc_tensor](repeating: kvc_tensor(), count: 3)
        var ov = [kvc_tensor](repeating: kvc_tensor(), count: 3)
        must(kvc_update_quantized(handle, &k, &v, stream, &ok, &ov))
        return ((A.view(ok[0]), A.view(ok[1]), A.view(ok[2])), (A.view(ov[0]), A.view(ov[1]), A.view(ov[2])))
    }
}

public final class TurboQuantKVCacheB200<A: DeviceArray>: B200KVCache<A> {
    override init(adopting h: OpaquePointer) { super.init(adopting: h) }

    public init(bits: Int = 4, keyBits: Int? = nil, valueBits: Int? = nil, seed: UInt64 = 42, keyGroupSize: Int = 64) {
        var cfg = defaults(KVC_KIND_TURBO)
        cfg.bits = Int32(bits)
        cfg.key_bits = Int32(keyBits ?? -1)
        cfg.value_bits = Int32(valueBits ?? -1)
        cfg.seed = seed
        cfg.key_group_size = Int32(keyGroupSize)
        super.init(config: cfg)
    }

    public var isCompressed: Bool { kvc_is_compressed(handle) != 0 }

    /// compressedAttention(queries:keys:values:scale:mask:) (TurboQuantKVCache.swift:1164-1446).
    public func compressedAttention(queries: A, keys: A, values: A, scale: Float, mask: MaskMode<A> = .none) -> A {
        attention(queries: queries, keys: keys, values: values, scale: scale, mask: mask)
    }

    /// The cache-side half of compressedAttention (compressRawCache :895 + encodeNewToken :1010-1147):
    /// chunked prefill straight into the compressed representation.
    public func encodeNewToken(keys: A, values: A) {
        var k = describe(keys), v = describe(values)
        must(kvc_turbo_encode_new_token(handle, &k, &v, stream))
    }
}

/// resolveTurboScheme (TurboQuantKVCache.swift:1611-1635).
public func resolveTurboSchemeB200(_ scheme: String?) -> (keyBits: Int, valueBits: Int)? {
    guard let scheme else { return nil }
    var kb: Int32 = 0, vb: Int32 = 0
    guard kvc_resolve_turbo_scheme(scheme, &kb, &vb) != 0 else { return nil }
    return (Int(kb), Int(vb))
}

/// maybeTurboQuantizeKVCache (TurboQuantKVCache.swift:1690-1762) over a flat layer list: converted
/// layers get a new handle (the library frees the old one), the wrappers are rebuilt around them.
@discardableResult
public func maybeTurboQuantizeKVCacheB200<A: DeviceArray>(
    cache: inout [B200KVCache<A>], keyBits: Int, valueBits: Int, quantizedKVStart: Int, stream: UnsafeMutableRawPointer? = nil
) -> Bool {
    var handles: [OpaquePointer?] = cache.map { $0.handle }
    var complete: Int32 = 0
    let status = handles.withUnsafeMutableBufferPointer {
        kvc_maybe_turbo_quantize($0.baseAddress, Int32($0.count), Int32(keyBits), Int32(valueBits), Int64(quantizedKVStart), stream, &complete)
    }
    precondition(status == KVC_OK, String(cString: kvc_last_error_message()))
    for i in cache.indices where handles[i] != cache[i].handle {
        cache[i].forgetHandle()     // already freed by the library
        cache[i] = B200KVCache<A>.wrap(adopting: handles[i]!)
    }
    return complete != 0
}

/// createCausalMask(n:offset:windowSize:lengths:) (KVCache.swift:253-275); `lengths` is a device int32 array.
public func createCausalMaskB200<A: DeviceArray>(
    n: Int, offset: Int, windowSize: Int? = nil, lengths: A? = nil, stream: UnsafeMutableRawPointer? = nil
) -> A {
    let batch = lengths?.shape[0] ?? 0
    let shape = lengths == nil ? [n, offset + n] : [batch, 1, n, offset + n]
    let out = A.empty(shape: shape, kvcDType: Int32(KVC_BOOL.rawValue))
    must(kvc_create_causal_mask(Int32(n), Int64(offset), Int64(windowSize ?? -1),
                                lengths?.devicePointer?.assumingMemoryBound(to: Int32.self), Int32(batch),
                                out.devicePointer, stream))
    return out
}

/// KVCacheStorage.beginRound / commit over the layer array (KVCachePlan.swift:219-347): one staged round
/// per cache, all or nothing; throws when some cache cannot stage the round (the caller decodes unstaged).
public final class StorageRoundB200<A: DeviceArray> {
    private var rounds: [OpaquePointer?]
    public init(caches: [B200KVCache<A>], maxPositions: Int) throws {
        var handles: [OpaquePointer?] = caches.map { $0.handle }
        rounds = [OpaquePointer?](repeating: nil, count: handles.count)
        try check(kvc_storage_begin_round(&handles, Int32(handles.count), Int32(maxPositions), &rounds))
    }
    deinit { for r in rounds where r != nil { kvc_round_free(r) } }

    /// The verify pass of every layer.
    public func attention(queries: [A], keys: [A], values: [A], scale: Float, causal: Bool, outs: [A],
                          stream: UnsafeMutableRawPointer? = nil) {
        var q = queries.map(describe), k = keys.map(describe), v = values.map(describe), o = outs.map(describe)
        let mode = Int32((causal ? KVC_MASK_CAUSAL : KVC_MASK_NONE).rawValue)
        must(kvc_storage_round_attention(&rounds, Int32(rounds.count), &q, &k, &v, scale, mode, &o, stream))
    }

    /// commit(retaining:): keeps the first `retaining` positions of the round in every cache (0 = rollback).
    public func commit(retaining: Int, stream: UnsafeMutableRawPointer? = nil) {
        must(kvc_storage_commit(&rounds, Int32(rounds.count), Int32(retaining), stream))
    }
}

/// The rewind at the end of speculateRound without staged rounds (Evaluate.swift:1262-1264).
@discardableResult
public func speculateRewindB200<A: DeviceArray>(caches: [B200KVCache<A>], numDraft: Int, accepted: Int, isDraft: Bool) -> Int {
    var handles: [OpaquePointer?] = caches.map { $0.handle }
    var trimmed: Int64 = 0
    must(kvc_speculate_rewind(&handles, Int32(handles.count), Int32(numDraft), Int32(accepted), isDraft ? 1 : 0, &trimmed))
    return Int(trimmed)
}

/// One decode step of a ragged batch held as one cache per sequence (kvc_attention_varlen): the
/// per-sequence attentionWithCacheUpdate calls of a layer in two launches.
public func attentionWithCacheUpdateVarlenB200<A: DeviceArray>(
    queries: [A], keys: [A], values: [A], caches: [B200KVCache<A>], scale: Float, outs: [A], stream: UnsafeMutableRawPointer? = nil
) {
    var handles: [OpaquePointer?] = caches.map { $0.handle }
    var q = queries.map(describe), k = keys.map(describe), v = values.map(describe), o = outs.map(describe)
    let status = kvc_attention_varlen(&handles, Int32(handles.count), &q, &k, &v, scale, &o, stream)
    precondition(status == KVC_OK, String(cString: kvc_last_error_message()))
}

/// maybeAffineQuantizeKVCache (KVCache.swift:2500-2520) over a flat layer list.
@discardableResult
public func maybeAffineQuantizeKVCacheB200<A: DeviceArray>(
    cache: inout [B200KVCache<A>], bits: Int, groupSize: Int, compressionStart: Int, stream: UnsafeMutableRawPointer? = nil
) -> Bool {
    var handles: [OpaquePointer?] = cache.map { $0.handle }
    var complete: Int32 = 0
    let status = handles.withUnsafeMutableBufferPointer {
        kvc_maybe_affine_quantize($0.baseAddress, Int32($0.count), Int32(bits), Int32(groupSize), Int64(compressionStart), stream, &complete)
    }
    precondition(status == KVC_OK, String(cString: kvc_last_error_message()))
    for i in cache.indices where handles[i] != cache[i].handle {
        cache[i].forgetHandle()     // already freed by the library
        cache[i] = B200KVCache<A>.wrap(adopting: handles[i]!)
    }
    return complete != 0
}

/// savePromptCache(url:cache:metadata:) (KVCache.swift:1797-1846) for caches held by the library. Model
/// state (`LMOutput.State`) is not a cache matter: callers that have one keep using the reference's
/// writer on `state` / `metaState`, which this wrapper exposes unchanged.
public func savePromptCacheB200<A: DeviceArray>(
    url: URL, cache: [B200KVCache<A>], metadata: [String: String] = [:], stream: UnsafeMutableRawPointer? = nil
) throws {
    var handles: [OpaquePointer?] = cache.map { $0.handle }
    let keys = metadata.keys.sorted()
    var cKeys: [UnsafePointer<CChar>?] = keys.map { UnsafePointer(strdup($0)) }
    var cValues: [UnsafePointer<CChar>?] = keys.map { UnsafePointer(strdup(metadata[$0]!)) }
    defer {
        for p in cKeys + cValues { free(UnsafeMutablePointer(mutating: p)) }
    }
    try check(kvc_save_prompt_cache(url.path, &handles, Int32(handles.count), &cKeys, &cValues, Int32(keys.count), stream))
}

/// loadPromptCache(url:) (KVCache.swift:1859-1871, restoreCacheFromMetaState :2031-2138). Files that
/// carry model state or cache classes outside this library make the call throw with the reference's
/// message; the caller then falls back to the reference's loader.
public func loadPromptCacheB200<A: DeviceArray>(
    url: URL, device: Int32 = -1, stream: UnsafeMutableRawPointer? = nil
) throws -> ([B200KVCache<A>], [String: String]) {
    var count: Int32 = 0
    var need = 0
    try check(kvc_load_prompt_cache(url.path, device, nil, 0, &count, nil, 0, &need, stream))
    var handles = [OpaquePointer?](repeating: nil, count: Int(count))
    var buffer = [CChar](repeating: 0, count: max(need, 1))
    try check(kvc_load_prompt_cache(url.path, device, &handles, count, &count, &buffer, buffer.count, &need, stream))
    // key NUL value NUL ... closed by an empty key
    var metadata: [String: String] = [:]
    var pos = 0
    while pos < buffer.count, buffer[pos] != 0 {
        let key = String(cString: Array(buffer[pos...]))
        pos += key.utf8.count + 1
        let value = String(cString: Array(buffer[pos...]))
        pos += value.utf8.count + 1
        metadata[key] = value
    }
    return (handles.prefix(Int(count)).map { B200KVCache<A>.wrap(adopting: $0!) }, metadata)
}
