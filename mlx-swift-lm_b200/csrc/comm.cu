// Multi-GPU plumbing: one process per GPU, each owning the cache rows of its
// KV heads (or of its batch slice). The only exchange on the path is the
// per-layer gather of attention outputs.
//
// Two forms of that exchange:
//  * peer stores (the fast one): when the caller's gathered-output buffer lies in
//    memory obtained from kvc_comm_symm_alloc, every rank's attention kernel writes
//    its slice straight into its own copy of the buffer in the final layout, and ONE
//    kernel per layer then pushes that slice into every peer's copy with ordinary
//    16-byte stores over NVLink, releases a per-source counter in the peer's memory
//    and waits (bounded) until every peer's slice has arrived here. No library
//    kernel, no TMA and no multicast touch peer memory: plain st.global only.
//  * ncclAllGather on the caller's stream (plus a re-ordering kernel when the heads
//    of a batch interleave) for any other buffer.
// NCCL is resolved with dlopen at first use so that the library loads (and every
// single-GPU entry point works) without it; the peer-store form uses it once per
// symmetric allocation, to hand the CUDA IPC handles round.
#include "cache.h"

#include <dlfcn.h>
#include <nccl.h>

#include <mutex>
#include <vector>

namespace kvc {
void cache_attention(kvc_cache *c, const kvc_tensor &q, const kvc_tensor &k, const kvc_tensor &v,
                     float scale, int32_t mask_mode, const kvc_tensor *mask, const kvc_tensor &out,
                     cudaStream_t s);

constexpr int KVC_MAX_RANKS = 8;

namespace {

struct NcclApi {
    void *handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
};

NcclApi &nccl() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        const char *names[] = {"libnccl.so.2", "libnccl.so"};
        for (const char *n : names) {
            api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
            if (api.handle) break;
        }
        if (!api.handle) return;
        api.GetUniqueId = (decltype(api.GetUniqueId))dlsym(api.handle, "ncclGetUniqueId");
        api.CommInitRank = (decltype(api.CommInitRank))dlsym(api.handle, "ncclCommInitRank");
        api.AllGather = (decltype(api.AllGather))dlsym(api.handle, "ncclAllGather");
        api.CommDestroy = (decltype(api.CommDestroy))dlsym(api.handle, "ncclCommDestroy");
        api.GetErrorString = (decltype(api.GetErrorString))dlsym(api.handle, "ncclGetErrorString");
    });
    if (!api.handle || !api.GetUniqueId || !api.CommInitRank || !api.AllGather || !api.CommDestroy)
        fail(KVC_ERR_COMM, "NCCL (libnccl.so.2) could not be loaded");
    return api;
}

void nccl_check(ncclResult_t r, const char *what) {
    if (r == ncclSuccess) return;
    const char *msg = nccl().GetErrorString ? nccl().GetErrorString(r) : "?";
    fail(KVC_ERR_COMM, std::string(what) + ": " + msg);
}

// [world, B, Hl, L*D] -> [B, world*Hl, L*D]
template <typename V>
__global__ void interleave_heads_kernel(const V *src, V *dst, int world, int B, int Hl, int64_t row_units,
                                        int64_t total) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int64_t u = i % row_units;
    int64_t r = i / row_units;
    const int h = (int)(r % Hl);
    r /= Hl;
    const int b = (int)(r % B);
    const int w = (int)(r / B);
    dst[(((int64_t)b * world + w) * Hl + h) * row_units + u] = src[i];
}

// One launch per layer of the peer-store exchange. Block (x, y): chunk x of the slice, peer slot y
// (the y-th rank other than this one). The slice is `rows` runs of `run16` 16-byte units, run r
// starting `row_stride16` units after run r - 1 (a rank's heads of one batch entry are one run).
// Each block copies its share of the runs from this rank's buffer to the same place in the peer's
// copy, makes the stores visible system-wide and bumps the counter this rank owns in the peer's
// flag array. Block (0, 0) then waits until every source's counter here has reached `expected`;
// a wait that runs out stores code 41 in the status word and returns.
struct ExchangeParams {
    const uint4 *src;                 // this rank's slice in its own copy
    uint4 *dst[KVC_MAX_RANKS];        // the same place in every rank's copy (dst[rank] unused)
    unsigned long long *peer_flags[KVC_MAX_RANKS];   // every rank's counter array as mapped here
    unsigned long long *my_flags;     // this rank's own counter array
    unsigned long long expected[KVC_MAX_RANKS];
    int64_t rows, run16, row_stride16;
    int32_t rank, world;
    uint32_t spin_limit;
    int *status;
};

__global__ void __launch_bounds__(256) exchange_kernel(const __grid_constant__ ExchangeParams p) {
    int peer = (int)blockIdx.y;
    if (peer >= p.rank) ++peer;   // skip this rank
    const int64_t total = p.rows * p.run16;
    uint4 *dst = p.dst[peer];
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / p.run16, u = i % p.run16;
        const int64_t off = r * p.row_stride16 + u;
        dst[off] = p.src[off];
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) atomicAdd_system(p.peer_flags[peer] + p.rank, 1ull);
    if (blockIdx.x != 0 || blockIdx.y != 0) return;
    // arrival wait: one lane per source rank
    if ((int)threadIdx.x < p.world && (int)threadIdx.x != p.rank) {
        const volatile unsigned long long *flag = p.my_flags + threadIdx.x;
        bool ok = false;
        for (uint32_t it = 0; it < p.spin_limit; ++it) {
            if (*flag >= p.expected[threadIdx.x]) { ok = true; break; }
            __nanosleep(64);
        }
        __threadfence_system();
        if (!ok) atomicExch(p.status, 41);
    }
}

}  // namespace
}  // namespace kvc

// Memory that exists on every rank at the same size and is mapped into every peer.
struct SymmRegion {
    void *local = nullptr;
    size_t bytes = 0;
    void *peer[kvc::KVC_MAX_RANKS] = {nullptr};   // peer[r]: rank r's copy as mapped here (peer[rank] = local)
};

struct kvc_comm {
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1;
    int device = 0;
    void *local = nullptr;
    size_t local_bytes = 0;
    void *gathered = nullptr;
    size_t gathered_bytes = 0;
    // peer-store exchange
    std::vector<SymmRegion> regions;
    SymmRegion flags;                                   // kvc::KVC_MAX_RANKS arrival counters (uint64) per rank
    unsigned long long expected[kvc::KVC_MAX_RANKS] = {0};   // arrivals this rank must have seen from each source so far
    uint32_t spin_limit = 1u << 26;                     // iterations of the bounded arrival wait
};

namespace {
thread_local std::string g_comm_error;

// Allocates `bytes` on this rank and maps every peer's allocation of the same call here. Collective:
// every rank of the communicator must make the call with the same size (the IPC handles travel in
// an ncclAllGather on `s`). The memory starts zeroed.
void symm_alloc(kvc_comm *c, size_t bytes, SymmRegion &r, cudaStream_t s) {
    using kvc::fail;
    KVC_REQUIRE(c->world <= kvc::KVC_MAX_RANKS, "symmetric memory supports at most 8 ranks");
    bytes = (bytes + 255) / 256 * 256;
    KVC_CUDA(cudaMalloc(&r.local, bytes));
    KVC_CUDA(cudaMemsetAsync(r.local, 0, bytes, s));
    r.bytes = bytes;
    r.peer[c->rank] = r.local;
    if (c->world == 1) {
        KVC_CUDA(cudaStreamSynchronize(s));
        return;
    }
    cudaIpcMemHandle_t mine;
    KVC_CUDA(cudaIpcGetMemHandle(&mine, r.local));
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    unsigned char *dev = nullptr;
    KVC_CUDA(cudaMalloc(&dev, 64 * (size_t)(c->world + 1)));
    std::vector<cudaIpcMemHandle_t> all((size_t)c->world);
    try {
        KVC_CUDA(cudaMemcpyAsync(dev, &mine, 64, cudaMemcpyHostToDevice, s));
        kvc::nccl_check(kvc::nccl().AllGather(dev, dev + 64, 64, ncclUint8, c->comm, s), "ncclAllGather (IPC handles)");
        KVC_CUDA(cudaMemcpyAsync(all.data(), dev + 64, 64 * (size_t)c->world, cudaMemcpyDeviceToHost, s));
        KVC_CUDA(cudaStreamSynchronize(s));
    } catch (...) {
        (void)cudaFree(dev);
        throw;
    }
    (void)cudaFree(dev);
    for (int p = 0; p < c->world; ++p) {
        if (p == c->rank) continue;
        void *mapped = nullptr;
        const cudaError_t e = cudaIpcOpenMemHandle(&mapped, all[(size_t)p], cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            (void)cudaGetLastError();
            fail(KVC_ERR_COMM, std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(e));
        }
        r.peer[p] = mapped;
    }
}

void symm_release(kvc_comm *c, SymmRegion &r) {
    for (int p = 0; p < c->world && p < kvc::KVC_MAX_RANKS; ++p)
        if (p != c->rank && r.peer[p]) (void)cudaIpcCloseMemHandle(r.peer[p]);
    if (r.local) (void)cudaFree(r.local);
    r = SymmRegion();
}

const SymmRegion *find_region(const kvc_comm *c, const void *ptr, size_t bytes) {
    for (const SymmRegion &r : c->regions) {
        const char *lo = (const char *)r.local;
        if ((const char *)ptr >= lo && (const char *)ptr + bytes <= lo + r.bytes) return &r;
    }
    return nullptr;
}

// Pushes this rank's slice of `full` (already written into this rank's copy) to every peer and waits for
// theirs. rows / run_bytes / row_stride_bytes describe the slice starting `slice_off` bytes into `full`.
void launch_exchange(kvc_comm *c, const SymmRegion &reg, void *full, size_t slice_off, int64_t rows, size_t run_bytes,
                     size_t row_stride_bytes, cudaStream_t s) {
    kvc::ExchangeParams p = {};
    const size_t base_off = (size_t)((char *)full - (char *)reg.local) + slice_off;
    p.src = (const uint4 *)((char *)reg.local + base_off);
    for (int r = 0; r < c->world; ++r) {
        p.dst[r] = (uint4 *)((char *)reg.peer[r] + base_off);
        p.peer_flags[r] = (unsigned long long *)c->flags.peer[r];
    }
    p.my_flags = (unsigned long long *)c->flags.local;
    p.rows = rows;
    p.run16 = (int64_t)(run_bytes / 16);
    p.row_stride16 = (int64_t)(row_stride_bytes / 16);
    p.rank = c->rank;
    p.world = c->world;
    p.spin_limit = c->spin_limit;
    p.status = kvc::device_status_word(c->device);
    const int64_t total16 = rows * p.run16;
    const unsigned gx = (unsigned)std::max<int64_t>(1, std::min<int64_t>(8, (total16 + 255) / 256));
    for (int r = 0; r < c->world; ++r) {
        if (r != c->rank) c->expected[r] += gx;   // every source rank launches the same grid
        p.expected[r] = c->expected[r];
    }
    kvc::exchange_kernel<<<dim3(gx, (unsigned)(c->world - 1)), 256, 0, s>>>(p);
    KVC_CUDA(cudaGetLastError());
    ++kvc::g_launch_count;
}
}  // namespace

extern "C" {

kvc_status kvc_comm_unique_id(uint8_t id[KVC_UNIQUE_ID_BYTES]) {
    try {
        static_assert(sizeof(ncclUniqueId) <= KVC_UNIQUE_ID_BYTES, "unique id does not fit");
        ncclUniqueId uid;
        kvc::nccl_check(kvc::nccl().GetUniqueId(&uid), "ncclGetUniqueId");
        memset(id, 0, KVC_UNIQUE_ID_BYTES);
        memcpy(id, &uid, sizeof(uid));
        return KVC_OK;
    } catch (const kvc::Error &e) {
        return kvc_internal_set_error(e.code, e.what());
    }
}

kvc_status kvc_comm_init(int32_t rank, int32_t world, const uint8_t id[KVC_UNIQUE_ID_BYTES], kvc_comm **out) {
    if (!out || !id) return kvc_internal_set_error(KVC_ERR_INVALID_ARG, "kvc_comm_init: null argument");
    *out = nullptr;
    try {
        KVC_REQUIRE(world >= 1 && rank >= 0 && rank < world, "kvc_comm_init: bad rank/world");
        kvc_comm *c = new kvc_comm();
        c->rank = rank;
        c->world = world;
        c->device = kvc::current_device();
        if (world > 1) {
            ncclUniqueId uid;
            memcpy(&uid, id, sizeof(uid));
            ncclResult_t r = kvc::nccl().CommInitRank(&c->comm, world, uid, rank);
            if (r != ncclSuccess) {
                delete c;
                kvc::nccl_check(r, "ncclCommInitRank");
            }
        }
        *out = c;
        return KVC_OK;
    } catch (const kvc::Error &e) {
        return kvc_internal_set_error(e.code, e.what());
    }
}

void kvc_comm_free(kvc_comm *c) {
    if (!c) return;
    if (c->comm) (void)kvc::nccl().CommDestroy(c->comm);
    if (c->local) (void)cudaFree(c->local);
    if (c->gathered) (void)cudaFree(c->gathered);
    for (SymmRegion &r : c->regions) symm_release(c, r);
    if (c->flags.local) symm_release(c, c->flags);
    (void)cudaGetLastError();
    delete c;
}

int32_t kvc_comm_rank(const kvc_comm *c) { return c ? c->rank : -1; }
int32_t kvc_comm_world(const kvc_comm *c) { return c ? c->world : -1; }

kvc_status kvc_comm_symm_alloc(kvc_comm *comm, size_t bytes, void *stream, void **out_ptr) {
    if (!comm || !out_ptr || bytes == 0)
        return kvc_internal_set_error(KVC_ERR_INVALID_ARG, "kvc_comm_symm_alloc: bad argument");
    *out_ptr = nullptr;
    try {
        cudaStream_t s = (cudaStream_t)stream;
        if (!comm->flags.local) symm_alloc(comm, 256, comm->flags, s);
        SymmRegion r;
        symm_alloc(comm, bytes, r, s);
        comm->regions.push_back(r);
        *out_ptr = r.local;
        return KVC_OK;
    } catch (const kvc::Error &e) {
        return kvc_internal_set_error(e.code, e.what());
    }
}

kvc_status kvc_comm_set_wait_limit(kvc_comm *comm, uint32_t iterations) {
    if (!comm || iterations == 0) return kvc_internal_set_error(KVC_ERR_INVALID_ARG, "kvc_comm_set_wait_limit: bad argument");
    comm->spin_limit = iterations;
    return KVC_OK;
}

kvc_status kvc_attention_sharded(kvc_comm *comm, kvc_cache *cache, const kvc_tensor *q,
                                 const kvc_tensor *k, const kvc_tensor *v, float scale,
                                 int32_t mask_mode, const kvc_tensor *mask,
                                 const kvc_tensor *out_full, int32_t shard_axis, void *stream) {
    if (!comm || !cache || !q || !k || !v || !out_full)
        return kvc_internal_set_error(KVC_ERR_INVALID_ARG, "kvc_attention_sharded: null argument");
    try {
        cudaStream_t s = (cudaStream_t)stream;
        KVC_REQUIRE(shard_axis == 0 || shard_axis == 1, "kvc_attention_sharded: shard_axis must be 0 (batch) or 1 (heads)");
        KVC_REQUIRE(q->ndim == 4 && out_full->ndim == 4, "kvc_attention_sharded: tensors must be 4-d");
        const int world = comm->world;
        const int64_t B = q->shape[0], Hl = q->shape[1], L = q->shape[2], D = q->shape[3];
        const size_t es = kvc::dtype_size(q->dtype);
        // contiguity of the gathered result
        int64_t expect = 1;
        for (int i = 3; i >= 0; --i) {
            KVC_REQUIRE(out_full->shape[i] == 1 || out_full->stride[i] == expect,
                        "kvc_attention_sharded: out_full must be contiguous");
            expect *= out_full->shape[i];
        }
        if (shard_axis == 1)
            KVC_REQUIRE(out_full->shape[0] == B && out_full->shape[1] == Hl * world && out_full->shape[2] == L &&
                            out_full->shape[3] == D,
                        "kvc_attention_sharded: out_full must be [B, Hq_local*world, L, D]");
        else
            KVC_REQUIRE(out_full->shape[0] == B * world && out_full->shape[1] == Hl && out_full->shape[2] == L &&
                            out_full->shape[3] == D,
                        "kvc_attention_sharded: out_full must be [B_local*world, Hq, L, D]");
        const size_t local_bytes = (size_t)(B * Hl * L * D) * es;
        auto fit = [&](void *&p, size_t &have, size_t need) {
            if (have >= need) return;
            if (p) KVC_CUDA(cudaFree(p));
            p = nullptr;
            KVC_CUDA(cudaMalloc(&p, need));
            have = need;
        };
        // Peer-store exchange: the gathered buffer lives in symmetric memory, this rank's slice is
        // written in place (final layout) and one kernel pushes it to the peers and waits for theirs.
        if (world > 1) {
            const size_t full_bytes = local_bytes * (size_t)world;
            const SymmRegion *reg = find_region(comm, out_full->data, full_bytes);
            const size_t run_bytes = shard_axis == 1 ? (size_t)(Hl * L * D) * es : local_bytes;
            const size_t row_stride_bytes = (size_t)(Hl * world * L * D) * es;
            if (reg && run_bytes % 16 == 0 && ((uintptr_t)out_full->data & 15) == 0) {
                kvc_tensor mine = *q;
                const size_t slice_off = (size_t)comm->rank * run_bytes;
                mine.data = (char *)out_full->data + slice_off;
                mine.stride[3] = 1; mine.stride[2] = D; mine.stride[1] = L * D;
                mine.stride[0] = shard_axis == 1 ? Hl * world * L * D : Hl * L * D;
                kvc::cache_attention(cache, *q, *k, *v, scale, mask_mode, mask, mine, s);
                launch_exchange(comm, *reg, out_full->data, slice_off, shard_axis == 1 ? B : 1, run_bytes, row_stride_bytes, s);
                return KVC_OK;
            }
        }
        kvc_tensor local = *q;
        if (world == 1) {
            local.data = out_full->data;
        } else if (shard_axis == 0) {
            // rank-contiguous: attend straight into this rank's slice of out_full
            local.data = (char *)out_full->data + (size_t)comm->rank * local_bytes;
        } else {
            fit(comm->local, comm->local_bytes, local_bytes);
            local.data = comm->local;
        }
        local.stride[3] = 1; local.stride[2] = D; local.stride[1] = L * D; local.stride[0] = Hl * L * D;
        kvc::cache_attention(cache, *q, *k, *v, scale, mask_mode, mask, local, s);
        if (world == 1) return KVC_OK;
        const ncclDataType_t dt = q->dtype == KVC_F32 ? ncclFloat32 : (q->dtype == KVC_F16 ? ncclFloat16 : ncclBfloat16);
        const size_t count = (size_t)(B * Hl * L * D);
        if (shard_axis == 0) {
            kvc::nccl_check(kvc::nccl().AllGather(local.data, out_full->data, count, dt, comm->comm, s), "ncclAllGather");
            return KVC_OK;
        }
        if (B == 1) {
            kvc::nccl_check(kvc::nccl().AllGather(local.data, out_full->data, count, dt, comm->comm, s), "ncclAllGather");
            return KVC_OK;
        }
        fit(comm->gathered, comm->gathered_bytes, local_bytes * world);
        kvc::nccl_check(kvc::nccl().AllGather(local.data, comm->gathered, count, dt, comm->comm, s), "ncclAllGather");
        const size_t row_bytes = (size_t)(L * D) * es;
        const int64_t rows = (int64_t)world * B * Hl;
        if (row_bytes % 16 == 0) {
            const int64_t ru = row_bytes / 16, total = rows * ru;
            kvc::interleave_heads_kernel<uint4><<<(unsigned)((total + 255) / 256), 256, 0, s>>>(
                (const uint4 *)comm->gathered, (uint4 *)out_full->data, world, (int)B, (int)Hl, ru, total);
        } else {
            const int64_t ru = row_bytes / 2, total = rows * ru;
            kvc::interleave_heads_kernel<uint16_t><<<(unsigned)((total + 255) / 256), 256, 0, s>>>(
                (const uint16_t *)comm->gathered, (uint16_t *)out_full->data, world, (int)B, (int)Hl, ru, total);
        }
        KVC_CUDA(cudaGetLastError());
        ++kvc::g_launch_count;
        return KVC_OK;
    } catch (const kvc::Error &e) {
        return kvc_internal_set_error(e.code, e.what());
    }
}

kvc_status kvc_attention_sharded_batch(kvc_comm *comm, kvc_cache *const *caches, int32_t count,
                                       const kvc_tensor *q, const kvc_tensor *k, const kvc_tensor *v,
                                       float scale, int32_t mask_mode, const kvc_tensor *outs_full,
                                       int32_t shard_axis, void *stream) {
    if (!caches || !q || !k || !v || !outs_full)
        return kvc_internal_set_error(KVC_ERR_INVALID_ARG, "kvc_attention_sharded_batch: null argument");
    for (int i = 0; i < count; ++i) {
        kvc_status st = kvc_attention_sharded(comm, caches[i], &q[i], &k[i], &v[i], scale, mask_mode, nullptr,
                                              &outs_full[i], shard_axis, stream);
        if (st != KVC_OK) return st;
    }
    return KVC_OK;
}

}  // extern "C"
