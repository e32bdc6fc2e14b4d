// Multi-GPU plumbing: one process per GPU, each owning the cache rows of its
// KV heads (or of its batch slice). The only exchange on the path is the
// per-layer all-gather of attention outputs; it runs as ncclAllGather on the
// caller's stream. NCCL is resolved with dlopen at first use so that the
// library loads (and every single-GPU entry point works) without it.
#include "cache.h"

#include <dlfcn.h>
#include <nccl.h>

#include <mutex>

namespace kvc {
void cache_attention(kvc_cache *c, const kvc_tensor &q, const kvc_tensor &k, const kvc_tensor &v,
                     float scale, int32_t mask_mode, const kvc_tensor *mask, const kvc_tensor &out,
                     cudaStream_t s);

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

}  // namespace
}  // namespace kvc

struct kvc_comm {
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1;
    int device = 0;
    void *local = nullptr;
    size_t local_bytes = 0;
    void *gathered = nullptr;
    size_t gathered_bytes = 0;
};

namespace {
thread_local std::string g_comm_error;
}

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
    (void)cudaGetLastError();
    delete c;
}

int32_t kvc_comm_rank(const kvc_comm *c) { return c ? c->rank : -1; }
int32_t kvc_comm_world(const kvc_comm *c) { return c ? c->world : -1; }

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
