// Device memory plumbing: stream-ordered allocation from the device's default
// memory pool (kept warm so re-allocation never goes back to the driver), and a
// per-device scratch arena for attention partials.
#include "common.h"

#include <mutex>
#include <vector>

namespace kvc {

thread_local int64_t g_launch_count = 0;

int current_device() {
    int dev = 0;
    KVC_CUDA(cudaGetDevice(&dev));
    return dev;
}

namespace {
struct DeviceInfo {
    bool pool_ready = false;
    int sms = 0;
    void *scratch = nullptr;
    size_t scratch_bytes = 0;
};
std::mutex g_mu;
std::vector<DeviceInfo> g_devices;

DeviceInfo &info_locked(int device) {
    if ((int)g_devices.size() <= device) g_devices.resize(device + 1);
    return g_devices[device];
}

void ensure_pool(int device) {
    std::lock_guard<std::mutex> lock(g_mu);
    DeviceInfo &di = info_locked(device);
    if (di.pool_ready) return;
    cudaMemPool_t pool;
    KVC_CUDA(cudaDeviceGetDefaultMemPool(&pool, device));
    // Keep freed blocks cached in the pool instead of returning them to the
    // driver at every synchronisation point.
    uint64_t threshold = UINT64_MAX;
    KVC_CUDA(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &threshold));
    di.pool_ready = true;
}
}  // namespace

int sm_count(int device) {
    {
        std::lock_guard<std::mutex> lock(g_mu);
        DeviceInfo &di = info_locked(device);
        if (di.sms > 0) return di.sms;
    }
    int sms = 0;
    KVC_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    std::lock_guard<std::mutex> lock(g_mu);
    info_locked(device).sms = sms;
    return sms;
}

void *dev_alloc(size_t bytes, cudaStream_t stream) {
    if (bytes == 0) bytes = 16;
    ensure_pool(current_device());
    void *p = nullptr;
    KVC_CUDA(cudaMallocAsync(&p, bytes, stream));
    return p;
}

void dev_free(void *ptr, cudaStream_t stream) {
    if (!ptr) return;
    cudaError_t e = cudaFreeAsync(ptr, stream);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
    }
}

void *scratch_get(int device, size_t bytes, cudaStream_t stream) {
    std::lock_guard<std::mutex> lock(g_mu);
    DeviceInfo &di = info_locked(device);
    if (di.scratch_bytes >= bytes) return di.scratch;
    // Grow geometrically. The old arena may still be read by work already
    // enqueued; cudaFree synchronises the device before releasing it.
    size_t want = di.scratch_bytes ? di.scratch_bytes : (size_t)8 << 20;
    while (want < bytes) want *= 2;
    if (di.scratch) {
        cudaError_t e = cudaFree(di.scratch);
        if (e != cudaSuccess) (void)cudaGetLastError();
        di.scratch = nullptr;
        di.scratch_bytes = 0;
    }
    (void)stream;
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, want);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        fail(KVC_ERR_OUT_OF_MEMORY, std::string("scratch cudaMalloc: ") + cudaGetErrorString(e));
    }
    di.scratch = p;
    di.scratch_bytes = want;
    return p;
}

}  // namespace kvc
