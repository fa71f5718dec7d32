#include "runtime.h"

#include <atomic>
#include <cstring>
#include <map>
#include <memory>

namespace sigb200 {

namespace {

thread_local char tls_error[1024] = {0};

std::mutex g_contexts_mu;
std::map<int, std::unique_ptr<DeviceContext>> g_contexts;
std::atomic<int> g_policy{0};
std::atomic<uint64_t> g_launches{0};
std::atomic<int> g_tile_pref{0};

}  // namespace

void set_last_error(const char* text) noexcept {
    std::strncpy(tls_error, text ? text : "", sizeof(tls_error) - 1);
    tls_error[sizeof(tls_error) - 1] = '\0';
}

void clear_last_error() noexcept { tls_error[0] = '\0'; }

const char* last_error() noexcept { return tls_error; }

void set_kernel_policy(int policy) noexcept { g_policy.store(policy); }
int kernel_policy() noexcept { return g_policy.load(); }

void set_tile_preference(int pref) noexcept { g_tile_pref.store(pref); }
int tile_preference() noexcept { return g_tile_pref.load(); }

void count_launch(uint64_t n) noexcept { g_launches.fetch_add(n, std::memory_order_relaxed); }
uint64_t launch_count() noexcept { return g_launches.load(std::memory_order_relaxed); }

PointerInfo classify_pointer(const void* p) {
    PointerInfo info{false, false, -1};
    if (p == nullptr) return info;
    cudaPointerAttributes attr{};
    const cudaError_t err = cudaPointerGetAttributes(&attr, p);
    if (err != cudaSuccess) {
        (void)cudaGetLastError();
        if (err == cudaErrorInvalidValue) return info;  // plain host memory on old drivers
        SIG_CUDA_CHECK(err);
    }
    if (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged) {
        info.on_device = true;
        info.device = attr.device;
    } else if (attr.type == cudaMemoryTypeHost) {
        info.pinned = true;
    }
    return info;
}

int current_device() {
    int dev = 0;
    SIG_CUDA_CHECK(cudaGetDevice(&dev));
    return dev;
}

int device_count() {
    int n = 0;
    SIG_CUDA_CHECK(cudaGetDeviceCount(&n));
    return n;
}

DeviceGuard::DeviceGuard(int device) {
    SIG_CUDA_CHECK(cudaGetDevice(&previous_));
    if (device >= 0 && device != previous_) {
        SIG_CUDA_CHECK(cudaSetDevice(device));
        switched_ = true;
    }
}

DeviceGuard::~DeviceGuard() {
    if (switched_) (void)cudaSetDevice(previous_);
}

Scratch::Scratch(size_t bytes, cudaStream_t stream) : stream_(stream) {
    if (bytes == 0) return;
    (void)device_context(current_device());  // first use on a device sets the pool to keep freed scratch
    const cudaError_t err = cudaMallocAsync(&ptr_, bytes, stream);
    if (err == cudaErrorMemoryAllocation) {
        (void)cudaGetLastError();
        throw std::bad_alloc();
    }
    SIG_CUDA_CHECK(err);
}

Scratch::~Scratch() {
    if (ptr_) (void)cudaFreeAsync(ptr_, stream_);
}

DeviceContext& device_context(int device) {
    std::lock_guard<std::mutex> lock(g_contexts_mu);
    auto it = g_contexts.find(device);
    if (it != g_contexts.end()) return *it->second;
    DeviceGuard guard(device);
    auto ctx = std::make_unique<DeviceContext>();
    ctx->device = device;
    SIG_CUDA_CHECK(cudaStreamCreateWithFlags(&ctx->copy_in, cudaStreamNonBlocking));
    SIG_CUDA_CHECK(cudaStreamCreateWithFlags(&ctx->compute, cudaStreamNonBlocking));
    SIG_CUDA_CHECK(cudaStreamCreateWithFlags(&ctx->copy_out, cudaStreamNonBlocking));
    SIG_CUDA_CHECK(cudaDeviceGetAttribute(&ctx->sm_count, cudaDevAttrMultiProcessorCount, device));
    // Keep freed scratch in the pool instead of returning it to the driver between calls.
    cudaMemPool_t pool;
    SIG_CUDA_CHECK(cudaDeviceGetDefaultMemPool(&pool, device));
    uint64_t threshold = UINT64_MAX;
    SIG_CUDA_CHECK(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &threshold));
    DeviceContext& ref = *ctx;
    g_contexts.emplace(device, std::move(ctx));
    return ref;
}

void shutdown_runtime() noexcept {
    std::lock_guard<std::mutex> lock(g_contexts_mu);
    for (auto& kv : g_contexts) {
        int prev = -1;
        if (cudaGetDevice(&prev) != cudaSuccess) { (void)cudaGetLastError(); continue; }
        if (cudaSetDevice(kv.first) != cudaSuccess) { (void)cudaGetLastError(); continue; }
        DeviceContext& c = *kv.second;
        if (c.copy_in) (void)cudaStreamDestroy(c.copy_in);
        if (c.compute) (void)cudaStreamDestroy(c.compute);
        if (c.copy_out) (void)cudaStreamDestroy(c.copy_out);
        cudaMemPool_t pool;
        if (cudaDeviceGetDefaultMemPool(&pool, kv.first) == cudaSuccess) (void)cudaMemPoolTrimTo(pool, 0);
        (void)cudaSetDevice(prev);
        (void)cudaGetLastError();
    }
    g_contexts.clear();
}

}  // namespace sigb200
