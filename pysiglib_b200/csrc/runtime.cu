#include "runtime.h"

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <string>

namespace sigb200 {

namespace {

thread_local char tls_error[1024] = {0};

std::mutex g_contexts_mu;
std::map<int, std::unique_ptr<DeviceContext>> g_contexts;
std::atomic<int> g_policy{0};
std::atomic<uint64_t> g_launches{0};
std::atomic<int> g_tile_pref{0};
std::atomic<uint64_t> g_forced[2] = {{~0ull}, {~0ull}};  // packed (P, G, segments); all ones = none

int alloc_failures_from_env() {
    const char* text = std::getenv("SIGB200_FAIL_ALLOCS");
    return text ? std::max(0, std::atoi(text)) : 0;
}
std::atomic<int> g_fail_allocs{alloc_failures_from_env()};

// true: this request must be reported as failed (consumes one injected failure)
bool injected_failure() noexcept {
    int n = g_fail_allocs.load(std::memory_order_relaxed);
    while (n > 0)
        if (g_fail_allocs.compare_exchange_weak(n, n - 1, std::memory_order_relaxed)) return true;
    return false;
}

void* pool_alloc(DeviceContext& ctx, size_t bytes, cudaStream_t stream) {
    if (injected_failure()) throw std::bad_alloc();
    void* ptr = nullptr;
    const cudaError_t err = cudaMallocFromPoolAsync(&ptr, bytes, ctx.pool, stream);
    if (err == cudaErrorMemoryAllocation) {
        (void)cudaGetLastError();
        throw std::bad_alloc();
    }
    SIG_CUDA_CHECK(err);
    return ptr;
}

}  // namespace

void set_last_error(const char* text) noexcept {
    std::strncpy(tls_error, text ? text : "", sizeof(tls_error) - 1);
    tls_error[sizeof(tls_error) - 1] = '\0';
}

void clear_last_error() noexcept { tls_error[0] = '\0'; }

const char* last_error() noexcept { return tls_error; }

void set_kernel_policy(int policy) noexcept { g_policy.store(policy); }
int kernel_policy() noexcept { return g_policy.load(); }

void set_forced_plan(bool backward, int P, int G, int segments) noexcept {
    const uint64_t packed = P < 0 ? ~0ull : (uint64_t(P & 0xffff) << 32) | (uint64_t(G & 0xffff) << 16) |
                                             uint64_t(std::max(segments, 1) & 0xffff);
    g_forced[backward ? 1 : 0].store(packed);
}
ForcedPlan forced_plan(bool backward) noexcept {
    const uint64_t packed = g_forced[backward ? 1 : 0].load();
    if (packed == ~0ull) return ForcedPlan{-1, -1, 1};
    return ForcedPlan{int((packed >> 32) & 0xffff), int((packed >> 16) & 0xffff), int(packed & 0xffff)};
}
void set_tile_preference(int pref) noexcept { g_tile_pref.store(pref); }
int tile_preference() noexcept { return g_tile_pref.load(); }

void count_launch(uint64_t n) noexcept { g_launches.fetch_add(n, std::memory_order_relaxed); }
uint64_t launch_count() noexcept { return g_launches.load(std::memory_order_relaxed); }

PointerInfo classify_pointer(const void* p) {
    PointerInfo info{false, false, -1, false};
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
        info.managed = attr.type == cudaMemoryTypeManaged;
    } else if (attr.type == cudaMemoryTypeHost) {
        info.pinned = true;
    }
    return info;
}

void require_on_device(std::initializer_list<const void*> ptrs, int device, const char* who) {
    for (const void* p : ptrs) {
        if (!p) continue;
        const PointerInfo info = classify_pointer(p);
        if (!info.on_device)
            throw std::invalid_argument(std::string(who) + ": all buffers must be device pointers or all host pointers");
        if (!info.managed && info.device != device)
            throw std::invalid_argument(std::string(who) + ": all buffers must live on the same device (found devices " +
                                        std::to_string(device) + " and " + std::to_string(info.device) + ")");
    }
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
    ptr_ = pool_alloc(device_context(current_device()), bytes, stream);
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
    SIG_CUDA_CHECK(cudaEventCreateWithFlags(&ctx->ready, cudaEventDisableTiming));
    for (StagingSlot& sl : ctx->slots) {
        SIG_CUDA_CHECK(cudaEventCreateWithFlags(&sl.copied_in, cudaEventDisableTiming));
        SIG_CUDA_CHECK(cudaEventCreateWithFlags(&sl.computed, cudaEventDisableTiming));
        SIG_CUDA_CHECK(cudaEventCreateWithFlags(&sl.copied_out, cudaEventDisableTiming));
    }
    // A pool of this library's own: freed scratch stays in it instead of going back to the driver
    // between calls, and the device's default pool keeps whatever policy the host process gave it.
    cudaMemPoolProps props{};
    props.allocType = cudaMemAllocationTypePinned;
    props.handleTypes = cudaMemHandleTypeNone;
    props.location.type = cudaMemLocationTypeDevice;
    props.location.id = device;
    SIG_CUDA_CHECK(cudaMemPoolCreate(&ctx->pool, &props));
    uint64_t threshold = UINT64_MAX;
    SIG_CUDA_CHECK(cudaMemPoolSetAttribute(ctx->pool, cudaMemPoolAttrReleaseThreshold, &threshold));
    DeviceContext& ref = *ctx;
    g_contexts.emplace(device, std::move(ctx));
    return ref;
}

void reserve_staging(DeviceContext& ctx, size_t bytes, int n_slots) {
    for (int i = 0; i < n_slots; ++i) {
        StagingSlot& sl = ctx.slots[i];
        if (sl.capacity >= bytes) continue;
        if (sl.buffer) {
            SIG_CUDA_CHECK(cudaFreeAsync(sl.buffer, ctx.compute));
            sl.buffer = nullptr;
            sl.capacity = 0;
        }
        sl.buffer = pool_alloc(ctx, bytes, ctx.compute);
        sl.capacity = bytes;
    }
}

void inject_alloc_failures(int n) noexcept { g_fail_allocs.store(n > 0 ? n : 0); }

uint64_t pool_reserved_bytes(int device) {
    std::lock_guard<std::mutex> lock(g_contexts_mu);
    auto it = g_contexts.find(device);
    if (it == g_contexts.end() || !it->second->pool) return 0;
    uint64_t value = 0;
    SIG_CUDA_CHECK(cudaMemPoolGetAttribute(it->second->pool, cudaMemPoolAttrReservedMemCurrent, &value));
    return value;
}

void shutdown_runtime() noexcept {
    std::lock_guard<std::mutex> lock(g_contexts_mu);
    for (auto& kv : g_contexts) {
        int prev = -1;
        if (cudaGetDevice(&prev) != cudaSuccess) { (void)cudaGetLastError(); continue; }
        if (cudaSetDevice(kv.first) != cudaSuccess) { (void)cudaGetLastError(); continue; }
        DeviceContext& c = *kv.second;
        (void)cudaDeviceSynchronize();
        for (StagingSlot& sl : c.slots) {
            if (sl.buffer) (void)cudaFreeAsync(sl.buffer, c.compute);
            if (sl.copied_in) (void)cudaEventDestroy(sl.copied_in);
            if (sl.computed) (void)cudaEventDestroy(sl.computed);
            if (sl.copied_out) (void)cudaEventDestroy(sl.copied_out);
        }
        if (c.ready) (void)cudaEventDestroy(c.ready);
        if (c.compute) (void)cudaStreamSynchronize(c.compute);
        if (c.copy_in) (void)cudaStreamDestroy(c.copy_in);
        if (c.compute) (void)cudaStreamDestroy(c.compute);
        if (c.copy_out) (void)cudaStreamDestroy(c.copy_out);
        if (c.pool) (void)cudaMemPoolDestroy(c.pool);
        (void)cudaSetDevice(prev);
        (void)cudaGetLastError();
    }
    g_contexts.clear();
}

}  // namespace sigb200
