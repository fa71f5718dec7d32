// Per-device runtime state of the library: an internal stream and pinned staging
// buffers for calls that pass host memory, device-pointer classification, a
// device guard, and stream-ordered scratch allocation.
//
// Replaces the reference's runtime helpers (siglib/cusig/cu_runtime_utils.h:53-260
// workspace allocation and launch checks, siglib/cusig/cu_path_reduction.h:29-48
// per-device cached workspaces under one mutex): scratch memory comes from a
// stream-ordered memory pool that this library creates per device (the device's
// default pool, which the host application may share with other users of
// cudaMallocAsync, is left untouched), so concurrent calls on different streams
// never share a buffer and no process-wide lock is held during a call.  Freed
// scratch stays in that pool until cusig_shutdown().
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <initializer_list>
#include <mutex>

#include "common.h"

namespace sigb200 {

struct PointerInfo {
    bool on_device;  // device (or managed) memory
    bool pinned;     // page-locked host memory (only meaningful when !on_device)
    int device;      // owning device for device memory, else -1
    bool managed;    // managed memory: reachable from every device, `device` is only its preferred home
};

PointerInfo classify_pointer(const void* p);

// Throws invalid_argument unless every non-null pointer is device memory that lives on `device`
// (managed memory counts as being on every device).  A kernel given a host pointer, or a
// pointer of another GPU without peer access, would fault; this rejects the call on the host.
void require_on_device(std::initializer_list<const void*> ptrs, int device, const char* who);

class DeviceGuard {
public:
    explicit DeviceGuard(int device);
    ~DeviceGuard();
    DeviceGuard(const DeviceGuard&) = delete;
    DeviceGuard& operator=(const DeviceGuard&) = delete;
private:
    int previous_ = -1;
    bool switched_ = false;
};

// Stream-ordered scratch: allocated on `stream`, released on `stream` in the destructor.
class Scratch {
public:
    Scratch(size_t bytes, cudaStream_t stream);
    ~Scratch();
    Scratch(const Scratch&) = delete;
    Scratch& operator=(const Scratch&) = delete;
    void* get() const { return ptr_; }
    template <typename T> T* as() const { return static_cast<T*>(ptr_); }
private:
    void* ptr_ = nullptr;
    cudaStream_t stream_;
};

// One staging slot of the host-memory pipeline: a device buffer that is carved into the
// operands of one batch chunk, and the events that order the three streams around it.  Slots
// are kept between calls (allocation and event creation cost more than a small call).
struct StagingSlot {
    void* buffer = nullptr;
    size_t capacity = 0;
    cudaEvent_t copied_in = nullptr, computed = nullptr, copied_out = nullptr;
};

struct DeviceContext {
    int device = -1;
    std::mutex mu;              // serialises host-memory calls that share the staging resources
    cudaStream_t copy_in = nullptr;   // non-blocking streams of the host-memory pipeline
    cudaStream_t compute = nullptr;
    cudaStream_t copy_out = nullptr;
    cudaEvent_t ready = nullptr;
    StagingSlot slots[2];
    cudaMemPool_t pool = nullptr;     // private stream-ordered pool of this library on this device
    int sm_count = 0;
};

// Makes both staging slots of `ctx` at least `bytes` large (ctx.mu must be held; uses
// ctx.compute).  Throws std::bad_alloc when the device cannot provide them.
void reserve_staging(DeviceContext& ctx, size_t bytes, int n_slots);

// Host-side failure injection for tests of the out-of-memory paths: the next `n` scratch
// or staging requests report cudaErrorMemoryAllocation without touching the device.  The
// environment variable SIGB200_FAIL_ALLOCS=n arms it at library load.
void inject_alloc_failures(int n) noexcept;

// Bytes currently reserved from the driver by this library's pool on `device` (0 before first use).
uint64_t pool_reserved_bytes(int device);

// Lazily created, lives until shutdown_runtime().
DeviceContext& device_context(int device);
int current_device();
int device_count();

// Frees every cached resource on every device (cusig_shutdown).
void shutdown_runtime() noexcept;

// 0 = automatic kernel choice, 1 = shape-generic kernels only (used by the tests
// to exercise the fallback on shapes the tile kernels would otherwise take).
void set_kernel_policy(int policy) noexcept;

// Tile-variant override for tests and tuning: 0 automatic, 1 biggest tile, 2 smallest tile,
// 3 automatic without time segmentation, 4 biggest tile with forced time segmentation.
void set_tile_preference(int pref) noexcept;
int tile_preference() noexcept;

// Test hook: pins the register-tile variant (chain length P, group G) and the number of time
// segments of the forward (backward = false) or backward sweep, for shapes that have such a
// variant compiled; P < 0 clears it.  Lets the tests run every compiled variant of a shape.
struct ForcedPlan { int P, G, segments; };
void set_forced_plan(bool backward, int P, int G, int segments) noexcept;
ForcedPlan forced_plan(bool backward) noexcept;

// Launch accounting (sigb200_launch_count).
void count_launch(uint64_t n = 1) noexcept;
uint64_t launch_count() noexcept;
int kernel_policy() noexcept;

}  // namespace sigb200
