// Per-device runtime state of the library: an internal stream and pinned staging
// buffers for calls that pass host memory, device-pointer classification, a
// device guard, and stream-ordered scratch allocation.
//
// Replaces the reference's runtime helpers (siglib/cusig/cu_runtime_utils.h:53-260
// workspace allocation and launch checks, siglib/cusig/cu_path_reduction.h:29-48
// per-device cached workspaces under one mutex): scratch memory comes from the
// CUDA stream-ordered pool of the device, so concurrent calls on different
// streams never share a buffer and no process-wide lock is held during a call.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <mutex>

#include "common.h"

namespace sigb200 {

struct PointerInfo {
    bool on_device;  // device (or managed) memory
    bool pinned;     // page-locked host memory (only meaningful when !on_device)
    int device;      // owning device for device memory, else -1
};

PointerInfo classify_pointer(const void* p);

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

struct DeviceContext {
    int device = -1;
    std::mutex mu;              // serialises host-memory calls that share the staging resources
    cudaStream_t copy_in = nullptr;   // non-blocking streams of the host-memory pipeline
    cudaStream_t compute = nullptr;
    cudaStream_t copy_out = nullptr;
    int sm_count = 0;
};

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

// Launch accounting (sigb200_launch_count).
void count_launch(uint64_t n = 1) noexcept;
uint64_t launch_count() noexcept;
int kernel_policy() noexcept;

}  // namespace sigb200
