// Host-side helpers shared by the tensor-algebra translation units (sig_algebra.cu, sig_log.cu):
// launch geometry, the level table with its limits, and staging of host-pointer calls.
#pragma once

#include <algorithm>
#include <initializer_list>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

#include "algebra_math.h"
#include "common.h"
#include "runtime.h"

namespace sigb200 {
namespace {

constexpr int kThreads = 256;

unsigned grid_1d(uint64_t work, int threads) {
    const uint64_t blocks = (work + threads - 1) / threads;
    if (blocks == 0) return 1;
    if (blocks > 0x7fffffffull) throw std::invalid_argument("problem too large for one kernel launch");
    return static_cast<unsigned>(blocks);
}

// Grid for kernels that give one thread to each of `per_item` elements and walk the batch along
// grid.y with stride gridDim.y: enough CTAs to fill the GPU several times over, but not one tiny
// CTA per (element block, batch entry) when the batch is large.
dim3 batched_grid(uint64_t per_item, uint64_t batch, int threads) {
    const unsigned gx = grid_1d(per_item, threads);
    const uint64_t target = 148ull * 64;  // CTAs
    const uint64_t gy = std::max<uint64_t>(1, std::min<uint64_t>(std::min<uint64_t>(batch, 65535), (target + gx - 1) / gx));
    return dim3(gx, static_cast<unsigned>(gy));
}

Levels checked_levels(uint64_t dim, uint64_t degree, const char* who) {
    if (degree > kAlgebraMaxDegree)
        throw std::invalid_argument(std::string(who) + ": degree above 64 is not supported");
    if (sig_length_full(dim, degree) > kAlgebraMaxLength)  // throws on overflow by itself
        throw std::invalid_argument(std::string(who) + ": signatures of 2^31 or more coefficients are not supported");
    return make_levels(dim, degree);
}

void check_launch(const char* what) {
    count_launch();
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(err));
}

// Runs `body(device pointers, stream)` with every host operand staged through one scratch block:
// inputs copied in, outputs copied back, all on the context's compute stream.
struct StagedOperand {
    const void* host_in;  // nullptr for pure outputs
    void* host_out;       // nullptr for pure inputs
    size_t bytes;
};

template <typename Body>
void run_staged(std::vector<StagedOperand> ops, int device, Body body) {
    DeviceGuard guard(device >= 0 ? device : current_device());
    DeviceContext& ctx = device_context(current_device());
    std::lock_guard<std::mutex> lock(ctx.mu);
    cudaStream_t st = ctx.compute;
    size_t total = 0;
    std::vector<size_t> offs;
    for (auto& op : ops) {
        offs.push_back(total);
        total += (op.bytes + 255) / 256 * 256;
    }
    Scratch buf(std::max<size_t>(total, 256), st);
    std::vector<void*> dev;
    for (size_t i = 0; i < ops.size(); ++i) {
        void* p = static_cast<unsigned char*>(buf.get()) + offs[i];
        dev.push_back(p);
        if (ops[i].host_in && ops[i].bytes)
            SIG_CUDA_CHECK(cudaMemcpyAsync(p, ops[i].host_in, ops[i].bytes, cudaMemcpyHostToDevice, st));
    }
    body(dev, st);
    for (size_t i = 0; i < ops.size(); ++i)
        if (ops[i].host_out && ops[i].bytes)
            SIG_CUDA_CHECK(cudaMemcpyAsync(ops[i].host_out, dev[i], ops[i].bytes, cudaMemcpyDeviceToHost, st));
    SIG_CUDA_CHECK(cudaStreamSynchronize(st));
}

// true: all device, false: all host; throws on a mix
bool all_on_device(std::initializer_list<const void*> ptrs, const char* who, int* device) {
    int on = 0, off = 0, home = -1;
    for (const void* p : ptrs) {
        if (!p) continue;
        const PointerInfo info = classify_pointer(p);
        if (!info.on_device) { ++off; continue; }
        ++on;
        if (info.managed) { if (home < 0) *device = info.device; continue; }
        if (home >= 0 && info.device != home)
            throw std::invalid_argument(std::string(who) + ": all buffers must live on the same device (found devices " +
                                        std::to_string(home) + " and " + std::to_string(info.device) + ")");
        home = info.device;
        *device = home;
    }
    if (on && off)
        throw std::invalid_argument(std::string(who) + ": all buffers must be device pointers or all host pointers");
    return on > 0;
}

}  // namespace
}  // namespace sigb200
