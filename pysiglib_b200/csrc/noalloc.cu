// sig_backprop for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc (or anything that allocates for
// them) at the moment they need a gradient: a serving or training process whose caching
// allocator has already reserved the GPU's memory, so a late cudaMalloc can fail although
// the process "has" the memory; and latency-sensitive loops, because cudaMalloc / cudaFree
// synchronise the device and stall every other stream.  The regular backward entry points
// take their increment-gradient scratch from the stream-ordered pool; the entry points here
// use a fixed buffer that is part of the library image instead.
//
// The scratch is a file-scope __device__ array of kNoAllocScratchBytes.  Every GPU on which
// this library's device code is loaded by a process holds that much memory until the
// process exits.  Host code cannot use the array's name as a pointer (on the host it names
// a stand-in object, not device memory), so the device address is looked up once per device
// with cudaGetSymbolAddress while that device is current, and cached.  That look-up happens
// in the first call on a device; make that first call before any stream capture.
//
// "Allocates nothing" holds from the second call of a shape onwards.  The CUDA runtime loads
// device code lazily: the module that holds the scratch array is brought onto a device by the
// first cudaGetSymbolAddress there, and each kernel variant (dimension, degree, flags, dtype)
// by its first launch or occupancy query, and both loads take device memory.  A host that is
// about to hand the GPU's memory to its own allocator should therefore make one warm-up call
// per device and per shape it will use while memory is still available; calls after that
// neither allocate nor load anything.
//
// All calls share the one buffer and it keeps whatever the previous call left in it: the
// part a call uses is cleared on the call's stream before the kernel runs, and two calls
// whose GPU work overlaps (different streams, no ordering between them) race on it.
#include <mutex>

#include "../../include/cusig_b200.h"
#include "dispatch.h"
#include "kernels.h"
#include "runtime.h"

namespace sigb200 {

constexpr size_t kNoAllocScratchBytes = size_t(32) << 20;  // 32 MiB per device
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

// defined in sig_tile_dispatch.cu: the tile backward with caller-provided scratch and SM count
template <typename T>
bool launch_tile_backward_prealloc(const T* path, T* out, const T* sig_derivs, const T* sig, const SigShape& s,
                                   T end_time, T* incr_grad, int sm_count, cudaStream_t stream);

namespace {

constexpr int kMaxDevices = 64;
std::mutex g_setup_mu;
void* g_scratch_ptr[kMaxDevices] = {nullptr};
int g_sm_count[kMaxDevices] = {0};

// Device address of the static scratch on `device` (which must be current); first use per
// device resolves it with cudaGetSymbolAddress.
void* scratch_on_current_device(int device, int* sm_count) {
    if (device < 0 || device >= kMaxDevices) throw std::invalid_argument("device ordinal out of range");
    std::lock_guard<std::mutex> lock(g_setup_mu);
    if (g_scratch_ptr[device] == nullptr) {
        void* ptr = nullptr;
        SIG_CUDA_CHECK(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
        int sms = 0;
        SIG_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
        g_scratch_ptr[device] = ptr;
        g_sm_count[device] = sms;
    }
    *sm_count = g_sm_count[device];
    return g_scratch_ptr[device];
}

template <typename T>
void sig_backprop_noalloc(const T* path, T* out, const T* sig_derivs, const T* sig, uint64_t batch, uint64_t d,
                          uint64_t L, uint64_t degree, bool time_aug, bool lead_lag, T end_time, bool scalar_term,
                          cudaStream_t stream, bool synchronize) {
    if (d == 0) throw std::invalid_argument("sig_backprop_cuda received path of dimension 0");
    if (batch == 0 || L == 0) return;
    const SigShape s = make_shape(batch, d, L, degree, time_aug, lead_lag, scalar_term);
    if (path == nullptr || out == nullptr) throw std::invalid_argument("sig_backprop_cuda received a null pointer");
    const PointerInfo pout = classify_pointer(out);
    if (!pout.on_device || !classify_pointer(path).on_device)
        throw std::invalid_argument("the no-alloc entry points take device pointers only");
    const bool needs_sig = !(s.len <= 1 || s.degree == 0);
    if (needs_sig && (sig == nullptr || sig_derivs == nullptr))
        throw std::invalid_argument("sig_backprop_cuda received a null pointer");
    // every buffer a kernel will dereference must be device memory of out's GPU: a host pointer
    // or another GPU's memory would fault on the device, so it is turned away here
    if (needs_sig && (!classify_pointer(sig).on_device || !classify_pointer(sig_derivs).on_device))
        throw std::invalid_argument("the no-alloc entry points take device pointers only");
    require_on_device({path}, pout.device, "sigb200_sig_backprop_noalloc");
    if (needs_sig) require_on_device({sig, sig_derivs}, pout.device, "sigb200_sig_backprop_noalloc");
    DeviceGuard guard(pout.device);
    const uint64_t out_elems = checked_mul(batch, checked_mul(L, d, "path gradient"), "path gradient");
    if (!needs_sig) {
        launch_fill<T>(out, out_elems, T(0), stream);
    } else if (s.degree == 1) {
        // closed form, needs no scratch at all
        launch_degree_one_backward<T>(path, out, sig_derivs, s, end_time, stream);
    } else {
        if (!tile_backward_available<T>(s))
            throw std::invalid_argument(
                "this (dimension, degree) is not covered by the register-tile kernels, the only ones that run "
                "without allocating; use sig_backprop_cuda_* instead");
        const uint64_t need = checked_mul(checked_mul(batch, checked_mul(L - 1, d, "scratch"), "scratch"),
                                          sizeof(T), "scratch");
        if (need > kNoAllocScratchBytes)
            throw std::invalid_argument("sig_backprop needs " + std::to_string(need) +
                                        " bytes of scratch (batch * (length - 1) * dimension values) but the static "
                                        "buffer of the no-alloc entry point holds " +
                                        std::to_string(kNoAllocScratchBytes) + "; split the batch");
        int sm_count = 0;
        T* scratch = static_cast<T*>(scratch_on_current_device(pout.device, &sm_count));
        if (!launch_tile_backward_prealloc<T>(path, out, sig_derivs, sig, s, end_time, scratch, sm_count, stream))
            throw std::runtime_error("no register-tile variant for this shape");
    }
    if (synchronize) SIG_CUDA_CHECK(cudaStreamSynchronize(stream));
}

}  // namespace
}  // namespace sigb200

using namespace sigb200;

extern "C" __attribute__((visibility("default")))
int sigb200_sig_backprop_noalloc_f(const float* path, float* out, const float* sig_derivs, const float* sig,
                                   uint64_t batch_size, uint64_t dimension, uint64_t length, uint64_t degree,
                                   bool time_aug, bool lead_lag, float end_time, bool scalar_term, void* stream,
                                   int synchronize) {
    SIG_SAFE_CALL(sig_backprop_noalloc<float>(path, out, sig_derivs, sig, batch_size, dimension, length, degree,
                                              time_aug, lead_lag, end_time, scalar_term,
                                              static_cast<cudaStream_t>(stream), synchronize != 0));
}

extern "C" __attribute__((visibility("default")))
int sigb200_sig_backprop_noalloc_d(const double* path, double* out, const double* sig_derivs, const double* sig,
                                   uint64_t batch_size, uint64_t dimension, uint64_t length, uint64_t degree,
                                   bool time_aug, bool lead_lag, double end_time, bool scalar_term, void* stream,
                                   int synchronize) {
    SIG_SAFE_CALL(sig_backprop_noalloc<double>(path, out, sig_derivs, sig, batch_size, dimension, length, degree,
                                               time_aug, lead_lag, end_time, scalar_term,
                                               static_cast<cudaStream_t>(stream), synchronize != 0));
}

extern "C" __attribute__((visibility("default")))
uint64_t sigb200_noalloc_scratch_bytes(void) { return kNoAllocScratchBytes; }
