// extern "C" surface of libcusig.so (declared in include/cusig_b200.h).
//
// The four compute symbols, cusig_last_error_message and cusig_shutdown keep the
// reference's names and signatures (siglib/cusig/cusig.h:43,312-314,342-344,1028)
// so that pysiglib/load_siglib.py:76-130,484-494 can load this library unchanged.
// Every other symbol that loader resolves at import time is exported as a stub
// that fails with code 10, so the import succeeds and only this path is served.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "../../include/cusig_b200.h"
#include "algebra.h"
#include "dispatch.h"
#include "kernels.h"
#include "runtime.h"

using namespace sigb200;

namespace {

CallOptions sync_options() { return CallOptions{}; }

CallOptions stream_options(void* stream, int synchronize, int* nonfinite) {
    CallOptions o;
    o.stream = static_cast<cudaStream_t>(stream);
    o.synchronize = synchronize != 0;
    o.nonfinite = nonfinite;
    return o;
}

// Contiguous shards, remainder to the first shards (the reference's thread split,
// siglib/cpsig/multithreading.cpp:66-78, applied to devices).
struct Shard { uint64_t begin, count; int device; };

std::vector<Shard> make_shards(uint64_t batch, const int* devices, int n_devices) {
    if (n_devices <= 0) throw std::invalid_argument("n_devices must be positive");
    const int available = device_count();
    std::vector<Shard> shards;
    const uint64_t n = std::min<uint64_t>(uint64_t(n_devices), std::max<uint64_t>(batch, 1));
    const uint64_t chunk = batch / n, rem = batch % n;
    for (uint64_t g = 0; g < n; ++g) {
        const int dev = devices ? devices[g] : int(g);
        if (dev < 0 || dev >= available)
            throw std::invalid_argument("device ordinal " + std::to_string(dev) + " is not available");
        const uint64_t begin = g * chunk + std::min(g, rem);
        shards.push_back({begin, chunk + (g < rem ? 1 : 0), dev});
    }
    return shards;
}

// Runs fn(shard) on one host thread per shard; the first failure (lowest shard) is rethrown.
template <typename Fn>
void run_sharded(const std::vector<Shard>& shards, Fn&& fn) {
    std::vector<std::exception_ptr> errors(shards.size());
    std::vector<std::thread> threads;
    for (size_t i = 1; i < shards.size(); ++i)
        threads.emplace_back([&, i] {
            try { fn(shards[i]); } catch (...) { errors[i] = std::current_exception(); }
        });
    try { fn(shards[0]); } catch (...) { errors[0] = std::current_exception(); }
    for (auto& t : threads) t.join();
    for (auto& e : errors) if (e) std::rethrow_exception(e);
}

template <typename T>
void signature_sharded(const T* path, T* out, uint64_t batch, uint64_t d, uint64_t L, uint64_t degree,
                       bool time_aug, bool lead_lag, T end_time, bool scalar_term, const int* devices,
                       int n_devices) {
    if (d == 0) throw std::invalid_argument("signature_cuda received path of dimension 0");
    if (batch == 0) return;
    const SigShape s = make_shape(batch, d, L, degree, time_aug, lead_lag, scalar_term);
    if (classify_pointer(out).on_device || classify_pointer(path).on_device)
        throw std::invalid_argument("the sharded entry points take host buffers");
    run_sharded(make_shards(batch, devices, n_devices), [&](const Shard& sh) {
        if (sh.count == 0) return;
        CallOptions o;
        o.device = sh.device;
        signature_entry<T>(path + sh.begin * L * d, out + sh.begin * s.stride, sh.count, d, L, degree, time_aug,
                           lead_lag, end_time, true, scalar_term, nullptr, 0, o);
    });
}

template <typename T>
void sig_backprop_sharded(const T* path, T* out, const T* sig_derivs, const T* sig, uint64_t batch, uint64_t d,
                          uint64_t L, uint64_t degree, bool time_aug, bool lead_lag, T end_time,
                          bool scalar_term, const int* devices, int n_devices) {
    if (d == 0) throw std::invalid_argument("sig_backprop_cuda received path of dimension 0");
    if (batch == 0) return;
    const SigShape s = make_shape(batch, d, L, degree, time_aug, lead_lag, scalar_term);
    if (classify_pointer(out).on_device || classify_pointer(path).on_device)
        throw std::invalid_argument("the sharded entry points take host buffers");
    run_sharded(make_shards(batch, devices, n_devices), [&](const Shard& sh) {
        if (sh.count == 0) return;
        CallOptions o;
        o.device = sh.device;
        sig_backprop_entry<T>(path + sh.begin * L * d, out + sh.begin * L * d,
                              sig_derivs ? sig_derivs + sh.begin * s.stride : nullptr,
                              sig ? sig + sh.begin * s.stride : nullptr, sh.count, d, L, degree, time_aug,
                              lead_lag, end_time, scalar_term, nullptr, 0, o);
    });
}

int stub_not_built(const char* name) noexcept {
    clear_last_error();
    std::string msg = std::string(name) +
        " is not part of this build of libcusig (it serves the signature, sig_backprop, sig_combine, sig_join, linear_sig, transform_path, sig_coef and sig_to_log_sig families)";
    set_last_error(msg.c_str());
    return 10;
}

}  // namespace

#define SIG_API extern "C" __attribute__((visibility("default")))

SIG_API int signature_cuda_f(const float* path, float* out, uint64_t batch_size, uint64_t dimension,
                             uint64_t length, uint64_t degree, bool time_aug, bool lead_lag, float end_time,
                             bool horner, bool scalar_term, const float* correction, uint64_t correction_len,
                             uint64_t correction_batch_stride, uint64_t correction_segment_stride) {
    SIG_SAFE_CALL(signature_entry<float>(path, out, batch_size, dimension, length, degree, time_aug, lead_lag,
                                         end_time, horner, scalar_term, correction, correction_len, sync_options(),
                        correction_batch_stride, correction_segment_stride));
}

SIG_API int signature_cuda_d(const double* path, double* out, uint64_t batch_size, uint64_t dimension,
                             uint64_t length, uint64_t degree, bool time_aug, bool lead_lag, double end_time,
                             bool horner, bool scalar_term, const double* correction, uint64_t correction_len,
                             uint64_t correction_batch_stride, uint64_t correction_segment_stride) {
    SIG_SAFE_CALL(signature_entry<double>(path, out, batch_size, dimension, length, degree, time_aug, lead_lag,
                                          end_time, horner, scalar_term, correction, correction_len, sync_options(),
                        correction_batch_stride, correction_segment_stride));
}

SIG_API int sig_backprop_cuda_f(const float* path, float* out, const float* sig_derivs, const float* sig,
                                uint64_t batch_size, uint64_t dimension, uint64_t length, uint64_t degree,
                                bool time_aug, bool lead_lag, float end_time, bool scalar_term,
                                const float* correction, uint64_t correction_len, uint64_t correction_batch_stride,
                                uint64_t correction_segment_stride) {
    SIG_SAFE_CALL(sig_backprop_entry<float>(path, out, sig_derivs, sig, batch_size, dimension, length, degree,
                                            time_aug, lead_lag, end_time, scalar_term, correction, correction_len,
                                            sync_options(), correction_batch_stride, correction_segment_stride));
}

SIG_API int sig_backprop_cuda_d(const double* path, double* out, const double* sig_derivs, const double* sig,
                                uint64_t batch_size, uint64_t dimension, uint64_t length, uint64_t degree,
                                bool time_aug, bool lead_lag, double end_time, bool scalar_term,
                                const double* correction, uint64_t correction_len, uint64_t correction_batch_stride,
                                uint64_t correction_segment_stride) {
    SIG_SAFE_CALL(sig_backprop_entry<double>(path, out, sig_derivs, sig, batch_size, dimension, length, degree,
                                             time_aug, lead_lag, end_time, scalar_term, correction, correction_len,
                                             sync_options(), correction_batch_stride, correction_segment_stride));
}

SIG_API int sig_combine_cuda_f(const float* sig1, const float* sig2, float* out, uint64_t batch_size,
                               uint64_t dimension, uint64_t degree, bool scalar_term) {
    SIG_SAFE_CALL(sig_combine_entry<float>(sig1, sig2, out, batch_size, dimension, degree, scalar_term, sync_options()));
}

SIG_API int sig_combine_cuda_d(const double* sig1, const double* sig2, double* out, uint64_t batch_size,
                               uint64_t dimension, uint64_t degree, bool scalar_term) {
    SIG_SAFE_CALL(sig_combine_entry<double>(sig1, sig2, out, batch_size, dimension, degree, scalar_term, sync_options()));
}

SIG_API int sig_combine_backprop_cuda_f(const float* sig_combined_deriv, float* sig1_deriv, float* sig2_deriv,
                                        const float* sig1, const float* sig2, uint64_t batch_size,
                                        uint64_t dimension, uint64_t degree, bool scalar_term) {
    SIG_SAFE_CALL(sig_combine_backprop_entry<float>(sig_combined_deriv, sig1_deriv, sig2_deriv, sig1, sig2, batch_size,
                                                    dimension, degree, scalar_term, sync_options()));
}

SIG_API int sig_combine_backprop_cuda_d(const double* sig_combined_deriv, double* sig1_deriv, double* sig2_deriv,
                                        const double* sig1, const double* sig2, uint64_t batch_size,
                                        uint64_t dimension, uint64_t degree, bool scalar_term) {
    SIG_SAFE_CALL(sig_combine_backprop_entry<double>(sig_combined_deriv, sig1_deriv, sig2_deriv, sig1, sig2, batch_size,
                                                     dimension, degree, scalar_term, sync_options()));
}

#define SIG_ALGEBRA_EXPORTS(SUF, T)                                                                                   \
    SIG_API int linear_sig_cuda_##SUF(const T* displacement, T* out, uint64_t batch_size, uint64_t dimension,         \
                                      uint64_t degree, bool scalar_term) {                                            \
        SIG_SAFE_CALL(linear_sig_entry<T>(displacement, out, batch_size, dimension, degree, scalar_term,              \
                                          sync_options()));                                                           \
    }                                                                                                                 \
    SIG_API int sig_join_cuda_##SUF(const T* sig, const T* displacement, T* out, uint64_t batch_size,                 \
                                    uint64_t dimension, uint64_t degree, bool prepend, bool scalar_term) {            \
        SIG_SAFE_CALL(sig_join_entry<T>(sig, displacement, out, batch_size, dimension, degree, prepend, scalar_term,  \
                                        sync_options()));                                                             \
    }                                                                                                                 \
    SIG_API int sig_join_backprop_cuda_##SUF(const T* d_out, T* d_sig, T* d_displacement, const T* sig,               \
                                             const T* displacement, uint64_t batch_size, uint64_t dimension,          \
                                             uint64_t degree, bool prepend, bool scalar_term) {                       \
        SIG_SAFE_CALL(sig_join_backprop_entry<T>(d_out, d_sig, d_displacement, sig, displacement, batch_size,         \
                                                 dimension, degree, prepend, scalar_term, sync_options()));           \
    }                                                                                                                 \
    SIG_API int transform_path_cuda_##SUF(const T* data_in, T* data_out, uint64_t batch_size, uint64_t dimension,     \
                                          uint64_t length, bool time_aug, bool lead_lag, T end_time) {                \
        SIG_SAFE_CALL(transform_path_entry<T>(data_in, data_out, batch_size, dimension, length, time_aug, lead_lag,   \
                                              end_time, sync_options()));                                             \
    }                                                                                                                 \
    SIG_API int transform_path_backprop_cuda_##SUF(const T* derivs, T* data_out, uint64_t batch_size,                 \
                                                   uint64_t dimension, uint64_t length, bool time_aug,                \
                                                   bool lead_lag, T end_time) {                                       \
        SIG_SAFE_CALL(transform_path_backprop_entry<T>(derivs, data_out, batch_size, dimension, length, time_aug,     \
                                                       lead_lag, end_time, sync_options()));                          \
    }                                                                                                                 \
    SIG_API int sig_to_log_sig_cuda_##SUF(const T* sig, T* out, uint64_t batch_size, uint64_t dimension,             \
                                          uint64_t degree, int method, bool scalar_term) {                            \
        SIG_SAFE_CALL(sig_to_log_sig_entry<T>(sig, out, batch_size, dimension, degree, method, scalar_term,           \
                                              sync_options()));                                                       \
    }                                                                                                                 \
    SIG_API int sig_to_log_sig_backprop_cuda_##SUF(const T* sig, T* out, const T* log_sig_derivs, uint64_t batch_size, \
                                                   uint64_t dimension, uint64_t degree, int method,                   \
                                                   bool scalar_term) {                                                \
        SIG_SAFE_CALL(sig_to_log_sig_backprop_entry<T>(sig, out, log_sig_derivs, batch_size, dimension, degree,       \
                                                       method, scalar_term, sync_options()));                         \
    }                                                                                                                 \
    SIG_API int sig_coef_cuda_##SUF(const T* path, T* out, const uint64_t* multi_idx, uint64_t num_multi_idx,         \
                                    const uint64_t* degrees, uint64_t batch_size, uint64_t dimension,                 \
                                    uint64_t length, bool prefixes) {                                                 \
        SIG_SAFE_CALL(sig_coef_entry<T>(path, out, multi_idx, num_multi_idx, degrees, batch_size, dimension, length,  \
                                        prefixes, sync_options()));                                                   \
    }                                                                                                                 \
    SIG_API int sig_coef_backprop_cuda_##SUF(const T* path, T* out, const T* coefs, const T* derivs,                  \
                                             const uint64_t* multi_idx, uint64_t num_multi_idx,                       \
                                             const uint64_t* degrees, uint64_t batch_size, uint64_t dimension,        \
                                             uint64_t length) {                                                       \
        SIG_SAFE_CALL(sig_coef_backprop_entry<T>(path, out, coefs, derivs, multi_idx, num_multi_idx, degrees,         \
                                                 batch_size, dimension, length, sync_options()));                     \
    }
SIG_ALGEBRA_EXPORTS(f, float)
SIG_ALGEBRA_EXPORTS(d, double)
#undef SIG_ALGEBRA_EXPORTS

SIG_API int prepare_log_sig_cuda(uint64_t dimension, uint64_t degree, int method, bool /*use_disk*/) {
    SIG_SAFE_CALL(prepare_log_sig_entry(dimension, degree, method));
}

SIG_API const char* cusig_last_error_message(void) { return last_error(); }

SIG_API void cusig_shutdown(void) {
    release_log_sig_tables();
    shutdown_runtime();
}

SIG_API int sigb200_signature_f(const float* path, float* out, uint64_t batch_size, uint64_t dimension,
                                uint64_t length, uint64_t degree, bool time_aug, bool lead_lag, float end_time,
                                bool scalar_term, void* stream, int synchronize, int* nonfinite) {
    SIG_SAFE_CALL(signature_entry<float>(path, out, batch_size, dimension, length, degree, time_aug, lead_lag,
                                         end_time, true, scalar_term, nullptr, 0,
                                         stream_options(stream, synchronize, nonfinite)));
}

SIG_API int sigb200_signature_d(const double* path, double* out, uint64_t batch_size, uint64_t dimension,
                                uint64_t length, uint64_t degree, bool time_aug, bool lead_lag, double end_time,
                                bool scalar_term, void* stream, int synchronize, int* nonfinite) {
    SIG_SAFE_CALL(signature_entry<double>(path, out, batch_size, dimension, length, degree, time_aug, lead_lag,
                                          end_time, true, scalar_term, nullptr, 0,
                                          stream_options(stream, synchronize, nonfinite)));
}

SIG_API int sigb200_sig_backprop_f(const float* path, float* out, const float* sig_derivs, const float* sig,
                                   uint64_t batch_size, uint64_t dimension, uint64_t length, uint64_t degree,
                                   bool time_aug, bool lead_lag, float end_time, bool scalar_term, void* stream,
                                   int synchronize) {
    SIG_SAFE_CALL(sig_backprop_entry<float>(path, out, sig_derivs, sig, batch_size, dimension, length, degree,
                                            time_aug, lead_lag, end_time, scalar_term, nullptr, 0,
                                            stream_options(stream, synchronize, nullptr)));
}

SIG_API int sigb200_sig_backprop_d(const double* path, double* out, const double* sig_derivs, const double* sig,
                                   uint64_t batch_size, uint64_t dimension, uint64_t length, uint64_t degree,
                                   bool time_aug, bool lead_lag, double end_time, bool scalar_term, void* stream,
                                   int synchronize) {
    SIG_SAFE_CALL(sig_backprop_entry<double>(path, out, sig_derivs, sig, batch_size, dimension, length, degree,
                                             time_aug, lead_lag, end_time, scalar_term, nullptr, 0,
                                             stream_options(stream, synchronize, nullptr)));
}

SIG_API int sigb200_log_sig_f(const float* path, float* out, uint64_t batch_size, uint64_t dimension, uint64_t length,
                              uint64_t degree, bool time_aug, bool lead_lag, float end_time, int method,
                              bool scalar_term, void* stream, int synchronize, int* nonfinite) {
    SIG_SAFE_CALL(log_sig_entry<float>(path, out, batch_size, dimension, length, degree, time_aug, lead_lag, end_time,
                                       method, scalar_term, stream_options(stream, synchronize, nonfinite)));
}

SIG_API int sigb200_log_sig_d(const double* path, double* out, uint64_t batch_size, uint64_t dimension, uint64_t length,
                              uint64_t degree, bool time_aug, bool lead_lag, double end_time, int method,
                              bool scalar_term, void* stream, int synchronize, int* nonfinite) {
    SIG_SAFE_CALL(log_sig_entry<double>(path, out, batch_size, dimension, length, degree, time_aug, lead_lag, end_time,
                                        method, scalar_term, stream_options(stream, synchronize, nonfinite)));
}

SIG_API int sigb200_signature_sharded_f(const float* path, float* out, uint64_t batch_size, uint64_t dimension,
                                        uint64_t length, uint64_t degree, bool time_aug, bool lead_lag,
                                        float end_time, bool scalar_term, const int* devices, int n_devices) {
    SIG_SAFE_CALL(signature_sharded<float>(path, out, batch_size, dimension, length, degree, time_aug, lead_lag,
                                           end_time, scalar_term, devices, n_devices));
}

SIG_API int sigb200_signature_sharded_d(const double* path, double* out, uint64_t batch_size, uint64_t dimension,
                                        uint64_t length, uint64_t degree, bool time_aug, bool lead_lag,
                                        double end_time, bool scalar_term, const int* devices, int n_devices) {
    SIG_SAFE_CALL(signature_sharded<double>(path, out, batch_size, dimension, length, degree, time_aug, lead_lag,
                                            end_time, scalar_term, devices, n_devices));
}

SIG_API int sigb200_sig_backprop_sharded_f(const float* path, float* out, const float* sig_derivs,
                                           const float* sig, uint64_t batch_size, uint64_t dimension,
                                           uint64_t length, uint64_t degree, bool time_aug, bool lead_lag,
                                           float end_time, bool scalar_term, const int* devices, int n_devices) {
    SIG_SAFE_CALL(sig_backprop_sharded<float>(path, out, sig_derivs, sig, batch_size, dimension, length, degree,
                                              time_aug, lead_lag, end_time, scalar_term, devices, n_devices));
}

SIG_API int sigb200_sig_backprop_sharded_d(const double* path, double* out, const double* sig_derivs,
                                           const double* sig, uint64_t batch_size, uint64_t dimension,
                                           uint64_t length, uint64_t degree, bool time_aug, bool lead_lag,
                                           double end_time, bool scalar_term, const int* devices, int n_devices) {
    SIG_SAFE_CALL(sig_backprop_sharded<double>(path, out, sig_derivs, sig, batch_size, dimension, length, degree,
                                               time_aug, lead_lag, end_time, scalar_term, devices, n_devices));
}

SIG_API uint64_t sigb200_sig_length(uint64_t dimension, uint64_t degree) {
    try { return sig_length_full(dimension, degree); } catch (...) { return 0; }
}

SIG_API void sigb200_set_kernel_policy(int policy) { set_kernel_policy(policy); }

SIG_API void sigb200_set_tile_preference(int preference) { set_tile_preference(preference); }

SIG_API const char* sigb200_kernel_family(uint64_t dimension, uint64_t degree, bool time_aug, bool lead_lag,
                                          int is_double, int backward) {
    try {
        const SigShape s = make_shape(1, dimension, 2, degree, time_aug, lead_lag, false);
        if (!backward && (degree <= 1 || s.dim == 1)) return "trivial";
        if (backward && degree == 0) return "trivial";
        if (kernel_policy() != 0) return "generic";
        bool tile;
        if (backward) tile = is_double ? tile_backward_available<double>(s) : tile_backward_available<float>(s);
        else tile = is_double ? tile_forward_available<double>(s) : tile_forward_available<float>(s);
        return tile ? "tile" : "generic";
    } catch (...) {
        return "invalid";
    }
}

SIG_API int sigb200_describe_plan(char* buffer, uint64_t buffer_len, uint64_t batch_size, uint64_t dimension,
                                  uint64_t length, uint64_t degree, bool time_aug, bool lead_lag, int is_double,
                                  int backward) {
    SIG_SAFE_CALL(
        const SigShape s = make_shape(batch_size, dimension, length, degree, time_aug, lead_lag, false);
        std::string text;
        if (!backward && (s.len <= 1 || degree <= 1 || s.dim == 1)) text = "closed form";
        else if (backward && (s.len <= 1 || degree == 0)) text = "zero fill";
        else if (kernel_policy() != 0) text = "generic";
        else text = describe_tile_plan(is_double != 0, backward != 0, s);
        if (buffer && buffer_len) {
            const size_t n = std::min<size_t>(text.size(), buffer_len - 1);
            std::memcpy(buffer, text.data(), n);
            buffer[n] = 0;
        });
}

SIG_API uint64_t sigb200_launch_count(void) { return launch_count(); }

SIG_API void sigb200_set_forced_plan(int backward, int chain_length, int group, int segments) {
    set_forced_plan(backward != 0, chain_length, group, segments);
}

SIG_API void sigb200_inject_alloc_failures(int count) { inject_alloc_failures(count); }

SIG_API uint64_t sigb200_pool_reserved_bytes(int device) {
    try { return pool_reserved_bytes(device); } catch (...) { return 0; }
}

// ---- stubs for the rest of the reference's CUDA surface (pysiglib/load_siglib.py:165-183,420-641) ----

#define SIG_STUB(name) SIG_API int name(...) { return stub_not_built(#name); }
#define SIG_STUB_PAIR(name) SIG_STUB(name##_f) SIG_STUB(name##_d)

SIG_STUB_PAIR(log_sig_combine_cuda) SIG_STUB_PAIR(log_sig_combine_backprop_cuda)
SIG_STUB_PAIR(log_sig_from_path_cuda) SIG_STUB_PAIR(log_sig_from_path_backprop_cuda)
SIG_STUB_PAIR(log_sig_join_cuda) SIG_STUB_PAIR(log_sig_join_backprop_cuda)
SIG_STUB_PAIR(logsig_to_sig_cuda) SIG_STUB_PAIR(logsig_to_sig_backprop_cuda)
SIG_STUB_PAIR(sig_kernel_cuda) SIG_STUB_PAIR(sig_kernel_backprop_cuda)
SIG_STUB_PAIR(sig_kernel_poly_cuda) SIG_STUB_PAIR(sig_kernel_poly_backprop_cuda)
SIG_STUB_PAIR(branched_sig_cuda) SIG_STUB_PAIR(branched_sig_backprop_cuda)
SIG_STUB_PAIR(branched_sig_coef_cuda) SIG_STUB_PAIR(branched_sig_coef_backprop_cuda)
SIG_STUB_PAIR(branched_sig_combine_cuda) SIG_STUB_PAIR(branched_sig_combine_backprop_cuda)
SIG_STUB_PAIR(branched_sig_kernel_cuda) SIG_STUB_PAIR(branched_sig_kernel_backprop_cuda)
SIG_STUB_PAIR(branched_sig_kernel_poly_cuda) SIG_STUB_PAIR(branched_sig_kernel_poly_backprop_cuda)
SIG_STUB_PAIR(branched_sig_to_log_sig_cuda) SIG_STUB_PAIR(branched_sig_to_log_sig_backprop_cuda)
SIG_STUB_PAIR(branched_log_sig_join_cuda) SIG_STUB_PAIR(branched_log_sig_join_backprop_cuda)
SIG_STUB_PAIR(branched_log_sig_from_path_cuda) SIG_STUB_PAIR(branched_log_sig_from_path_backprop_cuda)
SIG_STUB(clear_cache_cuda) SIG_STUB(set_cache_dir_cuda)
SIG_STUB(prepare_branched_sig_cuda) SIG_STUB(prepare_branched_log_sig_cuda)
SIG_STUB(prepare_branched_sig_coef_cuda)
