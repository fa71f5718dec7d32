// Entry points of the host dispatch layer (one per C-ABI symbol family).
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "common.h"

namespace sigb200 {

struct CallOptions {
    cudaStream_t stream = nullptr;  // stream for device-pointer calls (nullptr = legacy default stream)
    bool synchronize = true;        // wait for completion before returning (device-pointer calls)
    int device = -1;                // device used to stage host-pointer calls (-1 = current device)
    int* nonfinite = nullptr;       // host int: set to 1 if the forward output holds NaN / Inf
};

// `nonfinite`: device int that is set to 1 when the output holds NaN / Inf (nullptr = no check).
template <typename T>
void forward_on_device(const T* path, T* out, const SigShape& s, T end_time, cudaStream_t stream,
                       int* nonfinite = nullptr);

template <typename T>
void backward_on_device(const T* path, T* out, const T* sig_derivs, const T* sig, const SigShape& s,
                        T end_time, cudaStream_t stream);

template <typename T>
void signature_entry(const T* path, T* out, uint64_t batch, uint64_t dimension, uint64_t length,
                     uint64_t degree, bool time_aug, bool lead_lag, T end_time, bool horner,
                     bool scalar_term, const T* correction, uint64_t correction_len, const CallOptions& opt,
                     uint64_t correction_batch_stride = 0, uint64_t correction_segment_stride = 0);

template <typename T>
void sig_backprop_entry(const T* path, T* out, const T* sig_derivs, const T* sig, uint64_t batch,
                        uint64_t dimension, uint64_t length, uint64_t degree, bool time_aug, bool lead_lag,
                        T end_time, bool scalar_term, const T* correction, uint64_t correction_len,
                        const CallOptions& opt, uint64_t correction_batch_stride = 0,
                        uint64_t correction_segment_stride = 0);

// out = sig1 (x) sig2 (Chen's identity) for batches of signatures of a `dimension`-channel path.
template <typename T>
void sig_combine_entry(const T* sig1, const T* sig2, T* out, uint64_t batch, uint64_t dimension, uint64_t degree,
                       bool scalar_term, const CallOptions& opt);

// Adjoints of both factors of out = sig1 (x) sig2 given dLoss/d out.
template <typename T>
void sig_combine_backprop_entry(const T* deriv, T* sig1_deriv, T* sig2_deriv, const T* sig1, const T* sig2,
                                uint64_t batch, uint64_t dimension, uint64_t degree, bool scalar_term,
                                const CallOptions& opt);

}  // namespace sigb200
