// Host entry points of the tensor-algebra operations around the signature kernels:
// signatures with per-segment correction terms, linear signatures, sig_join and the
// standalone path transforms.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "common.h"
#include "dispatch.h"

namespace sigb200 {

// Per-segment correction terms as the C ABI passes them (siglib/cusig/cusig.h:312-314):
// `len` values per segment covering tensor levels 2..k of the DATA dimension; the segment of
// path b, step j starts at ptr + b * batch_stride + j * segment_stride (strides may be 0).
template <typename T>
struct CorrectionView {
    const T* ptr = nullptr;
    uint64_t len = 0, batch_stride = 0, segment_stride = 0;
};

// Throws std::invalid_argument unless the arguments are acceptable (same rules and wording
// as siglib/cusig/cu_signature.cu:2028-2055).
void validate_correction(const void* correction, uint64_t correction_len, uint64_t dimension, uint64_t degree,
                         bool lead_lag);

// Signature with segment signatures exp(increment + correction); device pointers, s.len >= 2,
// s.degree >= 2, no lead-lag.
template <typename T>
void correction_forward_on_device(const T* path, T* out, const SigShape& s, T end_time, const CorrectionView<T>& c,
                                  cudaStream_t stream);

// Gradient of sum(sig_derivs * sig) w.r.t. the path for the corrected signature.
template <typename T>
void correction_backward_on_device(const T* path, T* out, const T* sig_derivs, const T* sig, const SigShape& s,
                                   T end_time, const CorrectionView<T>& c, cudaStream_t stream);

// Signature of straight segments: out[b] = exp(displacement[b]).  Replaces linear_sig_cuda_
// (siglib/cusig/cu_sig_combine.cu).
template <typename T>
void linear_sig_entry(const T* displacement, T* out, uint64_t batch, uint64_t dimension, uint64_t degree,
                      bool scalar_term, const CallOptions& opt);

// out = sig (x) exp(displacement), or exp(displacement) (x) sig with prepend.  Replaces sig_join_cuda_
// (siglib/cusig/cu_sig_combine.cu:495-543).
template <typename T>
void sig_join_entry(const T* sig, const T* displacement, T* out, uint64_t batch, uint64_t dimension,
                    uint64_t degree, bool prepend, bool scalar_term, const CallOptions& opt);

// Adjoints of sig_join w.r.t. the signature and the displacement.  Replaces sig_join_backprop_cuda_
// (siglib/cusig/cu_sig_combine.cu:549-659), without its round trip through host memory.
template <typename T>
void sig_join_backprop_entry(const T* d_out, T* d_sig, T* d_displacement, const T* sig, const T* displacement,
                             uint64_t batch, uint64_t dimension, uint64_t degree, bool prepend, bool scalar_term,
                             const CallOptions& opt);

// Signature -> log signature.  method 0: the expanded tensor logarithm, in the layout of `sig`;
// method 1: its coordinates at the Lyndon words, method 2: in the Lyndon basis (log_sig_length
// values per signature each).  Replaces
// sig_to_log_sig_cuda_ / sig_to_log_sig_backprop_cuda_ (siglib/cusig/cu_log_signature.cu) for those
// methods; the backward writes dLoss/d sig in the layout of `sig` (scalar slots 0).
template <typename T>
void sig_to_log_sig_entry(const T* sig, T* out, uint64_t batch, uint64_t dimension, uint64_t degree, int method,
                          bool scalar_term, const CallOptions& opt);
template <typename T>
void sig_to_log_sig_backprop_entry(const T* sig, T* out, const T* log_sig_derivs, uint64_t batch, uint64_t dimension,
                                   uint64_t degree, int method, bool scalar_term, const CallOptions& opt);
// Builds (and caches per device) the Lyndon-word table of methods 1 and 2 and the inverse
// projection matrix of method 2; method 3 is not part of this build.
// Log signature from the path in one call (methods 0, 1, 2); `scalar_term` only matters for method 0,
// whose result has the layout of the signature.  opt.nonfinite reports NaN / Inf in the signature.
template <typename T>
void log_sig_entry(const T* path, T* out, uint64_t batch, uint64_t dimension, uint64_t length, uint64_t degree,
                   bool time_aug, bool lead_lag, T end_time, int method, bool scalar_term, const CallOptions& opt);

void prepare_log_sig_entry(uint64_t dimension, uint64_t degree, int method);
uint64_t log_sig_length_host(uint64_t dimension, uint64_t degree);
void release_log_sig_tables() noexcept;

// Coefficients of the signature at given words only (one thread per path and word), and the
// gradient w.r.t. the path given the adjoints of all prefix coefficients.  multi_idx / degrees
// (uint64, device or host memory) list the letters of all words back to back and the word lengths;
// `dimension` is the dimension of `path` as passed (no transforms here).  Replace sig_coef_cuda_ /
// sig_coef_backprop_cuda_ (siglib/cusig/cu_sig_coef.cu).
template <typename T>
void sig_coef_entry(const T* path, T* out, const uint64_t* multi_idx, uint64_t num_multi_idx, const uint64_t* degrees,
                    uint64_t batch, uint64_t dimension, uint64_t length, bool prefixes, const CallOptions& opt);
template <typename T>
void sig_coef_backprop_entry(const T* path, T* out, const T* coefs, const T* derivs, const uint64_t* multi_idx,
                             uint64_t num_multi_idx, const uint64_t* degrees, uint64_t batch, uint64_t dimension,
                             uint64_t length, const CallOptions& opt);

// Materialises the time-augmented / lead-lag path, and the adjoint of that map.  Replace
// transform_path_cuda_ and transform_path_backprop_cuda_ (siglib/cusig/cu_path_transforms.cu:100-205).
template <typename T>
void transform_path_entry(const T* data_in, T* data_out, uint64_t batch, uint64_t dimension, uint64_t length,
                          bool time_aug, bool lead_lag, T end_time, const CallOptions& opt);
template <typename T>
void transform_path_backprop_entry(const T* derivs, T* data_out, uint64_t batch, uint64_t dimension, uint64_t length,
                                   bool time_aug, bool lead_lag, T end_time, const CallOptions& opt);

// The tensor logarithm of a whole batch in one launch, one CTA per signature (sig_log_stream.cu): the
// expanded tensor (lyndon == nullptr, count = its length) or the coordinates at the Lyndon words
// (lyndon[i]: scalar-free position of coordinate i).  Returns false with nothing launched when the shape
// is not served (batch below the SM count, degree < 2, levels below N beyond shared memory).
template <typename T>
bool launch_log_forward_streamed(const T* x, uint64_t x_stride, T* out, uint64_t out_stride, const uint32_t* lyndon,
                                 uint32_t count, bool zero_scalar, uint64_t batch, uint64_t dim, uint64_t degree,
                                 cudaStream_t stream);

// The backward pass of the tensor logarithm for a whole batch in one launch, one CTA per signature
// (sig_log_stream.cu).  x / dsig: first level-1 coefficients; g: the gradient in expanded layout
// (rank == nullptr) or with respect to the Lyndon-word coordinates (rank[p]: coordinate at scalar-free
// position p, -1 if none).  Returns false with nothing launched when the shape is not served (batch
// below the SM count, dimension not a power of two, degree < 2, working set beyond shared memory).
template <typename T>
bool launch_log_adjoint_streamed(const T* x, uint64_t x_stride, const T* g, uint64_t g_stride, const int32_t* rank,
                                 T* dsig, uint64_t dsig_stride, bool zero_scalar, uint64_t batch, uint64_t dim,
                                 uint64_t degree, cudaStream_t stream);

}  // namespace sigb200
