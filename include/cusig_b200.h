/*
 * C ABI of libcusig.so, the sm_100a (B200) implementation of pySigLib's batched
 * truncated path signature and its backward pass.
 *
 * Every function returns 0 on success, or: 1 allocation failure, 2 invalid
 * argument, 3 out of range, 10 runtime error, 11 unknown, 100000 + cudaError_t
 * for CUDA failures.  A description of the last failure on the calling thread is
 * returned by cusig_last_error_message().
 *
 * Buffers are caller-owned, contiguous and row-major:
 *   path        (batch, length, dimension)
 *   out / sig / sig_derivs  (batch, S)  with S = sum_{k=1..degree} d'^k (+1 when
 *               scalar_term), d' = (lead_lag ? 2*dimension : dimension) + (time_aug ? 1 : 0)
 * Pointers are either all device pointers (work runs on the device that owns
 * them) or all host pointers (the library stages the batch through the current
 * device in overlapped chunks and returns the result in host memory).
 */
#ifndef CUSIG_B200_H_
#define CUSIG_B200_H_

#include <stdbool.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* --- symbols with the reference's names and signatures ------------------------------- */

/* Truncated signature of a batch of paths.
 * Replaces: siglib/cusig/cusig.h:312-314 (declaration),
 *           siglib/cusig/cu_signature.cu:3497-3517 (definition); bound by
 *           pysiglib/load_siglib.py:484-488.
 * `horner` is accepted for compatibility; both settings run the Horner kernels.
 * A non-empty `correction` (correction_len values per segment, a prefix of tensor levels
 * 2..degree of the data dimension; segment j of path b at correction + b * batch_stride +
 * j * segment_stride) makes every segment's signature exp(increment + correction)
 * (siglib/cusig/cu_signature.cu:2369-2427, 2503-2531); not allowed with lead_lag.  Synchronous. */
int signature_cuda_f(const float* path, float* out, uint64_t batch_size, uint64_t dimension,
                     uint64_t length, uint64_t degree, bool time_aug, bool lead_lag, float end_time,
                     bool horner, bool scalar_term, const float* correction, uint64_t correction_len,
                     uint64_t correction_batch_stride, uint64_t correction_segment_stride);
int signature_cuda_d(const double* path, double* out, uint64_t batch_size, uint64_t dimension,
                     uint64_t length, uint64_t degree, bool time_aug, bool lead_lag, double end_time,
                     bool horner, bool scalar_term, const double* correction, uint64_t correction_len,
                     uint64_t correction_batch_stride, uint64_t correction_segment_stride);

/* Gradient of a scalar loss with respect to the path, given dLoss/dSignature.
 * Replaces: siglib/cusig/cusig.h:342-344, siglib/cusig/cu_signature.cu:3524-3544; bound by
 *           pysiglib/load_siglib.py:490-494.  Note the order: sig_derivs before sig.
 * `out` has the shape of `path`.  With a non-empty `correction` the gradient is that of the
 * corrected signature, still with respect to the path only (siglib/cusig/cu_signature.cu:2659-2763).
 * Synchronous. */
int sig_backprop_cuda_f(const float* path, float* out, const float* sig_derivs, const float* sig,
                        uint64_t batch_size, uint64_t dimension, uint64_t length, uint64_t degree,
                        bool time_aug, bool lead_lag, float end_time, bool scalar_term,
                        const float* correction, uint64_t correction_len,
                        uint64_t correction_batch_stride, uint64_t correction_segment_stride);
int sig_backprop_cuda_d(const double* path, double* out, const double* sig_derivs, const double* sig,
                        uint64_t batch_size, uint64_t dimension, uint64_t length, uint64_t degree,
                        bool time_aug, bool lead_lag, double end_time, bool scalar_term,
                        const double* correction, uint64_t correction_len,
                        uint64_t correction_batch_stride, uint64_t correction_segment_stride);

/* Chen product of two batches of signatures: out = sig1 (x) sig2, the signature of the
 * concatenated paths.  All three arrays are (batch, S) in the layout above.
 * Replaces: siglib/cusig/cusig.h:363-365 (siglib/cusig/cu_sig_combine.cu); bound by
 *           pysiglib/load_siglib.py:450-453.  Synchronous; device or host pointers. */
int sig_combine_cuda_f(const float* sig1, const float* sig2, float* out, uint64_t batch_size,
                       uint64_t dimension, uint64_t degree, bool scalar_term);
int sig_combine_cuda_d(const double* sig1, const double* sig2, double* out, uint64_t batch_size,
                       uint64_t dimension, uint64_t degree, bool scalar_term);

/* Backward of sig_combine: given dLoss/d(sig1 (x) sig2), writes dLoss/d sig1 and dLoss/d sig2
 * (same layout; the scalar slots get 0).
 * Replaces: siglib/cusig/cusig.h:386-388 (siglib/cusig/cu_sig_combine.cu); bound by
 *           pysiglib/load_siglib.py:466-470.  Synchronous; device or host pointers. */
int sig_combine_backprop_cuda_f(const float* sig_combined_deriv, float* sig1_deriv, float* sig2_deriv,
                                const float* sig1, const float* sig2, uint64_t batch_size, uint64_t dimension,
                                uint64_t degree, bool scalar_term);
int sig_combine_backprop_cuda_d(const double* sig_combined_deriv, double* sig1_deriv, double* sig2_deriv,
                                const double* sig1, const double* sig2, uint64_t batch_size, uint64_t dimension,
                                uint64_t degree, bool scalar_term);

/* Signature of the straight segment with the given displacement: out[b] = exp(displacement[b]),
 * level k = displacement^(x)k / k!.
 * Replaces: siglib/cusig/cusig.h:942-944 (siglib/cusig/cu_sig_combine.cu); bound by
 *           pysiglib/load_siglib.py:618-622.  Synchronous; device or host pointers. */
int linear_sig_cuda_f(const float* displacement, float* out, uint64_t batch_size, uint64_t dimension,
                      uint64_t degree, bool scalar_term);
int linear_sig_cuda_d(const double* displacement, double* out, uint64_t batch_size, uint64_t dimension,
                      uint64_t degree, bool scalar_term);

/* Extends signatures by one straight segment: out = sig (x) exp(displacement), or
 * exp(displacement) (x) sig with `prepend`.
 * Replaces: siglib/cusig/cusig.h:962-964 (siglib/cusig/cu_sig_combine.cu:495-543); bound by
 *           pysiglib/load_siglib.py:455-459.  Synchronous; device or host pointers. */
int sig_join_cuda_f(const float* sig, const float* displacement, float* out, uint64_t batch_size,
                    uint64_t dimension, uint64_t degree, bool prepend, bool scalar_term);
int sig_join_cuda_d(const double* sig, const double* displacement, double* out, uint64_t batch_size,
                    uint64_t dimension, uint64_t degree, bool prepend, bool scalar_term);

/* Backward of sig_join: writes dLoss/d sig (scalar slots 0) and dLoss/d displacement.
 * Replaces: siglib/cusig/cusig.h:984-986 (siglib/cusig/cu_sig_combine.cu:549-659); bound by
 *           pysiglib/load_siglib.py:460-464.  Computed entirely on the device. */
int sig_join_backprop_cuda_f(const float* d_out, float* d_sig, float* d_displacement, const float* sig,
                             const float* displacement, uint64_t batch_size, uint64_t dimension,
                             uint64_t degree, bool prepend, bool scalar_term);
int sig_join_backprop_cuda_d(const double* d_out, double* d_sig, double* d_displacement, const double* sig,
                             const double* displacement, uint64_t batch_size, uint64_t dimension,
                             uint64_t degree, bool prepend, bool scalar_term);

/* Materialises the lead-lag / time-augmented path: (B, L, d) -> (B, L', d') with L' = 2L-1 under
 * lead_lag and d' = (lead_lag ? 2d : d) + (time_aug ? 1 : 0); and the adjoint of that map
 * ((B, L', d') -> (B, L, d), the time channel dropped).
 * Replaces: siglib/cusig/cusig.h:65-67, 90-92 (siglib/cusig/cu_path_transforms.cu:100-205); bound by
 *           pysiglib/load_siglib.py:420-429.  Synchronous; device or host pointers. */
int transform_path_cuda_f(const float* data_in, float* data_out, uint64_t batch_size, uint64_t dimension,
                          uint64_t length, bool time_aug, bool lead_lag, float end_time);
int transform_path_cuda_d(const double* data_in, double* data_out, uint64_t batch_size, uint64_t dimension,
                          uint64_t length, bool time_aug, bool lead_lag, double end_time);
int transform_path_backprop_cuda_f(const float* derivs, float* data_out, uint64_t batch_size, uint64_t dimension,
                                   uint64_t length, bool time_aug, bool lead_lag, float end_time);
int transform_path_backprop_cuda_d(const double* derivs, double* data_out, uint64_t batch_size, uint64_t dimension,
                                   uint64_t length, bool time_aug, bool lead_lag, double end_time);

/* Signature coefficients at given words only.  `multi_idx` lists the letters of all words back
 * to back, `degrees` their lengths (uint64 arrays, device or host memory); with `prefixes` every
 * non-empty word contributes the coefficients of all its prefixes, else one value per word (the
 * empty word gives 1).  `dimension` is the dimension of `path` as passed: no transform is applied.
 * The backward takes the forward result computed with prefixes (`coefs`) and the adjoints in the
 * same layout (`derivs`) and writes the gradient with respect to `path`.  Words up to 32 letters.
 * Replaces: siglib/cusig/cusig.h:468-470, 492-494 (siglib/cusig/cu_sig_coef.cu); bound by
 *           pysiglib/load_siglib.py:471-482.  Synchronous; device or host pointers. */
int sig_coef_cuda_f(const float* path, float* out, const uint64_t* multi_idx, uint64_t num_multi_idx,
                    const uint64_t* degrees, uint64_t batch_size, uint64_t dimension, uint64_t length, bool prefixes);
int sig_coef_cuda_d(const double* path, double* out, const uint64_t* multi_idx, uint64_t num_multi_idx,
                    const uint64_t* degrees, uint64_t batch_size, uint64_t dimension, uint64_t length, bool prefixes);
int sig_coef_backprop_cuda_f(const float* path, float* out, const float* coefs, const float* derivs,
                             const uint64_t* multi_idx, uint64_t num_multi_idx, const uint64_t* degrees,
                             uint64_t batch_size, uint64_t dimension, uint64_t length);
int sig_coef_backprop_cuda_d(const double* path, double* out, const double* coefs, const double* derivs,
                             const uint64_t* multi_idx, uint64_t num_multi_idx, const uint64_t* degrees,
                             uint64_t batch_size, uint64_t dimension, uint64_t length);

/* Signature -> log signature.  method 0: expanded tensor logarithm in the layout of `sig` (scalar
 * slot 0); method 1: its coordinates at the Lyndon words of length <= degree, by length then
 * lexicographically (log_sig_length values per signature); method 2: its coordinates in the Lyndon
 * (bracket) basis, same count.  Method 3 returns code 2.
 * The backward takes dLoss/d log_sig in the layout of the forward's output and writes dLoss/d sig
 * in the layout of `sig`.
 * Replaces: siglib/cusig/cusig.h:407-409, 427-429 (siglib/cusig/cu_log_signature.cu); bound by
 *           pysiglib/load_siglib.py:496-505.  Synchronous; device or host pointers. */
int sig_to_log_sig_cuda_f(const float* sig, float* out, uint64_t batch_size, uint64_t dimension, uint64_t degree,
                          int method, bool scalar_term);
int sig_to_log_sig_cuda_d(const double* sig, double* out, uint64_t batch_size, uint64_t dimension, uint64_t degree,
                          int method, bool scalar_term);
int sig_to_log_sig_backprop_cuda_f(const float* sig, float* out, const float* log_sig_derivs, uint64_t batch_size,
                                   uint64_t dimension, uint64_t degree, int method, bool scalar_term);
int sig_to_log_sig_backprop_cuda_d(const double* sig, double* out, const double* log_sig_derivs, uint64_t batch_size,
                                   uint64_t dimension, uint64_t degree, int method, bool scalar_term);

/* Builds the per-device tables of methods 1 and 2 ahead of the first call (optional: the
 * tables are built on demand); method 0 needs nothing; method 3 returns code 2.
 * Replaces: siglib/cusig/cusig.h:447; bound by pysiglib/load_siglib.py:165-183. */
int prepare_log_sig_cuda(uint64_t dimension, uint64_t degree, int method, bool use_disk);

/* Thread-local text of the last error; valid until the next call on this thread.
 * Replaces: siglib/cusig/cusig.h:43; bound by pysiglib/load_siglib.py:108-110. */
const char* cusig_last_error_message(void);

/* Releases streams and cached device memory on every device.
 * Replaces: siglib/cusig/cusig.h:1028 (siglib/cusig/cache_lifecycle/cusig_lifecycle.cu:35-50). */
void cusig_shutdown(void);

/* --- extensions used by this repository's Python layer and benchmark ------------------ */

/* As signature_cuda_* on an explicit stream (a cudaStream_t passed as void*).
 * synchronize = 0 returns as soon as the work is enqueued (device pointers only).
 * nonfinite: optional host int set to 1 when the output holds NaN or Inf (forces a
 * synchronisation); replaces the two isnan/isinf passes of pysiglib/sig.py:299-302.
 * The reference has no stream argument (siglib/cusig/cu_runtime_utils.h:53-56 synchronises
 * the whole device after every call). */
int sigb200_signature_f(const float* path, float* out, uint64_t batch_size, uint64_t dimension,
                        uint64_t length, uint64_t degree, bool time_aug, bool lead_lag, float end_time,
                        bool scalar_term, void* stream, int synchronize, int* nonfinite);
int sigb200_signature_d(const double* path, double* out, uint64_t batch_size, uint64_t dimension,
                        uint64_t length, uint64_t degree, bool time_aug, bool lead_lag, double end_time,
                        bool scalar_term, void* stream, int synchronize, int* nonfinite);
int sigb200_sig_backprop_f(const float* path, float* out, const float* sig_derivs, const float* sig,
                           uint64_t batch_size, uint64_t dimension, uint64_t length, uint64_t degree,
                           bool time_aug, bool lead_lag, float end_time, bool scalar_term, void* stream,
                           int synchronize);
int sigb200_sig_backprop_d(const double* path, double* out, const double* sig_derivs, const double* sig,
                           uint64_t batch_size, uint64_t dimension, uint64_t length, uint64_t degree,
                           bool time_aug, bool lead_lag, double end_time, bool scalar_term, void* stream,
                           int synchronize);

/* Single-box batch partitioner: host buffers, the batch cut into contiguous shards over
 * `n_devices` GPUs (device ordinals in `devices`, or 0..n_devices-1 when NULL), one host
 * thread and one stream set per device, no communication between devices.
 * No counterpart in the reference (it is single-device). */
int sigb200_signature_sharded_f(const float* path, float* out, uint64_t batch_size, uint64_t dimension,
                                uint64_t length, uint64_t degree, bool time_aug, bool lead_lag,
                                float end_time, bool scalar_term, const int* devices, int n_devices);
int sigb200_signature_sharded_d(const double* path, double* out, uint64_t batch_size, uint64_t dimension,
                                uint64_t length, uint64_t degree, bool time_aug, bool lead_lag,
                                double end_time, bool scalar_term, const int* devices, int n_devices);
int sigb200_sig_backprop_sharded_f(const float* path, float* out, const float* sig_derivs, const float* sig,
                                   uint64_t batch_size, uint64_t dimension, uint64_t length, uint64_t degree,
                                   bool time_aug, bool lead_lag, float end_time, bool scalar_term,
                                   const int* devices, int n_devices);
int sigb200_sig_backprop_sharded_d(const double* path, double* out, const double* sig_derivs, const double* sig,
                                   uint64_t batch_size, uint64_t dimension, uint64_t length, uint64_t degree,
                                   bool time_aug, bool lead_lag, double end_time, bool scalar_term,
                                   const int* devices, int n_devices);

/* Log signature straight from the path, methods 0 (expanded, layout of the signature; scalar_term
 * adds the leading slot, which is 0), 1 (Lyndon-word coordinates) and 2 (Lyndon-basis coordinates).
 * Replaces the two calls the reference's Python makes (pysiglib/log_sig.py:457: signature_cuda_* then
 * sig_to_log_sig_cuda_*) by one in which the signature is never written to a caller-visible array;
 * for shapes with a fused kernel it never reaches global memory at all.  `out` holds
 * batch * (method 0: signature length, else log-signature length) values.  Device or host pointers;
 * `nonfinite` (may be NULL) receives 1 when the signature holds NaN / Inf (then the call also waits
 * for completion).  No counterpart among the reference's C symbols. */
int sigb200_log_sig_f(const float* path, float* out, uint64_t batch_size, uint64_t dimension, uint64_t length,
                      uint64_t degree, bool time_aug, bool lead_lag, float end_time, int method, bool scalar_term,
                      void* stream, int synchronize, int* nonfinite);
int sigb200_log_sig_d(const double* path, double* out, uint64_t batch_size, uint64_t dimension, uint64_t length,
                      uint64_t degree, bool time_aug, bool lead_lag, double end_time, int method, bool scalar_term,
                      void* stream, int synchronize, int* nonfinite);

/* sig_backprop without any device-memory allocation, for hosts that cannot allocate when they
 * need the gradient: processes whose own allocator already owns the GPU's memory (a late
 * cudaMalloc can fail there), and latency-critical loops (cudaMalloc / cudaFree synchronise the
 * device).  This entry point has no counterpart in the reference.
 * The increment-gradient scratch (batch * (length-1) * dimension values) lives in a static
 * 32 MiB device buffer inside the library (sigb200_noalloc_scratch_bytes()); larger requests,
 * host pointers and shapes outside the register-tile kernel table are rejected with code 2.
 * Every buffer must be device memory of the GPU that holds `out`; anything else is rejected with
 * code 2 before a kernel is launched.
 * The first call on a device looks the buffer up (cudaGetSymbolAddress) and should come before
 * any stream capture.  That first call, and the first call of each (dimension, degree, flags,
 * dtype) on a device, make the CUDA runtime load device code, which does take device memory:
 * make one warm-up call per device and shape while memory is still available; later calls
 * allocate nothing.  All calls share the buffer: the used part is cleared on `stream` first,
 * and calls whose GPU work overlaps race on it.  Asynchronous on `stream` unless synchronize != 0. */
int sigb200_sig_backprop_noalloc_f(const float* path, float* out, const float* sig_derivs, const float* sig,
                                   uint64_t batch_size, uint64_t dimension, uint64_t length, uint64_t degree,
                                   bool time_aug, bool lead_lag, float end_time, bool scalar_term, void* stream,
                                   int synchronize);
int sigb200_sig_backprop_noalloc_d(const double* path, double* out, const double* sig_derivs, const double* sig,
                                   uint64_t batch_size, uint64_t dimension, uint64_t length, uint64_t degree,
                                   bool time_aug, bool lead_lag, double end_time, bool scalar_term, void* stream,
                                   int synchronize);
uint64_t sigb200_noalloc_scratch_bytes(void);

/* Number of coefficients of a signature, scalar term included; 0 on overflow.
 * Same contract as the CPU library's sig_length (siglib/cpsig/cp_utils.cpp:91-105). */
uint64_t sigb200_sig_length(uint64_t dimension, uint64_t degree);

/* 0 = automatic kernel choice (default), 1 = shape-generic kernels only. */
void sigb200_set_kernel_policy(int policy);

/* Register-tile variant choice, for tests and tuning: 0 automatic (default), 1 always the biggest
 * tile, 2 always the smallest, 3 automatic but without time segmentation of the forward sweep,
 * 4 biggest tile with the forward sweep always cut into three time segments (1-3 never segment). */
void sigb200_set_tile_preference(int preference);

/* Name of the kernel family the forward (backward = 1) pass would use for this shape:
 * "trivial", "tile", "generic".  Static string. */
const char* sigb200_kernel_family(uint64_t dimension, uint64_t degree, bool time_aug, bool lead_lag,
                                  int is_double, int backward);

/* Writes a description of the kernel variant this call shape would run on the current device
 * (tile parameters, time segments, resident CTAs per SM) into `buffer`.  Diagnostic only. */
int sigb200_describe_plan(char* buffer, uint64_t buffer_len, uint64_t batch_size, uint64_t dimension,
                          uint64_t length, uint64_t degree, bool time_aug, bool lead_lag, int is_double,
                          int backward);

/* Test hook: pins the register-tile variant (chain length, group) and the number of time segments
 * of the forward (backward = 0) or backward (1) sweep for shapes that have such a variant
 * compiled; chain_length < 0 clears it.  No counterpart in the reference. */
void sigb200_set_forced_plan(int backward, int chain_length, int group, int segments);

/* Test hook for the out-of-memory paths: the next `count` scratch / staging requests of this
 * library report cudaErrorMemoryAllocation on the host, without touching the device.  The calls
 * then recover by halving their batch piece, as the reference's workspace allocation does
 * (siglib/cusig/cu_runtime_utils.h:212-235).  SIGB200_FAIL_ALLOCS=<count> in the environment
 * arms the same thing at load time. */
void sigb200_inject_alloc_failures(int count);

/* Bytes this library's own stream-ordered memory pool currently holds on `device`
 * (scratch and staging buffers are kept there between calls until cusig_shutdown). */
uint64_t sigb200_pool_reserved_bytes(int device);

/* Number of kernels this library has launched in the calling process (all threads). */
uint64_t sigb200_launch_count(void);

#ifdef __cplusplus
}
#endif

#endif /* CUSIG_B200_H_ */
