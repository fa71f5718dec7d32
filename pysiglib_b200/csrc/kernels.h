// Host-side launch interface of the signature kernels.  Every function enqueues
// work on `stream` for the current device and returns without synchronising.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <string>

#include "common.h"

namespace sigb200 {

constexpr int kMaxDegree = 64;  // level-index table size; d >= 2 overflows 64 bits long before

struct LevelIndex {
    // li[k] = offset of level k in the scalar-term layout = (d^k - 1) / (d - 1); li[degree+1] = length
    uint32_t li[kMaxDegree + 2];
};

LevelIndex make_level_index(uint64_t dim, uint64_t degree);

// ---- closed forms: degree <= 1, augmented length <= 1, augmented dimension 1 ----
template <typename T>
void launch_trivial_forward(const T* path, T* out, const SigShape& s, T end_time, cudaStream_t stream);

// Degree-1 backward (closed form: only the end points of a path get a gradient).
template <typename T>
void launch_degree_one_backward(const T* path, T* out, const T* sig_derivs, const SigShape& s, T end_time,
                                cudaStream_t stream);

// ---- generic (any dimension / degree) level-synchronous kernels, one CTA per path ----
// scratch: generic_forward_scratch_elems(s) elements per CTA, `ctas` CTAs.
uint64_t generic_forward_scratch_elems(const SigShape& s);
uint64_t generic_backward_scratch_elems(const SigShape& s);
template <typename T>
void launch_generic_forward(const T* path, T* out, const SigShape& s, T end_time, T* scratch,
                            unsigned ctas, cudaStream_t stream);
template <typename T>
void launch_generic_backward(const T* path, T* out, const T* sig_derivs, const T* sig, const SigShape& s,
                             T end_time, T* scratch, unsigned ctas, cudaStream_t stream);

// ---- register-tile kernels for a table of (dimension, degree) shapes ----
// Return false when the shape is not in the table (nothing is enqueued).
// The backward variant accumulates increment gradients with atomics into
// `incr_grad` (batch x (data_len - 1) x data_dim, zeroed here) and then converts
// them to point gradients in `out`.
template <typename T>
bool tile_forward_available(const SigShape& s);
// `nonfinite` (device int, may be null): set to 1 when the stored signature holds NaN / Inf;
// *nonfinite_checked tells whether the launched kernels did that check themselves.
template <typename T>
bool launch_tile_forward(const T* path, T* out, const SigShape& s, T end_time, cudaStream_t stream,
                         int* nonfinite = nullptr, bool* nonfinite_checked = nullptr);
// Paths per full wave of the unsegmented register-tile sweep for this shape (0 = unknown).
template <typename T>
uint64_t tile_wave_paths(const SigShape& s, bool backward);
template <typename T>
bool tile_backward_available(const SigShape& s);
template <typename T>
bool launch_tile_backward(const T* path, T* out, const T* sig_derivs, const T* sig, const SigShape& s,
                          T end_time, T* incr_grad, cudaStream_t stream);

// log(signature) of every path in one launch, without the signature going to global memory (the
// fused sweep of sig_tile.cuh).  rank == nullptr: expanded logarithm, `out` laid out like the signature
// (out_shift = 1 leaves the scalar slot, set to 0); otherwise rank[p] = output index of the word at
// scalar-free position p, or -1 to drop it.  Returns false when nothing was launched: the shape has
// no fused kernel, or (unless `force`) the two-step route is the faster one for it.
template <typename T>
bool launch_tile_forward_log(const T* path, T* out, const SigShape& s, T end_time, uint32_t out_stride,
                             uint32_t out_shift, const int32_t* rank, int* nonfinite, cudaStream_t stream,
                             bool force = false);

// What the tile dispatcher would launch for this shape on the current device ("generic" if none).
std::string describe_tile_plan(bool is_double, bool backward, const SigShape& s);

// out[b] <- seg[b][0] (x) seg[b][1] (x) .. (x) seg[b][nseg-1]  (Chen products truncated at the
// degree), pairwise in ceil(log2 nseg) launches.  seg is (batch, nseg, S) without scalar terms;
// tmp holds chen_combine_tmp_elems(s, nseg) values.
uint64_t chen_combine_tmp_elems(const SigShape& s, int nseg);
template <typename T>
void launch_chen_combine(T* out, const T* seg, T* tmp, const SigShape& s, int nseg, cudaStream_t stream);

// The same join in one launch, one CTA per path with the running product in shared memory
// (sig_chen.cu); false, with nothing launched, when a signature does not fit there.
template <typename T>
bool launch_chen_chain(T* out, const T* seg, const SigShape& s, int nseg, cudaStream_t stream);

// C = A (x) B with one CTA per signature (sig_chen.cu): the levels below N of both factors in shared
// memory, the top level streamed with vector loads and stores.  A or B may be nullptr: that factor is
// then exp(disp[b]), the signature of the straight segment with displacement disp[b] (dimension values
// per signature), generated on the fly.  Returns false, with nothing launched, when the batch is too
// small to fill the GPU that way or the lower levels do not fit shared memory.
template <typename T>
bool launch_chen_product_streamed(const T* A, uint64_t a_stride, const T* B, uint64_t b_stride, const T* disp, T* C,
                                  uint64_t c_stride, const SigShape& s, cudaStream_t stream, bool write_scalar);

// Both adjoints of C = A (x) B from dC (dA[u] = sum_v dC[u v] B[v], dB[v] = sum_u A[u] dC[u v]) in one
// pass over dC, one CTA per signature; every pointer addresses a first level-1 coefficient.  Returns
// false, with nothing launched, under the same conditions as launch_chen_product_streamed.
// gen = 1 / 2: factor A / B is exp(disp[b]) (its pointers are ignored) and the adjoint of the
// displacement goes to d_disp (batch x dim) instead.
template <typename T>
bool launch_chen_adjoints_streamed(const T* dC, uint64_t dc_stride, const T* A, uint64_t a_stride, const T* B,
                                   uint64_t b_stride, T* dA, uint64_t da_stride, T* dB, uint64_t db_stride,
                                   const SigShape& s, cudaStream_t stream, int gen = 0, const T* disp = nullptr,
                                   T* d_disp = nullptr);

// C = A (x) B and the adjoint of the left factor, dX[u] = sum_v dS[u v] A[v], for batches of
// scalar-free signatures; every pointer addresses the first level-1 coefficient of path 0 and
// has its own batch stride (in elements).
template <typename T>
void launch_chen_product(const T* A, uint64_t a_stride, const T* B, uint64_t b_stride, T* C, uint64_t c_stride,
                         const SigShape& s, cudaStream_t stream, bool write_scalar = false);
template <typename T>
void launch_chen_left_adjoint(const T* dS, uint64_t ds_stride, const T* A, uint64_t a_stride, T* dX,
                              uint64_t dx_stride, const SigShape& s, cudaStream_t stream);
// dY[v] = sum_u dS[u v] A[u]: adjoint of the right factor of A (x) Y
template <typename T>
void launch_chen_right_adjoint(const T* dS, uint64_t ds_stride, const T* A, uint64_t a_stride, T* dY,
                               uint64_t dy_stride, const SigShape& s, cudaStream_t stream);

// out[t] = g[t-1] - g[t] over the raw path (g = increment gradients, (batch, L-1, d))
template <typename T>
void launch_increment_to_point_grad(const T* incr_grad, T* out, uint64_t batch, uint64_t L, uint64_t d,
                                    cudaStream_t stream);

template <typename T>
void launch_fill(T* dst, uint64_t n, T value, cudaStream_t stream);

// Scans `n` values for NaN / Inf and sets *flag (device int) to 1 if any is found.
template <typename T>
void launch_nonfinite_scan(const T* data, uint64_t n, int* flag, cudaStream_t stream);

}  // namespace sigb200
