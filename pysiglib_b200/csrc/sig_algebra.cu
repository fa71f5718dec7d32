// Tensor-algebra operations around the signature kernels, for sm_100a:
//   * signatures whose segment signatures are exp(increment + correction)  (forward and backward),
//   * linear signatures, sig_join and its adjoints,
//   * the standalone time-augmentation / lead-lag path transform and its adjoint.
//
// These follow the per-coefficient formulation of algebra_math.h: every phase of an algorithm
// assigns each output coefficient to exactly one thread, which reads only buffers finished in an
// earlier phase, so the only synchronisation is a CTA barrier (or a kernel boundary) between phases.
// The corrected signature runs one CTA per path, sequentially over the segments, with its working
// set (a dozen signature-sized vectors per path) in a scratch buffer that stays in L2.
#include <algorithm>
#include <stdexcept>
#include <string>
#include <vector>

#include "algebra.h"
#include "algebra_host.h"
#include "algebra_math.h"
#include "increments.cuh"
#include "kernels.h"
#include "runtime.h"

namespace sigb200 {

namespace {

// ----- linear signature and its adjoint ------------------------------------------------------

// out points at the level-1 coefficient of path 0; one thread per coefficient, paths along grid.y.
template <typename T>
__global__ void linear_sig_kernel(const T* __restrict__ disp, T* __restrict__ out, uint64_t out_stride, Levels lv,
                                  uint64_t batch, bool write_scalar) {
    const uint32_t j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= lv.total()) return;
    const uint32_t t = lv.level_of(j);
    const uint32_t w = j - lv.off[t];
    for (uint64_t b = blockIdx.y; b < batch; b += gridDim.y) {
        out[b * out_stride + j] = linear_sig_coeff(disp + b * lv.dim, lv, t, w);
        if (write_scalar && j == 0) out[b * out_stride - 1] = T(1);
    }
}

// d_disp[b][i] = sum over coefficients of dL[b] * d(linear signature)/d v_i.  One CTA per path;
// partial sums meet in shared memory (acc, dim values) when it fits, else directly in d_disp,
// which the caller has zeroed.
template <typename T>
__global__ void linear_sig_adjoint_kernel(const T* __restrict__ disp, const T* __restrict__ dL, uint64_t dl_stride,
                                          T* __restrict__ d_disp, Levels lv, bool use_shared) {
    extern __shared__ unsigned char smem_raw[];
    T* acc = reinterpret_cast<T*>(smem_raw);
    const uint64_t b = blockIdx.x;
    const T* v = disp + b * uint64_t(lv.dim);
    const T* g = dL + b * dl_stride;
    T* target = use_shared ? acc : d_disp + b * uint64_t(lv.dim);
    if (use_shared) {
        for (uint32_t i = threadIdx.x; i < lv.dim; i += blockDim.x) acc[i] = T(0);
        __syncthreads();
    }
    const uint32_t S = lv.total();
    for (uint32_t j = threadIdx.x; j < S; j += blockDim.x) {
        const uint32_t t = lv.level_of(j);
        linear_sig_adjoint_terms(v, g[j], lv, t, j - lv.off[t],
                                 [&](uint32_t letter, T value) { atomicAdd(&target[letter], value); });
    }
    if (use_shared) {
        __syncthreads();
        for (uint32_t i = threadIdx.x; i < lv.dim; i += blockDim.x) d_disp[b * lv.dim + i] = acc[i];
    }
}

// The same adjoint through the recursion L_k = L_{k-1} (x) v / k, for dim <= blockDim: first the
// adjoints are pushed down level by level (in place in dL, which is scratch),
//     dL_{k-1}[u] += (1/k) sum_c v[c] dL_k[u c]        (k = N .. 2),
// then every coefficient (u, c) of level k contributes one term L_{k-1}[u] dL_k[u c] / k to d v[c].
// blockDim is a multiple of dim, so a thread always meets the same letter c = threadIdx % dim and
// keeps its partial sum in a register; the partial sums meet in shared memory (dim values).
template <typename T>
__global__ void linear_sig_adjoint_recursive_kernel(const T* __restrict__ disp, const T* __restrict__ L,
                                                    T* __restrict__ dL, uint64_t stride, T* __restrict__ d_disp,
                                                    Levels lv) {
    extern __shared__ unsigned char smem_raw[];
    T* acc = reinterpret_cast<T*>(smem_raw);  // dim sums, then dim letters of v
    T* vs = acc + lv.dim;
    const uint64_t b = blockIdx.x;
    const uint32_t d = lv.dim, N = lv.degree;
    const T* lin = L + b * stride;
    T* g = dL + b * stride;
    for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) {
        acc[i] = T(0);
        vs[i] = disp[b * d + i];
    }
    __syncthreads();
    for (uint32_t k = N; k >= 2; --k) {
        const T inv_k = T(1) / static_cast<T>(k);
        const uint32_t count = lv.size(k - 1);
        const T* upper = g + lv.off[k];
        T* lower = g + lv.off[k - 1];
        for (uint32_t u = threadIdx.x; u < count; u += blockDim.x) {
            T sum = T(0);
            for (uint32_t c = 0; c < d; ++c) sum = alg_fma(vs[c], upper[u * d + c], sum);
            lower[u] += sum * inv_k;
        }
        __syncthreads();
    }
    const uint32_t c = threadIdx.x % d;
    T mine = threadIdx.x < d ? g[threadIdx.x] : T(0);  // level 1 passes straight through
    const uint32_t first = N >= 2 ? lv.off[2] : lv.total();
    for (uint32_t j = first + threadIdx.x; j < lv.total(); j += blockDim.x) {
        const uint32_t k = lv.level_of(j);
        const uint32_t u = (j - lv.off[k]) / d;  // (j - off[k]) % d == c because off[k] - off[2] and blockDim are multiples of d
        mine = alg_fma(lin[lv.off[k - 1] + u], g[j] * (T(1) / static_cast<T>(k)), mine);
    }
    atomicAdd(&acc[c], mine);
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) d_disp[b * d + i] = acc[i];
}

template <typename T>
void launch_linear_sig(const T* disp, T* out_level1, uint64_t out_stride, const Levels& lv, uint64_t batch,
                       bool write_scalar, cudaStream_t stream) {
    if (lv.degree == 0 || batch == 0) return;
    const dim3 grid = batched_grid(lv.total(), batch, kThreads);
    linear_sig_kernel<T><<<grid, kThreads, 0, stream>>>(disp, out_level1, out_stride, lv, batch, write_scalar);
    check_launch("linear_sig kernel");
}

// L: the linear signature itself (same stride as dL); dL is scratch and is overwritten when dim <= 256.
template <typename T>
void launch_linear_sig_adjoint(const T* disp, const T* L, T* dL_level1, uint64_t dl_stride, T* d_disp,
                               const Levels& lv, uint64_t batch, cudaStream_t stream) {
    if (batch == 0) return;
    if (batch > 0x7fffffffull) throw std::invalid_argument("batch too large for one kernel launch");
    if (lv.dim <= 256) {
        const unsigned threads = lv.dim * (256 / lv.dim);  // a multiple of dim, at most 256
        linear_sig_adjoint_recursive_kernel<T><<<static_cast<unsigned>(batch), threads, 2 * size_t(lv.dim) * sizeof(T),
                                                 stream>>>(disp, L, dL_level1, dl_stride, d_disp, lv);
        check_launch("linear_sig adjoint kernel");
        return;
    }
    const size_t smem = size_t(lv.dim) * sizeof(T);
    const bool use_shared = smem <= 32 * 1024;
    if (!use_shared) SIG_CUDA_CHECK(cudaMemsetAsync(d_disp, 0, batch * lv.dim * sizeof(T), stream));
    linear_sig_adjoint_kernel<T><<<static_cast<unsigned>(batch), kThreads, use_shared ? smem : 0, stream>>>(
        disp, dL_level1, dl_stride, d_disp, lv, use_shared);
    check_launch("linear_sig adjoint kernel");
}

// ----- corrected signature: one CTA per path --------------------------------------------------

template <typename T>
struct CorrectionArgs {
    const T* ptr;
    uint64_t len, batch_stride, segment_stride;
    uint64_t data_dim;
};

// X <- increment of augmented step `step` on level 1, the correction scattered from data-dimension
// words to augmented words on levels >= 2, zero elsewhere.  Ends with a CTA barrier.
template <typename T>
__device__ void build_segment_log(T* X, const PathView<T>& pv, const T* x, int step, const CorrectionArgs<T>& c,
                                  const T* corr_path, const Levels& lv) {
    const uint32_t S = lv.total();
    for (uint32_t j = threadIdx.x; j < S; j += blockDim.x)
        X[j] = j < lv.dim ? pv.increment(x, step, static_cast<int>(j)) : T(0);
    __syncthreads();
    const T* seg = corr_path + uint64_t(step) * c.segment_stride;
    const uint32_t data_dim = static_cast<uint32_t>(c.data_dim);
    uint32_t offset = 0, level_size = data_dim;  // the correction is shorter than a signature: 32-bit indices
    for (uint32_t level = 2; level <= lv.degree; ++level) {
        level_size *= data_dim;
        if (uint64_t(offset) + level_size > c.len) break;
        for (uint32_t w = threadIdx.x; w < level_size; w += blockDim.x) {
            const T value = seg[offset + w];
            if (value == T(0)) continue;
            uint32_t rest = w, aug = 0, pw = level_size / data_dim;
            for (uint32_t pos = 0; pos < level; ++pos) {
                const uint32_t label = rest / pw;
                rest -= label * pw;
                if (pos + 1 < level) pw /= data_dim;
                aug = aug * lv.dim + label;
            }
            X[lv.off[level] + aug] = value;
        }
        offset += level_size;
    }
    __syncthreads();
}

// E <- exp(X) (and Einv <- exp(-X) when asked), keeping the powers P_2..P_N in `powers`
// (N-1 vectors) when keep_powers, else ping-ponging inside the first two.  Ends with a barrier.
template <typename T>
__device__ void segment_exp(const T* X, T* E, T* Einv, T* powers, bool keep_powers, const Levels& lv) {
    const uint32_t S = lv.total();
    for (uint32_t j = threadIdx.x; j < S; j += blockDim.x) {
        E[j] = X[j];
        if (Einv) Einv[j] = -X[j];
    }
    const T* prev = X;
    for (uint32_t n = 2; n <= lv.degree; ++n) {
        T* cur = powers + (keep_powers ? uint64_t(n - 2) : uint64_t(n & 1)) * S;
        for (uint32_t j = threadIdx.x; j < S; j += blockDim.x) {
            const uint32_t t = lv.level_of(j);
            const T val = exp_power_coeff(X, prev, lv, n, t, j - lv.off[t]);
            cur[j] = val;
            E[j] += val;  // coefficient j belongs to this thread in every round
            if (Einv) Einv[j] += (n & 1) ? -val : val;
        }
        __syncthreads();
        prev = cur;
    }
    __syncthreads();
}

template <typename T>
__global__ void correction_forward_kernel(PathView<T> pv, CorrectionArgs<T> c, T* __restrict__ out,
                                          uint64_t out_stride, bool scalar_term, T* __restrict__ scratch, Levels lv,
                                          uint64_t batch_offset) {
    const uint32_t S = lv.total();
    const uint64_t b = batch_offset + blockIdx.x;
    const T* x = pv.base + b * pv.path_stride;
    const T* corr_path = c.ptr + b * c.batch_stride;
    // the six working vectors of the path: shared memory when they fit (scratch == nullptr), else global scratch
    extern __shared__ __align__(16) unsigned char correction_smem[];
    T* ws = scratch ? scratch + uint64_t(blockIdx.x) * 6 * S : reinterpret_cast<T*>(correction_smem);
    T *X = ws, *powers = ws + S, *E = ws + 3 * uint64_t(S), *cur = ws + 4 * uint64_t(S), *nxt = ws + 5 * uint64_t(S);

    for (int step = 0; step < pv.steps; ++step) {
        build_segment_log(X, pv, x, step, c, corr_path, lv);
        segment_exp<T>(X, E, nullptr, powers, false, lv);
        for (uint32_t j = threadIdx.x; j < S; j += blockDim.x) {
            if (step == 0) {
                nxt[j] = E[j];
            } else {
                const uint32_t t = lv.level_of(j);
                nxt[j] = product_coeff(cur, E, lv, t, j - lv.off[t]);
            }
        }
        __syncthreads();
        T* tmp = cur; cur = nxt; nxt = tmp;
    }
    T* o = out + b * out_stride;
    if (scalar_term) {
        if (threadIdx.x == 0) o[0] = T(1);
        ++o;
    }
    for (uint32_t j = threadIdx.x; j < S; j += blockDim.x) o[j] = cur[j];
}

// The splits of the coefficients a thread owns, decoded once: coefficient j = threadIdx.x + k * blockDim.x
// (k < K) of level t is the word u v for every left length 1 .. t-1, and a product needs A[off[left] + u]
// and B[off[t-left] + v].  The per-coefficient formulas of algebra_math.h decode these with two integer
// divisions per term and phase; for signatures of at most K * blockDim.x coefficients a thread keeps
// the index pairs of its coefficients in registers instead and every phase is loads and FMAs only.
template <int K, int NS>
struct SplitCache {
    uint32_t level[K];          // 0: slot unused
    uint32_t ia[K][NS];         // [left - 1]
    uint32_t ib[K][NS];

    __device__ void build(const Levels& lv) {
        const uint32_t S = lv.total();
#pragma unroll
        for (int k = 0; k < K; ++k) {
            const uint32_t j = threadIdx.x + k * blockDim.x;
            level[k] = 0;
#pragma unroll
            for (int i = 0; i < NS; ++i) ia[k][i] = ib[k][i] = 0;
            if (j < S) {
                const uint32_t t = lv.level_of(j), w = j - lv.off[t];
                level[k] = t;
                uint32_t right_size = lv.dim;   // d^(t - left), from left = t - 1 down
#pragma unroll
                for (int i = NS - 1; i >= 0; --i) {
                    const uint32_t left = i + 1;
                    if (left <= t - 1) {
                        const uint32_t u = w / right_size, v = w - u * right_size;
                        ia[k][i] = lv.off[left] + u;
                        ib[k][i] = lv.off[t - left] + v;
                        right_size *= lv.dim;
                    }
                }
            }
        }
    }
};

// The forward sweep of correction_forward_kernel with the cached splits; same sums in the same order.
// Requires lv.total() <= K * blockDim.x and lv.degree - 1 <= NS; working vectors in shared memory.
template <typename T, int K, int NS>
__global__ void correction_forward_cached_kernel(PathView<T> pv, CorrectionArgs<T> c, T* __restrict__ out,
                                                 uint64_t out_stride, bool scalar_term, Levels lv,
                                                 uint64_t batch_offset) {
    extern __shared__ __align__(16) unsigned char correction_smem[];
    const uint32_t S = lv.total(), N = lv.degree, nt = blockDim.x;
    const uint64_t b = batch_offset + blockIdx.x;
    const T* x = pv.base + b * pv.path_stride;
    const T* corr_path = c.ptr + b * c.batch_stride;
    T* ws = reinterpret_cast<T*>(correction_smem);
    T *X = ws, *powers = ws + S, *E = ws + 3 * S, *cur = ws + 4 * S, *nxt = ws + 5 * S;
    SplitCache<K, NS> sp;
    sp.build(lv);

    for (int step = 0; step < pv.steps; ++step) {
        build_segment_log(X, pv, x, step, c, corr_path, lv);
        // E = exp(X) = X + sum_n P_n, P_n = X (x) P_{n-1} / n on levels >= n
#pragma unroll
        for (int k = 0; k < K; ++k)
            if (sp.level[k]) E[threadIdx.x + k * nt] = X[threadIdx.x + k * nt];
        const T* prev = X;
        for (uint32_t n = 2; n <= N; ++n) {
            T* pw = powers + uint64_t(n & 1) * S;
            const T inv_n = T(1) / static_cast<T>(n);
#pragma unroll
            for (int k = 0; k < K; ++k) {
                const uint32_t t = sp.level[k];
                if (t) {
                    T acc = T(0);
                    if (t >= n) {
#pragma unroll
                        for (int i = 0; i < NS; ++i)          // left = 1 .. t - (n - 1)
                            if (uint32_t(i) + n <= t) acc = alg_fma(prev[sp.ib[k][i]], X[sp.ia[k][i]] * inv_n, acc);
                    }
                    const uint32_t j = threadIdx.x + k * nt;
                    pw[j] = acc;
                    E[j] += acc;
                }
            }
            __syncthreads();
            prev = pw;
        }
        __syncthreads();
        // running signature times exp(X)
#pragma unroll
        for (int k = 0; k < K; ++k) {
            const uint32_t t = sp.level[k];
            if (t) {
                const uint32_t j = threadIdx.x + k * nt;
                if (step == 0) {
                    nxt[j] = E[j];
                } else {
                    T acc = cur[j];
#pragma unroll
                    for (int i = NS - 1; i >= 0; --i)          // left = t - 1 .. 1
                        if (uint32_t(i) + 1 < t) acc = alg_fma(E[sp.ib[k][i]], cur[sp.ia[k][i]], acc);
                    nxt[j] = acc + E[j];
                }
            }
        }
        __syncthreads();
        T* tmp = cur; cur = nxt; nxt = tmp;
    }
    T* o = out + b * out_stride;
    if (scalar_term) {
        if (threadIdx.x == 0) o[0] = T(1);
        ++o;
    }
    for (uint32_t j = threadIdx.x; j < S; j += nt) o[j] = cur[j];
}

// Buffers per path: X, P_2..P_N (at least 2), E, Einv, S x2, dS x2, dE, dP x2.
__host__ __device__ inline uint64_t backward_vectors(uint32_t degree) {
    return 10 + (degree > 3 ? degree - 1 : 2);
}

template <typename T>
__global__ void correction_backward_kernel(PathView<T> pv, CorrectionArgs<T> c, const T* __restrict__ sig,
                                           const T* __restrict__ sig_derivs, uint64_t sig_stride, bool scalar_term,
                                           T* __restrict__ out, T* __restrict__ scratch, Levels lv,
                                           uint64_t batch_offset) {
    extern __shared__ unsigned char smem_raw[];
    T* g = reinterpret_cast<T*>(smem_raw);  // gradient w.r.t. this step's increment
    T* g_next = g + lv.dim;                 // the same for the step after it
    const uint32_t S = lv.total();
    const uint32_t N = lv.degree;
    const uint64_t b = batch_offset + blockIdx.x;
    const T* x = pv.base + b * pv.path_stride;
    const T* corr_path = c.ptr + b * c.batch_stride;
    const uint64_t npow = N > 3 ? N - 1 : 2;
    // working vectors: behind g / g_next in shared memory when they fit (scratch == nullptr), else global scratch
    T* ws = scratch ? scratch + uint64_t(blockIdx.x) * backward_vectors(N) * S : g + ((2 * lv.dim + 3) & ~3u);
    T* X = ws;
    T* powers = ws + S;                      // P_2 .. P_N
    T* E = powers + npow * S;
    T* Einv = E + S;
    T* Scur = Einv + S;
    T* Snxt = Scur + S;
    T* dScur = Snxt + S;
    T* dSnxt = dScur + S;
    T* dE = dSnxt + S;
    T* dPa = dE + S;
    T* dPb = dPa + S;
    T* o = out + b * pv.path_stride;
    const uint64_t shift = scalar_term ? 1 : 0;

    for (uint32_t j = threadIdx.x; j < S; j += blockDim.x) {
        Scur[j] = sig[b * sig_stride + shift + j];
        dScur[j] = sig_derivs[b * sig_stride + shift + j];
    }
    for (uint32_t i = threadIdx.x; i < lv.dim; i += blockDim.x) g_next[i] = T(0);
    __syncthreads();

    for (int step = pv.steps - 1; step >= 0; --step) {
        for (uint32_t i = threadIdx.x; i < lv.dim; i += blockDim.x) g[i] = T(0);
        build_segment_log(X, pv, x, step, c, corr_path, lv);
        segment_exp<T>(X, E, Einv, powers, true, lv);

        // signature of the path up to the start of this segment
        for (uint32_t j = threadIdx.x; j < S; j += blockDim.x) {
            const uint32_t t = lv.level_of(j);
            Snxt[j] = product_coeff(Scur, Einv, lv, t, j - lv.off[t]);
        }
        __syncthreads();
        { T* tmp = Scur; Scur = Snxt; Snxt = tmp; }

        // split the adjoint of (Scur (x) E) between its factors
        for (uint32_t j = threadIdx.x; j < S; j += blockDim.x) {
            const uint32_t t = lv.level_of(j);
            const uint32_t w = j - lv.off[t];
            dE[j] = right_adjoint_coeff(dScur, Scur, lv, t, w);
            dSnxt[j] = left_adjoint_coeff(dScur, E, lv, t, w);
        }
        __syncthreads();
        { T* tmp = dScur; dScur = dSnxt; dSnxt = tmp; }

        // adjoint of exp, keeping only the level-1 part of the result
        const T* dPn = nullptr;
        T* dPprev = dPa;
        for (uint32_t n = N; n >= 2; --n) {
            const T* prev = n == 2 ? X : powers + uint64_t(n - 3) * S;  // P_{n-1}
            for (uint32_t j = threadIdx.x; j < S; j += blockDim.x) {
                const uint32_t t = lv.level_of(j);
                const uint32_t w = j - lv.off[t];
                dPprev[j] = exp_adjoint_prev_coeff(dE, dPn, X, lv, n, t, w);
                if (t >= n) {
                    uint32_t letter;
                    const T term = exp_adjoint_level1_term(dE, dPn, prev, lv, n, t, w, &letter);
                    atomicAdd(&g[letter], term);
                }
            }
            __syncthreads();
            dPn = dPprev;
            dPprev = dPprev == dPa ? dPb : dPa;
        }
        for (uint32_t i = threadIdx.x; i < lv.dim; i += blockDim.x) {
            const T gi = g[i] + dE[i] + (dPn ? dPn[i] : T(0));
            if (i < uint32_t(pv.d)) o[uint64_t(step + 1) * pv.d + i] = gi - g_next[i];
            g_next[i] = gi;
        }
        __syncthreads();
    }
    for (uint32_t i = threadIdx.x; i < uint32_t(pv.d); i += blockDim.x) o[i] = -g_next[i];
}

constexpr uint64_t kScratchBudget = 1ull << 30;  // bytes of per-path working vectors held at once
constexpr uint64_t kCorrectionSharedBytes = 96 * 1024;  // working vectors of one path up to this size live in shared memory

template <typename T>
CorrectionArgs<T> make_args(const CorrectionView<T>& c, uint64_t data_dim) {
    return CorrectionArgs<T>{c.ptr, c.len, c.batch_stride, c.segment_stride, data_dim};
}

// ----- path transform --------------------------------------------------------------------------

// The transformed batch as one flat array: a thread takes VEC consecutive output values (they may
// run over the end of a point or of a path: the (path, point, channel) position is decoded once by
// division and then advanced with carries), gathers them and stores them with one vector store.  A
// path holds fewer than 2^32 values; `out` is aligned to VEC values.
template <typename T, int VEC>
__global__ void transform_path_kernel(const T* __restrict__ in, T* __restrict__ out, uint64_t total, uint32_t d,
                                      uint32_t L, uint32_t dim, uint32_t len, bool time_aug, bool lead_lag, T dt) {
    const uint32_t per = len * dim;
    const uint64_t stride = uint64_t(gridDim.x) * blockDim.x * VEC;
    // (path, offset in the path) of the first value: one 64-bit division, then advanced by the
    // (constant) grid stride with a carry
    const uint64_t stride_b = stride / per;
    const uint32_t stride_r = static_cast<uint32_t>(stride - stride_b * per);
    uint64_t e0 = (uint64_t(blockIdx.x) * blockDim.x + threadIdx.x) * VEC;
    uint64_t b0 = e0 / per;
    uint32_t r0 = static_cast<uint32_t>(e0 - b0 * per);
    for (; e0 < total; e0 += stride, b0 += stride_b, r0 += stride_r) {
        if (r0 >= per) {
            r0 -= per;
            ++b0;
        }
        uint32_t p = r0 / dim, ch = r0 - p * dim;
        const T* path = in + b0 * (uint64_t(L) * d);
        const uint32_t copied = lead_lag ? 2 * d : d;      // channels taken from the path; the rest is time
        // channel ch of point p reads path[lead + ch] (ch < d) or path[lag + ch] (d <= ch < 2d, lead-lag)
        uint32_t lead = lead_lag ? (p >> 1) * d : p * d;
        uint32_t lag = lead_lag ? ((p >> 1) + (p & 1)) * d - d : 0;
        T v[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            v[k] = T(0);
            if (e0 + k < total) {
                if (ch >= copied) v[k] = static_cast<T>(p) * dt;
                else v[k] = path[(ch < d ? lead : lag) + ch];
                if (++ch == dim) {
                    ch = 0;
                    if (++p == len) {
                        p = 0;
                        path += uint64_t(L) * d;
                    }
                    lead = lead_lag ? (p >> 1) * d : p * d;
                    lag = lead_lag ? ((p >> 1) + (p & 1)) * d - d : 0;
                }
            }
        }
        if (e0 + VEC <= total) {
            if constexpr (VEC == 4) {
                if constexpr (sizeof(T) == 4) *reinterpret_cast<float4*>(out + e0) = make_float4(v[0], v[1], v[2], v[3]);
                else {
                    *reinterpret_cast<double2*>(out + e0) = make_double2(v[0], v[1]);
                    *reinterpret_cast<double2*>(out + e0 + 2) = make_double2(v[2], v[3]);
                }
            } else {
                out[e0] = v[0];
            }
        } else {
#pragma unroll
            for (int k = 0; k < VEC; ++k)
                if (e0 + k < total) out[e0 + k] = v[k];
        }
    }
}

template <typename T>
__global__ void transform_path_backprop_kernel(const T* __restrict__ derivs, T* __restrict__ out, uint64_t batch,
                                               uint32_t d, uint32_t L, uint32_t dim, uint32_t len, bool lead_lag) {
    const uint32_t r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= L * d) return;
    const uint32_t k = r / d, j = r - k * d;
    for (uint64_t b = blockIdx.y; b < batch; b += gridDim.y) {
        const T* g = derivs + b * len * dim;
        T sum;
        if (lead_lag) {
            sum = g[(2 * k) * dim + j];
            sum += g[(2 * k) * dim + d + j];
            if (k + 1 < L) sum += g[(2 * k + 1) * dim + j];
            if (k >= 1) sum += g[(2 * k - 1) * dim + d + j];
        } else {
            sum = g[k * dim + j];
        }
        out[b * L * d + r] = sum;
    }
}

}  // namespace

void validate_correction(const void* correction, uint64_t correction_len, uint64_t dimension, uint64_t degree,
                         bool lead_lag) {
    if (correction == nullptr && correction_len != 0)
        throw std::invalid_argument("correction pointer is null but correction_len is nonzero");
    if (lead_lag && correction_len != 0) throw std::invalid_argument("correction cannot be used with lead_lag=true");
    if (correction_len == 0) return;
    if (degree < 2) throw std::invalid_argument("correction must be empty when degree < 2");
    uint64_t offset = 0, level_size = dimension;
    for (uint64_t level = 2; level <= degree; ++level) {
        if (level_size > correction_len) break;  // also keeps the product below from overflowing
        level_size *= dimension;
        offset += level_size;
        if (offset == correction_len) return;
        if (offset > correction_len) break;
    }
    throw std::invalid_argument("correction length must be a prefix of tensor levels 2..degree");
}

template <typename T>
void correction_forward_on_device(const T* path, T* out, const SigShape& s, T end_time, const CorrectionView<T>& c,
                                  cudaStream_t stream) {
    const Levels lv = checked_levels(s.dim, s.degree, "signature_cuda (correction)");
    const PathView<T> pv = make_path_view<T>(path, s.data_dim, s.data_len, s.time_aug, false, end_time);
    const uint64_t per_path = 6 * lv.total() * sizeof(T);
    // small signatures keep the working vectors of a path in shared memory (every phase of a segment
    // then waits on shared-memory instead of L2 round trips); larger ones use pooled global scratch
    const bool in_shared = per_path <= kCorrectionSharedBytes;
    // small signatures: every thread keeps the splits of its (at most four) coefficients in registers
    constexpr int kSplits = 5;
    if (in_shared && per_path <= 48 * 1024 && lv.total() <= 4 * kThreads && lv.degree >= 1 && lv.degree - 1 <= kSplits) {
        for (uint64_t b0 = 0; b0 < s.batch; b0 += 0x7fffffffull) {
            const uint64_t count = std::min<uint64_t>(0x7fffffffull, s.batch - b0);
            if (lv.total() <= 2 * kThreads)
                correction_forward_cached_kernel<T, 2, kSplits><<<static_cast<unsigned>(count), kThreads, per_path, stream>>>(
                    pv, make_args(c, s.data_dim), out, s.stride, s.scalar_term, lv, b0);
            else
                correction_forward_cached_kernel<T, 4, kSplits><<<static_cast<unsigned>(count), kThreads, per_path, stream>>>(
                    pv, make_args(c, s.data_dim), out, s.stride, s.scalar_term, lv, b0);
            check_launch("corrected signature kernel");
        }
        return;
    }
    if (in_shared && per_path > 48 * 1024)
        SIG_CUDA_CHECK(cudaFuncSetAttribute(correction_forward_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            int(per_path)));
    const uint64_t chunk = std::max<uint64_t>(1, std::min<uint64_t>(std::min<uint64_t>(s.batch, 0x7fffffffull),
                                                                   in_shared ? s.batch : kScratchBudget / std::max<uint64_t>(per_path, 1)));
    Scratch ws(in_shared ? 0 : chunk * per_path, stream);
    for (uint64_t b0 = 0; b0 < s.batch; b0 += chunk) {
        const uint64_t count = std::min(chunk, s.batch - b0);
        correction_forward_kernel<T><<<static_cast<unsigned>(count), kThreads, in_shared ? per_path : 0, stream>>>(
            pv, make_args(c, s.data_dim), out, s.stride, s.scalar_term, in_shared ? nullptr : ws.as<T>(), lv, b0);
        check_launch("corrected signature kernel");
    }
}

template <typename T>
void correction_backward_on_device(const T* path, T* out, const T* sig_derivs, const T* sig, const SigShape& s,
                                   T end_time, const CorrectionView<T>& c, cudaStream_t stream) {
    const Levels lv = checked_levels(s.dim, s.degree, "sig_backprop_cuda (correction)");
    const PathView<T> pv = make_path_view<T>(path, s.data_dim, s.data_len, s.time_aug, false, end_time);
    const size_t g_bytes = ((2 * s.dim + 3) & ~3ull) * sizeof(T);
    if (g_bytes > 48 * 1024) throw std::invalid_argument("sig_backprop_cuda (correction): dimension too large");
    const uint64_t per_path = backward_vectors(lv.degree) * lv.total() * sizeof(T);
    const bool in_shared = per_path + g_bytes <= kCorrectionSharedBytes;
    const size_t smem = g_bytes + (in_shared ? per_path : 0);
    if (smem > 48 * 1024)
        SIG_CUDA_CHECK(cudaFuncSetAttribute(correction_backward_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            int(smem)));
    const uint64_t chunk = std::max<uint64_t>(1, std::min<uint64_t>(std::min<uint64_t>(s.batch, 0x7fffffffull),
                                                                   in_shared ? s.batch : kScratchBudget / std::max<uint64_t>(per_path, 1)));
    Scratch ws(in_shared ? 0 : chunk * per_path, stream);
    for (uint64_t b0 = 0; b0 < s.batch; b0 += chunk) {
        const uint64_t count = std::min(chunk, s.batch - b0);
        correction_backward_kernel<T><<<static_cast<unsigned>(count), kThreads, smem, stream>>>(
            pv, make_args(c, s.data_dim), sig, sig_derivs, s.stride, s.scalar_term, out, in_shared ? nullptr : ws.as<T>(), lv,
            b0);
        check_launch("corrected signature backward kernel");
    }
}

template <typename T>
void linear_sig_entry(const T* displacement, T* out, uint64_t batch, uint64_t dimension, uint64_t degree,
                      bool scalar_term, const CallOptions& opt) {
    if (dimension == 0) throw std::invalid_argument("linear_sig_cuda received dimension 0");
    if (batch == 0) return;
    const SigShape s = make_shape(batch, dimension, 2, degree, false, false, scalar_term);
    if (s.stride == 0) return;
    if (!displacement || !out) throw std::invalid_argument("linear_sig_cuda received a null pointer");
    const Levels lv = checked_levels(dimension, degree, "linear_sig_cuda");
    const uint64_t shift = scalar_term ? 1 : 0;
    auto run = [&](const T* v, T* o, cudaStream_t st) {
        if (degree == 0) launch_fill<T>(o, batch * s.stride, T(1), st);
        else launch_linear_sig<T>(v, o + shift, s.stride, lv, batch, scalar_term, st);
    };
    int device = -1;
    if (all_on_device({displacement, out}, "linear_sig_cuda", &device)) {
        DeviceGuard guard(device);
        run(displacement, out, opt.stream);
        if (opt.synchronize) SIG_CUDA_CHECK(cudaStreamSynchronize(opt.stream));
        return;
    }
    run_staged({{displacement, nullptr, batch * dimension * sizeof(T)}, {nullptr, out, batch * s.stride * sizeof(T)}},
               opt.device, [&](const std::vector<void*>& d, cudaStream_t st) {
                   run(static_cast<const T*>(d[0]), static_cast<T*>(d[1]), st);
               });
}

template <typename T>
void sig_join_entry(const T* sig, const T* displacement, T* out, uint64_t batch, uint64_t dimension,
                    uint64_t degree, bool prepend, bool scalar_term, const CallOptions& opt) {
    if (dimension == 0) throw std::invalid_argument("sig_join_cuda received dimension 0");
    if (batch == 0) return;
    const SigShape s = make_shape(batch, dimension, 2, degree, false, false, scalar_term);
    if (s.stride == 0) return;
    if (!sig || !displacement || !out) throw std::invalid_argument("sig_join_cuda received a null pointer");
    const Levels lv = checked_levels(dimension, degree, "sig_join_cuda");
    const uint64_t shift = scalar_term ? 1 : 0;
    const uint64_t S = s.full_len - 1;
    auto run = [&](const T* a, const T* v, T* o, cudaStream_t st) {
        if (degree == 0) { launch_fill<T>(o, batch * s.stride, T(1), st); return; }
        // big batches: one pass, the segment's signature exp(v) is generated inside the product kernel
        if (launch_chen_product_streamed<T>(prepend ? nullptr : a + shift, s.stride, prepend ? a + shift : nullptr, s.stride,
                                            v, o + shift, s.stride, s, st, scalar_term))
            return;
        Scratch lin(batch * S * sizeof(T), st);
        launch_linear_sig<T>(v, lin.as<T>(), S, lv, batch, false, st);
        if (prepend) launch_chen_product<T>(lin.as<T>(), S, a + shift, s.stride, o + shift, s.stride, s, st, scalar_term);
        else launch_chen_product<T>(a + shift, s.stride, lin.as<T>(), S, o + shift, s.stride, s, st, scalar_term);
    };
    int device = -1;
    if (all_on_device({sig, displacement, out}, "sig_join_cuda", &device)) {
        DeviceGuard guard(device);
        run(sig, displacement, out, opt.stream);
        if (opt.synchronize) SIG_CUDA_CHECK(cudaStreamSynchronize(opt.stream));
        return;
    }
    const size_t nb = batch * s.stride * sizeof(T);
    run_staged({{sig, nullptr, nb}, {displacement, nullptr, batch * dimension * sizeof(T)}, {nullptr, out, nb}},
               opt.device, [&](const std::vector<void*>& d, cudaStream_t st) {
                   run(static_cast<const T*>(d[0]), static_cast<const T*>(d[1]), static_cast<T*>(d[2]), st);
               });
}

template <typename T>
void sig_join_backprop_entry(const T* d_out, T* d_sig, T* d_displacement, const T* sig, const T* displacement,
                             uint64_t batch, uint64_t dimension, uint64_t degree, bool prepend, bool scalar_term,
                             const CallOptions& opt) {
    if (dimension == 0) throw std::invalid_argument("sig_join_backprop_cuda received dimension 0");
    if (batch == 0) return;
    const SigShape s = make_shape(batch, dimension, 2, degree, false, false, scalar_term);
    if (!d_displacement || !displacement) throw std::invalid_argument("sig_join_backprop_cuda received a null pointer");
    if (s.stride != 0 && (!d_out || !d_sig || !sig))
        throw std::invalid_argument("sig_join_backprop_cuda received a null pointer");
    const Levels lv = checked_levels(dimension, degree, "sig_join_backprop_cuda");
    const uint64_t shift = scalar_term ? 1 : 0;
    const uint64_t S = s.full_len - 1;
    auto run = [&](const T* g, T* ds, T* dv, const T* a, const T* v, cudaStream_t st) {
        if (scalar_term) SIG_CUDA_CHECK(cudaMemsetAsync(ds, 0, batch * s.stride * sizeof(T), st));  // scalar slots
        if (degree == 0) {
            SIG_CUDA_CHECK(cudaMemsetAsync(dv, 0, batch * dimension * sizeof(T), st));
            return;
        }
        // big batches: one pass over the incoming gradient, exp(v) and its adjoint never leave the SM
        if (launch_chen_adjoints_streamed<T>(g + shift, s.stride, a + shift, s.stride, a + shift, s.stride, ds + shift,
                                             s.stride, ds + shift, s.stride, s, st, prepend ? 1 : 2, v, dv))
            return;
        Scratch tmp(2 * batch * S * sizeof(T), st);
        T* lin = tmp.as<T>();
        T* dlin = lin + batch * S;
        launch_linear_sig<T>(v, lin, S, lv, batch, false, st);
        if (prepend) {  // out = lin (x) sig
            launch_chen_left_adjoint<T>(g + shift, s.stride, a + shift, s.stride, dlin, S, s, st);
            launch_chen_right_adjoint<T>(g + shift, s.stride, lin, S, ds + shift, s.stride, s, st);
        } else {        // out = sig (x) lin
            launch_chen_left_adjoint<T>(g + shift, s.stride, lin, S, ds + shift, s.stride, s, st);
            launch_chen_right_adjoint<T>(g + shift, s.stride, a + shift, s.stride, dlin, S, s, st);
        }
        launch_linear_sig_adjoint<T>(v, lin, dlin, S, dv, lv, batch, st);
    };
    int device = -1;
    if (all_on_device({d_out, d_sig, d_displacement, sig, displacement}, "sig_join_backprop_cuda", &device)) {
        DeviceGuard guard(device);
        run(d_out, d_sig, d_displacement, sig, displacement, opt.stream);
        if (opt.synchronize) SIG_CUDA_CHECK(cudaStreamSynchronize(opt.stream));
        return;
    }
    const size_t nb = batch * s.stride * sizeof(T), vb = batch * dimension * sizeof(T);
    run_staged({{d_out, nullptr, nb}, {nullptr, d_sig, nb}, {nullptr, d_displacement, vb}, {sig, nullptr, nb},
                {displacement, nullptr, vb}},
               opt.device, [&](const std::vector<void*>& d, cudaStream_t st) {
                   run(static_cast<const T*>(d[0]), static_cast<T*>(d[1]), static_cast<T*>(d[2]),
                       static_cast<const T*>(d[3]), static_cast<const T*>(d[4]), st);
               });
}

template <typename T>
void transform_path_entry(const T* data_in, T* data_out, uint64_t batch, uint64_t dimension, uint64_t length,
                          bool time_aug, bool lead_lag, T end_time, const CallOptions& opt) {
    if (dimension == 0) throw std::invalid_argument("transform_path_cuda received path of dimension 0");
    if (batch == 0 || length == 0) return;
    if (!data_in || !data_out) throw std::invalid_argument("transform_path_cuda received a null pointer");
    const SigShape s = make_shape(batch, dimension, length, 1, time_aug, lead_lag, false);
    const T dt = s.len > 1 ? end_time / static_cast<T>(s.len - 1) : T(0);
    const uint64_t n_out = checked_mul(checked_mul(batch, s.len, "transformed path"), s.dim, "transformed path");
    if (s.len * s.dim >= (1ull << 32)) throw std::invalid_argument("transform_path_cuda: path too large");
    auto run = [&](const T* in, T* o, cudaStream_t st) {
        const uint64_t total = n_out;
        const bool wide = reinterpret_cast<uintptr_t>(o) % (4 * sizeof(T)) == 0;
        const uint64_t threads = (total + (wide ? 3 : 0)) / (wide ? 4 : 1);
        const int sms = device_context(current_device()).sm_count;
        const unsigned grid = static_cast<unsigned>(std::min<uint64_t>((threads + kThreads - 1) / kThreads, uint64_t(sms) * 32));
        if (wide)
            transform_path_kernel<T, 4><<<grid, kThreads, 0, st>>>(in, o, total, uint32_t(dimension), uint32_t(length),
                                                                   uint32_t(s.dim), uint32_t(s.len), time_aug, lead_lag, dt);
        else
            transform_path_kernel<T, 1><<<grid, kThreads, 0, st>>>(in, o, total, uint32_t(dimension), uint32_t(length),
                                                                   uint32_t(s.dim), uint32_t(s.len), time_aug, lead_lag, dt);
        check_launch("transform_path kernel");
    };
    int device = -1;
    if (all_on_device({data_in, data_out}, "transform_path_cuda", &device)) {
        DeviceGuard guard(device);
        run(data_in, data_out, opt.stream);
        if (opt.synchronize) SIG_CUDA_CHECK(cudaStreamSynchronize(opt.stream));
        return;
    }
    run_staged({{data_in, nullptr, batch * length * dimension * sizeof(T)}, {nullptr, data_out, n_out * sizeof(T)}},
               opt.device, [&](const std::vector<void*>& d, cudaStream_t st) {
                   run(static_cast<const T*>(d[0]), static_cast<T*>(d[1]), st);
               });
}

template <typename T>
void transform_path_backprop_entry(const T* derivs, T* data_out, uint64_t batch, uint64_t dimension, uint64_t length,
                                   bool time_aug, bool lead_lag, T, const CallOptions& opt) {
    if (dimension == 0) throw std::invalid_argument("transform_path_backprop_cuda received path of dimension 0");
    if (batch == 0 || length == 0) return;
    if (!derivs || !data_out) throw std::invalid_argument("transform_path_backprop_cuda received a null pointer");
    const SigShape s = make_shape(batch, dimension, length, 1, time_aug, lead_lag, false);
    const uint64_t n_in = checked_mul(checked_mul(batch, s.len, "transformed path"), s.dim, "transformed path");
    const uint64_t n_out = batch * length * dimension;
    if (s.len * s.dim >= (1ull << 32)) throw std::invalid_argument("transform_path_backprop_cuda: path too large");
    auto run = [&](const T* g, T* o, cudaStream_t st) {
        const dim3 grid = batched_grid(length * dimension, batch, kThreads);
        transform_path_backprop_kernel<T><<<grid, kThreads, 0, st>>>(g, o, batch, uint32_t(dimension), uint32_t(length),
                                                                     uint32_t(s.dim), uint32_t(s.len), lead_lag);
        check_launch("transform_path_backprop kernel");
    };
    int device = -1;
    if (all_on_device({derivs, data_out}, "transform_path_backprop_cuda", &device)) {
        DeviceGuard guard(device);
        run(derivs, data_out, opt.stream);
        if (opt.synchronize) SIG_CUDA_CHECK(cudaStreamSynchronize(opt.stream));
        return;
    }
    run_staged({{derivs, nullptr, n_in * sizeof(T)}, {nullptr, data_out, n_out * sizeof(T)}}, opt.device,
               [&](const std::vector<void*>& d, cudaStream_t st) {
                   run(static_cast<const T*>(d[0]), static_cast<T*>(d[1]), st);
               });
}

#define INSTANTIATE(T)                                                                                              \
    template void correction_forward_on_device<T>(const T*, T*, const SigShape&, T, const CorrectionView<T>&,       \
                                                  cudaStream_t);                                                    \
    template void correction_backward_on_device<T>(const T*, T*, const T*, const T*, const SigShape&, T,            \
                                                   const CorrectionView<T>&, cudaStream_t);                         \
    template void linear_sig_entry<T>(const T*, T*, uint64_t, uint64_t, uint64_t, bool, const CallOptions&);        \
    template void sig_join_entry<T>(const T*, const T*, T*, uint64_t, uint64_t, uint64_t, bool, bool,               \
                                    const CallOptions&);                                                            \
    template void sig_join_backprop_entry<T>(const T*, T*, T*, const T*, const T*, uint64_t, uint64_t, uint64_t,    \
                                             bool, bool, const CallOptions&);                                       \
    template void transform_path_entry<T>(const T*, T*, uint64_t, uint64_t, uint64_t, bool, bool, T,                \
                                          const CallOptions&);                                                      \
    template void transform_path_backprop_entry<T>(const T*, T*, uint64_t, uint64_t, uint64_t, bool, bool, T,       \
                                                   const CallOptions&);
INSTANTIATE(float)
INSTANTIATE(double)
#undef INSTANTIATE

}  // namespace sigb200
