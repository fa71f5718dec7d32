// Shape-generic signature kernels: any augmented dimension and degree.
//
// One CTA owns one path at a time and keeps the whole level structure in global
// memory (served from L1/L2); each Horner level is a data-parallel phase over the
// words of that level, separated by __syncthreads().  These kernels are the
// fallback behind the register-tile kernels (sig_tile.cuh), which cover the
// shapes that matter for throughput; here the goal is exact agreement with the
// reference's arithmetic for every shape.
//
// What is computed (reference: siglib/cpsig/cp_signature.h:426-500 forward,
// :549-603 in-place step, :1098-1203 reverse sweep; CUDA host dispatch being
// replaced: siglib/cusig/cu_signature.cu:2467-2657 and :2897-3488):
//   forward step, for target level T = N..2, with increment z:
//       W_1 = z / T;  W_{l+1} = ((W_l + S_l) / (T - l)) (x) z  for l = 1..T-2;
//       S_T += (W_{T-1} + S_{T-1}) (x) z;          finally S_1 += z.
//   backward step: rewind S with -z, then pull the adjoint through the same
//   recurrence level by level, accumulating the increment gradient g.
#include <cstdio>

#include "increments.cuh"
#include "kernels.h"
#include "runtime.h"

namespace sigb200 {

namespace {

constexpr int kGenericThreads = 256;

template <typename T>
__device__ __forceinline__ T fma_t(T a, T b, T c);
template <>
__device__ __forceinline__ float fma_t<float>(float a, float b, float c) { return fmaf(a, b, c); }
template <>
__device__ __forceinline__ double fma_t<double>(double a, double b, double c) { return fma(a, b, c); }

// ---- closed forms -----------------------------------------------------------

// mode 0: fill with zeros (+1 in the scalar slot); mode 1: degree-1 endpoint
// difference; mode 2: augmented dimension 1, level k = dx^k / k!.
template <typename T>
__global__ void trivial_forward_kernel(PathView<T> pv, T* out, uint64_t total, uint32_t stride, int degree,
                                       bool scalar, int mode) {
    const uint64_t idx = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const uint64_t b = idx / stride;
    const uint32_t i = static_cast<uint32_t>(idx - b * stride);
    if (scalar && i == 0) { out[idx] = T(1); return; }
    if (mode == 0) { out[idx] = T(0); return; }
    const T* x = pv.base + b * pv.path_stride;
    const int k = static_cast<int>(i) + (scalar ? 0 : 1);  // position in the scalar-term layout
    if (mode == 1) {
        const int c = k - 1;
        T v;
        if (c < pv.d) v = x[(pv.L - 1) * pv.d + c] - x[c];
        else if (pv.lead_lag && c < 2 * pv.d) v = x[(pv.L - 1) * pv.d + (c - pv.d)] - x[c - pv.d];
        else v = pv.dt * T(pv.steps);
        out[idx] = v;
        return;
    }
    // mode 2: raw dimension 1, no flags (siglib/cpsig/cp_signature.h:770-785)
    const T inc = x[pv.L - 1] - x[0];
    T v = T(1);
    for (int level = 1; level <= k; ++level) v *= inc / T(level);
    out[idx] = v;
}

// Degree-1 backward in closed form: S_1 is the total increment, so only the end points get a
// gradient (+-dS_1; with lead-lag the lag and lead halves add up, the time channel has none).
template <typename T>
__global__ void degree_one_backward_kernel(PathView<T> pv, T* out, const T* derivs, uint64_t total, uint32_t stride,
                                           bool scalar) {
    const uint64_t idx = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const uint64_t row = idx / uint32_t(pv.d);  // b * L + t
    const int c = int(idx - row * uint32_t(pv.d));
    const uint64_t b = row / uint32_t(pv.L);
    const int t = int(row - b * uint32_t(pv.L));
    T v = T(0);
    if (t == 0 || t == pv.L - 1) {
        const T* ds = derivs + b * stride + (scalar ? 1 : 0);
        T g = ds[c];
        if (pv.lead_lag) g += ds[pv.d + c];
        v = t == 0 ? -g : g;
    }
    out[idx] = v;
}

// ---- block-cooperative Horner step on a scalar-term layout signature --------

template <typename T>
__device__ void horner_step_block(T* S, const T* zs, const T* rcp, int D, int N, const uint32_t* li,
                                  T* wa, T* wb) {
    const unsigned tid = threadIdx.x, nt = blockDim.x;
    for (int target = N; target >= 2; --target) {
        const T r_target = rcp[target];
        const T* cur = nullptr;
        T* nxt = wa;
        for (int l = 1; l <= target - 2; ++l) {
            const T scale = rcp[target - l];
            const uint32_t out_size = (li[l + 1] - li[l]) * uint32_t(D);
            const T* s_l = S + li[l];
            for (uint32_t idx = tid; idx < out_size; idx += nt) {
                const uint32_t w = idx / uint32_t(D);
                const uint32_t c = idx - w * uint32_t(D);
                const T wv = (l == 1) ? zs[w] * r_target : cur[w];
                const T v = (wv + s_l[w]) * scale;
                nxt[idx] = zs[c] * v;
            }
            __syncthreads();
            cur = nxt;
            nxt = (nxt == wa) ? wb : wa;
        }
        const uint32_t out_size = li[target + 1] - li[target];
        const T* s_l = S + li[target - 1];
        T* s_t = S + li[target];
        for (uint32_t idx = tid; idx < out_size; idx += nt) {
            const uint32_t w = idx / uint32_t(D);
            const uint32_t c = idx - w * uint32_t(D);
            const T wv = (target == 2) ? zs[w] * r_target : cur[w];
            s_t[idx] = fma_t(zs[c], wv + s_l[w], s_t[idx]);
        }
        __syncthreads();
    }
    for (uint32_t c = tid; c < uint32_t(D); c += nt) S[1 + c] = fma_t(zs[c], T(1), S[1 + c]);
    __syncthreads();
}

template <typename T>
__global__ void __launch_bounds__(kGenericThreads)
generic_forward_kernel(PathView<T> pv, T* out, uint64_t batch, int N, uint32_t stride, bool scalar,
                       T* scratch, uint32_t work_elems, LevelIndex lev) {
    extern __shared__ unsigned char smem_raw[];
    T* zs = reinterpret_cast<T*>(smem_raw);
    T* rcp = zs + pv.dim;
    __shared__ uint32_t li[kMaxDegree + 2];
    const unsigned tid = threadIdx.x, nt = blockDim.x;
    const int D = pv.dim;
    for (unsigned i = tid; i < unsigned(N + 2); i += nt) li[i] = lev.li[i];
    for (unsigned i = tid; i <= unsigned(N); i += nt) rcp[i] = i ? T(1) / T(i) : T(0);
    T* wa = scratch + uint64_t(blockIdx.x) * 2 * work_elems;
    T* wb = wa + work_elems;
    __syncthreads();

    for (uint64_t b = blockIdx.x; b < batch; b += gridDim.x) {
        const T* x = pv.base + b * pv.path_stride;
        T* S = out + b * stride - (scalar ? 0 : 1);
        // first segment (siglib/cpsig/cp_signature.h:365-389)
        for (unsigned c = tid; c < unsigned(D); c += nt) {
            const T z = pv.increment(x, 0, c);
            zs[c] = z;
            S[1 + c] = z;
        }
        if (scalar && tid == 0) S[0] = T(1);
        __syncthreads();
        for (int k = 2; k <= N; ++k) {
            const uint32_t size = li[k + 1] - li[k];
            const T r = rcp[k];
            for (uint32_t idx = tid; idx < size; idx += nt) {
                const uint32_t w = idx / uint32_t(D);
                const uint32_t c = idx - w * uint32_t(D);
                S[li[k] + idx] = zs[c] * (S[li[k - 1] + w] * r);
            }
            __syncthreads();
        }
        for (int j = 1; j < pv.steps; ++j) {
            for (unsigned c = tid; c < unsigned(D); c += nt) zs[c] = pv.increment(x, j, c);
            __syncthreads();
            horner_step_block(S, zs, rcp, D, N, li, wa, wb);
        }
        __syncthreads();
    }
}

// column sums gpart[j] = sum_i rows[i*D + j] * val[i]
template <typename T>
__device__ void column_sums_block(const T* rows, const T* val, uint32_t size, int D, T* gpart) {
    const unsigned tid = threadIdx.x, nt = blockDim.x;
    if (unsigned(D) >= nt) {
        for (uint32_t j = tid; j < uint32_t(D); j += nt) {
            T acc = T(0);
            for (uint32_t i = 0; i < size; ++i) acc = fma_t(rows[uint64_t(i) * D + j], val[i], acc);
            gpart[j] = acc;
        }
    } else {
        const unsigned groups = nt / unsigned(D);
        if (tid < groups * unsigned(D)) {
            const unsigned grp = tid / unsigned(D), j = tid - grp * unsigned(D);
            if (grp < size) {
                T acc = T(0);
                for (uint32_t i = grp; i < size; i += groups) acc = fma_t(rows[uint64_t(i) * D + j], val[i], acc);
                atomicAdd(&gpart[j], acc);
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(kGenericThreads)
generic_backward_kernel(PathView<T> pv, T* out, const T* sig_derivs, const T* sig, uint64_t batch, int N,
                        uint32_t stride, bool scalar, T* scratch, uint64_t scratch_per_cta,
                        uint32_t work_elems, LevelIndex lev) {
    extern __shared__ unsigned char smem_raw[];
    const int D = pv.dim;
    T* zs = reinterpret_cast<T*>(smem_raw);
    T* g = zs + D;
    T* gpart = g + D;
    T* rcp = gpart + D;
    __shared__ uint32_t li[kMaxDegree + 2];
    const unsigned tid = threadIdx.x, nt = blockDim.x;
    for (unsigned i = tid; i < unsigned(N + 2); i += nt) li[i] = lev.li[i];
    for (unsigned i = tid; i <= unsigned(N); i += nt) rcp[i] = i ? T(1) / T(i) : T(0);
    __syncthreads();
    const uint32_t full_len = li[N + 1];
    T* Sc = scratch + uint64_t(blockIdx.x) * scratch_per_cta;
    T* dSc = Sc + full_len;
    T* HS = dSc + full_len;  // work levels 0..N-1, indexed with li[]
    T* hd0 = HS + li[N];
    T* hd1 = hd0 + work_elems;
    const int dd = pv.d;

    for (uint64_t b = blockIdx.x; b < batch; b += gridDim.x) {
        const T* x = pv.base + b * pv.path_stride;
        T* outb = out + b * pv.path_stride;
        const T* sig_b = sig + b * stride - (scalar ? 0 : 1);
        const T* der_b = sig_derivs + b * stride - (scalar ? 0 : 1);
        for (uint32_t i = tid; i < full_len; i += nt) {
            Sc[i] = i ? sig_b[i] : T(1);
            dSc[i] = i ? der_b[i] : T(0);
        }
        for (uint64_t i = tid; i < pv.path_stride; i += nt) outb[i] = T(0);
        __syncthreads();

        int pos = pv.L - 1;
        bool parity = false;
        for (int j = pv.steps - 1; j >= 0; --j) {
            for (unsigned c = tid; c < unsigned(D); c += nt) zs[c] = -pv.increment(x, j, c);
            __syncthreads();
            horner_step_block(Sc, zs, rcp, D, N, li, hd0, hd1);  // rewind to the state before step j
            for (unsigned c = tid; c < unsigned(D); c += nt) {
                zs[c] = -zs[c];
                g[c] = dSc[1 + c];
            }
            __syncthreads();

            for (int target = 2; target <= N; ++target) {
                const T r_target = rcp[target];
                for (unsigned c = tid; c < unsigned(D); c += nt) HS[1 + c] = zs[c] * r_target;
                __syncthreads();
                for (int level = 1; level + 1 < target; ++level) {
                    const T scale = rcp[target - level];
                    const uint32_t out_size = (li[level + 1] - li[level]) * uint32_t(D);
                    for (uint32_t idx = tid; idx < out_size; idx += nt) {
                        const uint32_t w = idx / uint32_t(D);
                        const uint32_t c = idx - w * uint32_t(D);
                        const T value = (HS[li[level] + w] + Sc[li[level] + w]) * scale;
                        HS[li[level + 1] + idx] = zs[c] * value;
                    }
                    __syncthreads();
                }
                const T* incoming = dSc + li[target];
                T* hd_cur = hd0;
                for (int level = target - 1; level > 0; --level) {
                    const T scale = rcp[target - level];
                    const uint32_t size = li[level + 1] - li[level];
                    for (unsigned c = tid; c < unsigned(D); c += nt) gpart[c] = T(0);
                    for (uint32_t i = tid; i < size; i += nt) {
                        const T value = (HS[li[level] + i] + Sc[li[level] + i]) * scale;
                        const T* row = incoming + uint64_t(i) * D;
                        T reduced = T(0);
                        for (int c = 0; c < D; ++c) reduced = fma_t(row[c], zs[c], reduced);
                        reduced *= scale;
                        hd_cur[i] = reduced;
                        dSc[li[level] + i] += reduced;
                        HS[li[level] + i] = value;
                    }
                    __syncthreads();
                    column_sums_block(incoming, HS + li[level], size, D, gpart);
                    __syncthreads();
                    for (unsigned c = tid; c < unsigned(D); c += nt) g[c] += gpart[c];
                    incoming = hd_cur;
                    hd_cur = (hd_cur == hd0) ? hd1 : hd0;
                    __syncthreads();
                }
                for (unsigned c = tid; c < unsigned(D); c += nt) g[c] += incoming[c] * r_target;
                __syncthreads();
            }

            const int half = (pv.lead_lag && parity) ? dd : 0;
            for (int c = tid; c < dd; c += nt) {
                const T s = g[c + half];
                outb[pos * dd + c] += s;
                outb[(pos - 1) * dd + c] -= s;
            }
            if (j > 0) {
                if (!pv.lead_lag || parity) pos -= 1;
                parity = !parity;
            }
            __syncthreads();
        }
    }
}

// One round of the pairwise joining of segment signatures with Chen's identity
// (reference arithmetic: siglib/cpsig/cp_sig_combine.h:34-66; here out of place, one thread
// per output coefficient, so all levels and all pairs of the batch run in one launch).
// in: (batch, n, slen) scalar-free; out: (batch, ceil(n/2), .): out[b][j] = in[b][2j] (x) in[b][2j+1]
// (a last unpaired segment is copied).
//   C_m[w] = A_m[w] + sum_{i=m-1..1} A_i[w_1..w_i] * B_{m-i}[w_{i+1}..w_m] + B_m[w]
// Exact division of a 32-bit index by the (runtime constant) dimension with a multiply and two
// shifts instead of the ~20-instruction integer division (Granlund-Montgomery, round-up variant).
struct FastDiv {
    uint32_t divisor, magic, shift1, shift2;
    __device__ __forceinline__ uint32_t div(uint32_t x) const {
        if (divisor == 1) return x;
        const uint32_t t = __umulhi(magic, x);
        return (t + ((x - t) >> shift1)) >> shift2;
    }
};

FastDiv make_fast_div(uint32_t d) {
    FastDiv f{d, 0, 0, 0};
    if (d <= 1) return f;
    uint32_t l = 0;
    while ((1ull << l) < d) ++l;  // ceil(log2 d)
    f.magic = static_cast<uint32_t>(((1ull << 32) * ((1ull << l) - d)) / d + 1);
    f.shift1 = 1;
    f.shift2 = l - 1;
    return f;
}

// One thread per output coefficient j of the scalar-free layout: j = p d + ch with p the slot of the
// prefix u (length m-1, all levels m = 1..N; level m starts at d li[m-1]) and ch the last letter, so
// consecutive threads read and write consecutive addresses.
template <typename T>
__device__ __forceinline__ T chen_product_coeff(const T* __restrict__ a, const T* __restrict__ bb, uint32_t j,
                                                const FastDiv& fd, int N, const uint32_t* li) {
    // a, bb address position 0 of the scalar-term layout
    const uint32_t d = fd.divisor;
    const uint32_t p = fd.div(j), ch = j - p * d;
    int m = 1;
    while (m < N && p >= li[m]) ++m;       // li[m-1] <= p < li[m]
    const uint32_t q = p - li[m - 1];      // index of the prefix inside level m-1
    T acc = a[1 + j];
    uint32_t left = q, pw = 1;             // left = q / d^(m-1-i), pw = d^(m-1-i)
    for (int i = m - 1; i >= 1; --i) {
        acc = fma_t(a[li[i] + left], bb[li[m - i] + (q - left * pw) * d + ch], acc);
        left = fd.div(left);
        pw *= d;
    }
    return acc + bb[1 + j];
}

template <typename T>
__global__ void __launch_bounds__(kGenericThreads)
chen_pair_kernel(const T* __restrict__ in, int n, T* __restrict__ out, uint64_t out_stride, bool out_scalar,
                 uint64_t pairs_total, uint32_t slen, FastDiv fd, int N, LevelIndex lev) {
    __shared__ uint32_t li[kMaxDegree + 2];
    for (unsigned i = threadIdx.x; i < unsigned(N + 2); i += blockDim.x) li[i] = lev.li[i];
    __syncthreads();
    const uint32_t j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= slen) return;
    const int n2 = (n + 1) / 2;
    for (uint64_t vb = blockIdx.y; vb < pairs_total; vb += gridDim.y) {  // vb = b * n2 + pair
        const uint64_t b = vb / uint64_t(n2);
        const int pair = int(vb - b * uint64_t(n2));
        const T* a = in + (b * uint64_t(n) + uint64_t(2 * pair)) * slen - 1;
        T* c = out + vb * out_stride - (out_scalar ? 0 : 1);
        c[1 + j] = 2 * pair + 1 < n ? chen_product_coeff<T>(a, a + slen, j, fd, N, li) : a[1 + j];
        if (out_scalar && j == 0) c[0] = T(1);  // the slot before level 1 is the scalar term
    }
}

// C = A (x) B for batches of scalar-free signatures with independent batch strides
// (the pointers address the first level-1 coefficient of path 0).
template <typename T>
__global__ void __launch_bounds__(kGenericThreads)
chen_product_kernel(const T* __restrict__ A, uint64_t a_stride, const T* __restrict__ B, uint64_t b_stride,
                    T* __restrict__ C, uint64_t c_stride, bool c_scalar, uint64_t batch, uint32_t slen, FastDiv fd,
                    int N, LevelIndex lev) {
    __shared__ uint32_t li[kMaxDegree + 2];
    for (unsigned i = threadIdx.x; i < unsigned(N + 2); i += blockDim.x) li[i] = lev.li[i];
    __syncthreads();
    const uint32_t j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= slen) return;
    for (uint64_t b = blockIdx.y; b < batch; b += gridDim.y) {
        T* c = C + b * c_stride - 1;
        c[1 + j] = chen_product_coeff<T>(A + b * a_stride - 1, B + b * b_stride - 1, j, fd, N, li);
        if (c_scalar && j == 0) c[0] = T(1);
    }
}

// Adjoint of the left factor of a Chen product: for S = X (x) A and a loss adjoint dS,
//   dX[u] = dS[u] + sum_{m >= 1, |u| + m <= N} sum_{|v| = m} dS[u v] * A[v].
// One thread per coefficient of dX.
template <typename T>
__global__ void __launch_bounds__(kGenericThreads)
chen_left_adjoint_kernel(const T* __restrict__ dS, uint64_t ds_stride, const T* __restrict__ A, uint64_t a_stride,
                         T* __restrict__ dX, uint64_t dx_stride, uint64_t total, uint32_t slen, int N,
                         LevelIndex lev) {
    __shared__ uint32_t li[kMaxDegree + 2];
    for (unsigned i = threadIdx.x; i < unsigned(N + 2); i += blockDim.x) li[i] = lev.li[i];
    __syncthreads();
    const uint64_t gid = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (gid >= total) return;
    const uint64_t b = gid / slen;
    const uint32_t pos = uint32_t(gid - b * slen) + 1;
    const T* ds = dS + b * ds_stride - 1;
    const T* a = A + b * a_stride - 1;
    int n = 1;
    while (n < N && pos >= li[n + 1]) ++n;
    const uint32_t idx = pos - li[n];
    T acc = ds[pos];
    for (int m = 1; n + m <= N; ++m) {
        const uint32_t pw = li[m + 1] - li[m];  // d^m
        const T* row = ds + li[n + m] + uint64_t(idx) * pw;
        const T* av = a + li[m];
        for (uint32_t v = 0; v < pw; ++v) acc = fma_t(row[v], av[v], acc);
    }
    (dX + b * dx_stride - 1)[pos] = acc;
}

// Adjoint of the right factor of a Chen product: for S = A (x) Y and a loss adjoint dS,
//   dY[v] = dS[v] + sum_{n >= 1, n + |v| <= N} sum_{|u| = n} dS[u v] * A[u].
// One thread per coefficient of dY.
template <typename T>
__global__ void __launch_bounds__(kGenericThreads)
chen_right_adjoint_kernel(const T* __restrict__ dS, uint64_t ds_stride, const T* __restrict__ A, uint64_t a_stride,
                          T* __restrict__ dY, uint64_t dy_stride, uint64_t total, uint32_t slen, int N,
                          LevelIndex lev) {
    __shared__ uint32_t li[kMaxDegree + 2];
    for (unsigned i = threadIdx.x; i < unsigned(N + 2); i += blockDim.x) li[i] = lev.li[i];
    __syncthreads();
    const uint64_t gid = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (gid >= total) return;
    const uint64_t b = gid / slen;
    const uint32_t pos = uint32_t(gid - b * slen) + 1;
    const T* ds = dS + b * ds_stride - 1;
    const T* a = A + b * a_stride - 1;
    int m = 1;
    while (m < N && pos >= li[m + 1]) ++m;
    const uint32_t idx = pos - li[m];
    const uint32_t pw = li[m + 1] - li[m];  // d^m
    T acc = ds[pos];
    for (int n = 1; n + m <= N; ++n) {
        const uint32_t count = li[n + 1] - li[n];  // d^n
        const T* col = ds + li[n + m] + idx;
        const T* av = a + li[n];
        for (uint32_t u = 0; u < count; ++u) acc = fma_t(col[uint64_t(u) * pw], av[u], acc);
    }
    (dY + b * dy_stride - 1)[pos] = acc;
}

// Gradient with respect to the points from the gradient with respect to the increments
// z_t = x_{t+1} - x_t:  dx_t = dz_{t-1} - dz_t.  Inside one path the flat index i = t * d + c of a
// point coordinate is also the index of dz_t[c], so dx[i] = dz[i - d] - dz[i] with the two ends cut
// off: no division.  Paths along grid.y.
template <typename T>
__global__ void increment_to_point_grad_kernel(const T* __restrict__ g, T* __restrict__ out, uint64_t batch,
                                               uint64_t per_path, uint64_t per_path_incr, uint32_t d) {
    const uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= per_path) return;
    for (uint64_t b = blockIdx.y; b < batch; b += gridDim.y) {
        const T* gb = g + b * per_path_incr;
        T v = T(0);
        if (i >= d) v = gb[i - d];
        if (i < per_path_incr) v -= gb[i];
        out[b * per_path + i] = v;
    }
}

template <typename T>
__global__ void fill_kernel(T* dst, uint64_t n, T value) {
    for (uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += uint64_t(gridDim.x) * blockDim.x)
        dst[i] = value;
}

template <typename T>
__global__ void nonfinite_scan_kernel(const T* __restrict__ data, uint64_t n, int* flag) {
    bool bad = false;
    for (uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += uint64_t(gridDim.x) * blockDim.x) {
        const T v = data[i];
        bad |= !(fabs(double(v)) <= 1.7976931348623157e308);
    }
    if (__syncthreads_or(bad) && threadIdx.x == 0) *flag = 1;
}

unsigned grid_1d(uint64_t total, unsigned block) {
    const uint64_t blocks = (total + block - 1) / block;
    if (blocks > 0x7fffffffull) throw std::out_of_range("launch grid too large");
    return static_cast<unsigned>(blocks ? blocks : 1);
}

uint32_t work_elems_of(const SigShape& s) {
    // size of level N-1 (largest Horner work level); at least 1 so pointers stay valid
    const uint64_t w = s.degree >= 2 ? ipow(s.dim, s.degree - 1) : 1;
    return static_cast<uint32_t>(w ? w : 1);
}

void check_generic_limits(const SigShape& s) {
    if (s.degree > kMaxDegree) throw std::invalid_argument("signature degree must be <= 64 on CUDA");
    if (s.full_len >= (1ull << 31) || s.dim >= (1ull << 24) || s.len >= (1ull << 30))
        throw std::invalid_argument("signature too large for the CUDA kernels (2^31 coefficients per path)");
}

}  // namespace

LevelIndex make_level_index(uint64_t dim, uint64_t degree) {
    LevelIndex l{};
    uint64_t v = 0;
    for (uint64_t k = 0; k <= degree + 1 && k < kMaxDegree + 2; ++k) {
        l.li[k] = static_cast<uint32_t>(v);
        v = v * dim + 1;
    }
    return l;
}

uint64_t generic_forward_scratch_elems(const SigShape& s) { return 2ull * work_elems_of(s); }

uint64_t generic_backward_scratch_elems(const SigShape& s) {
    const LevelIndex l = make_level_index(s.dim, s.degree);
    return 2ull * s.full_len + l.li[s.degree] + 2ull * work_elems_of(s);
}

template <typename T>
void launch_trivial_forward(const T* path, T* out, const SigShape& s, T end_time, cudaStream_t stream) {
    const uint64_t total = checked_mul(s.batch, s.stride, "signature output");
    if (total == 0) return;
    if (s.stride >= (1ull << 32)) throw std::invalid_argument("signature too large for the CUDA kernels");
    int mode;
    if (s.len <= 1 || s.degree == 0) mode = 0;
    else if (s.dim == 1) mode = 2;
    else mode = 1;  // degree == 1
    const PathView<T> pv = make_path_view(path, s.data_dim, s.data_len, s.time_aug, s.lead_lag, end_time);
    trivial_forward_kernel<T><<<grid_1d(total, 128), 128, 0, stream>>>(
        pv, out, total, static_cast<uint32_t>(s.stride), static_cast<int>(s.degree), s.scalar_term, mode);
    SIG_CUDA_CHECK(cudaGetLastError());
    count_launch();
}

template <typename T>
void launch_degree_one_backward(const T* path, T* out, const T* sig_derivs, const SigShape& s, T end_time,
                                cudaStream_t stream) {
    const uint64_t total = checked_mul(s.batch, checked_mul(s.data_len, s.data_dim, "path gradient"), "path gradient");
    if (total == 0) return;
    if (s.data_dim >= (1ull << 31) || s.data_len >= (1ull << 31) || s.stride >= (1ull << 32))
        throw std::invalid_argument("path too large for the CUDA kernels");
    const PathView<T> pv = make_path_view(path, s.data_dim, s.data_len, s.time_aug, s.lead_lag, end_time);
    degree_one_backward_kernel<T><<<grid_1d(total, 256), 256, 0, stream>>>(
        pv, out, sig_derivs, total, static_cast<uint32_t>(s.stride), s.scalar_term);
    SIG_CUDA_CHECK(cudaGetLastError());
    count_launch();
}

void check_generic_smem(size_t bytes) {
    if (bytes > 200 * 1024)
        throw std::invalid_argument("path dimension too large for the CUDA kernels at this degree (the increment "
                                    "vector of one step must fit in shared memory)");
}

template <typename T>
void launch_generic_forward(const T* path, T* out, const SigShape& s, T end_time, T* scratch, unsigned ctas,
                            cudaStream_t stream) {
    check_generic_limits(s);
    check_generic_smem((s.dim + s.degree + 1) * sizeof(T));
    const PathView<T> pv = make_path_view(path, s.data_dim, s.data_len, s.time_aug, s.lead_lag, end_time);
    const size_t smem = (s.dim + s.degree + 1) * sizeof(T);
    if (smem > 48 * 1024)
        SIG_CUDA_CHECK(cudaFuncSetAttribute(generic_forward_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            static_cast<int>(smem)));
    generic_forward_kernel<T><<<ctas, kGenericThreads, smem, stream>>>(
        pv, out, s.batch, static_cast<int>(s.degree), static_cast<uint32_t>(s.stride), s.scalar_term, scratch,
        work_elems_of(s), make_level_index(s.dim, s.degree));
    SIG_CUDA_CHECK(cudaGetLastError());
    count_launch();
}

template <typename T>
void launch_generic_backward(const T* path, T* out, const T* sig_derivs, const T* sig, const SigShape& s,
                             T end_time, T* scratch, unsigned ctas, cudaStream_t stream) {
    check_generic_limits(s);
    check_generic_smem((3 * s.dim + s.degree + 1) * sizeof(T));
    const PathView<T> pv = make_path_view(path, s.data_dim, s.data_len, s.time_aug, s.lead_lag, end_time);
    const size_t smem = (3 * s.dim + s.degree + 1) * sizeof(T);
    if (smem > 48 * 1024)
        SIG_CUDA_CHECK(cudaFuncSetAttribute(generic_backward_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            static_cast<int>(smem)));
    generic_backward_kernel<T><<<ctas, kGenericThreads, smem, stream>>>(
        pv, out, sig_derivs, sig, s.batch, static_cast<int>(s.degree), static_cast<uint32_t>(s.stride),
        s.scalar_term, scratch, generic_backward_scratch_elems(s), work_elems_of(s),
        make_level_index(s.dim, s.degree));
    SIG_CUDA_CHECK(cudaGetLastError());
    count_launch();
}

// Grid of the product kernels: x over the coefficients of one signature, y over the batch, which the
// threads walk with stride gridDim.y.  Enough CTAs to fill the GPU many times over, but not one
// CTA per (coefficient block, signature): at a few hundred thousand tiny CTAs their launch cost dominates.
dim3 batch_walk_grid(uint32_t slen, uint64_t batch) {
    const unsigned gx = grid_1d(slen, kGenericThreads);
    const uint64_t target = 148ull * 64;
    const uint64_t gy = std::max<uint64_t>(1, std::min<uint64_t>(std::min<uint64_t>(batch, 65535), (target + gx - 1) / gx));
    return dim3(gx, static_cast<unsigned>(gy));
}

uint64_t chen_combine_tmp_elems(const SigShape& s, int nseg) {
    // two ping-pong buffers: ceil(nseg/2) and ceil(nseg/4) signatures per path
    return s.batch * (s.full_len - 1) * uint64_t((nseg + 1) / 2 + (nseg + 3) / 4);
}

template <typename T>
void launch_chen_combine(T* out, const T* seg, T* tmp, const SigShape& s, int nseg, cudaStream_t stream) {
    if (nseg <= 1 || s.batch == 0) return;
    check_generic_limits(s);
    if (launch_chen_chain<T>(out, seg, s, nseg, stream)) return;   // one launch, running product in shared memory
    const uint32_t slen = static_cast<uint32_t>(s.full_len - 1);
    const LevelIndex lev = make_level_index(s.dim, s.degree);
    T* buf[2] = {tmp, tmp + s.batch * slen * uint64_t((nseg + 1) / 2)};
    const T* cur = seg;
    int n = nseg, round = 0;
    while (n > 1) {
        const int n2 = (n + 1) / 2;
        const bool final = n2 == 1;
        T* dst = final ? out : buf[round & 1];
        const uint64_t pairs = checked_mul(s.batch, uint64_t(n2), "signature output");
        const dim3 grid = batch_walk_grid(slen, pairs);
        chen_pair_kernel<T><<<grid, kGenericThreads, 0, stream>>>(
            cur, n, dst, final ? s.stride : slen, final && s.scalar_term, pairs, slen,
            make_fast_div(static_cast<uint32_t>(s.dim)), static_cast<int>(s.degree), lev);
        SIG_CUDA_CHECK(cudaGetLastError());
        count_launch();
        cur = dst;
        n = n2;
        ++round;
    }
}

template <typename T>
void launch_chen_product(const T* A, uint64_t a_stride, const T* B, uint64_t b_stride, T* C, uint64_t c_stride,
                         const SigShape& s, cudaStream_t stream, bool write_scalar) {
    check_generic_limits(s);
    const uint32_t slen = static_cast<uint32_t>(s.full_len - 1);
    if (s.batch == 0 || slen == 0) return;
    // big batches: one CTA per signature, operands streamed once (sig_chen.cu)
    if (launch_chen_product_streamed<T>(A, a_stride, B, b_stride, nullptr, C, c_stride, s, stream, write_scalar)) return;
    const dim3 grid = batch_walk_grid(slen, s.batch);
    chen_product_kernel<T><<<grid, kGenericThreads, 0, stream>>>(
        A, a_stride, B, b_stride, C, c_stride, write_scalar, s.batch, slen, make_fast_div(static_cast<uint32_t>(s.dim)),
        static_cast<int>(s.degree), make_level_index(s.dim, s.degree));
    SIG_CUDA_CHECK(cudaGetLastError());
    count_launch();
}

template <typename T>
void launch_chen_left_adjoint(const T* dS, uint64_t ds_stride, const T* A, uint64_t a_stride, T* dX,
                              uint64_t dx_stride, const SigShape& s, cudaStream_t stream) {
    check_generic_limits(s);
    const uint32_t slen = static_cast<uint32_t>(s.full_len - 1);
    const uint64_t total = checked_mul(s.batch, slen, "signature output");
    if (total == 0) return;
    chen_left_adjoint_kernel<T><<<grid_1d(total, kGenericThreads), kGenericThreads, 0, stream>>>(
        dS, ds_stride, A, a_stride, dX, dx_stride, total, slen, static_cast<int>(s.degree),
        make_level_index(s.dim, s.degree));
    SIG_CUDA_CHECK(cudaGetLastError());
    count_launch();
}

template <typename T>
void launch_chen_right_adjoint(const T* dS, uint64_t ds_stride, const T* A, uint64_t a_stride, T* dY,
                               uint64_t dy_stride, const SigShape& s, cudaStream_t stream) {
    check_generic_limits(s);
    const uint32_t slen = static_cast<uint32_t>(s.full_len - 1);
    const uint64_t total = checked_mul(s.batch, slen, "signature output");
    if (total == 0) return;
    chen_right_adjoint_kernel<T><<<grid_1d(total, kGenericThreads), kGenericThreads, 0, stream>>>(
        dS, ds_stride, A, a_stride, dY, dy_stride, total, slen, static_cast<int>(s.degree),
        make_level_index(s.dim, s.degree));
    SIG_CUDA_CHECK(cudaGetLastError());
    count_launch();
}

template <typename T>
void launch_increment_to_point_grad(const T* incr_grad, T* out, uint64_t batch, uint64_t L, uint64_t d,
                                    cudaStream_t stream) {
    const uint64_t total = checked_mul(batch, checked_mul(L, d, "path gradient"), "path gradient");
    if (total == 0) return;
    const uint64_t per_path = L * d;
    const dim3 grid(grid_1d(per_path, 256), static_cast<unsigned>(std::min<uint64_t>(batch, 65535)));
    increment_to_point_grad_kernel<T><<<grid, 256, 0, stream>>>(incr_grad, out, batch, per_path, (L - 1) * d,
                                                                static_cast<uint32_t>(d));
    SIG_CUDA_CHECK(cudaGetLastError());
    count_launch();
}

template <typename T>
void launch_fill(T* dst, uint64_t n, T value, cudaStream_t stream) {
    if (n == 0) return;
    const unsigned blocks = static_cast<unsigned>(std::min<uint64_t>((n + 255) / 256, 148 * 8));
    fill_kernel<T><<<blocks, 256, 0, stream>>>(dst, n, value);
    SIG_CUDA_CHECK(cudaGetLastError());
    count_launch();
}

template <typename T>
void launch_nonfinite_scan(const T* data, uint64_t n, int* flag, cudaStream_t stream) {
    if (n == 0) return;
    const unsigned blocks = static_cast<unsigned>(std::min<uint64_t>((n + 255) / 256, 148 * 8));
    nonfinite_scan_kernel<T><<<blocks, 256, 0, stream>>>(data, n, flag);
    SIG_CUDA_CHECK(cudaGetLastError());
    count_launch();
}

#define INSTANTIATE(T)                                                                                   \
    template void launch_trivial_forward<T>(const T*, T*, const SigShape&, T, cudaStream_t);             \
    template void launch_generic_forward<T>(const T*, T*, const SigShape&, T, T*, unsigned, cudaStream_t); \
    template void launch_generic_backward<T>(const T*, T*, const T*, const T*, const SigShape&, T, T*,   \
                                             unsigned, cudaStream_t);                                    \
    template void launch_increment_to_point_grad<T>(const T*, T*, uint64_t, uint64_t, uint64_t, cudaStream_t); \
    template void launch_chen_combine<T>(T*, const T*, T*, const SigShape&, int, cudaStream_t);                   \
    template void launch_chen_product<T>(const T*, uint64_t, const T*, uint64_t, T*, uint64_t, const SigShape&, cudaStream_t, bool); \
    template void launch_chen_left_adjoint<T>(const T*, uint64_t, const T*, uint64_t, T*, uint64_t, const SigShape&, cudaStream_t); \
    template void launch_degree_one_backward<T>(const T*, T*, const T*, const SigShape&, T, cudaStream_t); \
    template void launch_chen_right_adjoint<T>(const T*, uint64_t, const T*, uint64_t, T*, uint64_t, const SigShape&, cudaStream_t); \
    template void launch_fill<T>(T*, uint64_t, T, cudaStream_t);                                         \
    template void launch_nonfinite_scan<T>(const T*, uint64_t, int*, cudaStream_t);
INSTANTIATE(float)
INSTANTIATE(double)
#undef INSTANTIATE

}  // namespace sigb200
