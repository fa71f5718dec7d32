// The tensor logarithm and its backward pass at HBM speed: one CTA per signature.
//
// Forward (sig_log.cu): with x the signature without its scalar term, R_{N+1} = 0,
//     R_k = x / k - x (x) R_{k+1}   (k = N .. 2, needed on levels <= 1 + N - k),      y = x - x (x) R_2,
// where (x) is the product of tensors without scalar terms.  Backward, with Y = dLoss/dy:
//     dx  = Y + sum_k Q_k / k - sum_k (adjoint of the left factor of x (x) R_{k+1} at Q_k),    Q_1 = Y,
//     Q_{k+1} = dLoss/dR_{k+1} = -(adjoint of the right factor of x (x) R_{k+1} at Q_k).
// Only the first step touches the top level N, and there only through Y_N itself: dx_N = Y_N, and Y_N
// contracted with the levels below N of x and R_2.  So a CTA keeps the levels below N of x, of every
// R_k, of dx and of two Q buffers in shared memory, recomputes the R_k there, streams Y level by level
// from the caller's gradient (expanded, or scattered from the Lyndon-word coordinates through the
// rank table) while it writes the top level of dx, and runs the remaining steps entirely in shared
// memory.  Global traffic: the gradient and the levels below N of the signature in, dx out; the top
// level of the signature is never read.  The products are the register-resident adjoint of
// chen_stream.cuh with the negated factors -x and -R_{k+1}, which turns every minus sign above into
// the plain accumulation of that routine.
//
// Same values as the kernel sequence of sig_log.cu (log_seed / log_scatter / log_adjoint kernels),
// which stays for small batches, dimensions that are not powers of two and signatures too large for
// shared memory.  Reference: the derivative of siglib/cpsig/cp_tensor_log.h:47-122, evaluated there as
// cp_tensor_log.h:176-235; replaces sig_to_log_sig_backprop_cuda_ of siglib/cusig/cu_log_signature.cu.
#include <algorithm>
#include <type_traits>

#include "algebra.h"
#include "chen_stream.cuh"
#include "kernels.h"
#include "runtime.h"

namespace sigb200 {

namespace {

template <int VEC> struct IntPack;
template <> struct IntPack<4> { using type = int4; };
template <> struct IntPack<2> { using type = int2; };
template <> struct IntPack<1> { using type = int; };
__device__ __forceinline__ void unpack_int(const int4& p, int* v) { v[0] = p.x; v[1] = p.y; v[2] = p.z; v[3] = p.w; }
__device__ __forceinline__ void unpack_int(const int2& p, int* v) { v[0] = p.x; v[1] = p.y; }
__device__ __forceinline__ void unpack_int(const int& p, int* v) { v[0] = p; }

// The gradient with respect to the Lyndon-word coordinates, read as the expanded tensor it stands
// for: rank[p] is the coordinate that sits at scalar-free position p, -1 where the word is not Lyndon.
template <typename T, int VEC>
struct RankedGlobalLoader {
    using P = typename Pack<T, VEC>::type;
    const T* g;
    const int32_t* rank;
    // two phases: the ranks of a vector are read one batch of iterations before the coordinates they
    // point to, so the two dependent memory round trips of a vector do not add up inside one batch
    static constexpr bool kTwoPhase = true;
    using Handle = typename IntPack<VEC>::type;
    __device__ __forceinline__ Handle issue(uint32_t pos) const {
        return *reinterpret_cast<const Handle*>(rank + pos);
    }
    __device__ __forceinline__ P finish(const Handle& h) const {
        int r[VEC];
        unpack_int(h, r);
        T out[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) out[k] = r[k] >= 0 ? g[r[k]] : T(0);
        return make_pack(out);
    }
    __device__ __forceinline__ P vec(uint32_t pos) const { return finish(issue(pos)); }
    __device__ __forceinline__ T one(uint32_t c) const {
        const int r = rank[c];
        return r >= 0 ? g[r] : T(0);
    }
    __device__ __forceinline__ void prefetch(uint32_t) const {}
};

template <typename T, int VEC, int NS, bool RANKED>
__global__ void __launch_bounds__(kAdjointThreads, NS <= 3 ? kAdjointCtas : 1)
log_adjoint_cta_kernel(const T* __restrict__ x, uint64_t x_stride, const T* __restrict__ g, uint64_t g_stride,
                       uint32_t g_len, const int32_t* __restrict__ rank, T* __restrict__ dsig, uint64_t dsig_stride,
                       bool zero_scalar, uint64_t batch, int N, uint32_t d, int lgd, LevelIndex lev) {
    extern __shared__ __align__(16) unsigned char log_smem[];
    __shared__ uint32_t li[kMaxDegree + 2];
    __shared__ uint32_t ord_off[kMaxDegree + 2];
    __shared__ uint32_t r_off[kMaxDegree + 2];
    const uint32_t tid = threadIdx.x, nt = blockDim.x;
    for (uint32_t i = tid; i < uint32_t(N + 2); i += nt) li[i] = lev.li[i];
    __syncthreads();
    // every array with scalar-term addressing (array[li[m] + index]) and every level on a vector boundary
    const uint32_t low_len = (li[N] + 6) & ~3u;
    T* base = reinterpret_cast<T*>(log_smem);
    T* nx = base + (VEC - 1);                       // -x, levels 1 .. N-1
    T* ds = nx + low_len;                           // dLoss/dx, levels 1 .. N-1
    const uint32_t small_len = (li[N >= 3 ? N - 1 : 2] + 6) & ~3u;
    T* q0 = ds + low_len;                           // Q_2 (levels <= N-1), Q_4, ..
    T* q1 = q0 + low_len;                           // Q_3 (levels <= N-2), Q_5, ..
    T* nr = q1 + small_len;                         // -R_2, -R_3, .., -R_N, R_k (levels <= 1 + N - k) at nr + r_off[k]
    if (tid == 0) {
        uint32_t off = 0;
        for (int k = 2; k <= N; ++k) {
            r_off[k] = off;
            off += (li[2 + N - k] + 6) & ~3u;
        }
        r_off[N + 1] = off;
    }
    __syncthreads();
    AdjointShared<T> sm;
    sm.a_low = nx;
    sm.da_low = ds;
    sm.vs = sm.dvs = nullptr;
    sm.li = li;
    sm.ord_off = ord_off;
    uint32_t* order = reinterpret_cast<uint32_t*>(base + 3 * low_len + small_len + r_off[N + 1]);
    sm.order = order;
    fill_regular_order(order, ord_off, li, N, VEC, lgd);
    const uint32_t low_count = li[N] - 1;
    T unused[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) unused[k] = T(0);

    for (uint64_t b = blockIdx.x; b < batch; b += gridDim.x) {
        __syncthreads();
        const T* xb = x + b * x_stride;
        // What this CTA reads in scattered order or right at the start of a signature (the coordinate row
        // behind the rank table, a few tens of KB, and the levels below N of the signature) is pulled into
        // L2 one signature ahead, one 128-byte line per thread and round.
        {
            constexpr uint32_t kLine = 128 / sizeof(T);
            auto pull = [&](uint64_t which) {
                if (which >= batch) return;
                if constexpr (RANKED) {
                    const T* gb = g + which * g_stride;
                    for (uint32_t i = tid * kLine; i < g_len; i += nt * kLine)
                        asm volatile("prefetch.global.L2 [%0];" ::"l"(gb + i));
                }
                const T* xn = x + which * x_stride;
                for (uint32_t i = tid * kLine; i < low_count; i += nt * kLine)
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(xn + i));
            };
            if (b == blockIdx.x) pull(b);
            pull(b + gridDim.x);
        }
        for (uint32_t j = tid; j < low_count; j += nt) nx[1 + j] = -xb[j];
        for (uint32_t j = tid; j < li[N]; j += nt) ds[j] = q0[j] = T(0);
        __syncthreads();
        // -R_k = -x / k + (-x) (x) (-R_{k+1}), one thread per coefficient
        for (int k = N; k >= 2; --k) {
            const uint32_t levels = 1 + N - k;
            const T rk = T(1) / T(k);
            T* cur = nr + r_off[k];
            const T* next = k < N ? nr + r_off[k + 1] : nullptr;
            for (uint32_t pos = 1 + tid; pos < li[levels + 1]; pos += nt) {
                uint32_t t = 1;
                while (pos >= li[t + 1]) ++t;
                const uint32_t idx = pos - li[t];
                T value = nx[pos] * rk;
                for (uint32_t i = t - 1; i >= 1; --i) {
                    const uint32_t sh = (t - i) * uint32_t(lgd);
                    value = chen_fma(nx[li[i] + (idx >> sh)], next[li[t - i] + (idx & ((1u << sh) - 1u))], value);
                }
                cur[pos] = value;
            }
            __syncthreads();
        }
        // first step: Q_1 = Y from the caller's gradient, all levels; dx_N = Y_N goes straight out
        T* dtop = dsig + b * dsig_stride + low_count;
        sm.b_low = nr + r_off[2];
        sm.db_low = q0;
        if constexpr (RANKED) {
            const RankedGlobalLoader<T, VEC> load{g + b * g_stride, rank};
            adjoint_levels_regular<T, VEC, NS>(sm, load, N, true, dtop, static_cast<T*>(nullptr), T(1), T(0), 0, N, d, lgd,
                                               unused);
        } else {
            const DenseGlobalLoader<T, VEC> load{g + b * g_stride};
            adjoint_levels_regular<T, VEC, NS>(sm, load, N, true, dtop, static_cast<T*>(nullptr), T(1), T(0), 0, N, d, lgd,
                                               unused);
        }
        __syncthreads();
        // steps 2 .. N in shared memory: Q_k lives on levels <= 1 + N - k
        T* qc = q0;
        T* qn = q1;
        for (int k = 2; k <= N; ++k) {
            const int levels = 1 + N - k;
            if (levels >= 2) {
                for (uint32_t j = tid; j < li[levels]; j += nt) qn[j] = T(0);
                __syncthreads();
                sm.b_low = nr + r_off[k + 1];
            }
            sm.db_low = qn;
            const SharedLoader<T, VEC> load{qc};
            adjoint_levels_regular<T, VEC, NS>(sm, load, levels, false, static_cast<T*>(nullptr), static_cast<T*>(nullptr),
                                               T(1) / T(k), T(0), 0, N, d, lgd, unused);
            __syncthreads();
            T* t = qc;
            qc = qn;
            qn = t;
        }
        T* db = dsig + b * dsig_stride;
        for (uint32_t j = tid; j < low_count; j += nt) db[j] = ds[1 + j];
        if (zero_scalar && tid == 0) db[-1] = T(0);
    }
}

// Forward: y = x - x (x) R_2 for one signature per CTA, any dimension.  -x and the running -R_k
// (two buffers, R_k only needs R_{k+1}) live in shared memory on the levels below N; the outputs are
// then one thread each: coordinate i is the word at scalar-free position lyndon[i] (or i itself for
// the expanded layout), its value x[p] minus one product term per split, all operands of which are
// below level N.  The signature's top level is read only where an output needs it.
template <typename T>
__global__ void __launch_bounds__(kChenThreads)
log_forward_cta_kernel(const T* __restrict__ x, uint64_t x_stride, T* __restrict__ out, uint64_t out_stride,
                       const uint32_t* __restrict__ lyndon, uint32_t count, bool zero_scalar, uint64_t batch, int N,
                       uint32_t d, int lgd, LevelIndex lev) {
    extern __shared__ __align__(16) unsigned char log_smem[];
    __shared__ uint32_t li[kMaxDegree + 2];
    __shared__ uint32_t pw[kMaxDegree + 2];        // d^k
    const uint32_t tid = threadIdx.x, nt = blockDim.x;
    for (uint32_t i = tid; i < uint32_t(N + 2); i += nt) li[i] = lev.li[i];
    if (tid == 0) {
        uint32_t p = 1;
        for (int k = 0; k <= N; ++k) {
            pw[k] = p;
            p *= d;
        }
    }
    __syncthreads();
    const uint32_t low_len = (li[N] + 3) & ~3u;
    T* nx = reinterpret_cast<T*>(log_smem);        // -x, levels 1 .. N-1 (scalar-term addressing)
    T* ra = nx + low_len;                          // -R_k, alternating
    T* rb = ra + low_len;
    const uint32_t low_count = li[N] - 1;

    for (uint64_t b = blockIdx.x; b < batch; b += gridDim.x) {
        __syncthreads();
        const T* xb = x + b * x_stride;
        for (uint32_t j = tid; j < low_count; j += nt) nx[1 + j] = -xb[j];
        __syncthreads();
        T* cur = ra;
        T* next = rb;                              // holds -R_{k+1}
        for (int k = N; k >= 2; --k) {
            const uint32_t levels = 1 + N - k;
            const T rk = T(1) / T(k);
            for (uint32_t pos = 1 + tid; pos < li[levels + 1]; pos += nt) {
                uint32_t t = 1;
                while (pos >= li[t + 1]) ++t;
                const uint32_t idx = pos - li[t];
                T value = nx[pos] * rk;
                if (k < N) {
                    for (uint32_t i = t - 1; i >= 1; --i) {
                        const uint32_t left = idx / pw[t - i];
                        value = chen_fma(nx[li[i] + left], next[li[t - i] + idx - left * pw[t - i]], value);
                    }
                }
                cur[pos] = value;
            }
            __syncthreads();
            T* swap = cur;
            cur = next;
            next = swap;
        }
        const T* nr2 = next;                       // -R_2 on levels 1 .. N-1
        T* ob = out + b * out_stride;
        if (zero_scalar && tid == 0) ob[-1] = T(0);
        // kOutputs coordinates per thread and round: their position reads and then their (scattered) value
        // reads are issued together, so a round waits out one memory latency of each kind instead of kOutputs
        constexpr int kOutputs = 4;
        for (uint32_t i0 = tid; i0 < count; i0 += kOutputs * nt) {
            uint32_t pos[kOutputs];
            T val[kOutputs];
#pragma unroll
            for (int k = 0; k < kOutputs; ++k) {
                const uint32_t i = i0 + k * nt;
                pos[k] = i < count ? (lyndon ? lyndon[i] : i) : 0u;
            }
#pragma unroll
            for (int k = 0; k < kOutputs; ++k) val[k] = xb[pos[k]];
#pragma unroll
            for (int k = 0; k < kOutputs; ++k) {
                const uint32_t i = i0 + k * nt;
                if (i >= count) break;
                const uint32_t p = pos[k];
                uint32_t t = 1;
                while (p + 1 >= li[t + 1]) ++t;
                const uint32_t idx = p + 1 - li[t];
                T value = val[k];
                // y = x - x (x) R_2 = x - (-x) (x) (-R_2)
                if (lgd >= 0) {                          // power-of-two dimension: shifts instead of divisions
                    for (uint32_t s = t - 1; s >= 1; --s) {
                        const uint32_t sh = (t - s) * uint32_t(lgd);
                        value = chen_fma(-nx[li[s] + (idx >> sh)], nr2[li[t - s] + (idx & ((1u << sh) - 1u))], value);
                    }
                } else {
                    for (uint32_t s = t - 1; s >= 1; --s) {
                        const uint32_t left = idx / pw[t - s];
                        value = chen_fma(-nx[li[s] + left], nr2[li[t - s] + idx - left * pw[t - s]], value);
                    }
                }
                ob[i] = value;
            }
        }
    }
}

bool aligned_for(const void* p, size_t bytes) { return reinterpret_cast<uintptr_t>(p) % bytes == 0; }

}  // namespace

// y = log(1 + x) for a batch, one CTA per signature: the expanded tensor (lyndon == nullptr, count =
// coefficients of the signature) or its Lyndon-word coordinates (lyndon[i]: scalar-free position of
// coordinate i).  x / out address the first level-1 coefficient resp. the first output.  Returns false
// with nothing launched for batches below the SM count, degree < 2 or levels below N beyond shared memory.
template <typename T>
bool launch_log_forward_streamed(const T* x, uint64_t x_stride, T* out, uint64_t out_stride, const uint32_t* lyndon,
                                 uint32_t count, bool zero_scalar, uint64_t batch, uint64_t dim, uint64_t degree,
                                 cudaStream_t stream) {
    if (degree < 2 || degree > uint64_t(kMaxDegree) || dim < 1) return false;
    const int sms = device_context(current_device()).sm_count;
    if (batch < uint64_t(sms)) return false;
    if (sig_length_full(dim, degree) >= (1ull << 31)) return false;
    const LevelIndex lev = make_level_index(dim, degree);
    const uint64_t low_len = (uint64_t(lev.li[degree]) + 3) & ~3ull;
    const size_t smem = 3 * low_len * sizeof(T);
    if (smem > 200 * 1024) return false;
    const unsigned per_sm = static_cast<unsigned>(std::max<size_t>(1, std::min<size_t>(8, (220 * 1024) / (smem + 1024))));
    const unsigned grid = static_cast<unsigned>(std::min<uint64_t>(batch, uint64_t(sms) * per_sm));
    if (smem > 48 * 1024)
        SIG_CUDA_CHECK(cudaFuncSetAttribute(log_forward_cta_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    int lgd = -1;
    if ((dim & (dim - 1)) == 0 && dim >= 2) {
        lgd = 0;
        while ((1ull << lgd) < dim) ++lgd;
    }
    log_forward_cta_kernel<T><<<grid, kChenThreads, smem, stream>>>(x, x_stride, out, out_stride, lyndon, count, zero_scalar,
                                                                    batch, static_cast<int>(degree),
                                                                    static_cast<uint32_t>(dim), lgd, lev);
    SIG_CUDA_CHECK(cudaGetLastError());
    count_launch();
    return true;
}

template bool launch_log_forward_streamed<float>(const float*, uint64_t, float*, uint64_t, const uint32_t*, uint32_t, bool,
                                                 uint64_t, uint64_t, uint64_t, cudaStream_t);
template bool launch_log_forward_streamed<double>(const double*, uint64_t, double*, uint64_t, const uint32_t*, uint32_t, bool,
                                                  uint64_t, uint64_t, uint64_t, cudaStream_t);

// dLoss/d sig from dLoss/d log-signature for a batch, one CTA per signature.  x and dsig address first
// level-1 coefficients; g is the gradient in expanded layout (rank == nullptr, first level-1 coefficient)
// or with respect to the Lyndon-word coordinates (rank: the inverse position table).  Returns false,
// with nothing launched, when the batch does not fill the GPU, the dimension is not a power of two, the
// degree is below 2 or above the register-resident limit, or the working set exceeds shared memory.
template <typename T>
bool launch_log_adjoint_streamed(const T* x, uint64_t x_stride, const T* g, uint64_t g_stride, const int32_t* rank,
                                 T* dsig, uint64_t dsig_stride, bool zero_scalar, uint64_t batch, uint64_t dim,
                                 uint64_t degree, cudaStream_t stream) {
    // coordinates per signature when g is indexed through the rank table (its stride is their count)
    const uint32_t g_len = static_cast<uint32_t>(std::min<uint64_t>(g_stride, 0xffffffffull));
    if (degree < 2 || degree - 1 > uint64_t(kChenSplits) || dim < 2 || dim > uint64_t(kAdjointThreads) || (dim & (dim - 1)) != 0)
        return false;
    const int sms = device_context(current_device()).sm_count;
    if (batch < uint64_t(sms)) return false;
    if (sig_length_full(dim, degree) >= (1ull << 31)) return false;
    const LevelIndex lev = make_level_index(dim, degree);
    const uint64_t low_len = (uint64_t(lev.li[degree]) + 6) & ~3ull;
    uint64_t r_total = 0;
    for (uint64_t k = 2; k <= degree; ++k) r_total += (uint64_t(lev.li[2 + degree - k]) + 6) & ~3ull;
    int lgd = 0;
    while ((1ull << lgd) < dim) ++lgd;
    const uint64_t top_off = lev.li[degree] - 1;
    auto fits = [&](int vec) {
        const size_t bytes = vec * sizeof(T);
        return dim % vec == 0 && aligned_for(dsig + top_off, bytes) && dsig_stride % vec == 0 &&
               (rank != nullptr || (aligned_for(g + top_off, bytes) && g_stride % vec == 0));
    };
    bool launched = false;
    auto run = [&](auto kernel, int vec) {
        const uint64_t entries = regular_order_entries(lev, degree, kAdjointThreads, vec);
        const uint64_t small_len = (uint64_t(lev.li[degree >= 3 ? degree - 1 : 2]) + 6) & ~3ull;
        const size_t smem = (3 * low_len + small_len + r_total) * sizeof(T) + entries * sizeof(uint32_t);
        if (smem > 200 * 1024) return;
        const unsigned per_sm = static_cast<unsigned>(std::max<size_t>(1, std::min<size_t>(8, (220 * 1024) / (smem + 1024))));
        const unsigned grid = static_cast<unsigned>(std::min<uint64_t>(batch, uint64_t(sms) * per_sm));
        if (smem > 48 * 1024)
            SIG_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        kernel<<<grid, kAdjointThreads, smem, stream>>>(x, x_stride, g, g_stride, g_len, rank, dsig, dsig_stride, zero_scalar, batch,
                                                     static_cast<int>(degree), static_cast<uint32_t>(dim), lgd, lev);
        SIG_CUDA_CHECK(cudaGetLastError());
        count_launch();
        launched = true;
    };
    auto run_vec = [&](auto vec) {
        constexpr int V = decltype(vec)::value;
        if (rank) {
            if (degree <= 2) run(log_adjoint_cta_kernel<T, V, 1, true>, V);
            else if (degree <= 4) run(log_adjoint_cta_kernel<T, V, 3, true>, V);
            else run(log_adjoint_cta_kernel<T, V, kChenSplits, true>, V);
        } else {
            if (degree <= 2) run(log_adjoint_cta_kernel<T, V, 1, false>, V);
            else if (degree <= 4) run(log_adjoint_cta_kernel<T, V, 3, false>, V);
            else run(log_adjoint_cta_kernel<T, V, kChenSplits, false>, V);
        }
    };
    constexpr int kWide = sizeof(T) == 4 ? 4 : 2;
    if (fits(kWide)) run_vec(std::integral_constant<int, kWide>{});
    else if (fits(2)) run_vec(std::integral_constant<int, 2>{});
    else run_vec(std::integral_constant<int, 1>{});
    return launched;
}

template bool launch_log_adjoint_streamed<float>(const float*, uint64_t, const float*, uint64_t, const int32_t*, float*,
                                                 uint64_t, bool, uint64_t, uint64_t, uint64_t, cudaStream_t);
template bool launch_log_adjoint_streamed<double>(const double*, uint64_t, const double*, uint64_t, const int32_t*, double*,
                                                  uint64_t, bool, uint64_t, uint64_t, uint64_t, cudaStream_t);

}  // namespace sigb200
