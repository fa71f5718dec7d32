// Chen products of batches of signatures at HBM speed: one CTA per signature.
//
// C = A (x) B, level by level:  C_m[w] = sum_{i = 0..m} A_i[w_1..w_i] * B_{m-i}[w_{i+1}..w_m]  (A_0 = B_0 = 1).
// Nearly all coefficients sit in the top level N (a fraction (d-1)/d of them) and each of them needs,
// besides A_N[w] and B_N[w] themselves, only coefficients of the levels BELOW N of both factors: a few
// KB per signature.  So a CTA loads the levels below N of its two operands into shared memory once,
// writes the lower levels of the product from there, and then streams the top level: every thread
// takes VEC consecutive words (the same prefixes for every split, consecutive suffixes: one shared
// read of A_i and one vector read of B_{N-i} per split), with coalesced vector loads of A_N / B_N and
// a coalesced vector store of C_N.  Global traffic is the algorithmic minimum (each operand read
// once, the result written once).  One of the factors can be exp(v) of a displacement v (the
// signature of a straight segment, L_k = v^(x)k / k!): it is generated in shared memory and on the fly,
// never read from or written to global memory, which makes sig_join one pass over its input.
//
// Replaces, for batches that fill the GPU with one CTA per signature, the per-coefficient kernels of
// sig_generic.cu (kept for small batches and for signatures whose lower levels do not fit shared
// memory); same sums, same order over the splits (siglib/cpsig/cp_sig_combine.h:34-66 is the
// reference arithmetic, siglib/cusig/cu_sig_combine.cu:35-340 the reference kernels).
#include <cuda_pipeline.h>

#include <algorithm>
#include <type_traits>

#include "chen_stream.cuh"
#include "kernels.h"
#include "runtime.h"

namespace sigb200 {

namespace {

// Levels 0 .. N-1 of one operand into shared memory (scalar-term addressing: low[0] = 1,
// low[li[k] + index]).  src addresses the first level-1 coefficient; src == nullptr: the operand
// is exp(v), generated level by level (L_k[w c] = L_{k-1}[w] * v[c] / k).
template <typename T>
__device__ __forceinline__ void load_low(T* low, const T* __restrict__ src, const T* __restrict__ v, const uint32_t* li,
                                         int N, uint32_t d, uint32_t tid, uint32_t nt) {
    const uint32_t count = li[N] - 1;   // coefficients of levels 1 .. N-1
    if (tid == 0) low[0] = T(1);
    if (src != nullptr) {
        for (uint32_t j = tid; j < count; j += nt) low[1 + j] = src[j];
        return;
    }
    for (uint32_t c = tid; c < d && 1 < N; c += nt) low[1 + c] = v[c];
    for (int k = 2; k < N; ++k) {
        __syncthreads();
        const uint32_t n = li[k + 1] - li[k];
        const T r = T(1) / T(k);
        for (uint32_t j = tid; j < n; j += nt) {
            const uint32_t w = j / d, c = j - w * d;
            low[li[k] + j] = low[li[k - 1] + w] * (v[c] * r);
        }
    }
}

// A / B: first level-1 coefficient of signature 0 (nullptr: that factor is exp(v), v = disp + b * d).
template <typename T, int VEC>
__global__ void __launch_bounds__(kChenThreads)
chen_product_cta_kernel(const T* __restrict__ A, uint64_t a_stride, const T* __restrict__ B, uint64_t b_stride,
                        const T* __restrict__ disp, T* __restrict__ C, uint64_t c_stride, bool c_scalar, uint64_t batch,
                        int N, uint32_t d, LevelIndex lev) {
    extern __shared__ __align__(16) unsigned char chen_smem[];
    __shared__ uint32_t li[kMaxDegree + 2];
    const uint32_t tid = threadIdx.x, nt = blockDim.x;
    for (uint32_t i = tid; i < uint32_t(N + 2); i += nt) li[i] = lev.li[i];
    __syncthreads();
    // levels 0 .. N-1 of both factors.  li[k] - 1 is a multiple of d, hence of VEC: starting each array
    // VEC - 1 elements into a 16-byte aligned block puts every level on a vector boundary.
    const uint32_t low_len = (li[N] + 6) & ~3u;
    T* a_low = reinterpret_cast<T*>(chen_smem) + (VEC - 1);
    T* b_low = a_low + low_len;
    T* vs = reinterpret_cast<T*>(chen_smem) + 2 * low_len;   // the displacement, when a factor is generated
    const uint32_t top = li[N + 1] - li[N];              // d^N
    using P = typename Pack<T, VEC>::type;

    for (uint64_t b = blockIdx.x; b < batch; b += gridDim.x) {
        __syncthreads();                                  // the previous signature's reads are done
        const T* a = A ? A + b * a_stride : nullptr;
        const T* bb = B ? B + b * b_stride : nullptr;
        if (disp != nullptr) {
            for (uint32_t c = tid; c < d; c += nt) vs[c] = disp[b * d + c];
            __syncthreads();
        }
        load_low<T>(a_low, a, vs, li, N, d, tid, nt);
        load_low<T>(b_low, bb, vs, li, N, d, tid, nt);
        __syncthreads();
        T* c = C + b * c_stride;                          // first level-1 coefficient of the result
        if (c_scalar && tid == 0) c[-1] = T(1);
        // levels 1 .. N-1 of the product, one thread per coefficient, from shared memory
        for (uint32_t pos = 1 + tid; pos < li[N]; pos += nt) {
            int m = 1;
            while (pos >= li[m + 1]) ++m;
            const uint32_t idx = pos - li[m];
            T acc = a_low[pos] + b_low[pos];
            uint32_t left = idx, pw = 1;
            for (int i = m - 1; i >= 1; --i) {
                left /= d;
                pw *= d;
                acc = chen_fma(a_low[li[i] + left], b_low[li[m - i] + idx - left * pw], acc);
            }
            c[pos - 1] = acc;
        }
        // the top level, streamed: VEC consecutive words per thread
        const T* a_top = a ? a + (li[N] - 1) : nullptr;
        const T* b_top = bb ? bb + (li[N] - 1) : nullptr;
        T* c_top = c + (li[N] - 1);
        const T rn = T(1) / T(N);
        for (uint32_t idx = tid * VEC; idx < top; idx += nt * VEC) {
            T acc[VEC];
            // two streamed factors: the lines this thread's group reads two iterations from now go into L2
            // (one lane per 128 bytes).  Measured on B200, d = 16, degree 4: 0.83 ms without, 0.69 / 0.675 /
            // 0.69 / 0.78 ms at distances 1 / 2 / 3 / 6; with one generated factor the hint costs 2 %.
            if (a_top && b_top && (tid * VEC * sizeof(T)) % 128 == 0 && idx + 2 * nt * VEC < top) {
                asm volatile("prefetch.global.L2 [%0];" ::"l"(a_top + idx + 2 * nt * VEC));
                asm volatile("prefetch.global.L2 [%0];" ::"l"(b_top + idx + 2 * nt * VEC));
            }
            const uint32_t q = idx / d, c0 = idx - q * d;      // prefix of length N-1, first last letter
            if (a_top) {
                const P va = *reinterpret_cast<const P*>(a_top + idx);
#pragma unroll
                for (int k = 0; k < VEC; ++k) acc[k] = reinterpret_cast<const T*>(&va)[k];
            } else {
                const T s = a_low[li[N - 1] + q] * rn;          // exp(v) at the word: L_{N-1}[prefix] * v[c] / N
#pragma unroll
                for (int k = 0; k < VEC; ++k) acc[k] = s * vs[c0 + k];
            }
            if (b_top) {
                const P vb = *reinterpret_cast<const P*>(b_top + idx);
#pragma unroll
                for (int k = 0; k < VEC; ++k) acc[k] += reinterpret_cast<const T*>(&vb)[k];
            } else {
                const T s = b_low[li[N - 1] + q] * rn;
#pragma unroll
                for (int k = 0; k < VEC; ++k) acc[k] += s * vs[c0 + k];
            }
            uint32_t left = idx, pw = 1;
            for (int i = N - 1; i >= 1; --i) {
                left /= d;
                pw *= d;
                const T al = a_low[li[i] + left];
                T br[VEC];
                unpack(*reinterpret_cast<const P*>(b_low + li[N - i] + (idx - left * pw)), br);
#pragma unroll
                for (int k = 0; k < VEC; ++k) acc[k] = chen_fma(al, br[k], acc[k]);
            }
            P out;
#pragma unroll
            for (int k = 0; k < VEC; ++k) reinterpret_cast<T*>(&out)[k] = acc[k];
            *reinterpret_cast<P*>(c_top + idx) = out;
        }
    }
}

template <typename T, int VEC>
void launch_product(const T* A, uint64_t a_stride, const T* B, uint64_t b_stride, const T* disp, T* C, uint64_t c_stride,
                    bool c_scalar, const SigShape& s, size_t smem, unsigned grid, cudaStream_t stream) {
    if (smem > 48 * 1024)
        SIG_CUDA_CHECK(cudaFuncSetAttribute(chen_product_cta_kernel<T, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            int(smem)));
    chen_product_cta_kernel<T, VEC><<<grid, kChenThreads, smem, stream>>>(
        A, a_stride, B, b_stride, disp, C, c_stride, c_scalar, s.batch, static_cast<int>(s.degree),
        static_cast<uint32_t>(s.dim), make_level_index(s.dim, s.degree));
    SIG_CUDA_CHECK(cudaGetLastError());
    count_launch();
}

// Joins the consecutive segment signatures of every path in one launch: one CTA per path keeps the
// running product S in shared memory (levels below N twice, for the in-place update, and the whole top
// level), and multiplies one segment after the other onto it from the right:
//     S_N[w] += B_N[w] + sum_i S_i[prefix] B_{N-i}[suffix]   (every thread owns its words; reads only levels < N),
//     then S_m for m < N into the second buffer, from the old lower levels.
// seg: (batch, nseg, slen) scalar-free.  A segment comes in with asynchronous copies straight into
// shared memory, all of them in flight together (the kernel serves small batches: it is bound by the
// latency of those loads, not by their volume); the result is written once.
template <typename T, int VEC>
__global__ void __launch_bounds__(kChenThreads)
chen_chain_cta_kernel(const T* __restrict__ seg, int nseg, T* __restrict__ out, uint64_t out_stride, bool out_scalar,
                      uint64_t batch, int N, uint32_t d, LevelIndex lev) {
    extern __shared__ __align__(16) unsigned char chen_smem[];
    __shared__ uint32_t li[kMaxDegree + 2];
    const uint32_t tid = threadIdx.x, nt = blockDim.x;
    for (uint32_t i = tid; i < uint32_t(N + 2); i += nt) li[i] = lev.li[i];
    __syncthreads();
    const uint32_t low_len = (li[N] + 6) & ~3u;
    const uint32_t top = li[N + 1] - li[N], low_count = li[N] - 1, slen = li[N + 1] - 1;
    const uint32_t top_len = (top + 3) & ~3u;
    T* s_top = reinterpret_cast<T*>(chen_smem);            // top level of the running product
    T* b_top = s_top + top_len;                            // top level of the segment being multiplied on
    T* s_low = b_top + top_len + (VEC - 1);                // levels below N, every level on a vector boundary
    T* s_new = s_low + low_len;
    T* b_low = s_new + low_len;
    using P = typename Pack<T, VEC>::type;
    auto fetch = [&](const T* src, T* low, T* top_dst) {   // one segment, every copy in flight at once
        for (uint32_t j = tid; j < low_count; j += nt) __pipeline_memcpy_async(low + 1 + j, src + j, sizeof(T));
        for (uint32_t idx = tid * VEC; idx < top; idx += nt * VEC)
            __pipeline_memcpy_async(top_dst + idx, src + low_count + idx, VEC * sizeof(T));
        __pipeline_commit();
    };

    for (uint64_t b = blockIdx.x; b < batch; b += gridDim.x) {
        __syncthreads();
        const T* first = seg + b * uint64_t(nseg) * slen;
        if (tid == 0) s_low[0] = s_new[0] = b_low[0] = T(1);
        fetch(first, s_low, s_top);
        for (int k = 1; k < nseg; ++k) {
            __syncthreads();                               // the previous round is done with b_low / b_top
            fetch(first + uint64_t(k) * slen, b_low, b_top);
            __pipeline_wait_prior(0);
            __syncthreads();
            for (uint32_t idx = tid * VEC; idx < top; idx += nt * VEC) {
                T acc[VEC], bt[VEC];
                unpack(*reinterpret_cast<const P*>(s_top + idx), acc);
                unpack(*reinterpret_cast<const P*>(b_top + idx), bt);
#pragma unroll
                for (int v = 0; v < VEC; ++v) acc[v] += bt[v];
                uint32_t left = idx, pw = 1;
                for (int i = N - 1; i >= 1; --i) {
                    left /= d;
                    pw *= d;
                    const T al = s_low[li[i] + left];
                    T br[VEC];
                    unpack(*reinterpret_cast<const P*>(b_low + li[N - i] + (idx - left * pw)), br);
#pragma unroll
                    for (int v = 0; v < VEC; ++v) acc[v] = chen_fma(al, br[v], acc[v]);
                }
                *reinterpret_cast<P*>(s_top + idx) = make_pack(acc);
            }
            for (uint32_t pos = 1 + tid; pos < li[N]; pos += nt) {
                int m = 1;
                while (pos >= li[m + 1]) ++m;
                const uint32_t idx = pos - li[m];
                T acc = s_low[pos] + b_low[pos];
                uint32_t left = idx, pw = 1;
                for (int i = m - 1; i >= 1; --i) {
                    left /= d;
                    pw *= d;
                    acc = chen_fma(s_low[li[i] + left], b_low[li[m - i] + idx - left * pw], acc);
                }
                s_new[pos] = acc;
            }
            T* swap = s_low;
            s_low = s_new;
            s_new = swap;
        }
        __pipeline_wait_prior(0);
        __syncthreads();
        T* o = out + b * out_stride;
        if (out_scalar) {
            if (tid == 0) o[0] = T(1);
            ++o;
        }
        for (uint32_t j = tid; j < low_count; j += nt) o[j] = s_low[1 + j];
        for (uint32_t idx = tid; idx < top; idx += nt) o[low_count + idx] = s_top[idx];
    }
}

// Both adjoints of C = A (x) B in one pass over dC (the backward of sig_combine and of sig_join):
//     dA_i[u] = sum_v dC[u v] * B[v],   dB_j[v] = sum_u A[u] * dC[u v]      (v resp. u may be empty).
// Again the top level of dC carries nearly all the work and only touches the levels below N of A,
// B, dA and dB: those four live in shared memory (the two adjoints as accumulators), the top level of
// dC is streamed once with vector loads and copied to the top levels of dA and dB (their only
// contribution), and every word w of it adds dC[w] * B[suffix] to dA[prefix] and A[prefix] * dC[w]
// to dB[suffix] for each split.
//
// gen = 1 / 2: factor A / B is exp(v), v = disp[b] (sig_join).  Its levels below N are generated in
// shared memory, its adjoint X = dA / dB is not written but pulled back to d_disp[b] through the
// recursion exp(v)_k = exp(v)_{k-1} (x) v / k:
//     X_{k-1}[u] += (1/k) sum_c v[c] X_k[u c]   (k = N .. 2),     dv[c] = X_1[c] + sum_{k >= 2} sum_u exp(v)_{k-1}[u] X_k[u c] / k.
// The top level X_N is the streamed dC_N itself, so its two terms are taken in the streaming loop and
// X_N is never stored; the levels below are finished in shared memory after the loop.
// Any shape: every contribution is a shared-memory atomic, except that a prefix common to a group of
// lanes is pre-reduced by shuffles and the last-letter suffixes of a lane (fixed over its iterations
// when W is a multiple of d) are summed in registers.
template <typename T, int VEC>
__device__ __forceinline__ void adjoint_levels_generic(const AdjointShared<T>& sm, const T* __restrict__ g,
                                                       T* __restrict__ da_top, T* __restrict__ db_top, int gen, int N,
                                                       uint32_t d, T (&lastv)[VEC]) {
    using P = typename Pack<T, VEC>::type;
    const uint32_t tid = threadIdx.x, nt = blockDim.x, lane = tid & 31;
    const uint32_t* li = sm.li;
    const T* x_low = gen == 1 ? sm.a_low : sm.b_low;
    T* dx_low = gen == 1 ? sm.da_low : sm.db_low;
    const uint32_t top = li[N + 1] - li[N];
    const bool fixed_last = (nt * VEC) % d == 0;
    const T rn = T(1) / T(N);
    // levels below N of dC
    for (uint32_t pos = 1 + tid; pos < li[N]; pos += nt) {
        const T gv = g[pos - 1];
        int m = 1;
        while (pos >= li[m + 1]) ++m;
        const uint32_t idx = pos - li[m];
        atomicAdd(&sm.da_low[pos], gv);
        atomicAdd(&sm.db_low[pos], gv);
        uint32_t left = idx, pw = 1;
        for (int i = m - 1; i >= 1; --i) {
            left /= d;
            pw *= d;
            const uint32_t r = idx - left * pw;
            atomicAdd(&sm.da_low[li[i] + left], gv * sm.b_low[li[m - i] + r]);
            atomicAdd(&sm.db_low[li[m - i] + r], sm.a_low[li[i] + left] * gv);
        }
    }
    // the top level of dC, streamed
    const T* g_top = g + (li[N] - 1);
    T last[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) last[k] = T(0);
    for (uint32_t base = 0; base < top; base += nt * VEC) {
        const uint32_t idx = base + tid * VEC;
        const bool valid = idx < top;
        T gv[VEC];
        if (valid) {
            const P v = *reinterpret_cast<const P*>(g_top + idx);
            if (da_top) *reinterpret_cast<P*>(da_top + idx) = v;
            if (db_top) *reinterpret_cast<P*>(db_top + idx) = v;
            unpack(v, gv);
        } else {
#pragma unroll
            for (int k = 0; k < VEC; ++k) gv[k] = T(0);
        }
        const uint32_t at = valid ? idx : 0;
        uint32_t left = at, pw = 1;
        for (int i = N - 1; i >= 1; --i) {
            left /= d;
            pw *= d;                                       // d^(N-i): words per prefix of length i
            const uint32_t r = at - left * pw;
            const T al = sm.a_low[li[i] + left];
            const T* bs = sm.b_low + li[N - i] + r;
            T sa = T(0);
#pragma unroll
            for (int k = 0; k < VEC; ++k) sa = chen_fma(gv[k], bs[k], sa);
            const uint32_t share = lanes_per_block(pw, VEC);
            if (share) {
                sa = group_sum(sa, share);
                if ((lane & (share - 1)) == 0 && valid) atomicAdd(&sm.da_low[li[i] + left], sa);
            } else if (valid) {
                atomicAdd(&sm.da_low[li[i] + left], sa);
            }
            if (i == N - 1 && fixed_last) {
#pragma unroll
                for (int k = 0; k < VEC; ++k) last[k] = chen_fma(al, gv[k], last[k]);
            } else if (valid) {
                T* dst = sm.db_low + li[N - i] + r;
#pragma unroll
                for (int k = 0; k < VEC; ++k) atomicAdd(dst + k, al * gv[k]);
            }
        }
        if (gen) {
            const uint32_t q = at / d, c0 = at - q * d;
            T push = T(0);
#pragma unroll
            for (int k = 0; k < VEC; ++k) push = chen_fma(sm.vs[c0 + k], gv[k], push);
            push *= rn;
            const uint32_t share = lanes_per_block(d, VEC);
            if (share) {
                push = group_sum(push, share);
                if ((lane & (share - 1)) == 0 && valid) atomicAdd(&dx_low[li[N - 1] + q], push);
            } else if (valid) {
                atomicAdd(&dx_low[li[N - 1] + q], push);
            }
            const T xl = x_low[li[N - 1] + q] * rn;
            if (fixed_last) {
#pragma unroll
                for (int k = 0; k < VEC; ++k) lastv[k] = chen_fma(xl, gv[k], lastv[k]);
            } else if (valid) {
#pragma unroll
                for (int k = 0; k < VEC; ++k) atomicAdd(&sm.dvs[c0 + k], xl * gv[k]);
            }
        }
    }
    if (fixed_last) {
        const uint32_t c0 = (tid * VEC) % d;
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            atomicAdd(&sm.db_low[li[1] + c0 + k], last[k]);
            if (gen) atomicAdd(&sm.dvs[c0 + k], lastv[k]);
        }
    }
}

// NS = 0: generic shapes; NS > 0: regular shapes with at most NS splits (degree <= NS + 1), lgd = log2(d).
template <typename T, int VEC, int NS>
__global__ void __launch_bounds__(kAdjointThreads, NS > 0 && NS <= 3 ? kAdjointCtas : 1)
chen_adjoints_cta_kernel(const T* __restrict__ dC, uint64_t dc_stride, const T* __restrict__ A, uint64_t a_stride,
                         const T* __restrict__ B, uint64_t b_stride, T* __restrict__ dA, uint64_t da_stride,
                         T* __restrict__ dB, uint64_t db_stride, const T* __restrict__ disp, T* __restrict__ d_disp,
                         int gen, uint64_t batch, int N, uint32_t d, int lgd, LevelIndex lev) {
    extern __shared__ __align__(16) unsigned char chen_smem[];
    __shared__ uint32_t li[kMaxDegree + 2];
    __shared__ uint32_t ord_off[kMaxDegree + 2];
    const uint32_t tid = threadIdx.x, nt = blockDim.x;
    for (uint32_t i = tid; i < uint32_t(N + 2); i += nt) li[i] = lev.li[i];
    __syncthreads();
    const uint32_t low_len = (li[N] + 6) & ~3u;            // every level on a vector boundary, as above
    AdjointShared<T> sm;
    sm.a_low = reinterpret_cast<T*>(chen_smem) + (VEC - 1);
    sm.b_low = sm.a_low + low_len;
    sm.da_low = sm.b_low + low_len;
    sm.db_low = sm.da_low + low_len;
    sm.vs = reinterpret_cast<T*>(chen_smem) + 4 * low_len;
    sm.dvs = sm.vs + ((d + 3) & ~3u);
    sm.li = li;
    sm.order = nullptr;
    sm.ord_off = ord_off;
    if constexpr (NS > 0) {
        uint32_t* order = reinterpret_cast<uint32_t*>(sm.dvs + ((d + 3) & ~3u));
        sm.order = order;
        fill_regular_order(order, ord_off, li, N, VEC, lgd);
    }
    const T* x_low = gen == 1 ? sm.a_low : sm.b_low;
    T* dx_low = gen == 1 ? sm.da_low : sm.db_low;
    const uint32_t low_count = li[N] - 1;

    for (uint64_t b = blockIdx.x; b < batch; b += gridDim.x) {
        __syncthreads();
        const T* a = gen == 1 ? nullptr : A + b * a_stride;
        const T* bb = gen == 2 ? nullptr : B + b * b_stride;
        const T* g = dC + b * dc_stride;
        if (gen) {
            for (uint32_t c = tid; c < d; c += nt) {
                sm.vs[c] = disp[b * d + c];
                sm.dvs[c] = T(0);
            }
            __syncthreads();
        }
        load_low<T>(sm.a_low, a, sm.vs, li, N, d, tid, nt);
        load_low<T>(sm.b_low, bb, sm.vs, li, N, d, tid, nt);
        for (uint32_t j = tid; j < li[N]; j += nt) sm.da_low[j] = sm.db_low[j] = T(0);
        __syncthreads();
        T* da_top = gen == 1 ? nullptr : dA + b * da_stride + low_count;
        T* db_top = gen == 2 ? nullptr : dB + b * db_stride + low_count;
        T lastv[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) lastv[k] = T(0);
        if constexpr (NS > 0) {
            const DenseGlobalLoader<T, VEC> load{g};
            adjoint_levels_regular<T, VEC, NS>(sm, load, N, true, da_top, db_top, T(1), T(1), gen, N, d, lgd, lastv);
        }
        else adjoint_levels_generic<T, VEC>(sm, g, da_top, db_top, gen, N, d, lastv);
        __syncthreads();

        if (gen) {
            for (int k = N - 1; k >= 2; --k) {              // push the levels below N down, one at a time
                const uint32_t count = li[k] - li[k - 1];
                const T rk = T(1) / T(k);
                for (uint32_t u = tid; u < count; u += nt) {
                    const T* upper = dx_low + li[k] + u * d;
                    T sum = T(0);
                    for (uint32_t c = 0; c < d; ++c) sum = chen_fma(sm.vs[c], upper[c], sum);
                    dx_low[li[k - 1] + u] += sum * rk;
                }
                __syncthreads();
            }
            // dv[c]: every coefficient (u, c) of X_k gives exp(v)_{k-1}[u] X_k[u c] / k.  With nt a multiple
            // of d a thread meets one letter only (li[k] - 1 is a multiple of d) and sums in a register.
            const bool one_letter = nt % d == 0;
            T mine = T(0);
            for (uint32_t pos = 1 + tid; pos < li[N]; pos += nt) {
                int k = 1;
                while (pos >= li[k + 1]) ++k;
                const uint32_t j = pos - li[k], u = j / d, c = j - u * d;
                const T term = k == 1 ? dx_low[pos] : x_low[li[k - 1] + u] * dx_low[pos] * (T(1) / T(k));
                if (one_letter) mine += term;
                else atomicAdd(&sm.dvs[c], term);
            }
            if (one_letter) atomicAdd(&sm.dvs[tid % d], mine);
            __syncthreads();
            for (uint32_t c = tid; c < d; c += nt) d_disp[b * d + c] = sm.dvs[c];
        }
        if (gen != 1) {
            T* da = dA + b * da_stride;
            for (uint32_t j = tid; j < low_count; j += nt) da[j] = sm.da_low[1 + j];
        }
        if (gen != 2) {
            T* db = dB + b * db_stride;
            for (uint32_t j = tid; j < low_count; j += nt) db[j] = sm.db_low[1 + j];
        }
    }
}

bool aligned_to(const void* p, size_t bytes) { return p == nullptr || reinterpret_cast<uintptr_t>(p) % bytes == 0; }

}  // namespace

// C = A (x) B with one CTA per signature; A or B may be nullptr, that factor is then exp(disp[b]).
// Returns false (nothing launched) when the batch is too small to fill the GPU that way or the
// levels below N do not fit shared memory; the caller then uses the per-coefficient kernels.
template <typename T>
bool launch_chen_product_streamed(const T* A, uint64_t a_stride, const T* B, uint64_t b_stride, const T* disp, T* C,
                                  uint64_t c_stride, const SigShape& s, cudaStream_t stream, bool write_scalar) {
    if (s.degree < 2 || s.degree > uint64_t(kMaxDegree) || s.dim < 2 || s.full_len >= (1ull << 31)) return false;
    const int sms = device_context(current_device()).sm_count;
    if (s.batch < uint64_t(sms)) return false;
    const LevelIndex lev = make_level_index(s.dim, s.degree);
    const uint64_t low_len = (uint64_t(lev.li[s.degree]) + 6) & ~3ull;
    const size_t smem = (2 * low_len + ((s.dim + 3) & ~3ull)) * sizeof(T);
    if (smem > 160 * 1024) return false;
    const unsigned per_sm = static_cast<unsigned>(std::max<size_t>(1, std::min<size_t>(8, (200 * 1024) / (smem + 1024))));
    const unsigned grid = static_cast<unsigned>(std::min<uint64_t>(s.batch, uint64_t(sms) * per_sm));
    // vector width: the top level of every operand must start on a vector boundary in every signature
    const uint64_t top_off = lev.li[s.degree] - 1;
    auto fits = [&](int vec) {
        const size_t bytes = vec * sizeof(T);
        auto ok = [&](const T* p, uint64_t stride) {
            return p == nullptr || (aligned_to(p + top_off, bytes) && stride % vec == 0);
        };
        return s.dim % vec == 0 && ok(A, a_stride) && ok(B, b_stride) && ok(C, c_stride);
    };
    constexpr int kWide = sizeof(T) == 4 ? 4 : 2;
    if (fits(kWide)) launch_product<T, kWide>(A, a_stride, B, b_stride, disp, C, c_stride, write_scalar, s, smem, grid, stream);
    else if (sizeof(T) == 4 && fits(2)) launch_product<T, 2>(A, a_stride, B, b_stride, disp, C, c_stride, write_scalar, s, smem, grid, stream);
    else launch_product<T, 1>(A, a_stride, B, b_stride, disp, C, c_stride, write_scalar, s, smem, grid, stream);
    return true;
}

// out[b] = seg[b][0] (x) .. (x) seg[b][nseg-1] in one launch, one CTA per path (any batch size: the
// caller is the time-segmented sweep of a small batch).  Returns false with nothing launched when the
// running product does not fit shared memory.
template <typename T>
bool launch_chen_chain(T* out, const T* seg, const SigShape& s, int nseg, cudaStream_t stream) {
    if (nseg < 2 || s.batch == 0 || s.degree < 2 || s.degree > uint64_t(kMaxDegree) || s.dim < 2 ||
        s.full_len >= (1ull << 31))
        return false;
    const LevelIndex lev = make_level_index(s.dim, s.degree);
    const uint64_t low_len = (uint64_t(lev.li[s.degree]) + 6) & ~3ull;
    const uint64_t top = uint64_t(lev.li[s.degree + 1]) - lev.li[s.degree];
    const size_t smem = (2 * ((top + 3) & ~3ull) + 3 * low_len + 4) * sizeof(T);
    if (smem > 200 * 1024) return false;
    const int sms = device_context(current_device()).sm_count;
    const unsigned per_sm = static_cast<unsigned>(std::max<size_t>(1, std::min<size_t>(8, (220 * 1024) / (smem + 1024))));
    const unsigned grid = static_cast<unsigned>(std::min<uint64_t>(s.batch, uint64_t(sms) * per_sm));
    const uint64_t slen = s.full_len - 1;
    auto run = [&](auto kernel) {
        if (smem > 48 * 1024)
            SIG_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        kernel<<<grid, kChenThreads, smem, stream>>>(seg, nseg, out, s.stride, s.scalar_term, s.batch,
                                                     static_cast<int>(s.degree), static_cast<uint32_t>(s.dim), lev);
        SIG_CUDA_CHECK(cudaGetLastError());
        count_launch();
    };
    constexpr int kWide = sizeof(T) == 4 ? 4 : 2;
    auto fits = [&](int vec) { return s.dim % vec == 0 && aligned_to(seg, vec * sizeof(T)) && slen % vec == 0; };
    if (fits(kWide)) run(chen_chain_cta_kernel<T, kWide>);
    else if (fits(2)) run(chen_chain_cta_kernel<T, 2>);
    else run(chen_chain_cta_kernel<T, 1>);
    return true;
}

template bool launch_chen_chain<float>(float*, const float*, const SigShape&, int, cudaStream_t);
template bool launch_chen_chain<double>(double*, const double*, const SigShape&, int, cudaStream_t);

// dA and dB of C = A (x) B from dC in one launch, one CTA per signature.  Same contract as above:
// false means nothing was launched.  The scalar slots (if the caller's layout has them) are not touched.
// gen = 1 / 2: factor A / B is exp(disp[b]); its pointer and its adjoint's are ignored and the adjoint
// of the displacement is written to d_disp instead (batch x dim).
template <typename T>
bool launch_chen_adjoints_streamed(const T* dC, uint64_t dc_stride, const T* A, uint64_t a_stride, const T* B,
                                   uint64_t b_stride, T* dA, uint64_t da_stride, T* dB, uint64_t db_stride,
                                   const SigShape& s, cudaStream_t stream, int gen, const T* disp, T* d_disp) {
    if (s.degree < 2 || s.degree > uint64_t(kMaxDegree) || s.dim < 2 || s.full_len >= (1ull << 31)) return false;
    const int sms = device_context(current_device()).sm_count;
    if (s.batch < uint64_t(sms)) return false;
    const LevelIndex lev = make_level_index(s.dim, s.degree);
    const uint64_t low_len = (uint64_t(lev.li[s.degree]) + 6) & ~3ull;
    const size_t base_smem = (4 * low_len + 2 * ((s.dim + 3) & ~3ull)) * sizeof(T);
    if (base_smem > 160 * 1024) return false;
    if (gen == 1) A = nullptr, dA = nullptr;
    if (gen == 2) B = nullptr, dB = nullptr;
    const uint64_t top_off = lev.li[s.degree] - 1;
    auto fits = [&](int vec) {
        const size_t bytes = vec * sizeof(T);
        auto ok = [&](const T* p, uint64_t stride) {
            return p == nullptr || (aligned_to(p + top_off, bytes) && stride % vec == 0);
        };
        return s.dim % vec == 0 && ok(dC, dc_stride) && ok(dA, da_stride) && ok(dB, db_stride);
    };
    // the register-resident path needs power-of-two dimensions (then every vector width that divides d
    // also divides the words per iteration) and at most kChenSplits splits; otherwise the generic path
    int lgd = -1;
    if ((s.dim & (s.dim - 1)) == 0 && s.degree - 1 <= uint64_t(kChenSplits) && s.dim <= uint64_t(kAdjointThreads)) {
        lgd = 0;
        while ((1ull << lgd) < s.dim) ++lgd;
    }
    auto run = [&](auto kernel, int vec) {
        // regular shapes: plus one table entry per iteration of every level (W = threads * vec words each)
        const uint64_t entries = lgd >= 0 ? regular_order_entries(lev, s.degree, kAdjointThreads, vec) : 0;
        const size_t smem = base_smem + entries * sizeof(uint32_t);
        const unsigned per_sm = static_cast<unsigned>(std::max<size_t>(1, std::min<size_t>(8, (220 * 1024) / (smem + 1024))));
        const unsigned grid = static_cast<unsigned>(std::min<uint64_t>(s.batch, uint64_t(sms) * per_sm));
        if (smem > 48 * 1024)
            SIG_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        kernel<<<grid, kAdjointThreads, smem, stream>>>(dC, dc_stride, A, a_stride, B, b_stride, dA, da_stride, dB, db_stride,
                                                     disp, d_disp, gen, s.batch, static_cast<int>(s.degree),
                                                     static_cast<uint32_t>(s.dim), lgd, lev);
        SIG_CUDA_CHECK(cudaGetLastError());
        count_launch();
    };
    auto run_vec = [&](auto vec) {
        constexpr int V = decltype(vec)::value;
        if (lgd < 0) run(chen_adjoints_cta_kernel<T, V, 0>, V);
        else if (s.degree <= 2) run(chen_adjoints_cta_kernel<T, V, 1>, V);
        else if (s.degree <= 4) run(chen_adjoints_cta_kernel<T, V, 3>, V);
        else run(chen_adjoints_cta_kernel<T, V, kChenSplits>, V);
    };
    constexpr int kWide = sizeof(T) == 4 ? 4 : 2;
    if (fits(kWide)) run_vec(std::integral_constant<int, kWide>{});
    else if (fits(2)) run_vec(std::integral_constant<int, 2>{});
    else run_vec(std::integral_constant<int, 1>{});
    return true;
}

template bool launch_chen_adjoints_streamed<float>(const float*, uint64_t, const float*, uint64_t, const float*, uint64_t,
                                                   float*, uint64_t, float*, uint64_t, const SigShape&, cudaStream_t, int,
                                                   const float*, float*);
template bool launch_chen_adjoints_streamed<double>(const double*, uint64_t, const double*, uint64_t, const double*,
                                                    uint64_t, double*, uint64_t, double*, uint64_t, const SigShape&,
                                                    cudaStream_t, int, const double*, double*);

template bool launch_chen_product_streamed<float>(const float*, uint64_t, const float*, uint64_t, const float*, float*,
                                                  uint64_t, const SigShape&, cudaStream_t, bool);
template bool launch_chen_product_streamed<double>(const double*, uint64_t, const double*, uint64_t, const double*,
                                                   double*, uint64_t, const SigShape&, cudaStream_t, bool);

}  // namespace sigb200
