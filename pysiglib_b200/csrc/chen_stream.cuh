// Device code shared by the one-CTA-per-signature kernels that stream a tensor level by level
// (sig_chen.cu: Chen products and their adjoints; sig_log_stream.cu: the backward pass of the tensor
// logarithm): vector packs, lane-group sums, and the adjoint of a truncated tensor product for
// power-of-two dimensions with all partial sums in registers.
#pragma once

#include <algorithm>
#include <cstdint>

#include "kernels.h"

namespace sigb200 {

namespace {

constexpr int kChenThreads = 256;
// CTA size, CTAs per SM and vector loads in flight per thread of the adjoint kernels.  Measured on
// B200 at d = 16, degree 4 (sig_combine backward): 256 x 3 x 4 -> 1.25 ms; 512 threads x 2 CTAs -> 1.52-1.56 ms;
// 8 loads in flight -> 1.38 ms.
constexpr int kAdjointThreads = 256;
constexpr int kAdjointCtas = 3;
constexpr int kAdjointLoads = 4;
constexpr int kChenSplits = 7;    // register-resident suffix sums of the adjoint kernel: degrees up to 8

template <typename T> __device__ __forceinline__ T chen_fma(T a, T b, T c);
template <> __device__ __forceinline__ float chen_fma<float>(float a, float b, float c) { return fmaf(a, b, c); }
template <> __device__ __forceinline__ double chen_fma<double>(double a, double b, double c) { return fma(a, b, c); }

template <typename T, int VEC> struct Pack;
template <> struct Pack<float, 4> { using type = float4; };
template <> struct Pack<float, 2> { using type = float2; };
template <> struct Pack<float, 1> { using type = float; };
template <> struct Pack<double, 2> { using type = double2; };
template <> struct Pack<double, 1> { using type = double; };

__device__ __forceinline__ void unpack(const float4& p, float* v) { v[0] = p.x; v[1] = p.y; v[2] = p.z; v[3] = p.w; }
__device__ __forceinline__ void unpack(const float2& p, float* v) { v[0] = p.x; v[1] = p.y; }
__device__ __forceinline__ void unpack(const float& p, float* v) { v[0] = p; }
__device__ __forceinline__ void unpack(const double2& p, double* v) { v[0] = p.x; v[1] = p.y; }
__device__ __forceinline__ void unpack(const double& p, double* v) { v[0] = p; }

// Sum over groups of `width` consecutive lanes (a power of two, at most 32); every lane of the warp calls.
template <typename T>
__device__ __forceinline__ T group_sum(T x, uint32_t width) {
    // width is uniform over the warp; predicated steps measured faster than a switch over fixed widths
    if (width >= 32) x += __shfl_xor_sync(0xffffffffu, x, 16);
    if (width >= 16) x += __shfl_xor_sync(0xffffffffu, x, 8);
    if (width >= 8) x += __shfl_xor_sync(0xffffffffu, x, 4);
    if (width >= 4) x += __shfl_xor_sync(0xffffffffu, x, 2);
    if (width >= 2) x += __shfl_xor_sync(0xffffffffu, x, 1);
    return x;
}

// Threads take VEC consecutive words each, a warp 32 * VEC consecutive words starting at a multiple of
// that.  For blocks of `block` consecutive words (block a multiple of VEC, blocks starting at
// multiples of block): the number of consecutive lanes that always lie in one block, as a power of two
// (32: the whole warp), or 0 when lanes of one shuffle group could straddle two blocks.
__device__ __forceinline__ uint32_t lanes_per_block(uint32_t block, uint32_t vec) {
    if (block % (32 * vec) == 0) return 32;
    const uint32_t per = block / vec;
    return (block % vec == 0 && per < 32 && (per & (per - 1)) == 0) ? per : 0;
}

__device__ __forceinline__ float4 make_pack(const float (&v)[4]) { return make_float4(v[0], v[1], v[2], v[3]); }
__device__ __forceinline__ float2 make_pack(const float (&v)[2]) { return make_float2(v[0], v[1]); }
__device__ __forceinline__ float make_pack(const float (&v)[1]) { return v[0]; }
__device__ __forceinline__ double2 make_pack(const double (&v)[2]) { return make_double2(v[0], v[1]); }
__device__ __forceinline__ double make_pack(const double (&v)[1]) { return v[0]; }

// Loaders of the incoming gradient for adjoint_levels_regular, addressed by the position in a
// signature without scalar term: a dense array in global memory (g: the first level-1 coefficient) ...
template <typename T, int VEC>
struct DenseGlobalLoader {
    using P = typename Pack<T, VEC>::type;
    const T* g;
    static constexpr bool kTwoPhase = false;
    struct Handle {};
    __device__ __forceinline__ P vec(uint32_t pos) const { return *reinterpret_cast<const P*>(g + pos); }
    __device__ __forceinline__ T one(uint32_t c) const { return g[c]; }
    // hint: the line holding position pos will be read a few iterations from now
    __device__ __forceinline__ void prefetch(uint32_t pos) const { asm volatile("prefetch.global.L2 [%0];" ::"l"(g + pos)); }
};

// ... and an array in shared memory with scalar-term addressing (q[1 + position], every level on a
// vector boundary).
template <typename T, int VEC>
struct SharedLoader {
    using P = typename Pack<T, VEC>::type;
    const T* q;
    static constexpr bool kTwoPhase = false;
    struct Handle {};
    __device__ __forceinline__ P vec(uint32_t pos) const { return *reinterpret_cast<const P*>(q + 1 + pos); }
    __device__ __forceinline__ T one(uint32_t c) const { return q[1 + c]; }
    __device__ __forceinline__ void prefetch(uint32_t) const {}
};

template <typename T>
struct AdjointShared {
    T* a_low;            // levels 0 .. N-1 of A and B (scalar-term addressing)
    T* b_low;
    T* da_low;           // accumulators of the same shape
    T* db_low;
    T* vs;               // gen != 0: the displacement, the accumulator of its adjoint
    T* dvs;
    const uint32_t* order;     // regular shapes: the iteration order of every level, order[ord_off[m] + n]
    const uint32_t* ord_off;
    const uint32_t* li;
};

// The iteration order of level m for regular shapes: iteration n of 2^tb takes the words of block
// `it`, where the bit fields of `it` between consecutive log2(p_i) are filled from the bits of n with
// the highest field fastest (lgw = log2(W)).
__device__ __forceinline__ uint32_t regular_iteration(uint32_t n, int m, uint32_t tb, int lgd, uint32_t lgw) {
    uint32_t it = 0, pos = 0, hi = tb;
    for (int i = 1; i < m && hi > 0; ++i) {
        const int e_signed = (m - i) * lgd - int(lgw);
        const uint32_t e = e_signed > 0 ? uint32_t(e_signed) : 0u;
        if (e < hi) {
            it |= ((n >> pos) & ((1u << (hi - e)) - 1u)) << e;
            pos += hi - e;
            hi = e;
        }
    }
    return it;
}

// Regular shapes: d and the words per iteration W = nt * VEC are powers of two and N - 1 <= NS.
// Level after level from the top, each streamed in an order that keeps every suffix sum in registers.
// For the split after i letters of a level-m word a thread's suffix offset r depends only on
// it mod p_i, p_i = max(1, d^(m-i) / W), `it` the iteration; the iterations run with the low bit fields
// of `it` slowest, so r changes only p_i times per level and the partial sum is added to shared memory
// then.  Prefix sums are pre-reduced by shuffles over the lanes that share the prefix; where those lanes
// cover the prefix's whole block the sum has a single owner and needs no atomic.  Global loads are
// issued kBatch iterations at a time: a warp has that many vector loads in flight before it starts on
// the arithmetic of the first.
//
// The incoming gradient dC comes through `load` (load.vec(p): the VEC words from scalar-free position p,
// i.e. position p + 1 with a scalar term; load.one(c): letter c of level 1).  Levels 2 .. top_level are processed; the words of the top level
// are stored to da_top / db_top (each may be nullptr) when top_in_global, every other level adds
// a_direct * dC to da_low and b_direct * dC to db_low (the products with the scalar term 1 of the
// other factor: 1 for a Chen product, none for a product without scalar terms).  N is the degree of the
// signatures (only used when gen != 0, where top_level == N).
template <typename T, int VEC, int NS, typename Loader>
__device__ __forceinline__ void adjoint_levels_regular(const AdjointShared<T>& sm, const Loader& load, int top_level,
                                                       bool top_in_global, T* __restrict__ da_top,
                                                       T* __restrict__ db_top, T a_direct, T b_direct, int gen, int N,
                                                       uint32_t d, int lgd, T (&lastv)[VEC]) {
    using P = typename Pack<T, VEC>::type;
    constexpr int kBatch = kAdjointLoads;
    const uint32_t tid = threadIdx.x, nt = blockDim.x, lane = tid & 31;
    const uint32_t* li = sm.li;
    const uint32_t lgw = 31 - __clz(nt * VEC);
    const uint32_t first = tid * VEC;                      // this thread's word inside an iteration
    const T* x_low = gen == 1 ? sm.a_low : sm.b_low;       // the generated factor and its adjoint
    T* dx_low = gen == 1 ? sm.da_low : sm.db_low;
    const T rn = T(1) / T(N);
    // Per split q (d^(q+1) words per prefix), independent of the level: everything the iteration loop
    // needs is read from the level table once, here; the loop itself touches shared memory only for
    // operands and accumulators.
    uint32_t sh[NS], share[NS], flush_mask[NS];
    const T* b_at[NS];                                     // suffix operands of split q: level q + 1 of B
    T* db_at[NS];
    bool owner[NS];
#pragma unroll
    for (int q = 0; q < NS; ++q) {
        sh[q] = uint32_t(q + 1) * uint32_t(lgd);
        if (sh[q] > 31) sh[q] = 31;                        // splits beyond the degree: never used
        share[q] = lanes_per_block(1u << sh[q], VEC);      // never 0: powers of two
        owner[q] = share[q] * VEC == (1u << sh[q]);
        flush_mask[q] = sh[q] > lgw ? (1u << (sh[q] - lgw)) - 1u : 0u;
        const uint32_t level = q + 1 < uint32_t(top_level) ? q + 1 : 1;
        b_at[q] = sm.b_low + li[level];
        db_at[q] = sm.db_low + li[level];
    }
    const uint32_t gen_share = lanes_per_block(d, VEC);
    for (int m = top_level; m >= 2; --m) {
        const bool is_top = top_in_global && m == top_level;
        const uint32_t li_m = li[m];
        const uint32_t words = li[m + 1] - li_m;
        const uint32_t tb = words > nt * VEC ? (31 - __clz(words)) - lgw : 0;   // log2(iterations)
        const uint32_t iters = 1u << tb;
        const T* a_at[NS];                                 // prefix operands of split q: level m - 1 - q of A
        T* da_at[NS];
#pragma unroll
        for (int q = 0; q < NS; ++q) {
            const uint32_t level = m - 1 - q >= 1 ? m - 1 - q : 1;
            a_at[q] = sm.a_low + li[level];
            da_at[q] = sm.da_low + li[level];
        }
        T* da_own = sm.da_low + li_m;
        T* db_own = sm.db_low + li_m;
        const T* x_push = x_low + li[N - 1];
        T* dx_push = dx_low + li[N - 1];
        T acc[NS][VEC];
#pragma unroll
        for (int q = 0; q < NS; ++q)
#pragma unroll
            for (int k = 0; k < VEC; ++k) acc[q][k] = T(0);
        uint32_t prev_it = 0;
        const uint32_t* order = sm.order + sm.ord_off[m];
        auto flush = [&](int q, uint32_t it_of_sum) {
            const uint32_t r = ((it_of_sum << lgw) + first) & ((1u << sh[q]) - 1u);
            T* dst = db_at[q] + r;
#pragma unroll
            for (int k = 0; k < VEC; ++k) {
                atomicAdd(dst + k, acc[q][k]);
                acc[q][k] = T(0);
            }
        };
        // loaders that read through an index table issue the table reads one batch ahead
        typename Loader::Handle ahead[kBatch];
        if constexpr (Loader::kTwoPhase) {
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const uint32_t idx = ((uint32_t(u) < iters ? order[u] : 0u) << lgw) + first;
                ahead[u] = load.issue(li_m - 1 + (idx < words ? idx : 0u));
            }
        }
        for (uint32_t n0 = 0; n0 < iters; n0 += kBatch) {
            P v[kBatch];
            uint32_t its[kBatch];
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                its[u] = n0 + u < iters ? order[n0 + u] : 0u;
                const uint32_t idx = (its[u] << lgw) + first;
                v[u] = P{};
                if constexpr (Loader::kTwoPhase) {
                    if (n0 + u < iters && idx < words) v[u] = load.finish(ahead[u]);
                } else {
                    if (n0 + u < iters && idx < words) v[u] = load.vec(li_m - 1 + idx);
                    // the same words of the next batch: into L2 now (one lane per 128-byte line)
                    if (n0 + kBatch + u < iters && (first * sizeof(T)) % 128 == 0)
                        load.prefetch(li_m - 1 + (order[n0 + kBatch + u] << lgw) + first);
                }
            }
            if constexpr (Loader::kTwoPhase) {
#pragma unroll
                for (int u = 0; u < kBatch; ++u) {
                    const uint32_t nn = n0 + kBatch + u;
                    const uint32_t idx = ((nn < iters ? order[nn] : 0u) << lgw) + first;
                    ahead[u] = load.issue(li_m - 1 + (idx < words ? idx : 0u));
                }
            }
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                if (n0 + u >= iters) break;                // uniform over the CTA
                const uint32_t it = its[u];
                const uint32_t idx = (it << lgw) + first;
                const bool valid = idx < words;
                const uint32_t at = valid ? idx : 0;
                T gv[VEC];
                unpack(v[u], gv);
                if (valid) {
                    if (is_top) {
                        if (da_top) *reinterpret_cast<P*>(da_top + idx) = v[u];
                        if (db_top) *reinterpret_cast<P*>(db_top + idx) = v[u];
                    } else {                               // this thread owns these accumulators during this level
#pragma unroll
                        for (int k = 0; k < VEC; ++k) {
                            if (a_direct != T(0)) da_own[idx + k] += a_direct * gv[k];
                            if (b_direct != T(0)) db_own[idx + k] += b_direct * gv[k];
                        }
                    }
                }
                const uint32_t changed = it ^ prev_it;
#pragma unroll
                for (int q = 0; q < NS; ++q) {
                    if (m - 1 - q >= 1) {                  // split after m - 1 - q letters
                        const uint32_t left = at >> sh[q], r = at & ((1u << sh[q]) - 1u);
                        const T al = a_at[q][left];
                        T bs[VEC];
                        unpack(*reinterpret_cast<const P*>(b_at[q] + r), bs);
                        T sa = T(0);
#pragma unroll
                        for (int k = 0; k < VEC; ++k) sa = chen_fma(gv[k], bs[k], sa);
                        sa = group_sum(sa, share[q]);
                        if ((lane & (share[q] - 1)) == 0 && valid) {
                            if (owner[q]) da_at[q][left] += sa;   // the only contribution of this level
                            else atomicAdd(&da_at[q][left], sa);
                        }
                        if (changed & flush_mask[q]) flush(q, prev_it);
#pragma unroll
                        for (int k = 0; k < VEC; ++k) acc[q][k] = chen_fma(al, gv[k], acc[q][k]);
                    }
                }
                prev_it = it;
                if (gen && is_top) {
                    // X_N = dC_N: its push-down into X_{N-1}[prefix] and its term of dv[last letter]
                    const uint32_t q = at >> lgd, c0 = at & (d - 1);
                    T push = T(0);
#pragma unroll
                    for (int k = 0; k < VEC; ++k) push = chen_fma(sm.vs[c0 + k], gv[k], push);
                    push = group_sum(push * rn, gen_share);
                    if ((lane & (gen_share - 1)) == 0 && valid) atomicAdd(&dx_push[q], push);
                    const T xl = x_push[q] * rn;
#pragma unroll
                    for (int k = 0; k < VEC; ++k) lastv[k] = chen_fma(xl, gv[k], lastv[k]);
                }
            }
        }
#pragma unroll
        for (int q = 0; q < NS; ++q)
            if (m - 1 - q >= 1) flush(q, prev_it);
        __syncthreads();
    }
    for (uint32_t c = tid; c < d; c += nt) {               // level 1 of dC
        const T g1 = load.one(c);
        if (a_direct != T(0)) sm.da_low[1 + c] += a_direct * g1;
        if (b_direct != T(0)) sm.db_low[1 + c] += b_direct * g1;
    }
    if (gen) {
        const uint32_t c0 = first & (d - 1);
#pragma unroll
        for (int k = 0; k < VEC; ++k) atomicAdd(&sm.dvs[c0 + k], lastv[k]);
    }
}

// Fills the iteration-order table of adjoint_levels_regular for levels 2 .. N (the same for every
// signature of a launch); ends with a barrier.  Returns nothing: order / ord_off are shared memory.
__device__ __forceinline__ void fill_regular_order(uint32_t* order, uint32_t* ord_off, const uint32_t* li, int N, int vec,
                                                   int lgd) {
    const uint32_t tid = threadIdx.x, nt = blockDim.x;
    const uint32_t lgw = 31 - __clz(nt * vec);
    uint32_t off = 0;
    for (int m = N; m >= 2; --m) {
        const uint32_t words = li[m + 1] - li[m];
        const uint32_t tb = words > nt * vec ? (31 - __clz(words)) - lgw : 0;
        if (tid == 0) ord_off[m] = off;
        for (uint32_t n = tid; n < (1u << tb); n += nt) order[off + n] = regular_iteration(n, m, tb, lgd, lgw);
        off += 1u << tb;
    }
    __syncthreads();
}

}  // namespace

// Host side: entries of that table for a signature of `degree` levels over `dim` letters.
inline uint64_t regular_order_entries(const LevelIndex& lev, uint64_t degree, int threads, int vec) {
    uint64_t entries = 0;
    for (uint64_t m = 2; m <= degree; ++m)
        entries += std::max<uint64_t>(1, (uint64_t(lev.li[m + 1]) - lev.li[m]) / (uint64_t(threads) * vec));
    return entries;
}

}  // namespace sigb200
