// Register-tile signature kernels for sm_100a: forward Horner sweep and reverse
// (state-reconstructing) sweep, compiled per (dimension, degree, chain length, group).
//
// Mapping.  One CUDA thread = one execution unit of tile_math.h; the units of a path are
// laid out over ceil(UNITS / 32) warps, and every warp works on exactly one path, so all
// 32 lanes read the same increment and shared-memory reads of it are broadcasts.  Warps
// are fully independent: each one stages the increments of CH consecutive steps of its
// path into its own slice of shared memory with coalesced loads, synchronises with
// __syncwarp() only, and then runs the CH steps out of registers.  There is no block-wide
// barrier in either kernel.
//
// Forward: state in registers for the whole path, written once at the end.
// Backward: final signature and seeds loaded into registers; per step the state is
// rewound with the negated increment, the adjoint is pulled back, and the per-unit
// d'-vector of increment gradients is summed over the warp through a shared-memory
// transpose (every lane parks its vector in a row, then each lane sums one column),
// buffered per chunk in shared memory and added to the global increment-gradient buffer
// with one atomic per (step, channel, warp).
//
// These kernels replace the reference's thread-per-prefix kernels
// (siglib/cusig/cu_signature.cu:183-298 signature_per_word_ker,
// siglib/cusig/cu_signature_horner.cuh:219-249 forward_kernel, :309-363 backward_kernel).
#pragma once

#include <cooperative_groups.h>
#include <cuda_pipeline.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "increments.cuh"
#include "tile_math.h"

namespace sigb200 {

constexpr int kTileChunk = 32;  // steps staged per warp and chunk

constexpr int next_pow2_c(int v) {
    int r = 1;
    while (r < v) r *= 2;
    return r;
}

template <typename T> __device__ __forceinline__ T max_finite();
template <> __device__ __forceinline__ float max_finite<float>() { return 3.402823466e+38f; }
template <> __device__ __forceinline__ double max_finite<double>() { return 1.7976931348623157e+308; }

template <typename T> struct VecOf;
template <> struct VecOf<float> { using type = float4; static constexpr int n = 4; };
template <> struct VecOf<double> { using type = double2; static constexpr int n = 2; };

template <typename T, int D>
struct RowPad {
    static constexpr int V = VecOf<T>::n;
    static constexpr int DP = (D + V - 1) / V * V;  // padded row length (elements)
};

// dst[0..n) = src[0..n) with 16-byte shared-memory loads; src must be 16-byte aligned and
// readable up to the next multiple of the vector width.
template <typename T, int n>
__device__ __forceinline__ void load_row_vec(T (&dst)[n], const T* src) {
    using V = typename VecOf<T>::type;
    constexpr int W = VecOf<T>::n;
    constexpr int NV = (n + W - 1) / W;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const V v = reinterpret_cast<const V*>(src)[i];
        const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
        for (int k = 0; k < W; ++k)
            if (i * W + k < n) dst[i * W + k] = e[k];
    }
}

template <typename T, typename Sh>
struct StepOperands {
    T z[Sh::D];
    T zg[Sh::G];
    T zc[Sh::P > 0 ? Sh::P : 1];
};

template <typename T, typename Sh, bool NEGATE>
__device__ __forceinline__ void load_step(StepOperands<T, Sh>& op, const T* row, const UnitIndex<Sh>& ix) {
    load_row_vec<T, Sh::D>(op.z, row);
    if constexpr (Sh::G == Sh::D) {
#pragma unroll
        for (int j = 0; j < Sh::G; ++j) op.zg[j] = op.z[j];
    } else if constexpr (Sh::G % VecOf<T>::n == 0) {
        load_row_vec<T, Sh::G>(op.zg, row + ix.c0);
    } else {
#pragma unroll
        for (int j = 0; j < Sh::G; ++j) op.zg[j] = row[ix.c0 + j];
    }
#pragma unroll
    for (int k = 0; k < Sh::P; ++k) op.zc[k] = row[ix.p[k]];
    if constexpr (NEGATE) {
#pragma unroll
        for (int c = 0; c < Sh::D; ++c) op.z[c] = -op.z[c];
#pragma unroll
        for (int j = 0; j < Sh::G; ++j) op.zg[j] = -op.zg[j];
#pragma unroll
        for (int k = 0; k < Sh::P; ++k) op.zc[k] = -op.zc[k];
    }
}

// Register staging of the increments of steps [j0, j0 + cnt) of a plain float32 path (the forward
// sweep): prefetch() issues the global loads of the next chunk into registers while the current chunk
// is computed, commit() takes the differences and writes them to zs (row stride DP).
template <typename T, typename Sh>
struct ChunkRegs {
    static constexpr int K = (kTileChunk * Sh::D + 31) / 32;  // elements per lane and chunk
    T lo[K];
    T hi[K];
};

template <typename T, typename Sh>
__device__ __forceinline__ void prefetch_increments(ChunkRegs<T, Sh>& r, const T* x, int j0, int cnt, int lane) {
    constexpr int D = Sh::D;
    const T* src = x + size_t(j0) * D;
    const int total = cnt * D;
#pragma unroll
    for (int k = 0; k < ChunkRegs<T, Sh>::K; ++k) {
        const int i = lane + 32 * k;
        if (i < total) {
            r.lo[k] = src[i];
            r.hi[k] = src[i + D];
        }
    }
}

template <typename T, typename Sh>
__device__ __forceinline__ void commit_increments(T* zs, const ChunkRegs<T, Sh>& r, int cnt, int lane) {
    constexpr int D = Sh::D;
    constexpr int DP = RowPad<T, D>::DP;
    const int total = cnt * D;
#pragma unroll
    for (int k = 0; k < ChunkRegs<T, Sh>::K; ++k) {
        const int i = lane + 32 * k;
        if (i < total) {
            const int step = i / D, c = i - step * D;
            zs[step * DP + c] = r.hi[k] - r.lo[k];
        }
    }
}

// The raw points that the steps [j0, j0 + cnt) of a chunk need, staged in shared memory by asynchronous
// copies (fetch) and turned into the chunk's increments once they have arrived (commit).  With lead-lag
// the steps 2m, 2m + 1 both use the points m, m + 1; the time channel needs no data.
template <typename T, bool FLAGS>
struct ChunkPoints {
    const PathView<T>& pv;
    const T* x;
    T* raw;
    int lane;
    __device__ __forceinline__ int first_point(int j0) const { return FLAGS && pv.lead_lag ? j0 >> 1 : j0; }
    __device__ __forceinline__ void fetch(int j0, int cnt) const {
        const int from = first_point(j0);
        const int to = (FLAGS && pv.lead_lag ? (j0 + cnt - 1) >> 1 : j0 + cnt - 1) + 1;   // last point used
        const T* src = x + size_t(from) * pv.d;
        const int total = (to - from + 1) * pv.d;
        for (int i = lane; i < total; i += 32) __pipeline_memcpy_async(raw + i, src + i, sizeof(T));
        __pipeline_commit();
    }
    template <int D, int DP>
    __device__ __forceinline__ void commit(T* zs, int j0, int cnt) const {
        if constexpr (FLAGS) {
            // the generic increment formula, reading the staged points through a shifted base pointer
            const T* shifted = raw - size_t(first_point(j0)) * pv.d;
            for (int i = lane; i < cnt * D; i += 32) {
                const int step = i / D, c = i - step * D;
                zs[step * DP + c] = pv.increment(shifted, j0 + step, c);
            }
        } else {
            for (int i = lane; i < cnt * D; i += 32) {
                const int step = i / D, c = i - step * D;
                zs[step * DP + c] = raw[i + D] - raw[i];
            }
        }
    }
};

// Shared memory of one warp of the forward kernels: the increments of the current chunk and, for
// plain paths, the points of the next one (copied in asynchronously while the current chunk is swept).
template <typename T, int D>
struct ForwardSmem {
    static constexpr int DP = RowPad<T, D>::DP;
    static constexpr int RAW = ((kTileChunk + 1) * D + 3) / 4 * 4;
    static constexpr int PER_WARP = kTileChunk * DP + RAW;
};

// Forward sweep of one unit over the steps [j_begin, j_end) of the path starting at x; zs / raw are the
// warp's slices of shared memory.  The state is (re)initialised by the first step.
template <typename T, typename Sh, bool FLAGS>
__device__ __forceinline__ void tile_sweep_forward(TileState<T, Sh>& st, const PathView<T>& pv, const T* x, int j_begin,
                                                   int j_end, T* zs, T* raw, const UnitIndex<Sh>& ix, int lane) {
    constexpr int D = Sh::D;
    constexpr int DP = RowPad<T, D>::DP;
    StepOperands<T, Sh> op;
    constexpr bool OPERAND_PREFETCH = sizeof(T) == 4 && Sh::TS + 2 * (Sh::D + Sh::G + Sh::P) <= 170;
    // float32 plain paths keep the register prefetch of the next chunk (measured on B200 against the
    // asynchronous copies: C5 forward 48.3 vs 49.4 ms, C3 0.898 vs 0.913 ms); float64 and the flagged
    // paths, where those registers are not to be had, stage the points through shared memory
    // (C1 0.504 -> 0.481 ms, C2 0.580 -> 0.567 ms).
    constexpr bool EAGER = !FLAGS && sizeof(T) == 4;
    ChunkRegs<T, Sh> pre;
    const ChunkPoints<T, FLAGS> points{pv, x, raw, lane};
    if constexpr (EAGER) prefetch_increments<T, Sh>(pre, x, j_begin, min(kTileChunk, j_end - j_begin), lane);
    else if (j_end > j_begin) points.fetch(j_begin, min(kTileChunk, j_end - j_begin));
    for (int j0 = j_begin; j0 < j_end; j0 += kTileChunk) {
        const int cnt = min(kTileChunk, j_end - j0);
        __syncwarp();
        if constexpr (EAGER) {
            commit_increments<T, Sh>(zs, pre, cnt, lane);
            __syncwarp();
            if (j0 + kTileChunk < j_end)
                prefetch_increments<T, Sh>(pre, x, j0 + kTileChunk, min(kTileChunk, j_end - j0 - kTileChunk), lane);
        } else {
            __pipeline_wait_prior(0);
            __syncwarp();
            points.template commit<D, DP>(zs, j0, cnt);
            __syncwarp();
            if (j0 + kTileChunk < j_end) points.fetch(j0 + kTileChunk, min(kTileChunk, j_end - j0 - kTileChunk));
        }
        __syncwarp();
        int step = 0;
        if (j0 == j_begin) {
            load_step<T, Sh, false>(op, zs, ix);
            tile_init_first<T, Sh>(st, op.z, op.zg, op.zc);
            step = 1;
        }
        if constexpr (OPERAND_PREFETCH) {
            // The operands of the next step are loaded before the current step is computed, so
            // the shared-memory latency overlaps with the step's FMAs instead of preceding them.
            if (step < cnt) load_step<T, Sh, false>(op, zs + step * DP, ix);
#pragma unroll 2
            for (; step < cnt; ++step) {
                StepOperands<T, Sh> nxt;
                load_step<T, Sh, false>(nxt, zs + min(step + 1, cnt - 1) * DP, ix);
                tile_update<T, Sh>(st, op.z, op.zg, op.zc);
                op = nxt;
            }
        } else {
            for (; step < cnt; ++step) {
                load_step<T, Sh, false>(op, zs + step * DP, ix);
                tile_update<T, Sh>(st, op.z, op.zg, op.zc);
            }
        }
    }
}

// true when any coefficient the unit holds is NaN / Inf.  Every coefficient of the signature is
// owned by some unit (chain coefficients by all units sharing the prefix, which see the same
// value), so the union over units covers the whole signature.
template <typename T, typename Sh>
__device__ __forceinline__ bool tile_nonfinite(const TileState<T, Sh>& st) {
    bool bad = false;
#pragma unroll
    for (int k = 1; k <= Sh::P; ++k) bad |= !(fabs(st.ch[k]) <= max_finite<T>());
#pragma unroll
    for (int i = 0; i < Sh::TS; ++i) bad |= !(fabs(st.s[i]) <= max_finite<T>());
    return bad;
}

// Forward sweep.  With nseg > 1 every path is cut into nseg time segments that are swept
// independently (more warps for small batches) and written to `seg_out` ((batch, nseg, S),
// scalar-free); Chen-product launches then join them into `out`.
template <typename T, typename Sh, bool FLAGS, int WPB>
__global__ void __launch_bounds__(WPB * 32)
tile_forward_kernel(PathView<T> pv, T* __restrict__ out, T* __restrict__ seg_out, uint64_t batch, uint32_t stride,
                    bool scalar, int nseg, int* __restrict__ nonfinite) {
    constexpr int DP = RowPad<T, Sh::D>::DP;
    constexpr int WPP = (Sh::UNITS + 31) / 32;  // warps per (path, segment)
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    T* zs = reinterpret_cast<T*>(smem_raw) + size_t(warp) * ForwardSmem<T, Sh::D>::PER_WARP;
    T* raw = zs + kTileChunk * DP;

    const uint64_t gw = uint64_t(blockIdx.x) * WPB + warp;
    if (gw >= batch * uint64_t(nseg) * WPP) return;
    const uint64_t vp = gw / WPP;               // virtual path = b * nseg + segment
    const uint64_t b = vp / uint64_t(nseg);
    const int seg = int(vp - b * uint64_t(nseg));
    const int j_begin = int(int64_t(pv.steps) * seg / nseg);
    const int j_end = int(int64_t(pv.steps) * (seg + 1) / nseg);
    const int u = int(gw - vp * WPP) * 32 + lane;
    const bool active = u < Sh::UNITS;
    const UnitIndex<Sh> ix = decode_unit<Sh>(active ? u : 0);
    const T* x = pv.base + b * pv.path_stride;

    TileState<T, Sh> st;
    tile_sweep_forward<T, Sh, FLAGS>(st, pv, x, j_begin, j_end, zs, raw, ix, lane);
    if (active) {
        if (nseg == 1) {
            T* S = out + b * stride - (scalar ? 0 : 1);
            tile_store<T, Sh>(st, ix, S);
            if (scalar && u == 0) S[0] = T(1);
            // NaN / Inf check of what was just stored, on the registers (no pass over the output)
            if (nonfinite != nullptr && tile_nonfinite<T, Sh>(st)) *nonfinite = 1;
        } else {
            const uint32_t slen = stride - (scalar ? 1 : 0);
            T* S = seg_out + vp * slen - 1;
            tile_store<T, Sh>(st, ix, S);
        }
    }
}

// Shape of a fused log-signature launch: a path's units either fill CTAS_PER_PATH whole CTAs (a
// thread-block cluster, so that their shared memories can be written by each other) or several
// paths share one CTA.
template <typename Sh, int WPB>
struct LogSweepShape {
    static constexpr int WPP = (Sh::UNITS + 31) / 32;
    static constexpr int CTAS_PER_PATH = WPP >= WPB ? (WPP + WPB - 1) / WPB : 1;
    static constexpr int PATHS_PER_CTA = WPP >= WPB ? 1 : WPB / WPP;
    static constexpr int LOW = cgeom(Sh::D, Sh::N);   // coefficients of levels 0 .. N-1
};

// Forward sweep with the log-signature epilogue: computes log(signature) without the signature
// ever going to global memory.  The units of a path sweep as in tile_forward_kernel; then every
// unit publishes its coefficients BELOW level N into a shared-memory copy of those levels (a few
// KB per path; when the path spans several CTAs these form a cluster and every unit writes into
// all of their shared memories through distributed shared memory), the cluster synchronises, and
// every unit turns the level-N coefficients it still holds in registers into their logarithm
// (tile_log_top) while the threads share out the levels below N (log_low_prefix).
// `rank` == nullptr: expanded logarithm in the layout of the signature (out_shift = 1 reserves the
// scalar slot, which is 0).  Otherwise rank[p] is the output index of the word at scalar-free
// position p when it is a Lyndon word and -1 when it is not: Lyndon-word coordinates.
template <typename T, typename Sh, bool FLAGS, int WPB>
__global__ void __launch_bounds__(WPB * 32)
tile_forward_log_kernel(PathView<T> pv, T* __restrict__ out, uint64_t batch, uint32_t out_stride, uint32_t out_shift,
                        const int32_t* __restrict__ rank, int* __restrict__ nonfinite) {
    using Lay = LogSweepShape<Sh, WPB>;
    constexpr int D = Sh::D, N = Sh::N, Q = Sh::Q;
    constexpr int DP = RowPad<T, D>::DP;
    constexpr int WPP = Lay::WPP, C = Lay::CTAS_PER_PATH, PPC = Lay::PATHS_PER_CTA, LOW = Lay::LOW;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    T* zs = reinterpret_cast<T*>(smem_raw) + size_t(warp) * ForwardSmem<T, Sh::D>::PER_WARP;
    T* raw = zs + kTileChunk * DP;
    T* low_base = reinterpret_cast<T*>(smem_raw) + size_t(WPB) * ForwardSmem<T, Sh::D>::PER_WARP;

    // which path, which warp of it, which copy of the lower levels
    uint64_t b;
    int wip, slot;
    if constexpr (WPP >= WPB) {
        b = blockIdx.x / C;
        wip = int(blockIdx.x % C) * WPB + warp;
        slot = 0;
    } else {
        slot = warp / WPP;
        b = uint64_t(blockIdx.x) * PPC + slot;
        wip = warp - slot * WPP;
    }
    const bool valid = b < batch && wip < WPP && slot < PPC;
    const int u = wip * 32 + lane;
    const bool active = valid && u < Sh::UNITS;
    const UnitIndex<Sh> ix = decode_unit<Sh>(active ? u : 0);
    T* low = low_base + size_t(slot < PPC ? slot : 0) * LOW;

    TileState<T, Sh> st;
    if (valid) tile_sweep_forward<T, Sh, FLAGS>(st, pv, pv.base + b * pv.path_stride, 0, pv.steps, zs, raw, ix, lane);
    if (active && nonfinite != nullptr && tile_nonfinite<T, Sh>(st)) *nonfinite = 1;

    // levels below N of the whole path, in every CTA that holds units of it
    if constexpr (C > 1) {
        cooperative_groups::cluster_group cluster = cooperative_groups::this_cluster();
        for (int r = 0; r < C; ++r) {
            T* peer = cluster.map_shared_rank(low, r);
            if (active) tile_publish_low<T, Sh>(st, ix, peer);
            if (active && u == 0) peer[0] = T(1);
        }
        cluster.sync();
    } else {
        if (active) tile_publish_low<T, Sh>(st, ix, low);
        if (active && u == 0) low[0] = T(1);
        __syncthreads();
    }

    T* dst = out + b * uint64_t(out_stride);
    auto emit = [&](int pos0, T value) {   // pos0: position in the scalar-free layout
        if (rank == nullptr) dst[out_shift + pos0] = value;
        else {
            const int32_t r = rank[pos0];
            if (r >= 0) dst[r] = value;
        }
    };
    if (active) {
        if (rank == nullptr && out_shift != 0 && u == 0) dst[0] = T(0);
        tile_log_top<T, Sh>(st, ix, low);
        constexpr int top = cgeom(D, N) - 1;   // scalar-free position of the first level-N word
        if constexpr (Q >= 2) {
#pragma unroll
            for (int j = 0; j < Sh::nodes(Q - 1); ++j) {
                const int row = ((ix.pw * D + ix.c0) * cpow(D, Q - 2) + j) * D;
#pragma unroll
                for (int e = 0; e < D; ++e) emit(top + row + e, st.s[Sh::off(Q) + j * D + e]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < Sh::G; ++j) emit(top + ix.pw * D + ix.c0 + j, st.s[j]);
        }
    }
    // the levels below N: their prefixes are shared out over the threads that hold units of the path
    if (valid) {
        int first, stride;
        if constexpr (C > 1) {
            first = int(blockIdx.x % C) * (WPB * 32) + threadIdx.x;
            stride = C * WPB * 32;
        } else {
            first = wip * 32 + lane;
            stride = WPP * 32;
        }
        for (int prefix = first; prefix < cgeom(D, N - 1); prefix += stride)
            log_low_prefix<T, D, N>(low, prefix, [&](int pos, T value) { emit(pos - 1, value); });
    }
}

// Time segmentation of the reverse sweep (small batches): each path is cut into nseg segments
// that are swept by independent warps.  Segment k starts from the signature of the path up to
// its end (seg_sig for k = 0, state for 0 < k < nseg-1, the caller's sig for the last) and
// from the loss adjoint of that signature (adjoint; the caller's sig_derivs for the last).
// All three arrays are (batch, nseg, S) without scalar terms.
template <typename T>
struct BackwardSegments {
    int nseg = 1;
    const T* seg_sig = nullptr;
    const T* state = nullptr;
    const T* adjoint = nullptr;
};

constexpr int next_pow2(int v) { return v <= 1 ? 1 : 2 * next_pow2((v + 1) / 2); }
constexpr int ilog2(int v) { return v <= 1 ? 0 : 1 + ilog2(v / 2); }

// Shared-memory layout of one warp of the backward kernel (elements of T):
//   zs   [kTileChunk][DP]   increments of the chunk
//   gbuf [kTileChunk][D]    warp totals of the increment gradients, flushed once per chunk
//   tbuf [RS][32 rows][ROWP] (+16 between steps)  per-lane gradient vectors of RS steps,
//        written with vector stores and summed column-wise: the cross-lane reduction goes
//        through shared memory with independent loads instead of a chain of shuffles.
template <typename T, int D>
struct BackwardSmem {
    static constexpr int DP = RowPad<T, D>::DP;
    static constexpr int DP2 = next_pow2_c(D);
    static constexpr int RS = DP2 >= 32 ? 1 : 32 / DP2;      // steps per reduction group
    static constexpr int ROWP = DP2 + (DP2 >= 4 ? 4 : 1);    // padded row: conflict-free stores
    static constexpr int SLAB = 32 * ROWP + 16;              // one step; +16 words de-phases the banks
    static constexpr int RAW = ((kTileChunk + 1) * D + 3) / 4 * 4;   // points of the next chunk, copied in asynchronously
    static constexpr int PER_WARP = kTileChunk * (DP + D) + RS * SLAB + RAW;
};

// Resident CTAs per SM the backward kernel is compiled for: shallow float tiles of up to 68 values fit
// state + adjoint in 128 registers, which keeps four CTAs (16 warps) per SM; the reduction's
// shuffle / shared-atomic latencies need those warps more than they need spare registers.
template <typename T, typename Sh>
constexpr int backward_min_ctas() {
    return (sizeof(T) == 4 && Sh::TS <= 68 && Sh::Q <= 2) ? 4 : 1;
}

template <typename T, typename Sh, bool FLAGS, int WPB>
__global__ void __launch_bounds__(WPB * 32, backward_min_ctas<T, Sh>())
tile_backward_kernel(PathView<T> pv, const T* __restrict__ sig, const T* __restrict__ derivs,
                     T* __restrict__ incr_grad, uint64_t batch, uint32_t stride, bool scalar, BackwardSegments<T> segs) {
    constexpr int D = Sh::D, G = Sh::G, P = Sh::P;
    constexpr int DP = RowPad<T, D>::DP;
    constexpr int DP2 = next_pow2(D);
    constexpr int WPP = (Sh::UNITS + 31) / 32;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    using Lay = BackwardSmem<T, D>;
    constexpr int RS = Lay::RS, ROWP = Lay::ROWP, SLAB = Lay::SLAB;
    T* zs = reinterpret_cast<T*>(smem_raw) + size_t(warp) * Lay::PER_WARP;
    T* gbuf = zs + kTileChunk * DP;
    T* tbuf = gbuf + kTileChunk * D;
    T* raw = tbuf + RS * SLAB;

    const int nseg = segs.nseg;
    const uint64_t gw = uint64_t(blockIdx.x) * WPB + warp;
    if (gw >= batch * uint64_t(nseg) * WPP) return;
    const uint64_t vp = gw / WPP;               // virtual path = b * nseg + segment
    const uint64_t b = vp / uint64_t(nseg);
    const int seg = int(vp - b * uint64_t(nseg));
    const int j_begin = int(int64_t(pv.steps) * seg / nseg);
    const int j_end = int(int64_t(pv.steps) * (seg + 1) / nseg);
    const int u = int(gw - vp * WPP) * 32 + lane;
    const bool active = u < Sh::UNITS;
    const UnitIndex<Sh> ix = decode_unit<Sh>(active ? u : 0);
    const T* x = pv.base + b * pv.path_stride;
    T* gout = incr_grad + b * uint64_t(pv.L - 1) * pv.d;

    TileState<T, Sh, false> st;  // the reverse sweep keeps no level-N state (see TileState)
    TileAdjoint<T, Sh> ad;
    {
        // Signature and adjoint at the END of this time segment: the caller's arrays for the last
        // segment, else the prefix states / pulled-back adjoints prepared by the host (scalar-free).
        const uint32_t slen = stride - (scalar ? 1 : 0);
        const T* s_end = sig + b * stride - (scalar ? 0 : 1);
        const T* a_end = derivs + b * stride - (scalar ? 0 : 1);
        if (seg != nseg - 1) {
            s_end = (seg == 0 ? segs.seg_sig : segs.state) + vp * slen - 1;
            a_end = segs.adjoint + vp * slen - 1;
        }
        tile_load<T, Sh, false>(st, ad, ix, s_end, a_end);
    }
    if (!active) {
        // idle lanes carry a zero adjoint so that they add nothing to the warp sums
#pragma unroll
        for (int k = 0; k <= P; ++k) ad.ac[k] = T(0);
#pragma unroll
        for (int i = 0; i < Sh::TS; ++i) ad.a[i] = T(0);
    }

    // Warp-wide sum of one step's per-unit gradients into gbuf[step][letter] (every entry of the
    // chunk is written exactly once, by the lane that sums its column).
    auto reduce_step = [&](T (&v)[DP2], const T* gg, const T* gc, int step, int cnt) {
        // (1) letters with static indices:
        // every lane parks its vector in its own row of tbuf; once the RS steps of a group are
        // there, each lane sums one column (one letter of one step) over the 32 rows.
        {
            T* row = tbuf + (step % RS) * SLAB + lane * ROWP;
            if constexpr (DP2 >= 4) {
                using V = typename VecOf<T>::type;
                constexpr int W = VecOf<T>::n;
#pragma unroll
                for (int i = 0; i < DP2 / W; ++i) {
                    V pack;
                    T* e = reinterpret_cast<T*>(&pack);
#pragma unroll
                    for (int k = 0; k < W; ++k) e[k] = v[i * W + k];
                    reinterpret_cast<V*>(row)[i] = pack;
                }
            } else {
#pragma unroll
                for (int c = 0; c < DP2; ++c) row[c] = v[c];
            }
        }
        // The letters that depend on the unit (its own children c0 + j, its chain letters p[k])
        // are added to the lane's private row in place: plain read-modify-write, no atomics.
        {
            T* row = tbuf + (step % RS) * SLAB + lane * ROWP;
            if constexpr (G % VecOf<T>::n == 0 && DP2 >= 4) {
                using V = typename VecOf<T>::type;
                constexpr int W = VecOf<T>::n;
#pragma unroll
                for (int i = 0; i < G / W; ++i) {
                    V pack = reinterpret_cast<V*>(row + ix.c0)[i];
                    T* e = reinterpret_cast<T*>(&pack);
#pragma unroll
                    for (int k = 0; k < W; ++k) e[k] += gg[i * W + k];
                    reinterpret_cast<V*>(row + ix.c0)[i] = pack;
                }
            } else {
#pragma unroll
                for (int j = 0; j < G; ++j) row[ix.c0 + j] += gg[j];
            }
#pragma unroll
            for (int k = 0; k < P; ++k) row[ix.p[k]] += gc[k];
        }
        if (step % RS == 0) {
            const int in_group = min(RS, cnt - step);
            __syncwarp();
            if constexpr (DP2 < 32) {
                const int sl = lane / DP2, c = lane % DP2;
                if (sl < in_group && c < D) {
                    const T* col = tbuf + sl * SLAB + c;
                    T a0 = T(0), a1 = T(0), a2 = T(0), a3 = T(0);
#pragma unroll
                    for (int r = 0; r < 32; r += 4) {
                        a0 += col[(r + 0) * ROWP];
                        a1 += col[(r + 1) * ROWP];
                        a2 += col[(r + 2) * ROWP];
                        a3 += col[(r + 3) * ROWP];
                    }
                    gbuf[(step + sl) * D + c] = (a0 + a1) + (a2 + a3);   // the only writer of this (step, letter)
                }
            } else {
#pragma unroll
                for (int i = 0; i < DP2 / 32; ++i) {
                    const int c = lane + 32 * i;
                    if (c < D) {
                        const T* col = tbuf + c;
                        T a0 = T(0), a1 = T(0);
#pragma unroll
                        for (int r = 0; r < 32; r += 2) {
                            a0 += col[(r + 0) * ROWP];
                            a1 += col[(r + 1) * ROWP];
                        }
                        gbuf[step * D + c] = a0 + a1;
                    }
                }
            }
            __syncwarp();
        }
    };

    // (Neither a register prefetch of the next chunk nor a one-step-late reduction pays here:
    // both were measured on B200 and cost a resident CTA per SM, 233 -> 293 ms on the C5 shape.)
    StepOperands<T, Sh> op;
    // The points of a chunk come into shared memory with asynchronous copies issued one chunk ahead
    // (no registers held across the steps), so the global-memory latency of a chunk lies under the
    // arithmetic of the chunk before it; the increments are then built from shared values.
    const ChunkPoints<T, FLAGS> points{pv, x, raw, lane};
    if (j_end > j_begin) {
        const int first = max(j_begin, j_end - kTileChunk);
        points.fetch(first, j_end - first);
    }
    for (int j1 = j_end; j1 > j_begin;) {
        const int j0 = max(j_begin, j1 - kTileChunk);
        const int cnt = j1 - j0;
        __syncwarp();
        __pipeline_wait_prior(0);
        __syncwarp();
        points.template commit<D, DP>(zs, j0, cnt);
        __syncwarp();
        if (j0 > j_begin) {
            const int next = max(j_begin, j0 - kTileChunk);
            points.fetch(next, j0 - next);
        }
        __syncwarp();
        for (int step = cnt - 1; step >= 0; --step) {
            load_step<T, Sh, false>(op, zs + step * DP, ix);
            {
                // rewind to the state before this step: Horner step with the negated increment
                // (the negations fold into the operand modifiers of the consuming instructions)
                StepOperands<T, Sh> neg;
#pragma unroll
                for (int c = 0; c < D; ++c) neg.z[c] = -op.z[c];
#pragma unroll
                for (int j = 0; j < G; ++j) neg.zg[j] = -op.zg[j];
#pragma unroll
                for (int k = 0; k < P; ++k) neg.zc[k] = -op.zc[k];
                tile_update<T, Sh, false>(st, neg.z, neg.zg, neg.zc);
            }
            TileGrad<T, Sh> g;
#pragma unroll
            for (int c = 0; c < D; ++c) g.gz[c] = T(0);
#pragma unroll
            for (int j = 0; j < G; ++j) g.gg[j] = T(0);
#pragma unroll
            for (int k = 0; k < (P > 0 ? P : 1); ++k) g.gc[k] = T(0);
            tile_pullback<T, Sh, false>(st, ad, g, op.z, op.zg, op.zc);

            T v[DP2];
#pragma unroll
            for (int c = 0; c < DP2; ++c) v[c] = c < D ? g.gz[c] : T(0);
            reduce_step(v, g.gg, g.gc, step, cnt);
        }
        __syncwarp();
        // flush the chunk: one atomic per (step, channel)
        for (int i = lane; i < cnt * D; i += 32) {
            const int step = i / D, c = i - step * D;
            const int j = j0 + step;
            int m, cc;
            bool keep;
            if constexpr (FLAGS) {
                if (pv.lead_lag) {
                    m = j >> 1;
                    const bool odd = j & 1;
                    keep = odd ? (c < pv.d) : (c >= pv.d && c < 2 * pv.d);
                    cc = odd ? c : c - pv.d;
                } else {
                    m = j;
                    cc = c;
                    keep = c < pv.d;
                }
            } else {
                m = j;
                cc = c;
                keep = true;
            }
            if (keep) atomicAdd(gout + size_t(m) * pv.d + cc, gbuf[i]);
        }
        j1 = j0;
    }
}

}  // namespace sigb200
