// Host launchers and the registry entry type of the register-tile kernels.
#pragma once

#include <vector>

#include "kernels.h"
#include "runtime.h"
#include "sig_tile.cuh"

namespace sigb200 {

constexpr int kTileWarpsPerBlock = 4;

struct TileEntry {
    bool is_double;
    bool backward;
    int D, N, P, G;
    int units;       // execution units (threads) per path
    int tile_values; // register-resident coefficients per unit
    int est_instr;   // estimated issue slots per unit and step (cost model)
    int (*occupancy)(bool flags);  // resident CTAs per SM of the kernel on the current device
    // forward:  fn(pv, out, nullptr, nullptr, ...);  backward: fn(pv, incr_grad, sig, derivs, ...)
    // nseg / seg_out: time segmentation of the forward sweep (1 / nullptr = off; ignored backward)
    // nonfinite: device int set to 1 by an unsegmented forward sweep that stores NaN / Inf (nullptr = no check)
    void (*launch)(const void* pv, void* out, const void* sig, const void* derivs, uint64_t batch,
                   uint32_t stride, bool scalar, bool flags, int nseg, void* seg_out, int* nonfinite,
                   cudaStream_t stream);
    // Forward sweep with the log-signature epilogue (tile_forward_log_kernel); nullptr when it is not
    // compiled for this variant.  Returns false (nothing launched) when the shape does not fit: a
    // path must span at most 8 CTAs (portable cluster size) and the shared copy of the lower levels
    // must fit beside the increments.
    bool (*launch_log)(const void* pv, void* out, uint64_t batch, uint32_t out_stride, uint32_t out_shift,
                       const int32_t* rank, bool flags, int* nonfinite, cudaStream_t stream);
};

inline unsigned tile_grid(uint64_t batch, int units) {
    const uint64_t warps = batch * uint64_t((units + 31) / 32);
    const uint64_t blocks = (warps + kTileWarpsPerBlock - 1) / kTileWarpsPerBlock;
    if (blocks > 0x7fffffffull) throw std::out_of_range("launch grid too large");
    return static_cast<unsigned>(blocks);
}

template <typename Kernel>
inline void tile_set_smem(Kernel kernel, size_t smem) {
    if (smem > 48 * 1024)
        SIG_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
}

template <typename T, int D, int N, int P, int G>
void tile_forward_launch(const void* pv_, void* out, const void*, const void*, uint64_t batch, uint32_t stride,
                         bool scalar, bool flags, int nseg, void* seg_out, int* nonfinite, cudaStream_t stream) {
    using Sh = TileShape<D, N, P, G>;
    constexpr int W = kTileWarpsPerBlock;
    const PathView<T>& pv = *static_cast<const PathView<T>*>(pv_);
    const size_t smem = size_t(W) * ForwardSmem<T, D>::PER_WARP * sizeof(T);
    const unsigned grid = tile_grid(batch * uint64_t(nseg), Sh::UNITS);
    if (flags) {
        tile_set_smem(tile_forward_kernel<T, Sh, true, W>, smem);
        tile_forward_kernel<T, Sh, true, W><<<grid, W * 32, smem, stream>>>(pv, static_cast<T*>(out), static_cast<T*>(seg_out), batch, stride, scalar, nseg, nonfinite);
    } else {
        tile_set_smem(tile_forward_kernel<T, Sh, false, W>, smem);
        tile_forward_kernel<T, Sh, false, W><<<grid, W * 32, smem, stream>>>(pv, static_cast<T*>(out), static_cast<T*>(seg_out), batch, stride, scalar, nseg, nonfinite);
    }
    SIG_CUDA_CHECK(cudaGetLastError());
    count_launch();
}

template <typename T, int D, int N, int P, int G>
void tile_backward_launch(const void* pv_, void* incr_grad, const void* sig, const void* derivs, uint64_t batch,
                          uint32_t stride, bool scalar, bool flags, int nseg, void* segments, int* /*nonfinite*/,
                          cudaStream_t stream) {
    using Sh = TileShape<D, N, P, G>;
    constexpr int W = kTileWarpsPerBlock;
    const PathView<T>& pv = *static_cast<const PathView<T>*>(pv_);
    const size_t smem = size_t(W) * BackwardSmem<T, D>::PER_WARP * sizeof(T);
    BackwardSegments<T> segs;
    if (nseg > 1 && segments) segs = *static_cast<const BackwardSegments<T>*>(segments);
    const unsigned grid = tile_grid(batch * uint64_t(segs.nseg), Sh::UNITS);
    if (flags) {
        tile_set_smem(tile_backward_kernel<T, Sh, true, W>, smem);
        tile_backward_kernel<T, Sh, true, W><<<grid, W * 32, smem, stream>>>(
            pv, static_cast<const T*>(sig), static_cast<const T*>(derivs), static_cast<T*>(incr_grad), batch, stride,
            scalar, segs);
    } else {
        tile_set_smem(tile_backward_kernel<T, Sh, false, W>, smem);
        tile_backward_kernel<T, Sh, false, W><<<grid, W * 32, smem, stream>>>(
            pv, static_cast<const T*>(sig), static_cast<const T*>(derivs), static_cast<T*>(incr_grad), batch, stride,
            scalar, segs);
    }
    SIG_CUDA_CHECK(cudaGetLastError());
    count_launch();
}

template <typename T, int D, int N, int P, int G>
bool tile_forward_log_launch(const void* pv_, void* out, uint64_t batch, uint32_t out_stride, uint32_t out_shift,
                             const int32_t* rank, bool flags, int* nonfinite, cudaStream_t stream) {
    using Sh = TileShape<D, N, P, G>;
    constexpr int W = kTileWarpsPerBlock;
    using Lay = LogSweepShape<Sh, W>;
    const PathView<T>& pv = *static_cast<const PathView<T>*>(pv_);
    const size_t smem = (size_t(W) * ForwardSmem<T, D>::PER_WARP + size_t(Lay::PATHS_PER_CTA) * Lay::LOW) * sizeof(T);
    // deep tiles (many rows of level-N coefficients per unit) would turn the unrolled epilogue into
    // indexed register access; they take the two-step route
    constexpr bool shallow = Sh::Q <= 3 && (Sh::Q < 2 || Sh::nodes(Sh::Q - 1) <= 16);
    if (!shallow || Lay::CTAS_PER_PATH > 8 || smem > 200 * 1024) return false;
    const uint64_t blocks = Lay::CTAS_PER_PATH > 1 ? batch * Lay::CTAS_PER_PATH
                                                   : (batch + Lay::PATHS_PER_CTA - 1) / Lay::PATHS_PER_CTA;
    if (blocks > 0x7fffffffull) throw std::out_of_range("launch grid too large");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(blocks));
    cfg.blockDim = dim3(W * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = Lay::CTAS_PER_PATH;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = Lay::CTAS_PER_PATH > 1 ? 1 : 0;
    T* dst = static_cast<T*>(out);
    if (flags) {
        tile_set_smem(tile_forward_log_kernel<T, Sh, true, W>, smem);
        SIG_CUDA_CHECK(cudaLaunchKernelEx(&cfg, tile_forward_log_kernel<T, Sh, true, W>, pv, dst, batch, out_stride, out_shift,
                                          rank, nonfinite));
    } else {
        tile_set_smem(tile_forward_log_kernel<T, Sh, false, W>, smem);
        SIG_CUDA_CHECK(cudaLaunchKernelEx(&cfg, tile_forward_log_kernel<T, Sh, false, W>, pv, dst, batch, out_stride, out_shift,
                                          rank, nonfinite));
    }
    SIG_CUDA_CHECK(cudaGetLastError());
    count_launch();
    return true;
}

template <typename Kernel>
inline int tile_occupancy_of(Kernel kernel, size_t smem) {
    tile_set_smem(kernel, smem);
    int n = 0;
    SIG_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, kTileWarpsPerBlock * 32, smem));
    return n > 0 ? n : 1;
}

template <typename T, int D, int N, int P, int G>
int tile_forward_occupancy(bool flags) {
    using Sh = TileShape<D, N, P, G>;
    const size_t smem = size_t(kTileWarpsPerBlock) * ForwardSmem<T, D>::PER_WARP * sizeof(T);
    return flags ? tile_occupancy_of(tile_forward_kernel<T, Sh, true, kTileWarpsPerBlock>, smem)
                 : tile_occupancy_of(tile_forward_kernel<T, Sh, false, kTileWarpsPerBlock>, smem);
}

template <typename T, int D, int N, int P, int G>
int tile_backward_occupancy(bool flags) {
    using Sh = TileShape<D, N, P, G>;
    const size_t smem = size_t(kTileWarpsPerBlock) * BackwardSmem<T, D>::PER_WARP * sizeof(T);
    return flags ? tile_occupancy_of(tile_backward_kernel<T, Sh, true, kTileWarpsPerBlock>, smem)
                 : tile_occupancy_of(tile_backward_kernel<T, Sh, false, kTileWarpsPerBlock>, smem);
}

// BWD: 0 forward, 1 backward; LOG: 1 = also compile the fused log-signature sweep (forward only)
template <typename T, int D, int N, int P, int G, int BWD, int LOG>
TileEntry make_tile_entry(int est_instr) {
    using Sh = TileShape<D, N, P, G>;
    TileEntry e{sizeof(T) == 8, BWD != 0, D, N, P, G, Sh::UNITS, Sh::TS, est_instr, nullptr, nullptr, nullptr};
    if constexpr (BWD != 0) {
        e.occupancy = &tile_backward_occupancy<T, D, N, P, G>;
        e.launch = &tile_backward_launch<T, D, N, P, G>;
    } else {
        e.occupancy = &tile_forward_occupancy<T, D, N, P, G>;
        e.launch = &tile_forward_launch<T, D, N, P, G>;
        if constexpr (LOG != 0) e.launch_log = &tile_forward_log_launch<T, D, N, P, G>;
    }
    return e;
}

}  // namespace sigb200
