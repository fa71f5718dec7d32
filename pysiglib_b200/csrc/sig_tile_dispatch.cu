// Run-time choice among the compiled register-tile variants (tile_table.h).
#include <algorithm>
#include <mutex>

#include "sig_tile_launch.cuh"
#ifdef SIG_TILE_DEV
#include "tile_table_dev.h"  // development subset (quick builds)
#else
#include "tile_table.h"
#endif

namespace sigb200 {

#define SIG_DECLARE_PART(k) void register_tile_part_##k(std::vector<TileEntry>& table);
SIG_DECLARE_PART(0) SIG_DECLARE_PART(1) SIG_DECLARE_PART(2) SIG_DECLARE_PART(3)
SIG_DECLARE_PART(4) SIG_DECLARE_PART(5) SIG_DECLARE_PART(6) SIG_DECLARE_PART(7)
static_assert(SIG_TILE_PARTS == 8, "update the part list in sig_tile_dispatch.cu");

namespace {

const std::vector<TileEntry>& tile_table() {
    static std::vector<TileEntry> table;
    static std::once_flag once;
    std::call_once(once, [] {
        register_tile_part_0(table); register_tile_part_1(table); register_tile_part_2(table);
        register_tile_part_3(table); register_tile_part_4(table); register_tile_part_5(table);
        register_tile_part_6(table); register_tile_part_7(table);
        // big tiles first, so the first entry that yields enough warps is the most efficient one
        std::stable_sort(table.begin(), table.end(),
                         [](const TileEntry& a, const TileEntry& b) { return a.tile_values > b.tile_values; });
    });
    return table;
}

// Picks the variant for this shape: the biggest tile whose warp count fills the GPU
// (8 warps per SM), else the variant with the most warps.
const TileEntry* choose(bool is_double, bool backward, const SigShape& s, int sm_count) {
    if (s.dim > 64 || s.degree > 16 || s.full_len >= (1ull << 31)) return nullptr;
    const TileEntry* best = nullptr;
    const uint64_t want = uint64_t(sm_count > 0 ? sm_count : 148) * 8;
    for (const TileEntry& e : tile_table()) {
        if (e.is_double != is_double || e.backward != backward || e.D != int(s.dim) || e.N != int(s.degree)) continue;
        const uint64_t warps = s.batch * uint64_t((e.units + 31) / 32);
        if (warps >= want) return &e;
        if (!best || (e.units + 31) / 32 > (best->units + 31) / 32) best = &e;
    }
    return best;
}

}  // namespace

template <typename T>
bool tile_forward_available(const SigShape& s) {
    return choose(sizeof(T) == 8, false, s, 0) != nullptr;
}

template <typename T>
bool tile_backward_available(const SigShape& s) {
    return choose(sizeof(T) == 8, true, s, 0) != nullptr;
}

template <typename T>
bool launch_tile_forward(const T* path, T* out, const SigShape& s, T end_time, cudaStream_t stream) {
    const TileEntry* e = choose(sizeof(T) == 8, false, s, device_context(current_device()).sm_count);
    if (!e) return false;
    const PathView<T> pv = make_path_view(path, s.data_dim, s.data_len, s.time_aug, s.lead_lag, end_time);
    e->launch(&pv, out, nullptr, nullptr, s.batch, static_cast<uint32_t>(s.stride), s.scalar_term,
              s.time_aug || s.lead_lag, stream);
    return true;
}

template <typename T>
bool launch_tile_backward(const T* path, T* out, const T* sig_derivs, const T* sig, const SigShape& s,
                          T end_time, T* incr_grad, cudaStream_t stream) {
    const TileEntry* e = choose(sizeof(T) == 8, true, s, device_context(current_device()).sm_count);
    if (!e) return false;
    const PathView<T> pv = make_path_view(path, s.data_dim, s.data_len, s.time_aug, s.lead_lag, end_time);
    const uint64_t g_elems = s.batch * (s.data_len - 1) * s.data_dim;
    SIG_CUDA_CHECK(cudaMemsetAsync(incr_grad, 0, g_elems * sizeof(T), stream));
    e->launch(&pv, incr_grad, sig, sig_derivs, s.batch, static_cast<uint32_t>(s.stride), s.scalar_term,
              s.time_aug || s.lead_lag, stream);
    launch_increment_to_point_grad<T>(incr_grad, out, s.batch, s.data_len, s.data_dim, stream);
    return true;
}

// Tile backward for callers that bring their own scratch and SM count (used by the
// no-alloc entry points; touches neither the device context nor the memory pool).
template <typename T>
bool launch_tile_backward_prealloc(const T* path, T* out, const T* sig_derivs, const T* sig, const SigShape& s,
                                   T end_time, T* incr_grad, int sm_count, cudaStream_t stream) {
    const TileEntry* e = choose(sizeof(T) == 8, true, s, sm_count);
    if (!e) return false;
    const PathView<T> pv = make_path_view(path, s.data_dim, s.data_len, s.time_aug, s.lead_lag, end_time);
    const uint64_t g_elems = s.batch * (s.data_len - 1) * s.data_dim;
    SIG_CUDA_CHECK(cudaMemsetAsync(incr_grad, 0, g_elems * sizeof(T), stream));
    e->launch(&pv, incr_grad, sig, sig_derivs, s.batch, static_cast<uint32_t>(s.stride), s.scalar_term,
              s.time_aug || s.lead_lag, stream);
    launch_increment_to_point_grad<T>(incr_grad, out, s.batch, s.data_len, s.data_dim, stream);
    return true;
}

template bool launch_tile_backward_prealloc<float>(const float*, float*, const float*, const float*, const SigShape&,
                                                   float, float*, int, cudaStream_t);
template bool launch_tile_backward_prealloc<double>(const double*, double*, const double*, const double*,
                                                    const SigShape&, double, double*, int, cudaStream_t);

#define INSTANTIATE(T)                                                                              \
    template bool tile_forward_available<T>(const SigShape&);                                       \
    template bool tile_backward_available<T>(const SigShape&);                                      \
    template bool launch_tile_forward<T>(const T*, T*, const SigShape&, T, cudaStream_t);           \
    template bool launch_tile_backward<T>(const T*, T*, const T*, const T*, const SigShape&, T, T*, cudaStream_t);
INSTANTIATE(float)
INSTANTIATE(double)
#undef INSTANTIATE

}  // namespace sigb200
