// Run-time choice among the compiled register-tile variants (tile_table.h).
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <mutex>
#include <string>
#include <tuple>

#include "sig_tile_launch.cuh"
#ifndef SIG_TILE_TABLE
#define SIG_TILE_TABLE "tile_table.h"  // -DSIG_TILE_TABLE='"other.h"': a table restricted to the shapes a deployment needs
#endif
#include SIG_TILE_TABLE

namespace sigb200 {

#define SIG_DECLARE_PART(k) void register_tile_part_##k(std::vector<TileEntry>& table);
SIG_TILE_PART_LIST(SIG_DECLARE_PART)
#undef SIG_DECLARE_PART

namespace {

const std::vector<TileEntry>& tile_table() {
    static std::vector<TileEntry> table;
    static std::once_flag once;
    std::call_once(once, [] {
#define SIG_REGISTER_PART(k) register_tile_part_##k(table);
        SIG_TILE_PART_LIST(SIG_REGISTER_PART)
#undef SIG_REGISTER_PART
        // big tiles first, so the first entry that yields enough warps is the most efficient one
        std::stable_sort(table.begin(), table.end(),
                         [](const TileEntry& a, const TileEntry& b) { return a.tile_values > b.tile_values; });
    });
    return table;
}

struct Plan {
    const TileEntry* entry = nullptr;
    int nseg = 1;
    const TileEntry* forward_for_segments = nullptr;
};

// Resident CTAs per SM of a variant on a device, queried once and cached.
int occupancy_of(const TileEntry& e, bool flags, int device) {
    static std::mutex mu;
    static std::map<std::tuple<const TileEntry*, bool, int>, int> cache;
    std::lock_guard<std::mutex> lock(mu);
    const auto key = std::make_tuple(&e, flags, device);
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
    const int occ = e.occupancy(flags);
    cache.emplace(key, occ);
    return occ;
}

// Relative time of one wave in which every SM runs r CTAs of the same sweep, in units of
// the time a lone CTA needs.  Calibrated on B200 by forcing plans one by one (C4 shape,
// float32): a single CTA per SM already keeps the FMA pipe about half busy (a step is a long
// run of independent packed FMAs after a short dependent prologue), so co-resident CTAs
// mostly take turns: each extra CTA costs about 0.8 of a lone one.  Splitting a sweep into
// more CTAs therefore pays while SMs are idle and hardly at all afterwards.
double wave_cost(int r) { return 1.0 + 0.8 * (r - 1); }

// Modelled sweep time (issue slots of the busiest SM) of `blocks` CTAs of 4 warps, each
// running `steps` steps of e.est_instr slots, on `sms` SMs holding at most `occ` CTAs each.
double modelled_time(uint64_t blocks, int occ, int sms, double steps, const TileEntry& e) {
    const uint64_t capacity = uint64_t(occ) * sms;
    const uint64_t full = blocks / capacity, rem = blocks % capacity;
    double t = double(full) * wave_cost(occ);
    if (rem) t += wave_cost(int((rem + sms - 1) / sms));
    return t * steps * e.est_instr;
}

// Chooses the tile variant (and, forward only, the number of time segments) with the
// smallest modelled time.  tile_preference(): 1 = biggest tile, 2 = smallest, 3 = no
// segmentation, 4 = biggest tile with three segments (tests).
Plan choose(bool is_double, bool backward, const SigShape& s, int sm_count, bool flags, int device) {
    Plan plan;
    if (s.dim > 64 || s.degree > 16 || s.full_len >= (1ull << 31)) return plan;
    const int pref = tile_preference();
    const int sms = sm_count > 0 ? sm_count : 148;
    const uint64_t steps = s.len > 1 ? s.len - 1 : 1;
    const uint64_t seg_bytes = s.batch * (s.full_len - 1) * (is_double ? 8 : 4);
    static const int kSegments[] = {1, 2, 3, 4, 5, 6, 8, 10, 12, 16, 20, 24, 32};
    double best = 0;
    const TileEntry* first = nullptr;
    const TileEntry* last = nullptr;
    const TileEntry* fwd_big = nullptr;  // biggest forward tile: sweeps the segments of a segmented backward
    for (const TileEntry& e : tile_table())
        if (e.is_double == is_double && !e.backward && e.D == int(s.dim) && e.N == int(s.degree)) { fwd_big = &e; break; }
    // one pairwise Chen product / left adjoint over the batch: about 25 issue slots per term, plus launch
    const double join_cost = double(s.full_len) * s.degree / 32.0 * s.batch / (4.0 * sms) * 25.0 + 10000.0;
    for (const TileEntry& e : tile_table()) {
        if (e.is_double != is_double || e.backward != backward || e.D != int(s.dim) || e.N != int(s.degree)) continue;
        if (!first) first = &e;
        last = &e;
        if (pref == 1 || pref == 2 || pref == 4 || device < 0) continue;
        const int occ = occupancy_of(e, flags, device);
        const uint64_t wpp = uint64_t((e.units + 31) / 32);
        if (&e == first && (s.batch * wpp + kTileWarpsPerBlock - 1) / kTileWarpsPerBlock >= uint64_t(occ) * sms) {
            // the biggest tile already fills every SM to its occupancy: nothing to trade
            plan.entry = &e;
            plan.nseg = 1;
            break;
        }
        for (int nseg : kSegments) {
            // segment scratch: forward nseg + joins (about 2 nseg signatures), backward 3 nseg
            if (nseg > 1 && (pref == 3 || steps / nseg < 64 || seg_bytes * 3 * nseg > (1ull << 30))) break;
            if (nseg > 1 && backward && !fwd_big) break;
            const uint64_t blocks = (s.batch * nseg * wpp + kTileWarpsPerBlock - 1) / kTileWarpsPerBlock;
            // time segmentation only pays while one sweep leaves SMs idle
            if (nseg > 1 && (s.batch * (nseg - 1) * wpp + kTileWarpsPerBlock - 1) / kTileWarpsPerBlock >=
                                uint64_t(occ) * sms) break;
            const double seg_steps = double((steps + nseg - 1) / nseg);
            double t = modelled_time(blocks, occ, sms, seg_steps, e);
            if (nseg > 1 && !backward) t += (nseg - 1) * join_cost;  // joining the segments
            if (nseg > 1 && backward) {
                // segment signatures (one forward sweep), prefix states and pulled-back adjoints
                const uint64_t fwpp = uint64_t((fwd_big->units + 31) / 32);
                const uint64_t fblocks = (s.batch * nseg * fwpp + kTileWarpsPerBlock - 1) / kTileWarpsPerBlock;
                t += modelled_time(fblocks, occupancy_of(*fwd_big, flags, device), sms, seg_steps, *fwd_big);
                t += 2.0 * (nseg - 1) * join_cost;
            }
            if (!plan.entry || t < best) {
                best = t;
                plan.entry = &e;
                plan.nseg = nseg;
            }
        }
    }
    plan.forward_for_segments = fwd_big;
    // Test hook (set_forced_plan): pins the variant and segment count when such a variant is
    // compiled for the shape.
    const ForcedPlan forced = forced_plan(backward);
    if (forced.P >= 0) {
        for (const TileEntry& e : tile_table())
            if (e.is_double == is_double && e.backward == backward && e.D == int(s.dim) && e.N == int(s.degree) &&
                e.P == forced.P && e.G == forced.G) {
                plan.entry = &e;
                plan.nseg = int(std::max<uint64_t>(1, std::min<uint64_t>(uint64_t(forced.segments), steps)));
                if (backward && !fwd_big) plan.nseg = 1;
                return plan;
            }
    }
    if (pref == 1 || pref == 4 || (device < 0 && first)) plan.entry = first, plan.nseg = 1;
    if (pref == 2) plan.entry = last, plan.nseg = 1;
    if (pref == 4 && plan.entry && (!backward || fwd_big)) plan.nseg = int(std::min<uint64_t>(3, steps));
    return plan;
}

}  // namespace

template <typename T>
bool tile_forward_available(const SigShape& s) {
    return choose(sizeof(T) == 8, false, s, 0, false, -1).entry != nullptr;
}

template <typename T>
bool tile_backward_available(const SigShape& s) {
    return choose(sizeof(T) == 8, true, s, 0, false, -1).entry != nullptr;
}

// Paths that fill the GPU exactly once with the variant an unsegmented sweep of this shape
// would run (0 when the shape is outside the table or one path already overfills a wave).
template <typename T>
uint64_t tile_wave_paths(const SigShape& s, bool backward) {
    const int device = current_device();
    const bool flags = s.time_aug || s.lead_lag;
    SigShape big = s;
    big.batch = uint64_t(1) << 20;  // the variant a full GPU gets
    const DeviceContext& ctx = device_context(device);
    const Plan plan = choose(sizeof(T) == 8, backward, big, ctx.sm_count, flags, device);
    if (!plan.entry) return 0;
    const uint64_t wpp = uint64_t((plan.entry->units + 31) / 32);
    const uint64_t warps = uint64_t(occupancy_of(*plan.entry, flags, device)) * ctx.sm_count * kTileWarpsPerBlock;
    return warps / wpp;
}
template uint64_t tile_wave_paths<float>(const SigShape&, bool);
template uint64_t tile_wave_paths<double>(const SigShape&, bool);

template <typename T>
bool launch_tile_forward(const T* path, T* out, const SigShape& s, T end_time, cudaStream_t stream, int* nonfinite,
                         bool* nonfinite_checked) {
    if (nonfinite_checked) *nonfinite_checked = false;
    const int device = current_device();
    const bool flags = s.time_aug || s.lead_lag;
    const Plan plan = choose(sizeof(T) == 8, false, s, device_context(device).sm_count, flags, device);
    if (!plan.entry) return false;
    const PathView<T> pv = make_path_view(path, s.data_dim, s.data_len, s.time_aug, s.lead_lag, end_time);
    if (plan.nseg > 1) {
        // Small batch, long path: time is cut into segments swept by independent warps and the
        // segment signatures are joined with Chen's identity.
        const uint64_t per_buffer = s.batch * (s.full_len - 1);
        Scratch seg((per_buffer * uint64_t(plan.nseg) + chen_combine_tmp_elems(s, plan.nseg)) * sizeof(T), stream);
        plan.entry->launch(&pv, out, nullptr, nullptr, s.batch, static_cast<uint32_t>(s.stride), s.scalar_term, flags,
                           plan.nseg, seg.get(), nullptr, stream);
        launch_chen_combine<T>(out, seg.as<T>(), seg.as<T>() + per_buffer * uint64_t(plan.nseg), s, plan.nseg, stream);
        return true;
    }
    plan.entry->launch(&pv, out, nullptr, nullptr, s.batch, static_cast<uint32_t>(s.stride), s.scalar_term, flags, 1,
                       nullptr, nonfinite, stream);
    if (nonfinite_checked) *nonfinite_checked = true;
    return true;
}

// Forward sweep with the log-signature epilogue for the whole batch in one launch.  Used when the
// automatic plan for the shape is the unsegmented sweep of a variant that has the fused kernel
// compiled and the paths are short: on B200 the cluster launch costs about 9 % of the sweep
// (measured on d = 16, degree 4: 52.8 ms against 48.3 ms at 4096 steps) while computing the
// signature into scratch and running the tensor-logarithm kernels costs a fixed 0.37 us per
// path, so the fused sweep wins below about a thousand steps and loses above.  `force` skips that
// rule (tests).  Returns false when nothing was launched.
template <typename T>
bool launch_tile_forward_log(const T* path, T* out, const SigShape& s, T end_time, uint32_t out_stride,
                             uint32_t out_shift, const int32_t* rank, int* nonfinite, cudaStream_t stream, bool force) {
    if (s.degree < 2 || s.len <= 1) return false;
    const int device = current_device();
    const bool flags = s.time_aug || s.lead_lag;
    const Plan plan = choose(sizeof(T) == 8, false, s, device_context(device).sm_count, flags, device);
    const TileEntry* e = plan.entry;
    if (force && (!e || !e->launch_log)) {
        // tests: the variant that carries the fused kernel, whatever the batch size
        for (const TileEntry& cand : tile_table())
            if (cand.is_double == (sizeof(T) == 8) && !cand.backward && cand.D == int(s.dim) && cand.N == int(s.degree) &&
                cand.launch_log) { e = &cand; break; }
    }
    if (!e || !e->launch_log) return false;
    if (!force && (plan.nseg != 1 || s.len - 1 > 1024)) return false;
    const PathView<T> pv = make_path_view(path, s.data_dim, s.data_len, s.time_aug, s.lead_lag, end_time);
    return e->launch_log(&pv, out, s.batch, out_stride, out_shift, rank, flags, nonfinite, stream);
}
template bool launch_tile_forward_log<float>(const float*, float*, const SigShape&, float, uint32_t, uint32_t,
                                             const int32_t*, int*, cudaStream_t, bool);
template bool launch_tile_forward_log<double>(const double*, double*, const SigShape&, double, uint32_t, uint32_t,
                                              const int32_t*, int*, cudaStream_t, bool);

template <typename T>
bool launch_tile_backward(const T* path, T* out, const T* sig_derivs, const T* sig, const SigShape& s,
                          T end_time, T* incr_grad, cudaStream_t stream) {
    const int device = current_device();
    const bool flags = s.time_aug || s.lead_lag;
    const Plan plan = choose(sizeof(T) == 8, true, s, device_context(device).sm_count, flags, device);
    const TileEntry* e = plan.entry;
    if (!e) return false;
    const PathView<T> pv = make_path_view(path, s.data_dim, s.data_len, s.time_aug, s.lead_lag, end_time);
    const uint64_t g_elems = s.batch * (s.data_len - 1) * s.data_dim;
    const uint32_t stride = static_cast<uint32_t>(s.stride);
    SIG_CUDA_CHECK(cudaMemsetAsync(incr_grad, 0, g_elems * sizeof(T), stream));
    if (plan.nseg > 1) {
        // Small batch, long path: cut time into K segments swept by independent warps.  Needed per
        // segment k: the signature E_k of the path up to the segment's end and its loss adjoint
        // dE_k.  With A_k the signature of segment k alone (one forward sweep),
        //   E_0 = A_0, E_k = E_{k-1} (x) A_k, E_{K-1} = sig (given);
        //   dE_{K-1} = sig_derivs (given), dE_{k-1} = left adjoint of the product E_{k-1} (x) A_k.
        const int K = plan.nseg;
        const uint64_t slen = s.full_len - 1, row = uint64_t(K) * slen, per = s.batch * row;
        Scratch buf(3 * per * sizeof(T), stream);
        T* segA = buf.as<T>();
        T* E = segA + per;
        T* dE = E + per;
        plan.forward_for_segments->launch(&pv, nullptr, nullptr, nullptr, s.batch, stride, s.scalar_term, flags, K,
                                          segA, nullptr, stream);
        for (int k = 1; k <= K - 2; ++k)
            launch_chen_product<T>(k == 1 ? segA : E + uint64_t(k - 1) * slen, row, segA + uint64_t(k) * slen, row,
                                   E + uint64_t(k) * slen, row, s, stream);
        for (int k = K - 1; k >= 1; --k) {
            const bool top = k == K - 1;
            launch_chen_left_adjoint<T>(top ? sig_derivs + (s.scalar_term ? 1 : 0) : dE + uint64_t(k) * slen,
                                        top ? s.stride : row, segA + uint64_t(k) * slen, row,
                                        dE + uint64_t(k - 1) * slen, row, s, stream);
        }
        BackwardSegments<T> segs;
        segs.nseg = K;
        segs.seg_sig = segA;
        segs.state = E;
        segs.adjoint = dE;
        e->launch(&pv, incr_grad, sig, sig_derivs, s.batch, stride, s.scalar_term, flags, K, &segs, nullptr, stream);
    } else {
        e->launch(&pv, incr_grad, sig, sig_derivs, s.batch, stride, s.scalar_term, flags, 1, nullptr, nullptr, stream);
    }
    launch_increment_to_point_grad<T>(incr_grad, out, s.batch, s.data_len, s.data_dim, stream);
    return true;
}

// Tile backward for callers that bring their own scratch and SM count (used by the
// no-alloc entry points; touches neither the device context nor the memory pool).
template <typename T>
bool launch_tile_backward_prealloc(const T* path, T* out, const T* sig_derivs, const T* sig, const SigShape& s,
                                   T end_time, T* incr_grad, int sm_count, cudaStream_t stream) {
    int device = 0;
    SIG_CUDA_CHECK(cudaGetDevice(&device));
    // no extra scratch here: the choice is made among unsegmented sweeps only
    SigShape one = s;
    one.len = std::min<uint64_t>(s.len, 64);  // too short to be segmented, same variants otherwise
    const TileEntry* e = choose(sizeof(T) == 8, true, one, sm_count, s.time_aug || s.lead_lag, device).entry;
    if (!e) return false;
    const PathView<T> pv = make_path_view(path, s.data_dim, s.data_len, s.time_aug, s.lead_lag, end_time);
    const uint64_t g_elems = s.batch * (s.data_len - 1) * s.data_dim;
    SIG_CUDA_CHECK(cudaMemsetAsync(incr_grad, 0, g_elems * sizeof(T), stream));
    e->launch(&pv, incr_grad, sig, sig_derivs, s.batch, static_cast<uint32_t>(s.stride), s.scalar_term,
              s.time_aug || s.lead_lag, 1, nullptr, nullptr, stream);
    launch_increment_to_point_grad<T>(incr_grad, out, s.batch, s.data_len, s.data_dim, stream);
    return true;
}

template bool launch_tile_backward_prealloc<float>(const float*, float*, const float*, const float*, const SigShape&,
                                                   float, float*, int, cudaStream_t);
template bool launch_tile_backward_prealloc<double>(const double*, double*, const double*, const double*,
                                                    const SigShape&, double, double*, int, cudaStream_t);

// Human-readable description of what would be launched for a shape on the current device.
std::string describe_tile_plan(bool is_double, bool backward, const SigShape& s) {
    const int device = current_device();
    const bool flags = s.time_aug || s.lead_lag;
    const Plan plan = choose(is_double, backward, s, device_context(device).sm_count, flags, device);
    if (!plan.entry) return "generic";
    const TileEntry& e = *plan.entry;
    return std::string(backward ? "tile_backward" : "tile_forward") + "<D=" + std::to_string(e.D) + ",N=" +
           std::to_string(e.N) + ",P=" + std::to_string(e.P) + ",G=" + std::to_string(e.G) + "> units=" +
           std::to_string(e.units) + " segments=" + std::to_string(plan.nseg) + " ctas_per_sm=" +
           std::to_string(occupancy_of(e, flags, device));
}

#define INSTANTIATE(T)                                                                              \
    template bool tile_forward_available<T>(const SigShape&);                                       \
    template bool tile_backward_available<T>(const SigShape&);                                      \
    template bool launch_tile_forward<T>(const T*, T*, const SigShape&, T, cudaStream_t, int*, bool*); \
    template bool launch_tile_backward<T>(const T*, T*, const T*, const T*, const SigShape&, T, T*, cudaStream_t);
INSTANTIATE(float)
INSTANTIATE(double)
#undef INSTANTIATE

}  // namespace sigb200
