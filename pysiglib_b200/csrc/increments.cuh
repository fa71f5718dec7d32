// Path increments with the time-augmentation / lead-lag flags applied on the fly.
//
// The augmented path is never materialised: kernels ask for the increment of
// augmented step j, channel c, computed from the raw (L, d) points.
// Semantics follow the reference's point iterators (siglib/cpsig/cp_path.h:207-385):
//   lead-lag: 2L-1 points, channels [lag(d), lead(d)]; the lead channels move on
//             even steps, the lag channels on odd steps;
//   time-aug: one extra last channel running linearly from 0 to end_time.
#pragma once

#include <cstdint>

namespace sigb200 {

template <typename T>
struct PathView {
    const T* base;  // first point of the first path of the batch
    uint64_t path_stride;  // data_len * data_dim
    int d;          // raw dimension
    int L;          // raw length
    int dim;        // augmented dimension d'
    int steps;      // augmented length - 1
    bool time_aug;
    bool lead_lag;
    T dt;           // end_time / (augmented length - 1)

    __device__ __forceinline__ T increment(const T* x, int j, int c) const {
        if (lead_lag) {
            const int m = j >> 1;
            const bool odd = j & 1;
            if (c < d) return odd ? x[(m + 1) * d + c] - x[m * d + c] : T(0);
            if (c < 2 * d) return odd ? T(0) : x[(m + 1) * d + (c - d)] - x[m * d + (c - d)];
            return dt;
        }
        if (c < d) return x[(j + 1) * d + c] - x[j * d + c];
        return dt;
    }
};

template <typename T>
inline PathView<T> make_path_view(const T* path, uint64_t d, uint64_t L, bool time_aug, bool lead_lag,
                                  T end_time) {
    PathView<T> v;
    v.base = path;
    v.path_stride = d * L;
    v.d = static_cast<int>(d);
    v.L = static_cast<int>(L);
    v.dim = static_cast<int>((lead_lag ? 2 * d : d) + (time_aug ? 1 : 0));
    const uint64_t len = lead_lag ? (L ? 2 * L - 1 : 0) : L;
    v.steps = len > 0 ? static_cast<int>(len - 1) : 0;
    v.time_aug = time_aug;
    v.lead_lag = lead_lag;
    v.dt = len > 1 ? end_time / static_cast<T>(len - 1) : T(0);
    return v;
}

}  // namespace sigb200
