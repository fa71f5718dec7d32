// Host build of the register-tile arithmetic (pysiglib_b200/csrc/tile_math.h): every
// execution unit of a path is run sequentially on the CPU, so the tiling, indexing and
// adjoint logic of the CUDA kernels can be checked against the oracle without a GPU.
#include <cstdint>
#include <cstring>
#include <vector>

#include "../../pysiglib_b200/csrc/tile_math.h"

using namespace sigb200;

template <typename T, typename Sh>
static void gather_z(const T* zfull, const UnitIndex<Sh>& ix, T (&z)[Sh::D], T (&zg)[Sh::G], T* zc, T sign) {
    for (int c = 0; c < Sh::D; ++c) z[c] = sign * zfull[c];
    for (int j = 0; j < Sh::G; ++j) zg[j] = sign * zfull[ix.c0 + j];
    for (int k = 0; k < Sh::P; ++k) zc[k] = sign * zfull[ix.p[k]];
}

// path: (L, D) points; out: scalar-free signature
template <typename T, typename Sh>
static void forward_path(const T* path, int L, T* out) {
    constexpr int D = Sh::D;
    T* S = out - 1;
    for (int u = 0; u < Sh::UNITS; ++u) {
        const UnitIndex<Sh> ix = decode_unit<Sh>(u);
        TileState<T, Sh> st;
        T zf[D], z[D], zg[Sh::G], zc[Sh::P + 1];
        for (int step = 0; step + 1 < L; ++step) {
            for (int c = 0; c < D; ++c) zf[c] = path[(step + 1) * D + c] - path[step * D + c];
            gather_z<T, Sh>(zf, ix, z, zg, zc, T(1));
            if (step == 0) tile_init_first<T, Sh>(st, z, zg, zc);
            else tile_update<T, Sh>(st, z, zg, zc);
        }
        tile_store<T, Sh>(st, ix, S);
    }
}

// sig / seeds: scalar-free; grad: (L, D) point gradient
template <typename T, typename Sh>
static void backward_path(const T* path, int L, const T* sig, const T* seeds, T* grad) {
    constexpr int D = Sh::D;
    std::vector<T> incr(size_t(L - 1) * D, T(0));
    for (int u = 0; u < Sh::UNITS; ++u) {
        const UnitIndex<Sh> ix = decode_unit<Sh>(u);
        TileState<T, Sh, false> st;  // the reverse sweep keeps no level-N state
        TileAdjoint<T, Sh> ad;
        tile_load<T, Sh, false>(st, ad, ix, sig - 1, seeds - 1);
        T zf[D], z[D], zg[Sh::G], zc[Sh::P + 1];
        for (int step = L - 2; step >= 0; --step) {
            for (int c = 0; c < D; ++c) zf[c] = path[(step + 1) * D + c] - path[step * D + c];
            gather_z<T, Sh>(zf, ix, z, zg, zc, T(-1));
            tile_update<T, Sh, false>(st, z, zg, zc);
            gather_z<T, Sh>(zf, ix, z, zg, zc, T(1));
            TileGrad<T, Sh> g;
            for (int c = 0; c < D; ++c) g.gz[c] = T(0);
            for (int j = 0; j < Sh::G; ++j) g.gg[j] = T(0);
            for (int k = 0; k < (Sh::P > 0 ? Sh::P : 1); ++k) g.gc[k] = T(0);
            tile_pullback<T, Sh, false>(st, ad, g, z, zg, zc);
            T* row = incr.data() + size_t(step) * D;
            for (int c = 0; c < D; ++c) row[c] += g.gz[c];
            for (int j = 0; j < Sh::G; ++j) row[ix.c0 + j] += g.gg[j];
            for (int k = 0; k < Sh::P; ++k) row[ix.p[k]] += g.gc[k];
        }
    }
    for (int t = 0; t < L; ++t)
        for (int c = 0; c < D; ++c) {
            T v = T(0);
            if (t > 0) v += incr[size_t(t - 1) * D + c];
            if (t + 1 < L) v -= incr[size_t(t) * D + c];
            grad[t * D + c] = v;
        }
}

// expanded log signature (scalar-free layout) through the epilogue of the fused forward sweep:
// every unit sweeps the path, publishes its coefficients below level N, then turns its level-N
// coefficients into their logarithm; the levels below N are taken from the published ones
template <typename T, typename Sh>
static void forward_log_path(const T* path, int L, T* out) {
    constexpr int D = Sh::D, N = Sh::N;
    std::vector<TileState<T, Sh>> states(Sh::UNITS);
    std::vector<T> low(cgeom(D, N), T(0));
    low[0] = T(1);
    for (int u = 0; u < Sh::UNITS; ++u) {
        const UnitIndex<Sh> ix = decode_unit<Sh>(u);
        TileState<T, Sh>& st = states[u];
        T zf[D], z[D], zg[Sh::G], zc[Sh::P + 1];
        for (int step = 0; step + 1 < L; ++step) {
            for (int c = 0; c < D; ++c) zf[c] = path[(step + 1) * D + c] - path[step * D + c];
            gather_z<T, Sh>(zf, ix, z, zg, zc, T(1));
            if (step == 0) tile_init_first<T, Sh>(st, z, zg, zc);
            else tile_update<T, Sh>(st, z, zg, zc);
        }
        tile_publish_low<T, Sh>(st, ix, low.data());
    }
    T* S = out - 1;
    for (int u = 0; u < Sh::UNITS; ++u) {
        const UnitIndex<Sh> ix = decode_unit<Sh>(u);
        tile_log_top<T, Sh>(states[u], ix, low.data());
        // only the deepest tile level is final; tile_store also writes the others, overwritten below
        tile_store<T, Sh>(states[u], ix, S);
    }
    for (int prefix = 0; prefix < cgeom(D, N - 1); ++prefix)
        log_low_prefix<T, D, N>(low.data(), prefix, [&](int pos, T value) { S[pos] = value; });
}

#define HARNESS(D, N, P, G)                                                                              \
    extern "C" void fwd_f_##D##_##N##_##P##_##G(const float* p, int L, float* o) {                       \
        forward_path<float, TileShape<D, N, P, G>>(p, L, o);                                             \
    }                                                                                                    \
    extern "C" void fwd_d_##D##_##N##_##P##_##G(const double* p, int L, double* o) {                     \
        forward_path<double, TileShape<D, N, P, G>>(p, L, o);                                            \
    }                                                                                                    \
    extern "C" void log_f_##D##_##N##_##P##_##G(const float* p, int L, float* o) {                       \
        forward_log_path<float, TileShape<D, N, P, G>>(p, L, o);                                         \
    }                                                                                                    \
    extern "C" void log_d_##D##_##N##_##P##_##G(const double* p, int L, double* o) {                     \
        forward_log_path<double, TileShape<D, N, P, G>>(p, L, o);                                        \
    }                                                                                                    \
    extern "C" void bwd_f_##D##_##N##_##P##_##G(const float* p, int L, const float* s, const float* ds,  \
                                                float* g) {                                              \
        backward_path<float, TileShape<D, N, P, G>>(p, L, s, ds, g);                                     \
    }                                                                                                    \
    extern "C" void bwd_d_##D##_##N##_##P##_##G(const double* p, int L, const double* s, const double* ds, \
                                                double* g) {                                             \
        backward_path<double, TileShape<D, N, P, G>>(p, L, s, ds, g);                                    \
    }

HARNESS(2, 2, 1, 2)
HARNESS(2, 2, 0, 2)
HARNESS(2, 5, 2, 2)
HARNESS(2, 5, 3, 1)
HARNESS(2, 6, 1, 1)
HARNESS(3, 3, 0, 3)
HARNESS(3, 3, 2, 1)
HARNESS(3, 4, 1, 3)
HARNESS(3, 4, 2, 3)
HARNESS(4, 3, 1, 2)
HARNESS(4, 4, 2, 4)
HARNESS(5, 3, 1, 5)
HARNESS(6, 3, 1, 3)
HARNESS(8, 3, 1, 4)
// long chains over few tile values: the deep-degree variants of the table
HARNESS(3, 7, 5, 3)
HARNESS(4, 6, 4, 2)
HARNESS(2, 8, 6, 1)
