// Register-tile arithmetic of the signature kernels, shared by device code and by
// a host build used for CPU-side testing of the tiling logic.
//
// Decomposition.  A level-k coefficient of the signature, indexed by the word
// w = (i_1 .. i_k), is updated by one Horner step from the coefficients of the
// prefixes of w only.  So the level structure splits into independent pieces: one
// execution unit (a CUDA thread) owns
//     * a prefix word p of length P ("chain": the P coefficients S(p_1), S(p_1 p_2), ..,
//       kept redundantly by every unit that shares a prefix), and
//     * below p, G consecutive children c0 .. c0+G-1 at level P+1 with their complete
//       subtrees down to level N ("tile", depth Q = N - P, TS values held in registers).
// Units never communicate in the forward pass.  In the backward pass the adjoint of a
// chain coefficient is the sum of per-unit partial adjoints (the pull-back is linear in
// the adjoint), so units again work independently and only the d'-vector of increment
// gradients is summed across units.
//
// Arithmetic (reference: siglib/cpsig/cp_signature.h:464-499 forward step,
// :1137-1187 reverse step; the thread-per-prefix idea is the one of
// siglib/cusig/cu_signature_horner.cuh:27-216, re-tiled here so that a thread's useful
// FMAs dominate the redundant chain work):
//   for T = N..1:  W_1 = z/T, W_{l+1} = ((W_l + S_l)/(T-l)) (x) z,  S_T += (W_{T-1} + S_{T-1}) (x) z
// The operation order inside a coefficient equals the reference's CPU order, so float32
// results track it closely.
#pragma once

#if defined(__CUDACC__)
#define SIG_HD __host__ __device__ __forceinline__
#else
#include <cmath>
#define SIG_HD inline
#endif

namespace sigb200 {

constexpr int cpow(int d, int k) {
    int r = 1;
    for (int i = 0; i < k; ++i) r *= d;
    return r;
}
// 1 + d + .. + d^(k-1)
constexpr int cgeom(int d, int k) {
    int r = 0;
    for (int i = 0; i < k; ++i) r = r * d + 1;
    return r;
}

template <typename T> SIG_HD T sig_fma(T a, T b, T c);
#if defined(__CUDA_ARCH__)
template <> SIG_HD float sig_fma<float>(float a, float b, float c) { return fmaf(a, b, c); }
template <> SIG_HD double sig_fma<double>(double a, double b, double c) { return fma(a, b, c); }
#else
template <> SIG_HD float sig_fma<float>(float a, float b, float c) { return ::fmaf(a, b, c); }
template <> SIG_HD double sig_fma<double>(double a, double b, double c) { return ::fma(a, b, c); }
#endif

// Row primitives over the D children of one node.  In device code for float they use the
// packed two-wide FP32 instructions of sm_100 (fma/mul.rn.f32x2 through __ffma2_rn / __fmul2_rn):
// one issue slot performs two operations, which relieves the issue pressure of these
// FMA-bound kernels; every element still gets one correctly rounded FMA, so results are
// identical to the scalar form.  Host builds and double use the scalar loops.
#if defined(__CUDA_ARCH__)
#define SIG_PACKED_F32 1
#else
#define SIG_PACKED_F32 0
#endif

template <typename T> struct is_f32 { static constexpr bool value = false; };
template <> struct is_f32<float> { static constexpr bool value = true; };

// s[c] = fma(z[c], v, s[c])
template <typename T, int n>
SIG_HD void row_axpy(T* s, const T* z, T v) {
#if SIG_PACKED_F32
    if constexpr (is_f32<T>::value) {
        const float2 vv = make_float2(v, v);
#pragma unroll
        for (int c = 0; c + 1 < n; c += 2) {
            const float2 r = __ffma2_rn(make_float2(z[c], z[c + 1]), vv, make_float2(s[c], s[c + 1]));
            s[c] = r.x;
            s[c + 1] = r.y;
        }
        if (n % 2) s[n - 1] = sig_fma(z[n - 1], v, s[n - 1]);
    } else
#endif
    {
#pragma unroll
        for (int c = 0; c < n; ++c) s[c] = sig_fma(z[c], v, s[c]);
    }
}

// w[c] = z[c] * v
template <typename T, int n>
SIG_HD void row_scale(T* w, const T* z, T v) {
#if SIG_PACKED_F32
    if constexpr (is_f32<T>::value) {
        const float2 vv = make_float2(v, v);
#pragma unroll
        for (int c = 0; c + 1 < n; c += 2) {
            const float2 r = __fmul2_rn(make_float2(z[c], z[c + 1]), vv);
            w[c] = r.x;
            w[c + 1] = r.y;
        }
        if (n % 2) w[n - 1] = z[n - 1] * v;
    } else
#endif
    {
#pragma unroll
        for (int c = 0; c < n; ++c) w[c] = z[c] * v;
    }
}

// g[c] = fma(a[c], v, g[c]);  returns sum_c a[c] * z[c]
template <typename T, int n>
SIG_HD T row_pull(T* g, const T* a, const T* z, T v) {
#if SIG_PACKED_F32
    if constexpr (is_f32<T>::value) {
        const float2 vv = make_float2(v, v);
        float2 acc = make_float2(0.f, 0.f);
#pragma unroll
        for (int c = 0; c + 1 < n; c += 2) {
            const float2 aa = make_float2(a[c], a[c + 1]);
            const float2 r = __ffma2_rn(aa, vv, make_float2(g[c], g[c + 1]));
            g[c] = r.x;
            g[c + 1] = r.y;
            acc = __ffma2_rn(aa, make_float2(z[c], z[c + 1]), acc);
        }
        float total = acc.x + acc.y;
        if (n % 2) {
            g[n - 1] = sig_fma(a[n - 1], v, g[n - 1]);
            total = sig_fma(a[n - 1], z[n - 1], total);
        }
        return total;
    } else
#endif
    {
        T acc = T(0);
#pragma unroll
        for (int c = 0; c < n; ++c) {
            g[c] = sig_fma(a[c], v, g[c]);
            acc = sig_fma(a[c], z[c], acc);
        }
        return acc;
    }
}

// a[c] += x[c]
template <typename T, int n>
SIG_HD void row_add(T* a, const T* x) {
#if SIG_PACKED_F32
    if constexpr (is_f32<T>::value) {
#pragma unroll
        for (int c = 0; c + 1 < n; c += 2) {
            const float2 r = __fadd2_rn(make_float2(a[c], a[c + 1]), make_float2(x[c], x[c + 1]));
            a[c] = r.x;
            a[c + 1] = r.y;
        }
        if (n % 2) a[n - 1] += x[n - 1];
    } else
#endif
    {
#pragma unroll
        for (int c = 0; c < n; ++c) a[c] += x[c];
    }
}

template <int D_, int N_, int P_, int G_>
struct TileShape {
    static constexpr int D = D_;   // augmented path dimension
    static constexpr int N = N_;   // signature degree
    static constexpr int P = P_;   // chain (prefix) length, 0 <= P < N
    static constexpr int G = G_;   // children owned at level P+1, G divides D
    static constexpr int Q = N - P;          // tile depth
    static constexpr int NG = D / G;         // child groups per prefix
    static constexpr int UNITS = cpow(D, P) * NG;  // execution units per path
    // tile nodes at depth q (1..Q): G * D^(q-1); offset of depth q inside the tile array
    static constexpr int nodes(int q) { return G * cpow(D, q - 1); }
    static constexpr int off(int q) { return G * cgeom(D, q - 1); }
    static constexpr int TS = G * cgeom(D, Q);       // tile values per unit
    static constexpr int WS = G * cgeom(D, Q - 1) > G ? G * cgeom(D, Q - 1) : G;  // work values (depth < Q)
    static_assert(P >= 0 && P < N, "chain length out of range");
    static_assert(D % G == 0, "G must divide D");
};

template <typename T> SIG_HD T rcp_of(int k) { return T(1) / T(k); }

// Per-unit state: chain coefficients ch[0..P] (ch[0] = 1) and the tile s[0..TS).
// TOP = false drops the deepest tile level (the level-N coefficients).  The reverse sweep
// never reads them: the pull-back of a step only needs the rewound levels below N, and
// rewinding those does not involve level N either.  Leaving them out removes most of the
// state registers, most of the signature reads and the largest FMA block of the rewind.
template <typename T, typename Sh, bool TOP = true>
struct TileState {
    static constexpr int SIZE = TOP ? Sh::TS : (Sh::off(Sh::Q) > 0 ? Sh::off(Sh::Q) : 1);
    T ch[Sh::P + 1];
    T s[SIZE];
};

// First segment: S_k = S_{k-1} (x) z / k   (siglib/cpsig/cp_signature.h:365-389)
template <typename T, typename Sh>
SIG_HD void tile_init_first(TileState<T, Sh>& st, const T (&z)[Sh::D], const T (&zg)[Sh::G],
                            const T* zc /* [P] */) {
    st.ch[0] = T(1);
#pragma unroll
    for (int k = 1; k <= Sh::P; ++k) st.ch[k] = zc[k - 1] * (st.ch[k - 1] * rcp_of<T>(k));
#pragma unroll
    for (int j = 0; j < Sh::G; ++j) st.s[j] = zg[j] * (st.ch[Sh::P] * rcp_of<T>(Sh::P + 1));
#pragma unroll
    for (int q = 2; q <= Sh::Q; ++q) {
#pragma unroll
        for (int j = 0; j < Sh::nodes(q - 1); ++j) {
            const T v = st.s[Sh::off(q - 1) + j] * rcp_of<T>(Sh::P + q);
            row_scale<T, Sh::D>(&st.s[Sh::off(q) + j * Sh::D], z, v);
        }
    }
}

// Chain part of target level T: returns h = W^{(T)}_{K}[p_1..p_K] and fills hist[k] = W_k + S_k.
template <typename T, typename Sh, int K>
SIG_HD T tile_chain(const T* ch, const T* zc, int target, T* hist) {
    T h = T(0);
#pragma unroll
    for (int k = 0; k < K; ++k) {
        const T a = h + ch[k];
        if (hist) hist[k] = a;
        h = zc[k] * (a * rcp_of<T>(target - k));
    }
    return h;
}

// Levels of one Horner step with increment z (zg = z at the unit's children, zc = z at its chain
// letters): tile depths FIRST_T .. 1 in descending order, then the chain.  FIRST_T = Q is the whole
// step; FIRST_T = Q - 1 leaves the deepest tile level (the level-N coefficients) alone.
template <typename T, typename Sh, bool TOP, int FIRST_T>
SIG_HD void tile_update_levels(TileState<T, Sh, TOP>& st, const T (&z)[Sh::D], const T (&zg)[Sh::G], const T* zc) {
    constexpr int P = Sh::P, Q = Sh::Q, D = Sh::D, G = Sh::G;
    static_assert(FIRST_T <= (TOP ? Q : Q - 1), "the state does not hold that depth");
    T w[Sh::WS];
#pragma unroll
    for (int t = FIRST_T; t >= 1; --t) {
        const int target = P + t;
        const T base = tile_chain<T, Sh, P>(st.ch, zc, target, nullptr) + st.ch[P];
        if (t == 1) {
#pragma unroll
            for (int j = 0; j < G; ++j) st.s[j] = sig_fma(zg[j], base, st.s[j]);
        } else {
            const T v0 = base * rcp_of<T>(t);
#pragma unroll
            for (int j = 0; j < G; ++j) w[j] = zg[j] * v0;
#pragma unroll
            for (int q = 2; q <= Q - 1; ++q) {
                if (q <= t - 1) {
#pragma unroll
                    for (int j = 0; j < Sh::nodes(q - 1); ++j) {
                        const T v = (w[Sh::off(q - 1) + j] + st.s[Sh::off(q - 1) + j]) * rcp_of<T>(t - q + 1);
                        row_scale<T, D>(&w[Sh::off(q) + j * D], z, v);
                    }
                }
            }
#pragma unroll
            for (int q = 2; q <= Q; ++q) {
                if (q == t) {
#pragma unroll
                    for (int j = 0; j < Sh::nodes(q - 1); ++j) {
                        const T v = w[Sh::off(q - 1) + j] + st.s[Sh::off(q - 1) + j];
                        row_axpy<T, D>(&st.s[Sh::off(q) + j * D], z, v);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int target = P; target >= 1; --target) {
        T h = T(0);
#pragma unroll
        for (int k = 0; k < P; ++k)
            if (k < target - 1) h = zc[k] * ((h + st.ch[k]) * rcp_of<T>(target - k));
        st.ch[target] = sig_fma(zc[target - 1], h + st.ch[target - 1], st.ch[target]);
    }
}

// One whole Horner step.
template <typename T, typename Sh, bool TOP = true>
SIG_HD void tile_update(TileState<T, Sh, TOP>& st, const T (&z)[Sh::D], const T (&zg)[Sh::G], const T* zc) {
    tile_update_levels<T, Sh, TOP, (TOP ? Sh::Q : Sh::Q - 1)>(st, z, zg, zc);
}

// Which words a unit owns.  Units of a path are numbered u = pw * NG + grp with pw the
// chain word read as a base-D number (first letter most significant).
template <typename Sh>
struct UnitIndex {
    int p[Sh::P > 0 ? Sh::P : 1];  // chain letters
    int pw;                        // chain word
    int c0;                        // first owned child letter at level P+1
    bool chain_owner[Sh::P + 1];   // chain_owner[k]: this unit reports / seeds the level-k chain coefficient
};

template <typename Sh>
SIG_HD UnitIndex<Sh> decode_unit(int u) {
    UnitIndex<Sh> ix;
    const int grp = u % Sh::NG;
    ix.pw = u / Sh::NG;
    ix.c0 = grp * Sh::G;
    int rest = ix.pw;
#pragma unroll
    for (int k = Sh::P - 1; k >= 0; --k) {
        ix.p[k] = rest % Sh::D;
        rest /= Sh::D;
    }
    // level-k chain word is pw / D^(P-k); exactly one unit (all later letters and the group zero) owns it
    ix.chain_owner[0] = false;
#pragma unroll
    for (int k = 1; k <= Sh::P; ++k) ix.chain_owner[k] = grp == 0 && (ix.pw % cpow(Sh::D, Sh::P - k)) == 0;
    return ix;
}

// Writes the unit's coefficients into a signature laid out with the scalar term at S[0]
// (S may point one element before a scalar-free buffer; S[0] is then never touched here).
template <typename T, typename Sh>
SIG_HD void tile_store(const TileState<T, Sh>& st, const UnitIndex<Sh>& ix, T* S) {
#pragma unroll
    for (int k = 1; k <= Sh::P; ++k)
        if (ix.chain_owner[k]) S[cgeom(Sh::D, k) + ix.pw / cpow(Sh::D, Sh::P - k)] = st.ch[k];
#pragma unroll
    for (int q = 1; q <= Sh::Q; ++q) {
        T* dst = S + cgeom(Sh::D, Sh::P + q) + (ix.pw * Sh::D + ix.c0) * cpow(Sh::D, q - 1);
#pragma unroll
        for (int j = 0; j < Sh::nodes(q); ++j) dst[j] = st.s[Sh::off(q) + j];
    }
}

// Adjoint state of one unit: partial adjoints of the chain (ac[0] unused) and the tile.
template <typename T, typename Sh>
struct TileAdjoint {
    T ac[Sh::P + 1];
    T a[Sh::TS];
};

// Loads the final signature and the seeds (dLoss/dSignature) of a unit; chain adjoints
// are taken by the owning unit only, so that their sum over units is the true adjoint.
template <typename T, typename Sh, bool TOP>
SIG_HD void tile_load(TileState<T, Sh, TOP>& st, TileAdjoint<T, Sh>& ad, const UnitIndex<Sh>& ix, const T* S,
                      const T* dS) {
    st.ch[0] = T(1);
    ad.ac[0] = T(0);
#pragma unroll
    for (int k = 1; k <= Sh::P; ++k) {
        const int idx = cgeom(Sh::D, k) + ix.pw / cpow(Sh::D, Sh::P - k);
        st.ch[k] = S[idx];
        ad.ac[k] = ix.chain_owner[k] ? dS[idx] : T(0);
    }
#pragma unroll
    for (int q = 1; q <= Sh::Q; ++q) {
        const int base = cgeom(Sh::D, Sh::P + q) + (ix.pw * Sh::D + ix.c0) * cpow(Sh::D, q - 1);
#pragma unroll
        for (int j = 0; j < Sh::nodes(q); ++j) {
            if (TOP || q < Sh::Q) st.s[Sh::off(q) + j] = S[base + j];
            ad.a[Sh::off(q) + j] = dS[base + j];
        }
    }
}

// Per-step increment gradient of one unit, by letter class:
//   gz[c]  letters 0..D-1 reached through tile depths >= 2 (static indices),
//   gg[j]  letter c0 + j (the unit's own children at depth 1),
//   gc[k]  chain letter p_{k+1}.
template <typename T, typename Sh>
struct TileGrad {
    T gz[Sh::D];
    T gg[Sh::G];
    T gc[Sh::P > 0 ? Sh::P : 1];
};

// Pull the adjoint back through one Horner step taken with increment z from the
// (already rewound) state st.  Accumulates into ad and into g (which the caller zeroes).
template <typename T, typename Sh, bool TOP>
SIG_HD void tile_pullback(const TileState<T, Sh, TOP>& st, TileAdjoint<T, Sh>& ad, TileGrad<T, Sh>& g,
                          const T (&z)[Sh::D], const T (&zg)[Sh::G], const T* zc) {
    constexpr int P = Sh::P, Q = Sh::Q, D = Sh::D, G = Sh::G;
    T hist[P > 0 ? P : 1];
    // targets inside the chain, ascending
#pragma unroll
    for (int target = 1; target <= P; ++target) {
        // forward: ch[target] += (h_{target-1} + ch[target-1]) * zc[target-1]
        T h = T(0);
#pragma unroll
        for (int k = 0; k < P; ++k)
            if (k < target) {
                hist[k] = h + st.ch[k];
                if (k < target - 1) h = zc[k] * (hist[k] * rcp_of<T>(target - k));
            }
        T y = ad.ac[target];
        g.gc[target - 1] = sig_fma(y, hist[target - 1], g.gc[target - 1]);
        y *= zc[target - 1];
#pragma unroll
        for (int k = P - 1; k >= 0; --k)
            if (k <= target - 2) {
                ad.ac[k + 1] += y;  // adjoint of ch[k+1] through hist[k+1]
                const T r = rcp_of<T>(target - k);
                g.gc[k] = sig_fma(y, hist[k] * r, g.gc[k]);
                y *= r * zc[k];
            }
        // for k == target-1 the adjoint of ch[target-1] is added here:
        // (the loop above adds into ac[k+1] for k <= target-2, i.e. ac[1..target-1])
    }
    // targets inside the tile, ascending depth
    T w[Sh::WS];
    T wa[Sh::WS];
#pragma unroll
    for (int t = 1; t <= Q; ++t) {
        const int target = P + t;
        const T hP = tile_chain<T, Sh, P>(st.ch, zc, target, hist);
        const T base = hP + st.ch[P];
        T wa0 = T(0);
        if (t == 1) {
#pragma unroll
            for (int j = 0; j < G; ++j) {
                g.gg[j] = sig_fma(ad.a[j], base, g.gg[j]);
                wa0 = sig_fma(ad.a[j], zg[j], wa0);
            }
        } else {
            const T v0 = base * rcp_of<T>(t);
#pragma unroll
            for (int j = 0; j < G; ++j) w[j] = zg[j] * v0;
#pragma unroll
            for (int q = 2; q <= Q - 1; ++q) {
                if (q <= t - 1) {
#pragma unroll
                    for (int j = 0; j < Sh::nodes(q - 1); ++j) {
                        const T v = (w[Sh::off(q - 1) + j] + st.s[Sh::off(q - 1) + j]) * rcp_of<T>(t - q + 1);
                        row_scale<T, D>(&w[Sh::off(q) + j * D], z, v);
                    }
                }
            }
            // depth t: S_t[j, c] += (w_{t-1}[j] + s_{t-1}[j]) * z[c]
#pragma unroll
            for (int q = 2; q <= Q; ++q) {
                if (q == t) {
#pragma unroll
                    for (int j = 0; j < Sh::nodes(q - 1); ++j) {
                        const T v = w[Sh::off(q - 1) + j] + st.s[Sh::off(q - 1) + j];
                        wa[Sh::off(q - 1) + j] = row_pull<T, D>(g.gz, &ad.a[Sh::off(q) + j * D], z, v);
                    }
                }
            }
            // depths t-1 .. 2: node (j, c) = child c of depth-(q-1) node j
#pragma unroll
            for (int q = Q - 1; q >= 2; --q) {
                if (q <= t - 1) {
                    const T r = rcp_of<T>(t - q + 1);
#pragma unroll
                    for (int j = 0; j < Sh::nodes(q - 1); ++j) {
                        const T v = (w[Sh::off(q - 1) + j] + st.s[Sh::off(q - 1) + j]) * r;
                        row_add<T, D>(&ad.a[Sh::off(q) + j * D], &wa[Sh::off(q) + j * D]);
                        wa[Sh::off(q - 1) + j] = row_pull<T, D>(g.gz, &wa[Sh::off(q) + j * D], z, v) * r;
                    }
                }
            }
            // depth 1: w_1[j] = zg[j] * (base / t)
#pragma unroll
            for (int j = 0; j < G; ++j) {
                const T x = wa[j];
                ad.a[j] += x;
                g.gg[j] = sig_fma(x, v0, g.gg[j]);
                wa0 = sig_fma(x, zg[j], wa0);
            }
            wa0 *= rcp_of<T>(t);
        }
        // chain: base = h_P + ch[P]
        if (P > 0) {
            T y = wa0;
            ad.ac[P] += y;
#pragma unroll
            for (int k = P - 1; k >= 0; --k) {
                const T r = rcp_of<T>(target - k);
                g.gc[k] = sig_fma(y, hist[k] * r, g.gc[k]);
                y *= r * zc[k];
                if (k >= 1) ad.ac[k] += y;
            }
        }
    }
}

// ---- log-signature epilogue --------------------------------------------------------------------
//
// log S = sum_{k >= 1} (-1)^(k+1)/k x^(x)k with x = S - 1.  For a word w = u e (prefix u of length n1,
// last letter e) the coefficient of x^(x)k splits by the position of the last cut, so
//     log S[u e] = sum_{i = 0..n1} h[i] * S[u_{i+1} .. u_{n1} e],
//     h[i] = sum_{m = 0..i} (-1)^m / (m + 1) * g_m[i],   g_m[i] = coefficient of x^(x)m at u_1 .. u_i
// (g_0 = 1 at the empty word).  The weights h depend on the prefix only and involve coefficients
// of levels below |w|, so a unit of the forward sweep can turn the level-N coefficients it holds
// in registers into their logarithm as soon as the levels below N of the whole signature can be
// read from somewhere: `low`, levels 0 .. N-1 in the scalar-term layout (low[0] = 1).
// Same values as the tensor logarithm of the reference (siglib/cpsig/cp_tensor_log.h:47-122), summed
// in a different order.

// h[0 .. n1] for the prefix word of level n1 with index uidx inside that level (n1 <= N - 1).
// pre[i] receives the index of u_1 .. u_i inside level i.  All loops have compile-time bounds and
// are predicated on n1, so that with a constant n1 everything stays in registers.
template <typename T, int D, int N>
SIG_HD void log_prefix_weights(const T* low, int n1, int uidx, T* h, int* pre) {
    int rest = uidx;
#pragma unroll
    for (int i = N - 1; i >= 0; --i) {
        if (i <= n1) {
            pre[i] = rest;
            rest /= D;
        }
    }
    T prev[N], cur[N];
#pragma unroll
    for (int i = 0; i < N; ++i) {
        prev[i] = i == 0 ? T(1) : T(0);
        h[i] = prev[i];
        cur[i] = T(0);
    }
#pragma unroll
    for (int m = 1; m < N; ++m) {
        if (m <= n1) {
            const T c = (m % 2 ? T(-1) : T(1)) / T(m + 1);
#pragma unroll
            for (int i = 1; i < N; ++i) {
                if (i >= m && i <= n1) {
                    T acc = T(0);
#pragma unroll
                    for (int ip = 0; ip < N - 1; ++ip)
                        if (ip >= m - 1 && ip < i)
                            acc = sig_fma(prev[ip], low[cgeom(D, i - ip) + pre[i] - pre[ip] * cpow(D, i - ip)], acc);
                    cur[i] = acc;
                    h[i] = sig_fma(c, acc, h[i]);
                }
            }
#pragma unroll
            for (int i = 0; i < N; ++i) prev[i] = i >= m ? cur[i] : T(0);
        }
    }
}

// log S at the word u e of level n = n1 + 1 given the weights of u; `own` = S[u e] itself.
template <typename T, int D, int N>
SIG_HD T log_word(const T* low, int n1, const T* h, const int* pre, int e, T own) {
    T acc = h[0] * own;
#pragma unroll
    for (int k = 1; k < N; ++k) {          // k = n1 - i + 1: length of the piece u_{i+1} .. u_{n1} e
        const int i = n1 - k + 1;
        if (i >= 1) acc = sig_fma(h[i], low[cgeom(D, k) + (pre[n1] - pre[i] * cpow(D, k - 1)) * D + e], acc);
    }
    return acc;
}

// The unit's coefficients below level N, written to `low` (scalar-term layout of levels 0 .. N-1).
template <typename T, typename Sh>
SIG_HD void tile_publish_low(const TileState<T, Sh>& st, const UnitIndex<Sh>& ix, T* low) {
#pragma unroll
    for (int k = 1; k <= Sh::P; ++k)
        if (ix.chain_owner[k]) low[cgeom(Sh::D, k) + ix.pw / cpow(Sh::D, Sh::P - k)] = st.ch[k];
#pragma unroll
    for (int q = 1; q < Sh::Q; ++q) {
        T* dst = low + cgeom(Sh::D, Sh::P + q) + (ix.pw * Sh::D + ix.c0) * cpow(Sh::D, q - 1);
#pragma unroll
        for (int j = 0; j < Sh::nodes(q); ++j) dst[j] = st.s[Sh::off(q) + j];
    }
}

// Replaces the unit's level-N coefficients by those of log S (in place, in the registers).
template <typename T, typename Sh>
SIG_HD void tile_log_top(TileState<T, Sh>& st, const UnitIndex<Sh>& ix, const T* low) {
    constexpr int D = Sh::D, N = Sh::N, Q = Sh::Q;
    T h[N];
    int pre[N];
    if constexpr (Q >= 2) {
#pragma unroll
        for (int j = 0; j < Sh::nodes(Q - 1); ++j) {
            const int uidx = (ix.pw * D + ix.c0) * cpow(D, Q - 2) + j;
            log_prefix_weights<T, D, N>(low, N - 1, uidx, h, pre);
#pragma unroll
            for (int e = 0; e < D; ++e) {
                T& own = st.s[Sh::off(Q) + j * D + e];
                own = log_word<T, D, N>(low, N - 1, h, pre, e, own);
            }
        }
    } else {
        log_prefix_weights<T, D, N>(low, N - 1, ix.pw, h, pre);
#pragma unroll
        for (int j = 0; j < Sh::G; ++j) st.s[j] = log_word<T, D, N>(low, N - 1, h, pre, ix.c0 + j, st.s[j]);
    }
}

// log S at the words of the levels below N that share the prefix number `prefix` (0 <= prefix <
// cgeom(D, N - 1): prefixes of all lengths 0 .. N-2, shortest first), from `low` alone; calls
// emit(position in the scalar-term layout, value) for each of the D words.
template <typename T, int D, int N, typename Emit>
SIG_HD void log_low_prefix(const T* low, int prefix, Emit&& emit) {
    int n1 = 0, start = 0, count = 1;     // prefixes of length n1 are numbered start .. start + count - 1
    while (prefix >= start + count) {
        start += count;
        count *= D;
        ++n1;
    }
    T h[N];
    int pre[N];
    log_prefix_weights<T, D, N>(low, n1, prefix - start, h, pre);
    const int level_offset = cgeom(D, n1 + 1);
    for (int e = 0; e < D; ++e) {
        const int pos = level_offset + (prefix - start) * D + e;
        emit(pos, log_word<T, D, N>(low, n1, h, pre, e, low[pos]));
    }
}

}  // namespace sigb200
