// Per-coefficient arithmetic of the truncated tensor algebra: Chen product and its two
// adjoints, the power series of the tensor exponential and its adjoint, linear signatures.
//
// Every function computes ONE output coefficient from read-only inputs, so a caller may
// evaluate any set of coefficients concurrently (one thread per coefficient, a CTA striding
// over a level, or a plain loop on the host: the file compiles as ordinary C++ and is
// exercised that way by tests/cpu_harness).
//
// Layout: arrays hold levels 1..N without the scalar term; level t (d^t coefficients) starts
// at Levels::off[t]; word (i_1..i_t) sits at i_1 d^(t-1) + .. + i_t inside its level.
//
// The arithmetic follows, term for term, what the reference evaluates in
//   siglib/cpsig/cp_sig_combine.h:34-66, 125-176 (product, adjoints),
//   siglib/cpsig/cp_exp_signature.h:43-210       (exponential and its adjoint),
//   siglib/cpsig/cp_sig_join.h:36-57             (linear signature),
// with the loops turned inside out so that each coefficient is owned by one evaluator.
#pragma once

#include <cmath>
#include <cstdint>

#if defined(__CUDACC__)
#define SIG_HD __host__ __device__ __forceinline__
#else
#define SIG_HD inline
#endif

namespace sigb200 {

constexpr int kAlgebraMaxDegree = 64;

// Indices inside one signature are 32-bit: a signature of 2^31 coefficients is far beyond what
// these operators are used for, and 32-bit division is several times cheaper on the GPU.
constexpr uint64_t kAlgebraMaxLength = 1ull << 31;

struct Levels {
    uint32_t dim;
    uint32_t degree;
    uint32_t off[kAlgebraMaxDegree + 2];  // off[t], t = 1..degree+1; off[degree+1] = total length S

    SIG_HD uint32_t size(uint32_t t) const { return off[t + 1] - off[t]; }
    SIG_HD uint32_t total() const { return off[degree + 1]; }
    // level of flat index j (0 <= j < total())
    SIG_HD uint32_t level_of(uint32_t j) const {
        uint32_t t = 1;
        while (off[t + 1] <= j) ++t;
        return t;
    }
};

// The caller has checked that dim^1 + .. + dim^degree < kAlgebraMaxLength and degree <= kAlgebraMaxDegree.
inline Levels make_levels(uint64_t dim, uint64_t degree) {
    Levels lv{};
    lv.dim = static_cast<uint32_t>(dim);
    lv.degree = static_cast<uint32_t>(degree);
    uint64_t size = 1, offset = 0;
    lv.off[0] = 0;
    for (uint64_t t = 1; t <= degree + 1; ++t) {
        lv.off[t] = static_cast<uint32_t>(offset);
        size *= dim;
        offset += size;
    }
    return lv;
}

SIG_HD float alg_fma(float a, float b, float c) { return ::fmaf(a, b, c); }
SIG_HD double alg_fma(double a, double b, double c) { return ::fma(a, b, c); }

// C = A (x) B (both with implicit scalar 1): coefficient w of level t.
template <typename T>
SIG_HD T product_coeff(const T* A, const T* B, const Levels& lv, uint32_t t, uint32_t w) {
    T acc = A[lv.off[t] + w];
    uint32_t right_size = lv.dim;  // d^(t-left)
    for (uint32_t left = t - 1; left >= 1; --left) {
        const uint32_t u = w / right_size, v = w - u * right_size;
        acc = alg_fma(B[lv.off[t - left] + v], A[lv.off[left] + u], acc);
        right_size *= lv.dim;
    }
    return acc + B[lv.off[t] + w];
}

// Adjoint of the left factor of C = A (x) B: dA_l[u] = dC_l[u] + sum_{m,v} dC_{l+m}[u v] B_m[v].
template <typename T>
SIG_HD T left_adjoint_coeff(const T* dC, const T* B, const Levels& lv, uint32_t l, uint32_t u) {
    T acc = dC[lv.off[l] + u];
    uint32_t msize = lv.dim;
    for (uint32_t m = 1; l + m <= lv.degree; ++m) {
        const T* row = dC + lv.off[l + m] + u * msize;
        const T* b = B + lv.off[m];
        T dot = T(0);
        for (uint32_t v = 0; v < msize; ++v) dot = alg_fma(row[v], b[v], dot);
        acc += dot;
        msize *= lv.dim;
    }
    return acc;
}

// Adjoint of the right factor of C = A (x) B: dB_m[v] = dC_m[v] + sum_{l,u} dC_{l+m}[u v] A_l[u].
template <typename T>
SIG_HD T right_adjoint_coeff(const T* dC, const T* A, const Levels& lv, uint32_t m, uint32_t v) {
    T acc = dC[lv.off[m] + v];
    const uint32_t msize = lv.size(m);
    uint32_t lsize = lv.dim;
    for (uint32_t l = 1; l + m <= lv.degree; ++l) {
        const T* col = dC + lv.off[l + m] + v;
        const T* a = A + lv.off[l];
        for (uint32_t u = 0; u < lsize; ++u) acc = alg_fma(col[u * msize], a[u], acc);
        lsize *= lv.dim;
    }
    return acc;
}

// Product without the unit terms: sum_{l=1..t-1} A_l[u] B_{t-l}[v] for the word w = u v of level t.
template <typename T>
SIG_HD T nonunital_product_coeff(const T* A, const T* B, const Levels& lv, uint32_t t, uint32_t w) {
    T acc = T(0);
    uint32_t right_size = t > 1 ? lv.size(t - 1) : 1;  // d^(t-left), left = 1
    for (uint32_t left = 1; left < t; ++left) {
        const uint32_t u = w / right_size, v = w - u * right_size;
        acc = alg_fma(B[lv.off[t - left] + v], A[lv.off[left] + u], acc);
        right_size /= lv.dim;
    }
    return acc;
}

// Adjoints of C = (product without unit terms) of A and B:
//   dA_l[u] = sum_{m,v} dC_{l+m}[u v] B_m[v],   dB_m[v] = sum_{l,u} dC_{l+m}[u v] A_l[u].
// `top`: dC is known to vanish above that level (the sums stop there).
template <typename T>
SIG_HD T nonunital_left_adjoint_coeff(const T* dC, const T* B, const Levels& lv, uint32_t l, uint32_t u,
                                      uint32_t top) {
    T acc = T(0);
    uint32_t msize = lv.dim;
    for (uint32_t m = 1; l + m <= top; ++m) {
        const T* row = dC + lv.off[l + m] + u * msize;
        const T* b = B + lv.off[m];
        T dot = T(0);
        for (uint32_t v = 0; v < msize; ++v) dot = alg_fma(row[v], b[v], dot);
        acc += dot;
        msize *= lv.dim;
    }
    return acc;
}
template <typename T>
SIG_HD T nonunital_right_adjoint_coeff(const T* dC, const T* A, const Levels& lv, uint32_t m, uint32_t v,
                                       uint32_t top) {
    T acc = T(0);
    const uint32_t msize = lv.size(m);
    uint32_t lsize = lv.dim;
    for (uint32_t l = 1; l + m <= top; ++l) {
        const T* col = dC + lv.off[l + m] + v;
        const T* a = A + lv.off[l];
        for (uint32_t u = 0; u < lsize; ++u) acc = alg_fma(col[u * msize], a[u], acc);
        lsize *= lv.dim;
    }
    return acc;
}

// Power series of exp: P_1 = X, P_n = X (x) P_{n-1} / n (no scalar terms; P_n lives on levels >= n).
// Returns coefficient w of level t of P_n given P_{n-1} (Pprev), 0 below level n.
template <typename T>
SIG_HD T exp_power_coeff(const T* X, const T* Pprev, const Levels& lv, uint32_t n, uint32_t t, uint32_t w) {
    if (t < n) return T(0);
    const T inv_n = T(1) / static_cast<T>(n);
    T acc = T(0);
    uint32_t right_size = lv.size(t - 1);  // d^(t-left), left = 1
    const uint32_t max_left = t - (n - 1);
    for (uint32_t left = 1; left <= max_left; ++left) {
        const uint32_t u = w / right_size, v = w - u * right_size;
        acc = alg_fma(Pprev[lv.off[t - left] + v], X[lv.off[left] + u] * inv_n, acc);
        right_size /= lv.dim;
    }
    return acc;
}

// Adjoint of the power series, one round (n = degree .. 2).  With U = (dE + dPn) / n on levels >= n
// (dE = dLoss/d exp(X), dPn = adjoint of P_n accumulated so far, all zero for n = degree):
//   adjoint of P_{n-1}:  dPprev_m[v] = sum_{l,u} U_{l+m}[u v] X_l[u]           (m >= n-1)
template <typename T>
SIG_HD T exp_adjoint_prev_coeff(const T* dE, const T* dPn, const T* X, const Levels& lv, uint32_t n, uint32_t m,
                                uint32_t v) {
    if (m + 1 < n) return T(0);
    const T inv_n = T(1) / static_cast<T>(n);
    const uint32_t msize = lv.size(m);
    T acc = T(0);
    uint32_t lsize = lv.dim;
    for (uint32_t l = 1; l + m <= lv.degree; ++l) {
        const uint32_t base = lv.off[l + m] + v;
        const T* x = X + lv.off[l];
        for (uint32_t u = 0; u < lsize; ++u) {
            const T up = (dE[base + u * msize] + (dPn ? dPn[base + u * msize] : T(0))) * inv_n;
            acc = alg_fma(up, x[u], acc);
        }
        lsize *= lv.dim;
    }
    return acc;
}

//   contribution of coefficient w of level t >= n to the adjoint of the level-1 part of X:
//   d X_1[i] += U_t[i v] P_{n-1, t-1}[v] with i = w / d^(t-1), v = w % d^(t-1); returns the product and i.
template <typename T>
SIG_HD T exp_adjoint_level1_term(const T* dE, const T* dPn, const T* Pprev, const Levels& lv, uint32_t n, uint32_t t,
                                 uint32_t w, uint32_t* letter) {
    *letter = 0;
    if (t < n || t < 2) return T(0);
    const uint32_t vsize = lv.size(t - 1);
    const uint32_t i = w / vsize, v = w - i * vsize;
    *letter = i;
    const T inv_n = T(1) / static_cast<T>(n);
    const uint32_t j = lv.off[t] + w;
    const T up = (dE[j] + (dPn ? dPn[j] : T(0))) * inv_n;
    return up * Pprev[lv.off[t - 1] + v];
}

// Signature of a straight segment: L_t[w] = v[i_t] * (L_{t-1}[i_1..i_{t-1}] / t), built letter by letter.
template <typename T>
SIG_HD T linear_sig_coeff(const T* disp, const Levels& lv, uint32_t t, uint32_t w) {
    uint32_t div = t > 1 ? lv.size(t - 1) : 1;
    uint32_t rest = w;
    T acc = T(0);
    for (uint32_t k = 1; k <= t; ++k) {
        const uint32_t letter = rest / div;
        rest -= letter * div;
        if (k < t) div /= lv.dim;
        acc = k == 1 ? disp[letter] : disp[letter] * (acc * (T(1) / static_cast<T>(k)));
    }
    return acc;
}

// Adjoint of the linear signature w.r.t. the displacement: coefficient w of level t contributes
// dL_t[w] * (prod_{q != p} v[i_q]) / t! to d v[i_p] for every position p.  `emit(letter, value)`.
template <typename T, typename Emit>
SIG_HD void linear_sig_adjoint_terms(const T* disp, T dL, const Levels& lv, uint32_t t, uint32_t w, Emit emit) {
    // suffix products from the right, prefix running from the left
    T inv_fact = T(1);
    for (uint32_t k = 2; k <= t; ++k) inv_fact /= static_cast<T>(k);
    const T scale = dL * inv_fact;
    for (uint32_t p = 1; p <= t; ++p) {
        T prod = scale;
        uint32_t div = t > 1 ? lv.size(t - 1) : 1, rest = w, own = 0;
        for (uint32_t k = 1; k <= t; ++k) {
            const uint32_t letter = rest / div;
            rest -= letter * div;
            if (k < t) div /= lv.dim;
            if (k == p) own = letter;
            else prod *= disp[letter];
        }
        emit(own, prod);
    }
}

}  // namespace sigb200
