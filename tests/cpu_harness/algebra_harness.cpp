// Host build of pysiglib_b200/csrc/algebra_math.h: runs the per-coefficient functions over every
// coefficient in plain loops, phase by phase in the order the CUDA kernels of sig_algebra.cu use
// (a loop over all coefficients stands for "every thread, then a barrier").
#include <cstdint>
#include <vector>

#include "../../pysiglib_b200/csrc/algebra_math.h"

using namespace sigb200;

namespace {

template <typename T, typename F>
void for_each_coeff(const Levels& lv, F f) {
    for (uint32_t j = 0; j < lv.total(); ++j) {
        const uint32_t t = lv.level_of(j);
        f(j, t, j - lv.off[t]);
    }
}

// E = exp(X), optionally Einv = exp(-X); powers holds P_2..P_N (N-1 vectors)
template <typename T>
void run_exp(const T* X, T* E, T* Einv, T* powers, const Levels& lv) {
    const uint64_t S = lv.total();
    for (uint64_t j = 0; j < S; ++j) {
        E[j] = X[j];
        if (Einv) Einv[j] = -X[j];
    }
    const T* prev = X;
    for (uint32_t n = 2; n <= lv.degree; ++n) {
        T* cur = powers + uint64_t(n - 2) * S;
        for_each_coeff<T>(lv, [&](uint32_t j, uint32_t t, uint32_t w) {
            const T val = exp_power_coeff(X, prev, lv, n, t, w);
            cur[j] = val;
            E[j] += val;
            if (Einv) Einv[j] += (n & 1) ? -val : val;
        });
        prev = cur;
    }
}

// level-1 part of the adjoint of exp at X for upstream dE
template <typename T>
void run_exp_adjoint_level1(const T* X, const T* powers, const T* dE, T* g, const Levels& lv) {
    const uint64_t S = lv.total();
    std::vector<T> a(S), b(S);
    for (uint64_t i = 0; i < lv.dim; ++i) g[i] = T(0);
    const T* dPn = nullptr;
    T* dPprev = a.data();
    for (uint32_t n = lv.degree; n >= 2; --n) {
        const T* prev = n == 2 ? X : powers + uint64_t(n - 3) * S;
        for_each_coeff<T>(lv, [&](uint32_t j, uint32_t t, uint32_t w) {
            dPprev[j] = exp_adjoint_prev_coeff(dE, dPn, X, lv, n, t, w);
            if (t >= n) {
                uint32_t letter;
                const T term = exp_adjoint_level1_term(dE, dPn, prev, lv, n, t, w, &letter);
                g[letter] += term;
            }
        });
        dPn = dPprev;
        dPprev = dPprev == a.data() ? b.data() : a.data();
    }
    for (uint64_t i = 0; i < lv.dim; ++i) g[i] += dE[i] + (dPn ? dPn[i] : T(0));
}

template <typename T>
void build_log(T* X, const T* path, uint64_t d, int step, const T* corr, uint64_t corr_len, const Levels& lv) {
    for (uint64_t j = 0; j < lv.total(); ++j) X[j] = T(0);
    for (uint64_t i = 0; i < d; ++i) X[i] = path[(step + 1) * d + i] - path[step * d + i];
    uint64_t offset = 0, level_size = d;
    for (uint32_t level = 2; level <= lv.degree; ++level) {
        level_size *= d;
        if (offset + level_size > corr_len) break;
        for (uint64_t w = 0; w < level_size; ++w) X[lv.off[level] + w] = corr[offset + w];  // data dim == dim here
        offset += level_size;
    }
}

template <typename T>
void correction_forward(const T* path, uint64_t L, uint64_t d, uint64_t degree, const T* corr, uint64_t corr_len,
                        uint64_t seg_stride, T* out) {
    const Levels lv = make_levels(d, degree);
    const uint64_t S = lv.total();
    std::vector<T> X(S), powers(S * degree), E(S), cur(S), nxt(S);
    for (uint64_t step = 0; step + 1 < L; ++step) {
        build_log(X.data(), path, d, int(step), corr + step * seg_stride, corr_len, lv);
        run_exp<T>(X.data(), E.data(), nullptr, powers.data(), lv);
        for_each_coeff<T>(lv, [&](uint32_t j, uint32_t t, uint32_t w) {
            nxt[j] = step == 0 ? E[j] : product_coeff(cur.data(), E.data(), lv, t, w);
        });
        cur.swap(nxt);
    }
    for (uint64_t j = 0; j < S; ++j) out[j] = cur[j];
}

template <typename T>
void correction_backward(const T* path, uint64_t L, uint64_t d, uint64_t degree, const T* corr, uint64_t corr_len,
                         uint64_t seg_stride, const T* sig, const T* derivs, T* out) {
    const Levels lv = make_levels(d, degree);
    const uint64_t S = lv.total();
    std::vector<T> X(S), powers(S * degree), E(S), Einv(S), Scur(sig, sig + S), Snxt(S), dScur(derivs, derivs + S),
        dSnxt(S), dE(S), g(d), g_next(d, T(0));
    for (int64_t step = int64_t(L) - 2; step >= 0; --step) {
        build_log(X.data(), path, d, int(step), corr + step * seg_stride, corr_len, lv);
        run_exp<T>(X.data(), E.data(), Einv.data(), powers.data(), lv);
        for_each_coeff<T>(lv, [&](uint32_t j, uint32_t t, uint32_t w) {
            Snxt[j] = product_coeff(Scur.data(), Einv.data(), lv, t, w);
        });
        Scur.swap(Snxt);
        for_each_coeff<T>(lv, [&](uint32_t j, uint32_t t, uint32_t w) {
            dE[j] = right_adjoint_coeff(dScur.data(), Scur.data(), lv, t, w);
            dSnxt[j] = left_adjoint_coeff(dScur.data(), E.data(), lv, t, w);
        });
        dScur.swap(dSnxt);
        run_exp_adjoint_level1<T>(X.data(), powers.data(), dE.data(), g.data(), lv);
        for (uint64_t i = 0; i < d; ++i) {
            out[(step + 1) * d + i] = g[i] - g_next[i];
            g_next[i] = g[i];
        }
    }
    for (uint64_t i = 0; i < d; ++i) out[i] = -g_next[i];
}

// Tensor logarithm in the phase order of sig_log.cu: R_k for k = N..2, then y = x - x (x) R_2.
template <typename T>
void run_log(const T* x, T* y, T* keep /* (N-1) vectors */, const Levels& lv) {
    const uint64_t S = lv.total();
    const uint32_t N = lv.degree;
    const T* r_old = nullptr;
    for (uint32_t k = N; k >= 2; --k) {
        T* r_new = keep + uint64_t(k - 2) * S;
        const T constant = T(1) / static_cast<T>(k);
        for_each_coeff<T>(lv, [&](uint32_t j, uint32_t t, uint32_t w) {
            T value = T(0);
            if (t <= 1 + N - k) {
                value = constant * x[j];
                if (r_old) value -= nonunital_product_coeff(x, r_old, lv, t, w);
            }
            r_new[j] = value;
        });
        r_old = r_new;
    }
    for_each_coeff<T>(lv, [&](uint32_t j, uint32_t t, uint32_t w) {
        T value = x[j];
        if (r_old && t >= 2) value -= nonunital_product_coeff(x, r_old, lv, t, w);
        y[j] = value;
    });
}

template <typename T>
void run_log_backprop(const T* x, const T* dy, T* dx, const Levels& lv) {
    const uint64_t S = lv.total();
    const uint32_t N = lv.degree;
    std::vector<T> keep(S * (N > 1 ? N - 1 : 1)), y(S), qa(S), qb(S), D(dy, dy + S);
    for (uint64_t j = 0; j < S; ++j) dx[j] = dy[j];
    if (N < 2) return;
    run_log<T>(x, y.data(), keep.data(), lv);
    const T* q = D.data();
    T* q_new = qa.data();
    for (uint32_t k = 1; k <= N; ++k) {
        const T* r_next = k < N ? keep.data() + uint64_t(k - 1) * S : nullptr;
        const T constant = T(1) / static_cast<T>(k);
        const uint32_t top = k == 1 ? N : 1 + N - k;
        for_each_coeff<T>(lv, [&](uint32_t j, uint32_t t, uint32_t w) {
            T add = (k >= 2 && t <= top) ? q[j] * constant : T(0);
            if (r_next) add -= nonunital_left_adjoint_coeff(q, r_next, lv, t, w, top);
            if (t <= top) dx[j] += add;
            if (k < N) q_new[j] = -nonunital_right_adjoint_coeff(q, x, lv, t, w, top);
        });
        q = q_new;
        q_new = q_new == qa.data() ? qb.data() : qa.data();
    }
}

}  // namespace

#define HARNESS(SUF, T)                                                                                               \
    extern "C" void alg_exp_##SUF(const T* X, T* E, uint64_t dim, uint64_t degree) {                                  \
        const Levels lv = make_levels(dim, degree);                                                                   \
        std::vector<T> powers(lv.total() * degree);                                                                   \
        run_exp<T>(X, E, nullptr, powers.data(), lv);                                                                 \
    }                                                                                                                 \
    extern "C" void alg_exp_adjoint_level1_##SUF(const T* X, const T* dE, T* g, uint64_t dim, uint64_t degree) {      \
        const Levels lv = make_levels(dim, degree);                                                                   \
        std::vector<T> powers(lv.total() * degree), E(lv.total());                                                    \
        run_exp<T>(X, E.data(), nullptr, powers.data(), lv);                                                          \
        run_exp_adjoint_level1<T>(X, powers.data(), dE, g, lv);                                                       \
    }                                                                                                                 \
    extern "C" void alg_product_##SUF(const T* A, const T* B, T* C, uint64_t dim, uint64_t degree) {                  \
        const Levels lv = make_levels(dim, degree);                                                                   \
        for_each_coeff<T>(lv, [&](uint32_t j, uint32_t t, uint32_t w) { C[j] = product_coeff(A, B, lv, t, w); });     \
    }                                                                                                                 \
    extern "C" void alg_adjoints_##SUF(const T* dC, const T* A, const T* B, T* dA, T* dB, uint64_t dim,               \
                                       uint64_t degree) {                                                             \
        const Levels lv = make_levels(dim, degree);                                                                   \
        for_each_coeff<T>(lv, [&](uint32_t j, uint32_t t, uint32_t w) {                                               \
            dA[j] = left_adjoint_coeff(dC, B, lv, t, w);                                                              \
            dB[j] = right_adjoint_coeff(dC, A, lv, t, w);                                                             \
        });                                                                                                           \
    }                                                                                                                 \
    extern "C" void alg_linear_sig_##SUF(const T* v, T* out, uint64_t dim, uint64_t degree) {                         \
        const Levels lv = make_levels(dim, degree);                                                                   \
        for_each_coeff<T>(lv, [&](uint32_t j, uint32_t t, uint32_t w) { out[j] = linear_sig_coeff(v, lv, t, w); });   \
    }                                                                                                                 \
    extern "C" void alg_linear_sig_adjoint_##SUF(const T* v, const T* dL, T* dv, uint64_t dim, uint64_t degree) {     \
        const Levels lv = make_levels(dim, degree);                                                                   \
        for (uint64_t i = 0; i < dim; ++i) dv[i] = T(0);                                                              \
        for_each_coeff<T>(lv, [&](uint32_t j, uint32_t t, uint32_t w) {                                               \
            linear_sig_adjoint_terms(v, dL[j], lv, t, w, [&](uint32_t letter, T value) { dv[letter] += value; });     \
        });                                                                                                           \
    }                                                                                                                 \
    extern "C" void alg_log_##SUF(const T* x, T* y, uint64_t dim, uint64_t degree) {                                  \
        const Levels lv = make_levels(dim, degree);                                                                   \
        std::vector<T> keep(lv.total() * degree);                                                                     \
        run_log<T>(x, y, keep.data(), lv);                                                                            \
    }                                                                                                                 \
    extern "C" void alg_log_backprop_##SUF(const T* x, const T* dy, T* dx, uint64_t dim, uint64_t degree) {           \
        run_log_backprop<T>(x, dy, dx, make_levels(dim, degree));                                                     \
    }                                                                                                                 \
    extern "C" void alg_correction_forward_##SUF(const T* path, uint64_t L, uint64_t d, uint64_t degree,              \
                                                 const T* corr, uint64_t corr_len, uint64_t seg_stride, T* out) {     \
        correction_forward<T>(path, L, d, degree, corr, corr_len, seg_stride, out);                                   \
    }                                                                                                                 \
    extern "C" void alg_correction_backward_##SUF(const T* path, uint64_t L, uint64_t d, uint64_t degree,             \
                                                  const T* corr, uint64_t corr_len, uint64_t seg_stride,              \
                                                  const T* sig, const T* derivs, T* out) {                            \
        correction_backward<T>(path, L, d, degree, corr, corr_len, seg_stride, sig, derivs, out);                     \
    }

HARNESS(f, float)
HARNESS(d, double)
