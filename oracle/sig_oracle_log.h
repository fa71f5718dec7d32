/*
 * CPU oracle, third part: signature -> log signature (expanded tensor log and its
 * Lyndon-word coordinates) and the backward pass.
 *
 * TEST INFRASTRUCTURE ONLY.  Include after sig_oracle_impl.h in the same REAL / SUF / FMA context.
 *
 * Restates:
 *   siglib/cpsig/cp_tensor_log.h:47-122    tensor_log_ (Horner form of log(1+x), in place)
 *   siglib/cpsig/cp_tensor_log.h:128-158   log_sig_expanded, log_sig_lyndon_words
 *   siglib/cpsig/cp_tensor_log.h:176-259   tensor_log_backprop_, ..._lyndon_words
 *   siglib/cpsig/cp_sig_combine.h:178-230  uncombine_sig_deriv_zero
 *   siglib/cpsig/cp_log_signature.h:62-124, 140-226  batch drivers (scalar-term handling)
 *   siglib/shared/preparation/log_sig/lyndon_words.cpp:25-112  Lyndon words by length (Duval),
 *                                                              word -> flat index
 *
 * Parity pin: tests/test_oracle_log.py (log of a linear signature is the displacement, the
 * closed form of level 2, exp(log) round trip through tensor_exp_, log_sig_length against the
 * necklace formula of pysiglib/sig_length.py:97-163, backward against finite differences).
 */

#define CAT_(a, b) a##b
#define CAT(a, b) CAT_(a, b)
#define FN(name) CAT(name, SUF)

#ifndef SIG_ORACLE_LYNDON_ONCE
#define SIG_ORACLE_LYNDON_ONCE
/* Flat indices (scalar slot = 0) of the Lyndon words of length 1..degree over `dim` letters, by
 * length then lexicographically; returns the count, writes at most `cap` entries when out != NULL. */
uint64_t oracle_lyndon_indices(uint64_t dim, uint64_t degree, uint64_t* out, uint64_t cap) {
    uint64_t count = 0;
    uint64_t* w = (uint64_t*)malloc((degree + 1) * sizeof(uint64_t));
    if (!w) return 0;
    for (uint64_t n = 1; n <= degree; ++n) {
        uint64_t size = 1;
        w[0] = 0;
        while (size > 0) {
            const uint64_t m = size;
            if (m == n) {
                uint64_t idx = 0;
                for (uint64_t i = 0; i < n; ++i) idx = idx * dim + w[i] + 1;
                if (out && count < cap) out[count] = idx;
                ++count;
            }
            while (size < n) { w[size] = w[size - m]; ++size; }
            while (size > 0 && w[size - 1] == dim - 1) --size;
            if (size > 0) ++w[size - 1];
        }
    }
    free(w);
    return count;
}
#endif

/* cp_tensor_log.h:47-122; partial_logs (optional) receives the intermediate buff1 states */
static int FN(tensor_log_)(REAL* sig, uint64_t dim, uint64_t degree, REAL* partial_logs) {
    sig[0] = (REAL)0.;
    if (degree == 1) return 0;
    uint64_t* li = (uint64_t*)malloc((degree + 2) * sizeof(uint64_t));
    if (!li) return 1;
    populate_level_index(li, dim, degree + 2);
    const uint64_t buff1_size = oracle_sig_length(dim, degree - 1);
    const uint64_t buff2_size = oracle_sig_length(dim, degree);
    REAL* buff1 = (REAL*)calloc(buff1_size + buff2_size, sizeof(REAL));
    if (!buff1) { free(li); return 1; }
    REAL* buff2 = buff1 + buff1_size;

    for (int64_t k = (int64_t)degree; k > 0; --k) {
        const REAL constant = (REAL)1. / (REAL)k;
        for (uint64_t target = 2; target <= 1 + degree - (uint64_t)k; ++target) {
            memset(buff2 + li[target], 0, (li[target + 1] - li[target]) * sizeof(REAL));
            for (uint64_t left = 1; left < target; ++left) {
                const uint64_t right = target - left;
                REAL* res = buff2 + li[target];
                const REAL* left_end = sig + li[left + 1];
                const uint64_t right_size = li[right + 1] - li[right];
                const REAL* right_start = buff1 + li[right];
                for (const REAL* lp = sig + li[left]; lp < left_end; ++lp) {
                    FN(vec_mult_add_)(res, right_start, *lp, right_size);
                    res += right_size;
                }
            }
        }
        if (k == 1) continue;
        for (uint64_t target = 1; target <= 1 + degree - (uint64_t)k; ++target) {
            const uint64_t size = li[target + 1] - li[target];
            REAL* res = buff1 + li[target];
            const REAL* p1 = sig + li[target];
            const REAL* p2 = buff2 + li[target];
            for (uint64_t i = 0; i < size; ++i) res[i] = constant * p1[i] - p2[i];
        }
        if (partial_logs && k > 2 && k != (int64_t)degree) {
            memcpy(partial_logs, buff1, sizeof(REAL) * buff1_size);
            partial_logs += buff1_size;
        }
    }
    for (uint64_t target = 2; target <= degree; ++target) {
        const uint64_t size = li[target + 1] - li[target];
        REAL* res = sig + li[target];
        const REAL* p = buff2 + li[target];
        for (uint64_t i = 0; i < size; ++i) res[i] -= p[i];
    }
    if (partial_logs) memcpy(partial_logs, buff1, sizeof(REAL) * buff1_size);
    free(buff1);
    free(li);
    return 0;
}

/* cp_sig_combine.h:178-230: like uncombine_sig_deriv but sig2_deriv starts from zero, the unit
 * terms are left out and the result levels of concat_deriv below `degree` are rebuilt from zero */
static void FN(uncombine_sig_deriv_zero_)(const REAL* sig1, const REAL* sig2, REAL* concat_deriv, REAL* sig2_deriv,
                                          uint64_t dim, uint64_t degree, const uint64_t* li) {
    const uint64_t n = oracle_sig_length(dim, degree - 1);
    for (uint64_t i = 0; i < n; ++i) sig2_deriv[i] = (REAL)0.;
    for (int64_t level = (int64_t)degree; level > 0; --level) {
        for (int64_t left = level - 1, right = 1; left > 0; --left, ++right) {
            const REAL* res = concat_deriv + li[level];
            REAL* right_base = sig2_deriv + li[right];
            const uint64_t right_size = li[right + 1] - li[right];
            const uint64_t left_size = li[left + 1] - li[left];
            const REAL* left_base = sig1 + li[left];
            for (uint64_t i = 0; i < left_size; ++i) {
                const REAL scalar = left_base[i];
                for (uint64_t k = 0; k < right_size; ++k) right_base[k] += res[k] * scalar;
                res += right_size;
            }
        }
    }
    for (uint64_t left = 1; left < degree; ++left) {
        for (uint64_t i = li[left]; i < li[left + 1]; ++i) concat_deriv[i] = (REAL)0.;
        for (uint64_t level = left + 1, right = 1; level <= degree; ++level, ++right) {
            const REAL* res = concat_deriv + li[level];
            REAL* left_base = concat_deriv + li[left];
            const uint64_t left_size = li[left + 1] - li[left];
            const REAL* right_base = sig2 + li[right];
            const uint64_t right_size = li[right + 1] - li[right];
            for (uint64_t i = 0; i < left_size; ++i) {
                REAL accum = (REAL)0;
                for (uint64_t k = 0; k < right_size; ++k) accum += res[k] * right_base[k];
                left_base[i] += accum;
                res += right_size;
            }
        }
    }
}

/* cp_tensor_log.h:176-235; derivs is overwritten (callers pass a copy) */
static int FN(tensor_log_backprop_)(REAL* out, REAL* derivs, const REAL* sig, uint64_t dim, uint64_t degree) {
    const uint64_t sig_len = oracle_sig_length(dim, degree);
    const uint64_t sig_len2 = oracle_sig_length(dim, degree - 1);
    uint64_t* li = (uint64_t*)malloc((degree + 2) * sizeof(uint64_t));
    if (!li) return 1;
    populate_level_index(li, dim, degree + 2);
    memcpy(out, derivs, sig_len * sizeof(REAL));
    out[0] = (REAL)0.;
    if (degree <= 1) { free(li); return 0; }
    REAL* buf = (REAL*)calloc(2 * sig_len + sig_len2 * (degree - 1), sizeof(REAL));
    if (!buf) { free(li); return 1; }
    REAL* sig_copy = buf;
    REAL* other = buf + sig_len;
    REAL* partial_logs = buf + 2 * sig_len;
    memcpy(sig_copy, sig, sig_len * sizeof(REAL));
    int rc = FN(tensor_log_)(sig_copy, dim, degree, partial_logs);
    REAL* cur = derivs;
    REAL factor = (REAL)-1.;
    for (uint64_t depth = 1; depth + 1 < degree; ++depth) {
        const REAL scalar = (REAL)1. / (REAL)(1 + depth);
        REAL* partial = partial_logs + (degree - 2 - depth) * sig_len2;
        FN(uncombine_sig_deriv_zero_)(sig, partial, cur, other, dim, degree + 1 - depth, li);
        for (uint64_t lev = 1; lev <= degree - depth; ++lev)
            for (uint64_t i = li[lev]; i < li[lev + 1]; ++i) out[i] += factor * (cur[i] + scalar * other[i]);
        REAL* t = other; other = cur; cur = t;
        factor = -factor;
    }
    const REAL scalar = factor / (REAL)degree;
    REAL* out1 = out + li[1];
    const REAL* d2 = cur + li[2];
    const REAL* s1 = sig + li[1];
    for (uint64_t i = 0; i < dim; ++i)
        for (uint64_t j = 0; j < dim; ++j) {
            out1[i] += d2[i + dim * j] * s1[j] * scalar;
            out1[j] += d2[i + dim * j] * s1[i] * scalar;
        }
    free(buf);
    free(li);
    return rc;
}

/* cp_log_signature.h:62-124.  method 0: expanded (out has the layout of sig); 1: Lyndon words. */
int FN(oracle_sig_to_log_sig_)(const REAL* sig, REAL* out, uint64_t batch, uint64_t dim, uint64_t degree, int method,
                               int scalar_term) {
    if (dim == 0 || degree == 0 || method < 0 || method > 1) return 2;
    const uint64_t full = oracle_sig_length(dim, degree);
    const uint64_t in_stride = scalar_term ? full : full - 1;
    const uint64_t m = method ? oracle_lyndon_indices(dim, degree, NULL, 0) : 0;
    const uint64_t out_stride = method ? m : in_stride;
    REAL* work = (REAL*)malloc(full * sizeof(REAL));
    uint64_t* idx = method ? (uint64_t*)malloc((m + 1) * sizeof(uint64_t)) : NULL;
    if (!work || (method && !idx)) { free(work); free(idx); return 1; }
    if (method) oracle_lyndon_indices(dim, degree, idx, m);
    int rc = 0;
    for (uint64_t b = 0; b < batch && !rc; ++b) {
        work[0] = (REAL)1;
        memcpy(work + 1, sig + b * in_stride + (scalar_term ? 1 : 0), (full - 1) * sizeof(REAL));
        rc = FN(tensor_log_)(work, dim, degree, NULL);
        if (method) for (uint64_t i = 0; i < m; ++i) out[b * out_stride + i] = work[idx[i]];
        else memcpy(out + b * out_stride, work + (scalar_term ? 0 : 1), out_stride * sizeof(REAL));
    }
    free(work);
    free(idx);
    return rc;
}

/* cp_log_signature.h:140-226: out (layout of sig) = dF/d sig given dF/d log_sig */
int FN(oracle_sig_to_log_sig_backprop_)(const REAL* sig, REAL* out, const REAL* log_sig_derivs, uint64_t batch,
                                        uint64_t dim, uint64_t degree, int method, int scalar_term) {
    if (dim == 0 || degree == 0 || method < 0 || method > 1) return 2;
    const uint64_t full = oracle_sig_length(dim, degree);
    const uint64_t stride = scalar_term ? full : full - 1;
    const uint64_t m = method ? oracle_lyndon_indices(dim, degree, NULL, 0) : 0;
    const uint64_t lsd_stride = method ? m : stride;
    REAL* buf = (REAL*)malloc(3 * full * sizeof(REAL));
    uint64_t* idx = method ? (uint64_t*)malloc((m + 1) * sizeof(uint64_t)) : NULL;
    if (!buf || (method && !idx)) { free(buf); free(idx); return 1; }
    if (method) oracle_lyndon_indices(dim, degree, idx, m);
    REAL *sig_full = buf, *derivs = buf + full, *out_full = buf + 2 * full;
    int rc = 0;
    for (uint64_t b = 0; b < batch && !rc; ++b) {
        sig_full[0] = (REAL)1;
        memcpy(sig_full + 1, sig + b * stride + (scalar_term ? 1 : 0), (full - 1) * sizeof(REAL));
        for (uint64_t i = 0; i < full; ++i) derivs[i] = (REAL)0;
        if (method) for (uint64_t i = 0; i < m; ++i) derivs[idx[i]] = log_sig_derivs[b * lsd_stride + i];
        else memcpy(derivs + 1, log_sig_derivs + b * lsd_stride + (scalar_term ? 1 : 0), (full - 1) * sizeof(REAL));
        rc = FN(tensor_log_backprop_)(out_full, derivs, sig_full, dim, degree);
        memcpy(out + b * stride, out_full + (scalar_term ? 0 : 1), stride * sizeof(REAL));
    }
    free(buf);
    free(idx);
    return rc;
}

#undef FN
#undef CAT
#undef CAT_
