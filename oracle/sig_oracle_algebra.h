/*
 * CPU oracle, second part: tensor exponential, signatures with per-segment
 * correction terms, linear signatures and sig_join.
 *
 * TEST INFRASTRUCTURE ONLY, like sig_oracle_impl.h (which must be included first
 * in the same REAL / SUF / FMA context: it provides the path iterator, the fused
 * vector helpers and sig_combine_inplace_).
 *
 * Restates, operation for operation:
 *   siglib/cpsig/cp_exp_signature.h:43-101   tensor_exp_          (power series)
 *   siglib/cpsig/cp_exp_signature.h:108-210  tensor_exp_backprop_
 *   siglib/cpsig/cp_sig_combine.h:125-176    uncombine_sig_deriv
 *   siglib/cpsig/cp_sig_combine.h:232-262    linear_sig_deriv_to_increment_deriv
 *   siglib/cpsig/cp_signature.h:229-256      correction argument checks
 *   siglib/cpsig/cp_signature.h:263-305      apply_segment_correction_
 *   siglib/cpsig/cp_signature.h:319-359      signature_correction_inplace_
 *   siglib/cpsig/cp_signature.h:1021-1096    sig_backprop_correction_inplace_
 *   siglib/cpsig/cp_sig_join.h:36-57         linear_sig_with_level_index_
 *   siglib/cpsig/cp_sig_join.h:111-166       sig_join_
 *   siglib/cpsig/cp_sig_join.h:173-238       sig_join_backprop_
 *
 * Parity pin: tests/test_oracle_algebra.py checks these against the known answers
 * written out in the reference's tests/test_signature.py:126-188 (correction) and
 * against identities the reference's tests use (sig_join == sig of the extended
 * path, tests/test_linear_and_branched_join.py:86-112; zero correction == plain
 * signature), and the backward passes against central finite differences.
 */

#define CAT_(a, b) a##b
#define CAT(a, b) CAT_(a, b)
#define FN(name) CAT(name, SUF)

/* ----- cp_exp_signature.h:43-101 ----------------------------------------- */

static int FN(tensor_exp_)(const REAL* log_sig, REAL* out, uint64_t dim, uint64_t degree) {
    const uint64_t sig_len = oracle_sig_length(dim, degree);
    uint64_t* li = (uint64_t*)malloc((degree + 2) * sizeof(uint64_t));
    if (!li) return 1;
    populate_level_index(li, dim, degree + 2);
    out[0] = (REAL)1.;
    if (degree == 0) { free(li); return 0; }
    memcpy(out + li[1], log_sig + li[1], (li[degree + 1] - li[1]) * sizeof(REAL));
    if (degree <= 1) { free(li); return 0; }

    REAL* buf = (REAL*)malloc(2 * sig_len * sizeof(REAL));
    if (!buf) { free(li); return 1; }
    REAL* p_prev = buf;
    REAL* p_curr = buf + sig_len;
    memcpy(p_prev, log_sig, sig_len * sizeof(REAL));

    for (uint64_t n = 2; n <= degree; ++n) {
        const REAL inv_n = (REAL)1. / (REAL)n;
        for (uint64_t target = n; target <= degree; ++target) {
            const uint64_t begin = li[target], end = li[target + 1];
            memset(p_curr + begin, 0, (end - begin) * sizeof(REAL));
            const uint64_t max_left = target - (n - 1);
            for (uint64_t left = 1; left <= max_left; ++left) {
                const uint64_t right = target - left;
                REAL* res = p_curr + begin;
                const REAL* left_end = log_sig + li[left + 1];
                const uint64_t right_size = li[right + 1] - li[right];
                const REAL* right_start = p_prev + li[right];
                for (const REAL* lp = log_sig + li[left]; lp < left_end; ++lp) {
                    FN(vec_mult_add_)(res, right_start, *lp * inv_n, right_size);
                    res += right_size;
                }
            }
            for (uint64_t i = begin; i < end; ++i) out[i] += p_curr[i];
        }
        REAL* t = p_prev; p_prev = p_curr; p_curr = t;
    }
    free(buf);
    free(li);
    return 0;
}

/* ----- cp_exp_signature.h:108-210 ---------------------------------------- */

static int FN(tensor_exp_backprop_)(REAL* d_logsig, const REAL* d_sig, const REAL* log_sig, uint64_t dim,
                                    uint64_t degree) {
    const uint64_t sig_len = oracle_sig_length(dim, degree);
    uint64_t* li = (uint64_t*)malloc((degree + 2) * sizeof(uint64_t));
    if (!li) return 1;
    populate_level_index(li, dim, degree + 2);
    for (uint64_t i = 0; i < sig_len; ++i) d_logsig[i] = (REAL)0.;
    if (degree <= 1) {
        for (uint64_t i = li[1]; i < li[degree + 1]; ++i) d_logsig[i] = d_sig[i];
        free(li);
        return 0;
    }
    const uint64_t max_right = li[degree] - li[degree - 1];
    REAL* p_all = (REAL*)calloc(sig_len * degree + 2 * sig_len + max_right, sizeof(REAL));
    if (!p_all) { free(li); return 1; }
    REAL* dP = p_all + sig_len * degree;
    REAL* dP_next = dP + sig_len;
    REAL* upstream = dP_next + sig_len;
    memcpy(p_all, log_sig, sig_len * sizeof(REAL));

    for (uint64_t n = 2; n <= degree; ++n) {
        const REAL inv_n = (REAL)1. / (REAL)n;
        REAL* p_curr = p_all + (n - 1) * sig_len;
        const REAL* p_prev = p_all + (n - 2) * sig_len;
        for (uint64_t target = n; target <= degree; ++target) {
            const uint64_t max_left = target - (n - 1);
            for (uint64_t left = 1; left <= max_left; ++left) {
                const uint64_t right = target - left;
                REAL* res = p_curr + li[target];
                const REAL* left_end = log_sig + li[left + 1];
                const uint64_t right_size = li[right + 1] - li[right];
                const REAL* right_start = p_prev + li[right];
                for (const REAL* lp = log_sig + li[left]; lp < left_end; ++lp) {
                    FN(vec_mult_add_)(res, right_start, *lp * inv_n, right_size);
                    res += right_size;
                }
            }
        }
    }
    for (uint64_t i = li[1]; i < li[degree + 1]; ++i) d_logsig[i] = d_sig[i];

    for (int64_t n = (int64_t)degree; n >= 2; --n) {
        const REAL inv_n = (REAL)1. / (REAL)n;
        const REAL* p_prev = p_all + (n - 2) * sig_len;
        for (uint64_t i = 0; i < sig_len; ++i) dP_next[i] = (REAL)0.;
        for (uint64_t target = (uint64_t)n; target <= degree; ++target) {
            const uint64_t max_left = target - (uint64_t)(n - 1);
            for (uint64_t left = 1; left <= max_left; ++left) {
                const uint64_t right = target - left;
                const REAL* gp = d_sig + li[target];
                const REAL* dp = dP + li[target];
                REAL* d_left = d_logsig + li[left];
                const REAL* lp_end = log_sig + li[left + 1];
                REAL* d_right = dP_next + li[right];
                const REAL* rp_start = p_prev + li[right];
                const uint64_t right_size = li[right + 1] - li[right];
                for (const REAL* lp = log_sig + li[left]; lp < lp_end; ++lp) {
                    /* vec_add_scaled: upstream = (grad + dP) * inv_n */
                    for (uint64_t k = 0; k < right_size; ++k) upstream[k] = (gp[k] + dp[k]) * inv_n;
                    gp += right_size;
                    dp += right_size;
                    REAL dot = (REAL)0.;
                    for (uint64_t k = 0; k < right_size; ++k) dot = FMA(upstream[k], rp_start[k], dot);
                    *(d_left++) += dot;
                    FN(vec_mult_add_)(d_right, upstream, *lp, right_size);
                }
            }
        }
        REAL* t = dP; dP = dP_next; dP_next = t;
    }
    for (uint64_t i = li[1]; i < li[degree + 1]; ++i) d_logsig[i] += dP[i];
    free(p_all);
    free(li);
    return 0;
}

/* ----- cp_sig_combine.h:125-176 ------------------------------------------ */
/* In: concat_deriv = dF/d(sig1 (x) sig2).  Out: concat_deriv = dF/d sig1, sig2_deriv = dF/d sig2. */

static void FN(uncombine_sig_deriv_)(const REAL* sig1, const REAL* sig2, REAL* concat_deriv, REAL* sig2_deriv,
                                     uint64_t dim, uint64_t degree, const uint64_t* li) {
    memcpy(sig2_deriv, concat_deriv, oracle_sig_length(dim, degree) * sizeof(REAL));
    for (uint64_t level = degree; level > 0; --level) {
        for (uint64_t left = level - 1, right = 1; left > 0; --left, ++right) {
            REAL* res = concat_deriv + li[level];
            REAL* right_deriv = sig2_deriv + li[right];
            const uint64_t right_size = li[right + 1] - li[right];
            const uint64_t left_size = li[left + 1] - li[left];
            const REAL* left_base = sig1 + li[left];
            for (uint64_t i = 0; i < left_size; ++i) {
                FN(vec_mult_add_)(right_deriv, res, left_base[i], right_size);
                res += right_size;
            }
        }
    }
    for (uint64_t left = 1; left < degree; ++left) {
        for (uint64_t level = left + 1, right = 1; level <= degree; ++level, ++right) {
            REAL* res = concat_deriv + li[level];
            REAL* left_base = concat_deriv + li[left];
            const uint64_t left_size = li[left + 1] - li[left];
            const REAL* right_base = sig2 + li[right];
            const uint64_t right_size = li[right + 1] - li[right];
            for (uint64_t i = 0; i < left_size; ++i) {
                REAL dot = (REAL)0.;
                for (uint64_t k = 0; k < right_size; ++k) dot = FMA(res[k], right_base[k], dot);
                left_base[i] += dot;
                res += right_size;
            }
        }
    }
}

/* ----- cp_signature.h:263-305 -------------------------------------------- */

static void FN(apply_segment_correction_)(REAL* local_log, const REAL* corr, uint64_t corr_len, uint64_t data_dim,
                                          uint64_t dim, uint64_t degree, const uint64_t* li) {
    const uint64_t sig_len = li[degree + 1];
    for (uint64_t i = 0; i < sig_len; ++i) local_log[i] = (REAL)0;
    if (corr == NULL || corr_len == 0) return;
    uint64_t offset = 0, level_size = data_dim;
    for (uint64_t level = 2; level <= degree; ++level) {
        level_size *= data_dim;
        if (offset + level_size > corr_len) break;
        for (uint64_t w = 0; w < level_size; ++w) {
            const REAL value = corr[offset + w];
            if (value == (REAL)0) continue;
            uint64_t tmp = w, aug = 0, pw = level_size / data_dim;
            for (uint64_t pos = 0; pos < level; ++pos) {
                const uint64_t label = tmp / pw;
                tmp -= label * pw;
                if (pos + 1 < level) pw /= data_dim;
                aug = aug * dim + label;
            }
            local_log[li[level] + aug] += value;
        }
        offset += level_size;
    }
}

/* cp_signature.h:229-256; returns 0 if the arguments are acceptable */
static int FN(correction_args_bad_)(const void* corr, uint64_t corr_len, uint64_t d, uint64_t degree, int lead_lag) {
    if (corr == NULL && corr_len != 0) return 1;
    if (lead_lag && corr_len != 0) return 1;
    if (corr_len == 0) return 0;
    if (degree < 2) return 1;
    uint64_t offset = 0, level_size = d;
    for (uint64_t level = 2; level <= degree; ++level) {
        level_size *= d;
        offset += level_size;
        if (offset == corr_len) return 0;
        if (offset > corr_len) break;
    }
    return 1;
}

/* ----- cp_signature.h:319-359 (one path; out has the scalar term) -------- */

static int FN(signature_correction_one_)(const FN(opath_)* path, REAL* out, uint64_t degree, const REAL* corr,
                                         uint64_t corr_len, uint64_t seg_stride, const uint64_t* li) {
    const uint64_t dim = path->dim, sig_len = li[degree + 1];
    REAL* local_log = (REAL*)malloc(2 * sig_len * sizeof(REAL));
    if (!local_log) return 1;
    REAL* local_sig = local_log + sig_len;
    FN(opoint_) prev = FN(opoint_at_)(path, 0);
    FN(opoint_) next = FN(opoint_at_)(path, 0);
    FN(opoint_inc_)(&next);
    int rc = 0;
    for (uint64_t step = 0; step + 1 < path->len && !rc; ++step, FN(opoint_inc_)(&prev), FN(opoint_inc_)(&next)) {
        FN(apply_segment_correction_)(local_log, corr + step * seg_stride, corr_len, path->data_dim, dim, degree, li);
        for (uint64_t i = 0; i < dim; ++i) local_log[i + 1] = FN(opoint_get_)(&next, i) - FN(opoint_get_)(&prev, i);
        if (step == 0) {
            rc = FN(tensor_exp_)(local_log, out, dim, degree);
        } else {
            rc = FN(tensor_exp_)(local_log, local_sig, dim, degree);
            FN(sig_combine_inplace_)(out, local_sig, degree, li);
        }
    }
    free(local_log);
    return rc;
}

/* ----- cp_signature.h:1021-1096 (sig, sig_derivs: scalar-padded private copies, overwritten) */

static int FN(sig_backprop_correction_one_)(const FN(opath_)* path, REAL* out, REAL* sig_derivs, REAL* sig,
                                            uint64_t degree, const REAL* corr, uint64_t corr_len,
                                            uint64_t seg_stride, const uint64_t* li) {
    const uint64_t dim = path->dim, data_dim = path->data_dim, sig_len = li[degree + 1];
    REAL* buf = (REAL*)malloc(6 * sig_len * sizeof(REAL));
    if (!buf) return 1;
    REAL *local_derivs = buf, *local_log_derivs = buf + sig_len, *local_log = buf + 2 * sig_len,
         *inverse = buf + 3 * sig_len, *local_sig = buf + 4 * sig_len, *inverse_sig = buf + 5 * sig_len;
    int rc = 0;
    for (uint64_t step = path->len - 1; step-- > 0 && !rc;) {
        FN(opoint_) prev = FN(opoint_at_)(path, step);
        FN(opoint_) next = FN(opoint_at_)(path, step + 1);
        FN(apply_segment_correction_)(local_log, corr + step * seg_stride, corr_len, data_dim, dim, degree, li);
        for (uint64_t i = 0; i < dim; ++i) local_log[i + 1] = FN(opoint_get_)(&next, i) - FN(opoint_get_)(&prev, i);
        rc = FN(tensor_exp_)(local_log, local_sig, dim, degree);
        inverse[0] = (REAL)0;
        for (uint64_t i = 1; i < sig_len; ++i) inverse[i] = -local_log[i];
        if (!rc) rc = FN(tensor_exp_)(inverse, inverse_sig, dim, degree);
        FN(sig_combine_inplace_)(sig, inverse_sig, degree, li);
        FN(uncombine_sig_deriv_)(sig, local_sig, sig_derivs, local_derivs, dim, degree, li);
        if (!rc) rc = FN(tensor_exp_backprop_)(local_log_derivs, local_derivs, local_log, dim, degree);
        REAL* pos = out + (step + 1) * data_dim;
        REAL* neg = out + step * data_dim;
        for (uint64_t dd = 0; dd < data_dim; ++dd) {
            pos[dd] += local_log_derivs[1 + dd];
            neg[dd] -= local_log_derivs[1 + dd];
        }
    }
    free(buf);
    return rc;
}

/* Batch drivers for the correction variants (serial; 0 ok, 1 allocation failure, 2 invalid argument). */
int FN(oracle_signature_correction_)(const REAL* path, REAL* out, uint64_t batch, uint64_t d, uint64_t L,
                                     uint64_t degree, int time_aug, REAL end_time, int scalar_term,
                                     const REAL* corr, uint64_t corr_len, uint64_t batch_stride,
                                     uint64_t seg_stride) {
    if (d == 0 || corr_len == 0 || FN(correction_args_bad_)(corr, corr_len, d, degree, 0)) return 2;
    FN(opath_) p;
    FN(opath_init_)(&p, path, d, L, time_aug, 0, end_time);
    const uint64_t full = oracle_sig_length(p.dim, degree);
    const uint64_t stride = scalar_term ? full : full - 1;
    if (p.len <= 1) {
        for (uint64_t b = 0; b < batch; ++b) {
            for (uint64_t i = 0; i < stride; ++i) out[b * stride + i] = (REAL)0;
            if (scalar_term) out[b * stride] = (REAL)1;
        }
        return 0;
    }
    uint64_t* li = (uint64_t*)malloc((degree + 2) * sizeof(uint64_t));
    REAL* full_out = (REAL*)malloc(full * sizeof(REAL));
    if (!li || !full_out) { free(li); free(full_out); return 1; }
    populate_level_index(li, p.dim, degree + 2);
    int rc = 0;
    for (uint64_t b = 0; b < batch && !rc; ++b) {
        FN(opath_init_)(&p, path + b * d * L, d, L, time_aug, 0, end_time);
        rc = FN(signature_correction_one_)(&p, full_out, degree, corr + b * batch_stride, corr_len, seg_stride, li);
        memcpy(out + b * stride, full_out + (scalar_term ? 0 : 1), stride * sizeof(REAL));
    }
    free(li);
    free(full_out);
    return rc;
}

int FN(oracle_sig_backprop_correction_)(const REAL* path, REAL* out, const REAL* sig_derivs, const REAL* sig,
                                        uint64_t batch, uint64_t d, uint64_t L, uint64_t degree, int time_aug,
                                        REAL end_time, int scalar_term, const REAL* corr, uint64_t corr_len,
                                        uint64_t batch_stride, uint64_t seg_stride) {
    if (d == 0 || corr_len == 0 || FN(correction_args_bad_)(corr, corr_len, d, degree, 0)) return 2;
    for (uint64_t i = 0; i < batch * d * L; ++i) out[i] = (REAL)0;
    FN(opath_) p;
    FN(opath_init_)(&p, path, d, L, time_aug, 0, end_time);
    if (p.len <= 1 || degree == 0) return 0;
    const uint64_t full = oracle_sig_length(p.dim, degree);
    const uint64_t stride = scalar_term ? full : full - 1;
    uint64_t* li = (uint64_t*)malloc((degree + 2) * sizeof(uint64_t));
    REAL* copies = (REAL*)malloc(2 * full * sizeof(REAL));
    if (!li || !copies) { free(li); free(copies); return 1; }
    populate_level_index(li, p.dim, degree + 2);
    int rc = 0;
    for (uint64_t b = 0; b < batch && !rc; ++b) {
        REAL* dcopy = copies;
        REAL* scopy = copies + full;
        dcopy[0] = (REAL)0;
        scopy[0] = (REAL)1;
        memcpy(dcopy + 1, sig_derivs + b * stride + (scalar_term ? 1 : 0), (full - 1) * sizeof(REAL));
        memcpy(scopy + 1, sig + b * stride + (scalar_term ? 1 : 0), (full - 1) * sizeof(REAL));
        if (scalar_term) dcopy[0] = sig_derivs[b * stride];
        FN(opath_init_)(&p, path + b * d * L, d, L, time_aug, 0, end_time);
        rc = FN(sig_backprop_correction_one_)(&p, out + b * d * L, dcopy, scopy, degree, corr + b * batch_stride,
                                              corr_len, seg_stride, li);
    }
    free(li);
    free(copies);
    return rc;
}

/* Exposed so that the device kernels for exp / its adjoint can be checked on their own. */
int FN(oracle_tensor_exp_)(const REAL* log_sig, REAL* out, uint64_t dim, uint64_t degree) {
    return FN(tensor_exp_)(log_sig, out, dim, degree);
}
int FN(oracle_tensor_exp_backprop_)(REAL* d_logsig, const REAL* d_sig, const REAL* log_sig, uint64_t dim,
                                    uint64_t degree) {
    return FN(tensor_exp_backprop_)(d_logsig, d_sig, log_sig, dim, degree);
}

/* ----- cp_sig_join.h:36-57 (out always carries the scalar slot here) ----- */

static void FN(linear_sig_full_)(const REAL* disp, REAL* out, uint64_t dim, uint64_t degree, const uint64_t* li) {
    out[0] = (REAL)1;
    if (degree == 0) return;
    memcpy(out + 1, disp, dim * sizeof(REAL));
    for (uint64_t level = 2; level <= degree; ++level) {
        const REAL one_over_level = (REAL)1. / (REAL)level;
        REAL* res = out + li[level];
        const REAL* left_end = out + li[level];
        for (const REAL* lp = out + li[level - 1]; lp != left_end; ++lp, res += dim)
            FN(vec_mult_assign_)(res, out + 1, (*lp) * one_over_level, dim);
    }
}

int FN(oracle_linear_sig_)(const REAL* disp, REAL* out, uint64_t batch, uint64_t dim, uint64_t degree,
                           int scalar_term) {
    if (dim == 0) return 2;
    const uint64_t full = oracle_sig_length(dim, degree);
    const uint64_t stride = scalar_term ? full : full - 1;
    uint64_t* li = (uint64_t*)malloc((degree + 2) * sizeof(uint64_t));
    REAL* buf = (REAL*)malloc(full * sizeof(REAL));
    if (!li || !buf) { free(li); free(buf); return 1; }
    populate_level_index(li, dim, degree + 2);
    for (uint64_t b = 0; b < batch; ++b) {
        FN(linear_sig_full_)(disp + b * dim, buf, dim, degree, li);
        memcpy(out + b * stride, buf + (scalar_term ? 0 : 1), stride * sizeof(REAL));
    }
    free(li);
    free(buf);
    return 0;
}

/* ----- cp_sig_join.h:111-166 --------------------------------------------- */

int FN(oracle_sig_join_)(const REAL* sig, const REAL* disp, REAL* out, uint64_t batch, uint64_t dim,
                         uint64_t degree, int prepend, int scalar_term) {
    if (dim == 0) return 2;
    const uint64_t full = oracle_sig_length(dim, degree);
    const uint64_t stride = scalar_term ? full : full - 1;
    uint64_t* li = (uint64_t*)malloc((degree + 2) * sizeof(uint64_t));
    REAL* buf = (REAL*)malloc(2 * full * sizeof(REAL));
    if (!li || !buf) { free(li); free(buf); return 1; }
    REAL* lsig = buf;
    REAL* acc = buf + full;
    populate_level_index(li, dim, degree + 2);
    for (uint64_t b = 0; b < batch; ++b) {
        FN(linear_sig_full_)(disp + b * dim, lsig, dim, degree, li);
        if (prepend) {
            /* out = lsig (x) sig */
            REAL* s = (REAL*)malloc(full * sizeof(REAL));
            if (!s) { free(li); free(buf); return 1; }
            s[0] = (REAL)1;
            memcpy(s + 1, sig + b * stride + (scalar_term ? 1 : 0), (full - 1) * sizeof(REAL));
            memcpy(acc, lsig, full * sizeof(REAL));
            FN(sig_combine_inplace_)(acc, s, degree, li);
            free(s);
        } else {
            acc[0] = (REAL)1;
            memcpy(acc + 1, sig + b * stride + (scalar_term ? 1 : 0), (full - 1) * sizeof(REAL));
            FN(sig_combine_inplace_)(acc, lsig, degree, li);
        }
        memcpy(out + b * stride, acc + (scalar_term ? 0 : 1), stride * sizeof(REAL));
    }
    free(li);
    free(buf);
    return 0;
}

/* ----- cp_sig_combine.h:232-262 ------------------------------------------ */

static void FN(linear_sig_deriv_to_increment_deriv_)(const REAL* sig, REAL* sig_deriv, REAL* inc_deriv, uint64_t dim,
                                                     uint64_t degree, const uint64_t* li) {
    for (uint64_t i = 0; i < dim; ++i) inc_deriv[i] = (REAL)0.;
    if (degree == 0) return; /* no level 1 to read (the reference reads past its buffer here) */
    for (uint64_t level = degree; level > 1; --level) {
        const REAL one_over_level = (REAL)(1. / (double)level);
        const uint64_t level_size = li[level] - li[level - 1];
        for (uint64_t j = 0; j < level_size; ++j) {
            const REAL* level_deriv = sig_deriv + li[level] + dim * j;
            const uint64_t offs2 = li[level - 1] + j;
            /* dot_product_mult_add: inc_deriv += level_deriv * scalar; returns <sig+1, level_deriv> */
            const REAL scalar = sig[offs2] * one_over_level;
            REAL dot = (REAL)0.;
            for (uint64_t k = 0; k < dim; ++k) {
                dot = FMA(sig[1 + k], level_deriv[k], dot);
                inc_deriv[k] = FMA(level_deriv[k], scalar, inc_deriv[k]);
            }
            sig_deriv[offs2] += dot * one_over_level;
        }
    }
    FN(vec_mult_add_)(inc_deriv, sig_deriv + 1, (REAL)1., dim);
}

/* ----- cp_sig_join.h:173-238 --------------------------------------------- */

int FN(oracle_sig_join_backprop_)(const REAL* d_out, REAL* d_sig, REAL* d_disp, const REAL* sig, const REAL* disp,
                                  uint64_t batch, uint64_t dim, uint64_t degree, int prepend, int scalar_term) {
    if (dim == 0) return 2;
    const uint64_t full = oracle_sig_length(dim, degree);
    const uint64_t stride = scalar_term ? full : full - 1;
    const uint64_t off = scalar_term ? 1 : 0;
    uint64_t* li = (uint64_t*)malloc((degree + 2) * sizeof(uint64_t));
    REAL* buf = (REAL*)malloc(5 * full * sizeof(REAL));
    if (!li || !buf) { free(li); free(buf); return 1; }
    REAL *lsig = buf, *d_lsig = buf + full, *d_out_full = buf + 2 * full, *d_sig_full = buf + 3 * full,
         *sig_full = buf + 4 * full;
    populate_level_index(li, dim, degree + 2);
    for (uint64_t b = 0; b < batch; ++b) {
        FN(linear_sig_full_)(disp + b * dim, lsig, dim, degree, li);
        d_out_full[0] = scalar_term ? d_out[b * stride] : (REAL)0;
        memcpy(d_out_full + 1, d_out + b * stride + off, (full - 1) * sizeof(REAL));
        sig_full[0] = scalar_term ? sig[b * stride] : (REAL)1;
        memcpy(sig_full + 1, sig + b * stride + off, (full - 1) * sizeof(REAL));
        if (prepend) {
            memcpy(d_lsig, d_out_full, full * sizeof(REAL));
            FN(uncombine_sig_deriv_)(lsig, sig_full, d_lsig, d_sig_full, dim, degree, li);
        } else {
            memcpy(d_sig_full, d_out_full, full * sizeof(REAL));
            FN(uncombine_sig_deriv_)(sig_full, lsig, d_sig_full, d_lsig, dim, degree, li);
        }
        d_sig_full[0] = (REAL)0;
        d_lsig[0] = (REAL)0;
        memcpy(d_sig + b * stride, d_sig_full + (scalar_term ? 0 : 1), stride * sizeof(REAL));
        FN(linear_sig_deriv_to_increment_deriv_)(lsig, d_lsig, d_disp + b * dim, dim, degree, li);
    }
    free(li);
    free(buf);
    return 0;
}

#undef FN
#undef CAT
#undef CAT_
