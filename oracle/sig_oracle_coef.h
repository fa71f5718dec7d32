/*
 * CPU oracle, fourth part: individual signature coefficients (sig_coef) and the backward pass.
 *
 * TEST INFRASTRUCTURE ONLY.  Include after sig_oracle_impl.h in the same REAL / SUF / FMA context
 * (it uses the augmented-path iterator defined there).
 *
 * Restates siglib/cpsig/cp_sig_coef_impl.cpp:
 *   36-80     single_sig_coef_        (prefix chain of one word, Chen update per step)
 *   139-211   sig_coef_               (words of one path, prefixes, trivial cases)
 *   354-431   uncombine_coefs_, backprop_horner_
 *   433-486   single_sig_coef_backprop_ (reverse sweep, lead-lag / time-aug channel selection)
 *   545-611   sig_coef_backprop_      (words of one path)
 *
 * Parity pin: tests/test_oracle_coef.py (coefficients equal the entries of the oracle's full
 * signature, which the reference's golden vectors pin; backward against finite differences).
 */

#define CAT_(a, b) a##b
#define CAT(a, b) CAT_(a, b)
#define FN(name) CAT(name, SUF)

static void FN(single_sig_coef_)(const FN(opath_)* path, REAL* out, const uint64_t* word, uint64_t degree,
                                 REAL* coefs, REAL* incr, const REAL* f, int prefixes) {
    FN(opoint_) prev = FN(opoint_at_)(path, 0);
    FN(opoint_) next = FN(opoint_at_)(path, 0);
    FN(opoint_inc_)(&next);
    coefs[0] = (REAL)1.;
    REAL product = (REAL)1.;
    for (uint64_t i = 0; i < degree; ++i) {
        incr[i] = FN(opoint_get_)(&next, word[i]) - FN(opoint_get_)(&prev, word[i]);
        product *= incr[i];
        coefs[i + 1] = product * f[i + 1];
    }
    FN(opoint_inc_)(&prev);
    FN(opoint_inc_)(&next);
    for (uint64_t step = 1; step + 1 < path->len; ++step, FN(opoint_inc_)(&prev), FN(opoint_inc_)(&next)) {
        for (uint64_t i = 0; i < degree; ++i)
            incr[i] = FN(opoint_get_)(&next, word[i]) - FN(opoint_get_)(&prev, word[i]);
        for (uint64_t i = degree; i > 0; --i) {
            REAL acc = f[i];
            for (uint64_t j = 0; j + 1 < i; ++j) acc = acc * incr[j] + coefs[j + 1] * f[i - j - 1];
            coefs[i] += acc * incr[i - 1];
        }
    }
    if (!prefixes) *out = coefs[degree];
    else for (uint64_t i = 0; i < degree; ++i) out[i] = coefs[i + 1];
}

int FN(oracle_sig_coef_)(const REAL* path, REAL* out, const uint64_t* multi_idx, uint64_t num, const uint64_t* degrees,
                         uint64_t batch, uint64_t d, uint64_t L, int time_aug, int lead_lag, REAL end_time,
                         int prefixes) {
    if (d == 0) return 2;
    uint64_t max_degree = 0, result_len = 0, total = 0;
    for (uint64_t i = 0; i < num; ++i) {
        if (degrees[i] > max_degree) max_degree = degrees[i];
        result_len += (prefixes && degrees[i]) ? degrees[i] : 1;
        total += degrees[i];
    }
    const uint64_t aug = (lead_lag ? 2 * d : d) + (time_aug ? 1 : 0);
    for (uint64_t k = 0; k < total; ++k) if (multi_idx[k] >= aug) return 2;
    REAL* ws = (REAL*)malloc((3 * max_degree + 2) * sizeof(REAL));
    if (!ws) return 1;
    REAL *incr = ws, *f = ws + max_degree, *coefs = f + max_degree + 1;
    f[0] = (REAL)1.;
    for (uint64_t i = 1; i <= max_degree; ++i) f[i] = f[i - 1] / (REAL)i;
    for (uint64_t b = 0; b < batch; ++b) {
        REAL* o = out + b * result_len;
        FN(opath_) p;
        FN(opath_init_)(&p, path + b * d * L, d, L, time_aug, lead_lag, end_time);
        const uint64_t* w = multi_idx;
        for (uint64_t i = 0; i < num; ++i) {
            const uint64_t k = degrees[i];
            if (!k) { *o++ = (REAL)1.; continue; }
            if (L <= 1) { for (uint64_t q = 0; q < (prefixes ? k : 1); ++q) *o++ = (REAL)0.; w += k; continue; }
            FN(single_sig_coef_)(&p, o, w, k, coefs, incr, f, prefixes);
            o += prefixes ? k : 1;
            w += k;
        }
    }
    free(ws);
    return 0;
}

static void FN(single_sig_coef_backprop_)(const FN(opath_)* path, REAL* out, const uint64_t* word, uint64_t degree,
                                          REAL* coefs, REAL* incr, REAL* states, REAL* incr_derivs, REAL* derivs,
                                          const REAL* f, const REAL* sf) {
    const int lead_lag = path->lead_lag;
    const uint64_t pre_time = path->dim - (path->time_aug ? 1 : 0);
    const uint64_t dd = path->data_dim;
    REAL* pos = out + dd * (path->data_len - 1);
    REAL* neg = pos - dd;
    int parity = 0;
    for (uint64_t step = path->len - 1; step-- > 0;) {
        FN(opoint_) prev = FN(opoint_at_)(path, step);
        FN(opoint_) next = FN(opoint_at_)(path, step + 1);
        for (uint64_t i = 0; i < degree; ++i)
            incr[i] = FN(opoint_get_)(&next, word[i]) - FN(opoint_get_)(&prev, word[i]);
        if (step == 0) {
            for (uint64_t i = 1; i <= degree; ++i) coefs[i] = (REAL)0;
        } else {
            for (uint64_t i = degree; i > 0; --i) {
                REAL acc = sf[i];
                for (uint64_t j = 0; j + 1 < i; ++j) acc = acc * incr[j] + coefs[j + 1] * sf[i - j - 1];
                coefs[i] += acc * incr[i - 1];
            }
        }
        for (uint64_t i = 0; i < degree; ++i) incr_derivs[i] = (REAL)0.;
        for (uint64_t i = 1; i < degree + 1; ++i) {
            states[0] = f[i];
            for (uint64_t j = 0; j + 1 < i; ++j) states[j + 1] = states[j] * incr[j] + coefs[j + 1] * f[i - j - 1];
            const REAL output_deriv = derivs[i - 1];
            incr_derivs[i - 1] += output_deriv * states[i - 1];
            REAL state_deriv = output_deriv * incr[i - 1];
            for (uint64_t j = i - 1; j-- > 0;) {
                incr_derivs[j] += state_deriv * states[j];
                derivs[j] += state_deriv * f[i - j - 1];
                state_deriv *= incr[j];
            }
        }
        for (uint64_t i = 0; i < degree; ++i) {
            uint64_t idx = word[i];
            if (idx >= pre_time || (lead_lag && ((parity != 0) == (idx < dd)))) continue;
            if (lead_lag && parity) idx -= dd;
            pos[idx] += incr_derivs[i];
            neg[idx] -= incr_derivs[i];
        }
        if (step > 0) {
            if (!lead_lag || parity) { pos -= dd; neg -= dd; }
            parity = !parity;
        }
    }
}

int FN(oracle_sig_coef_backprop_)(const REAL* path, REAL* out, const REAL* coefs, const REAL* derivs,
                                  const uint64_t* multi_idx, uint64_t num, const uint64_t* degrees, uint64_t batch,
                                  uint64_t d, uint64_t L, int time_aug, int lead_lag, REAL end_time) {
    if (d == 0) return 2;
    uint64_t max_degree = 0, coefs_len = 0, total = 0;
    for (uint64_t i = 0; i < num; ++i) {
        if (degrees[i] > max_degree) max_degree = degrees[i];
        coefs_len += degrees[i] ? degrees[i] : 1;
        total += degrees[i];
    }
    const uint64_t aug = (lead_lag ? 2 * d : d) + (time_aug ? 1 : 0);
    for (uint64_t k = 0; k < total; ++k) if (multi_idx[k] >= aug) return 2;
    for (uint64_t i = 0; i < batch * d * L; ++i) out[i] = (REAL)0.;
    if (L <= 1) return 0;
    REAL* ws = (REAL*)malloc((7 * max_degree + 3) * sizeof(REAL));
    if (!ws) return 1;
    REAL *f = ws, *sf = f + max_degree + 1, *cc = sf + max_degree + 1, *incr = cc + max_degree + 1,
         *states = incr + max_degree, *incr_derivs = states + max_degree, *dc = incr_derivs + max_degree;
    f[0] = sf[0] = (REAL)1.;
    REAL sgn = (REAL)-1.;
    for (uint64_t i = 1; i <= max_degree; ++i, sgn = -sgn) { f[i] = f[i - 1] / (REAL)i; sf[i] = sgn * f[i]; }
    for (uint64_t b = 0; b < batch; ++b) {
        FN(opath_) p;
        FN(opath_init_)(&p, path + b * d * L, d, L, time_aug, lead_lag, end_time);
        const REAL* c = coefs + b * coefs_len;
        const REAL* g = derivs + b * coefs_len;
        const uint64_t* w = multi_idx;
        for (uint64_t i = 0; i < num; ++i) {
            const uint64_t k = degrees[i];
            if (!k) { ++c; ++g; continue; }
            cc[0] = (REAL)1.;
            memcpy(cc + 1, c, k * sizeof(REAL));
            memcpy(dc, g, k * sizeof(REAL));
            FN(single_sig_coef_backprop_)(&p, out + b * d * L, w, k, cc, incr, states, incr_derivs, dc, f, sf);
            c += k; g += k; w += k;
        }
    }
    free(ws);
    return 0;
}

#undef FN
#undef CAT
#undef CAT_
