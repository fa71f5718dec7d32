/*
 * CPU oracle for the truncated path signature and its backward pass.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is compared
 * against; nothing in the shipped package may call it.
 *
 * It is a plain-C restatement of the arithmetic of pySigLib's CPU library
 * (cpsig), written against the reference's source so that the order of
 * floating point operations, and where they are fused, follows it:
 *
 *   forward   siglib/cpsig/cp_signature.h:365-389  (first segment)
 *             siglib/cpsig/cp_signature.h:426-500  (Horner update per increment)
 *             siglib/cpsig/cp_signature.h:719-889  (trivial cases / dispatch)
 *             siglib/cpsig/cp_signature.h:391-424 + cp_sig_combine.h:34-66
 *                                                  (horner=false: Chen product)
 *   backward  siglib/cpsig/cp_signature.h:549-603  (in-place Horner step)
 *             siglib/cpsig/cp_signature.h:909-1019 (scalar re-padding, dispatch)
 *             siglib/cpsig/cp_signature.h:1098-1203 (reverse sweep)
 *   flags     siglib/cpsig/cp_path.h:46-385        (time-aug / lead-lag points)
 *   layout    siglib/cpsig/cp_utils.cpp:37-47,91-105 (level index, sig_length)
 *   fusing    siglib/cpsig/cp_simd-inl.h:44-137    (vec_mult_add = FMA,
 *                                                   vec_mult_assign = MUL)
 *
 * Parity pin: tests/test_oracle_golden.py checks this oracle against the
 * reference's own golden vectors (tests/fixtures/reference_data.npz, extracted
 * to tests/golden/) and the hand-computed vectors of
 * siglib/cpsig_unit_testing/cp_test_signature.cpp:140-405.
 *
 * The file is included twice by sig_oracle.c with REAL = float / double and
 * SUF = f / d.  Compile with -ffp-contract=off so that only the explicit
 * FMA() calls fuse, as in the reference.
 */

#define CAT_(a, b) a##b
#define CAT(a, b) CAT_(a, b)
#define FN(name) CAT(name, SUF)

/* ----- the augmented path: cp_path.h ------------------------------------ */

typedef struct {
    const REAL* data;
    uint64_t data_dim, data_len;
    uint64_t dim, len;
    int time_aug, lead_lag;
    REAL time_step;
} FN(opath_);

/* A point iterator.  `time` is carried by repeated addition exactly as the
 * reference's PointImplTimeAug does (cp_path.h:222-223, 335-344). */
typedef struct {
    const FN(opath_)* p;
    const REAL* ptr;
    int parity;
    REAL time;
} FN(opoint_);

static void FN(opath_init_)(FN(opath_)* p, const REAL* data, uint64_t d, uint64_t L,
                            int time_aug, int lead_lag, REAL end_time) {
    p->data = data;
    p->data_dim = d;
    p->data_len = L;
    p->dim = (lead_lag ? 2 * d : d) + (time_aug ? 1 : 0);
    p->len = lead_lag ? 2 * L - 1 : L;
    p->time_aug = time_aug;
    p->lead_lag = lead_lag;
    p->time_step = p->len > 1 ? end_time / (REAL)(p->len - 1) : (REAL)0;
}

static FN(opoint_) FN(opoint_at_)(const FN(opath_)* p, uint64_t index) {
    FN(opoint_) q;
    q.p = p;
    if (p->lead_lag) {
        q.ptr = p->data + (index / 2) * p->data_dim;
        q.parity = (int)(index % 2);
    } else {
        q.ptr = p->data + index * p->data_dim;
        q.parity = 0;
    }
    q.time = (REAL)index * p->time_step;
    return q;
}

static REAL FN(opoint_get_)(const FN(opoint_)* q, uint64_t i) {
    const FN(opath_)* p = q->p;
    if (i < p->data_dim) return q->ptr[i];
    if (p->lead_lag && i < 2 * p->data_dim) {
        /* lead channel: the next data point once the lead has moved */
        uint64_t lead = q->parity ? i : i - p->data_dim;
        return q->ptr[lead];
    }
    return q->time;
}

static void FN(opoint_inc_)(FN(opoint_)* q) {
    const FN(opath_)* p = q->p;
    if (p->lead_lag) {
        if (q->parity) q->ptr += p->data_dim;
        q->parity = !q->parity;
    } else {
        q->ptr += p->data_dim;
    }
    if (p->time_aug) q->time += p->time_step;
}

static void FN(opoint_dec_)(FN(opoint_)* q) {
    const FN(opath_)* p = q->p;
    if (p->lead_lag) {
        if (!q->parity) q->ptr -= p->data_dim;
        q->parity = !q->parity;
    } else {
        q->ptr -= p->data_dim;
    }
    if (p->time_aug) q->time -= p->time_step;
}

/* ----- fused / unfused vector helpers: cp_simd-inl.h -------------------- */

static void FN(vec_mult_add_)(REAL* out, const REAL* other, REAL scalar, uint64_t n) {
    for (uint64_t i = 0; i < n; ++i) out[i] = FMA(other[i], scalar, out[i]);
}

static void FN(vec_mult_assign_)(REAL* out, const REAL* other, REAL scalar, uint64_t n) {
    for (uint64_t i = 0; i < n; ++i) out[i] = other[i] * scalar;
}

/* ----- first segment: cp_signature.h:365-389 ---------------------------- */

static void FN(linear_signature_)(const FN(opoint_)* a, const FN(opoint_)* b, REAL* out,
                                  uint64_t dim, uint64_t degree, const uint64_t* li,
                                  int scalar_term) {
    if (scalar_term) out[0] = (REAL)1;
    if (degree == 0) return;
    const uint64_t off = scalar_term ? 0 : 1;
    for (uint64_t i = 0; i < dim; ++i)
        out[i + 1 - off] = FN(opoint_get_)(b, i) - FN(opoint_get_)(a, i);
    for (uint64_t level = 2; level <= degree; ++level) {
        const REAL one_over_level = (REAL)1. / (REAL)level;
        REAL* result = out + li[level] - off;
        const REAL* left_end = out + li[level] - off;
        for (const REAL* left = out + li[level - 1] - off; left != left_end; ++left, result += dim)
            FN(vec_mult_assign_)(result, out + 1 - off, (*left) * one_over_level, dim);
    }
}

/* ----- Horner forward: cp_signature.h:426-500 --------------------------- */

static int FN(signature_horner_)(const FN(opath_)* path, REAL* out, uint64_t degree, int scalar_term) {
    const uint64_t dim = path->dim;
    uint64_t* li = (uint64_t*)malloc((degree + 2) * sizeof(uint64_t));
    if (!li) return 1;
    populate_level_index(li, dim, degree + 2);

    FN(opoint_) prev = FN(opoint_at_)(path, 0);
    FN(opoint_) next = FN(opoint_at_)(path, 0);
    FN(opoint_inc_)(&next);
    FN(linear_signature_)(&prev, &next, out, dim, degree, li, scalar_term);
    if (path->len == 2) { free(li); return 0; }
    if (!scalar_term)
        for (uint64_t level = 1; level <= degree + 1; ++level) --li[level];

    FN(opoint_inc_)(&prev);
    FN(opoint_inc_)(&next);

    const uint64_t work_size = li[degree] - li[degree - 1];
    REAL* horner_step = (REAL*)malloc((work_size + degree + 1 + dim) * sizeof(REAL));
    if (!horner_step) { free(li); return 1; }
    REAL* reciprocals = horner_step + work_size;
    REAL* inc = reciprocals + degree + 1;
    for (uint64_t level = 1; level <= degree; ++level) reciprocals[level] = (REAL)1 / (REAL)level;

    for (uint64_t step = 1; step + 1 < path->len; ++step, FN(opoint_inc_)(&prev), FN(opoint_inc_)(&next)) {
        for (uint64_t i = 0; i < dim; ++i)
            inc[i] = FN(opoint_get_)(&next, i) - FN(opoint_get_)(&prev, i);

        for (int64_t target = (int64_t)degree; target > 1; --target) {
            for (uint64_t i = 0; i < dim; ++i) horner_step[i] = inc[i] * reciprocals[target];

            for (int64_t left = 1, right = target - 1; left < target - 1; ++left, --right) {
                const uint64_t left_size = li[left + 1] - li[left];
                const REAL one_over = reciprocals[right];
                REAL* lp = horner_step + left_size;
                const REAL* op = out + li[left + 1];
                REAL* rp = horner_step + left_size * dim;
                while (lp != horner_step) {
                    const REAL scalar = (*(--lp) + *(--op)) * one_over;
                    rp -= dim;
                    FN(vec_mult_assign_)(rp, inc, scalar, dim);
                }
            }

            const uint64_t left_size = li[target] - li[target - 1];
            const REAL* lp = horner_step + left_size;
            const REAL* op = out + li[target];
            REAL* rp = out + li[target + 1];
            while (lp != horner_step) {
                const REAL scalar = *(--lp) + *(--op);
                rp -= dim;
                FN(vec_mult_add_)(rp, inc, scalar, dim);
            }
        }
        FN(vec_mult_add_)(out + (scalar_term ? 1 : 0), inc, (REAL)1., dim);
    }
    free(horner_step);
    free(li);
    return 0;
}

/* ----- horner=false: cp_signature.h:391-424 + cp_sig_combine.h:34-66 ---- */

static void FN(sig_combine_inplace_)(REAL* s1, const REAL* s2, uint64_t degree, const uint64_t* li) {
    s1[0] = (REAL)1.;
    for (int64_t target = (int64_t)degree; target > 0; --target) {
        for (int64_t left = target - 1, right = 1; left > 0; --left, ++right) {
            REAL* rp = s1 + li[target];
            const REAL* left_end = s1 + li[left + 1];
            const uint64_t right_size = li[right + 1] - li[right];
            const REAL* right_start = s2 + li[right];
            for (REAL* lp = s1 + li[left]; lp != left_end; ++lp) {
                FN(vec_mult_add_)(rp, right_start, *lp, right_size);
                rp += right_size;
            }
        }
        const uint64_t level_size = li[target + 1] - li[target];
        FN(vec_mult_add_)(s1 + li[target], s2 + li[target], (REAL)1., level_size);
    }
}

static int FN(signature_naive_)(const FN(opath_)* path, REAL* out, uint64_t degree) {
    const uint64_t dim = path->dim;
    uint64_t* li = (uint64_t*)malloc((degree + 2) * sizeof(uint64_t));
    if (!li) return 1;
    populate_level_index(li, dim, degree + 2);
    FN(opoint_) prev = FN(opoint_at_)(path, 0);
    FN(opoint_) next = FN(opoint_at_)(path, 0);
    FN(opoint_inc_)(&next);
    FN(linear_signature_)(&prev, &next, out, dim, degree, li, 1);
    if (path->len == 2) { free(li); return 0; }
    REAL* lin = (REAL*)malloc(oracle_sig_length(dim, degree) * sizeof(REAL));
    if (!lin) { free(li); return 1; }
    FN(opoint_inc_)(&prev);
    FN(opoint_inc_)(&next);
    for (uint64_t step = 1; step + 1 < path->len; ++step, FN(opoint_inc_)(&prev), FN(opoint_inc_)(&next)) {
        FN(linear_signature_)(&prev, &next, lin, dim, degree, li, 1);
        FN(sig_combine_inplace_)(out, lin, degree, li);
    }
    free(lin);
    free(li);
    return 0;
}

/* ----- one path, forward: the per-path body of signature_ --------------- */

static int FN(signature_one_)(const REAL* path, REAL* out, uint64_t d, uint64_t L, uint64_t degree,
                              int time_aug, int lead_lag, REAL end_time, int horner, int scalar_term) {
    FN(opath_) p;
    FN(opath_init_)(&p, path, d, L, time_aug, lead_lag, end_time);
    const uint64_t full_len = oracle_sig_length(p.dim, degree);
    const uint64_t stride = scalar_term ? full_len : full_len - 1;

    if (p.len <= 1) {
        for (uint64_t i = 0; i < stride; ++i) out[i] = (REAL)0.;
        if (scalar_term) out[0] = (REAL)1.;
        return 0;
    }
    if (degree == 0) {
        if (scalar_term) out[0] = (REAL)1.;
        return 0;
    }
    if (p.dim == 1) { /* cp_signature.h:770-785 */
        const REAL increment = path[L - 1] - path[0];
        REAL value = (REAL)1;
        if (scalar_term) *(out++) = value;
        for (uint64_t level = 1; level <= degree; ++level) {
            value *= increment / (REAL)level;
            *(out++) = value;
        }
        return 0;
    }
    if (degree == 1) { /* cp_signature.h:842-848 */
        FN(opoint_) first = FN(opoint_at_)(&p, 0);
        FN(opoint_) last = FN(opoint_at_)(&p, p.len);
        FN(opoint_dec_)(&last);
        if (scalar_term) *(out++) = (REAL)1.;
        for (uint64_t i = 0; i < p.dim; ++i)
            out[i] = FN(opoint_get_)(&last, i) - FN(opoint_get_)(&first, i);
        return 0;
    }
    if (horner) return FN(signature_horner_)(&p, out, degree, scalar_term);
    if (scalar_term) return FN(signature_naive_)(&p, out, degree);
    REAL* buf = (REAL*)malloc(full_len * sizeof(REAL));
    if (!buf) return 1;
    int rc = FN(signature_naive_)(&p, buf, degree);
    memcpy(out, buf + 1, (full_len - 1) * sizeof(REAL));
    free(buf);
    return rc;
}

/* ----- in-place Horner step on a full signature: cp_signature.h:549-603 -- */

static void FN(signature_horner_step_)(REAL* sig, const REAL* inc, uint64_t dim, uint64_t degree,
                                       const uint64_t* li, REAL* horner_step) {
    for (int64_t target = (int64_t)degree; target > 1; --target) {
        REAL one_over = (REAL)1. / (REAL)target;
        for (uint64_t i = 0; i < dim; ++i) horner_step[i] = inc[i] * one_over;
        for (int64_t left = 1, right = target - 1; left < target - 1; ++left, --right) {
            const uint64_t left_size = li[left + 1] - li[left];
            one_over = (REAL)(1. / (double)right);
            REAL* sp = sig + li[left + 1];
            REAL* rp = horner_step + li[left + 2] - li[left + 1] - dim;
            for (REAL* lp = horner_step + left_size - 1; lp != horner_step - 1; --lp, rp -= dim) {
                const REAL v = (*lp + *(--sp)) * one_over;
                FN(vec_mult_assign_)(rp, inc, v, dim);
            }
        }
        const uint64_t left_size = li[target] - li[target - 1];
        REAL* sp = sig + li[target];
        REAL* rp = sig + li[target + 1] - dim;
        for (REAL* lp = horner_step + left_size - 1; lp != horner_step - 1; --lp, rp -= dim) {
            const REAL scalar = *lp + *(--sp);
            FN(vec_mult_add_)(rp, inc, scalar, dim);
        }
    }
    FN(vec_mult_add_)(sig + 1, inc, (REAL)1., dim);
}

/* ----- reverse sweep: cp_signature.h:1098-1203 -------------------------- */
/* sig / sig_derivs are scalar-padded private copies and are overwritten. */

static int FN(sig_backprop_inplace_)(const FN(opath_)* path, REAL* out, REAL* sig_derivs, REAL* sig,
                                     uint64_t degree) {
    const uint64_t data_dim = path->data_dim;
    const uint64_t dim = path->dim;
    const uint64_t data_len = path->data_len;
    const int lead_lag = path->lead_lag;

    uint64_t* li = (uint64_t*)malloc((degree + 2) * sizeof(uint64_t));
    if (!li) return 1;
    populate_level_index(li, dim, degree + 2);
    const uint64_t top = li[degree] - li[degree - 1];
    REAL* buf = (REAL*)malloc((li[degree] + top + 3 * dim + degree + 1) * sizeof(REAL));
    if (!buf) { free(li); return 1; }
    REAL* horner_step = buf;
    REAL* horner_derivs = horner_step + li[degree];
    REAL* inc = horner_derivs + top;
    REAL* inc_derivs = inc + dim;
    REAL* inc_partials = inc_derivs + dim;
    REAL* reciprocals = inc_partials + dim;
    for (uint64_t level = 1; level <= degree; ++level) reciprocals[level] = (REAL)1 / (REAL)level;

    FN(opoint_) prev = FN(opoint_at_)(path, path->len);
    FN(opoint_) next = FN(opoint_at_)(path, path->len);
    FN(opoint_dec_)(&prev);
    FN(opoint_dec_)(&prev);
    FN(opoint_dec_)(&next);
    REAL* pos = out + (data_len - 1) * data_dim;
    int parity = 0;

    for (uint64_t remaining = path->len - 1; remaining > 0; --remaining) {
        for (uint64_t i = 0; i < dim; ++i)
            inc[i] = FN(opoint_get_)(&prev, i) - FN(opoint_get_)(&next, i);
        FN(signature_horner_step_)(sig, inc, dim, degree, li, horner_step);
        for (uint64_t i = 0; i < dim; ++i) {
            inc[i] = -inc[i];
            inc_derivs[i] = sig_derivs[1 + i];
        }

        for (uint64_t target = 2; target <= degree; ++target) {
            for (uint64_t i = 0; i < dim; ++i) horner_step[1 + i] = inc[i] * reciprocals[target];
            for (uint64_t level = 1; level + 1 < target; ++level) {
                const uint64_t size = li[level + 1] - li[level];
                const REAL scale = reciprocals[target - level];
                for (uint64_t i = 0; i < size; ++i) {
                    const REAL value = (horner_step[li[level] + i] + sig[li[level] + i]) * scale;
                    FN(vec_mult_assign_)(horner_step + li[level + 1] + i * dim, inc, value, dim);
                }
            }
            const REAL* incoming = sig_derivs + li[target];
            for (uint64_t level = target - 1; level > 0; --level) {
                const uint64_t size = li[level + 1] - li[level];
                const REAL scale = reciprocals[target - level];
                for (uint64_t j = 0; j < dim; ++j) inc_partials[j] = (REAL)0;
                for (uint64_t i = 0; i < size; ++i) {
                    const REAL value = (horner_step[li[level] + i] + sig[li[level] + i]) * scale;
                    const REAL* row = incoming + i * dim;
                    REAL reduced = (REAL)0;
                    /* dimension-generic branch (dim == 0 template): FMA accumulate + dot product */
                    FN(vec_mult_add_)(inc_partials, row, value, dim);
                    for (uint64_t j = 0; j < dim; ++j) reduced = FMA(row[j], inc[j], reduced);
                    reduced *= scale;
                    horner_derivs[i] = reduced;
                    sig_derivs[li[level] + i] += reduced;
                }
                FN(vec_mult_add_)(inc_derivs, inc_partials, (REAL)1, dim);
                incoming = horner_derivs;
            }
            for (uint64_t i = 0; i < dim; ++i) inc_derivs[i] += horner_derivs[i] * reciprocals[target];
        }

        REAL* neg = pos - data_dim;
        const REAL* s = inc_derivs + (lead_lag && parity ? data_dim : 0);
        for (uint64_t dd = 0; dd < data_dim; ++dd) {
            pos[dd] += s[dd];
            neg[dd] -= s[dd];
        }
        FN(opoint_dec_)(&next);
        if (remaining > 1) {
            FN(opoint_dec_)(&prev);
            if (!lead_lag || parity) pos -= data_dim;
            parity = !parity;
        }
    }
    free(buf);
    free(li);
    return 0;
}

static int FN(sig_backprop_one_)(const REAL* path, REAL* out, const REAL* sig_derivs, const REAL* sig,
                                 uint64_t d, uint64_t L, uint64_t degree, int time_aug, int lead_lag,
                                 REAL end_time, int scalar_term) {
    FN(opath_) p;
    FN(opath_init_)(&p, path, d, L, time_aug, lead_lag, end_time);
    for (uint64_t i = 0; i < d * L; ++i) out[i] = (REAL)0.;
    if (p.len <= 1 || degree == 0) return 0;
    const uint64_t sig_len = oracle_sig_length(p.dim, degree);
    const uint64_t in_stride = scalar_term ? sig_len : sig_len - 1;
    REAL* copies = (REAL*)malloc(2 * sig_len * sizeof(REAL));
    if (!copies) return 1;
    REAL* derivs_copy = copies;
    REAL* sig_copy = copies + sig_len;
    if (scalar_term) {
        memcpy(derivs_copy, sig_derivs, sig_len * sizeof(REAL));
        memcpy(sig_copy, sig, sig_len * sizeof(REAL));
    } else { /* cp_signature.h:965-974 */
        derivs_copy[0] = (REAL)0;
        memcpy(derivs_copy + 1, sig_derivs, in_stride * sizeof(REAL));
        sig_copy[0] = (REAL)1;
        memcpy(sig_copy + 1, sig, in_stride * sizeof(REAL));
    }
    int rc = FN(sig_backprop_inplace_)(&p, out, derivs_copy, sig_copy, degree);
    free(copies);
    return rc;
}

/* ----- batch drivers (static contiguous chunks: multithreading.cpp:66-78) - */

typedef struct {
    const REAL* path; REAL* out; const REAL* sig_derivs; const REAL* sig;
    uint64_t d, L, degree; int time_aug, lead_lag; REAL end_time; int horner, scalar_term;
    uint64_t begin, end; uint64_t path_stride, sig_stride; int backward; int rc;
} FN(job_);

static void* FN(worker_)(void* arg) {
    FN(job_)* j = (FN(job_)*)arg;
    j->rc = 0;
    for (uint64_t b = j->begin; b < j->end && !j->rc; ++b) {
        if (j->backward)
            j->rc = FN(sig_backprop_one_)(j->path + b * j->path_stride, j->out + b * j->path_stride,
                                          j->sig_derivs + b * j->sig_stride, j->sig + b * j->sig_stride,
                                          j->d, j->L, j->degree, j->time_aug, j->lead_lag, j->end_time,
                                          j->scalar_term);
        else
            j->rc = FN(signature_one_)(j->path + b * j->path_stride, j->out + b * j->sig_stride,
                                       j->d, j->L, j->degree, j->time_aug, j->lead_lag, j->end_time,
                                       j->horner, j->scalar_term);
    }
    return NULL;
}

static int FN(run_batch_)(FN(job_)* proto, uint64_t batch, int n_threads) {
    if (batch == 0) return 0;
    uint64_t nt = n_threads < 1 ? 1 : (uint64_t)n_threads;
    if (nt > batch) nt = batch;
    if (nt == 1) {
        proto->begin = 0; proto->end = batch;
        FN(worker_)(proto);
        return proto->rc;
    }
    FN(job_)* jobs = (FN(job_)*)malloc(nt * sizeof(FN(job_)));
    pthread_t* th = (pthread_t*)malloc(nt * sizeof(pthread_t));
    if (!jobs || !th) { free(jobs); free(th); return 1; }
    const uint64_t chunk = batch / nt, rem = batch % nt;
    for (uint64_t t = 0; t < nt; ++t) {
        jobs[t] = *proto;
        jobs[t].begin = t * chunk + (t < rem ? t : rem);
        jobs[t].end = jobs[t].begin + chunk + (t < rem ? 1 : 0);
        pthread_create(&th[t], NULL, FN(worker_), &jobs[t]);
    }
    int rc = 0;
    for (uint64_t t = 0; t < nt; ++t) {
        pthread_join(th[t], NULL);
        if (jobs[t].rc) rc = jobs[t].rc;
    }
    free(jobs);
    free(th);
    return rc;
}

/* returns 0 ok, 1 allocation failure, 2 invalid argument (same codes as the reference's C ABI) */
int FN(oracle_signature_)(const REAL* path, REAL* out, uint64_t batch, uint64_t d, uint64_t L,
                          uint64_t degree, int time_aug, int lead_lag, REAL end_time, int horner,
                          int scalar_term, int n_threads) {
    if (d == 0) return 2;
    const uint64_t dim = (lead_lag ? 2 * d : d) + (time_aug ? 1 : 0);
    const uint64_t full = oracle_sig_length(dim, degree);
    FN(job_) j;
    memset(&j, 0, sizeof j);
    j.path = path; j.out = out; j.d = d; j.L = L; j.degree = degree;
    j.time_aug = time_aug; j.lead_lag = lead_lag; j.end_time = end_time;
    j.horner = horner; j.scalar_term = scalar_term;
    j.path_stride = d * L; j.sig_stride = scalar_term ? full : full - 1; j.backward = 0;
    return FN(run_batch_)(&j, batch, n_threads);
}

int FN(oracle_sig_backprop_)(const REAL* path, REAL* out, const REAL* sig_derivs, const REAL* sig,
                             uint64_t batch, uint64_t d, uint64_t L, uint64_t degree, int time_aug,
                             int lead_lag, REAL end_time, int scalar_term, int n_threads) {
    if (d == 0) return 2;
    const uint64_t dim = (lead_lag ? 2 * d : d) + (time_aug ? 1 : 0);
    const uint64_t full = oracle_sig_length(dim, degree);
    FN(job_) j;
    memset(&j, 0, sizeof j);
    j.path = path; j.out = out; j.sig_derivs = sig_derivs; j.sig = sig;
    j.d = d; j.L = L; j.degree = degree;
    j.time_aug = time_aug; j.lead_lag = lead_lag; j.end_time = end_time;
    j.scalar_term = scalar_term;
    j.path_stride = d * L; j.sig_stride = scalar_term ? full : full - 1; j.backward = 1;
    return FN(run_batch_)(&j, batch, n_threads);
}

/* out = sig1 (x) sig2 per batch entry (cp_sig_combine.h:34-66 on scalar-padded copies) */
int FN(oracle_sig_combine_)(const REAL* sig1, const REAL* sig2, REAL* out, uint64_t batch, uint64_t dim,
                            uint64_t degree, int scalar_term) {
    if (dim == 0) return 2;
    const uint64_t full = oracle_sig_length(dim, degree);
    const uint64_t stride = scalar_term ? full : full - 1;
    uint64_t* li = (uint64_t*)malloc((degree + 2) * sizeof(uint64_t));
    REAL* a = (REAL*)malloc(2 * full * sizeof(REAL));
    if (!li || !a) { free(li); free(a); return 1; }
    REAL* b = a + full;
    populate_level_index(li, dim, degree + 2);
    for (uint64_t i = 0; i < batch; ++i) {
        a[0] = b[0] = (REAL)1;
        memcpy(a + 1, sig1 + i * stride + (scalar_term ? 1 : 0), (full - 1) * sizeof(REAL));
        memcpy(b + 1, sig2 + i * stride + (scalar_term ? 1 : 0), (full - 1) * sizeof(REAL));
        FN(sig_combine_inplace_)(a, b, degree, li);
        memcpy(out + i * stride, a + (scalar_term ? 0 : 1), stride * sizeof(REAL));
    }
    free(li);
    free(a);
    return 0;
}

/* Adjoints of both factors of a (x) b: d1[u] = sum_v deriv[uv] b[v], d2[v] = sum_u deriv[uv] a[u]
 * (what siglib/cpsig/cp_sig_combine.h sig_combine_backprop_ computes; scalar slots get 0).
 * Written from the definition, level pair by level pair. */
int FN(oracle_sig_combine_backprop_)(const REAL* deriv, REAL* d1, REAL* d2, const REAL* sig1, const REAL* sig2,
                                     uint64_t batch, uint64_t dim, uint64_t degree, int scalar_term) {
    if (dim == 0) return 2;
    const uint64_t full = oracle_sig_length(dim, degree);
    const uint64_t stride = scalar_term ? full : full - 1;
    uint64_t* li = (uint64_t*)malloc((degree + 2) * sizeof(uint64_t));
    REAL* buf = (REAL*)malloc(5 * full * sizeof(REAL));
    if (!li || !buf) { free(li); free(buf); return 1; }
    populate_level_index(li, dim, degree + 2);
    REAL *ds = buf, *a = buf + full, *b = buf + 2 * full, *o1 = buf + 3 * full, *o2 = buf + 4 * full;
    const uint64_t off = scalar_term ? 1 : 0;
    for (uint64_t i = 0; i < batch; ++i) {
        ds[0] = (REAL)0; a[0] = b[0] = (REAL)1;
        memcpy(ds + 1, deriv + i * stride + off, (full - 1) * sizeof(REAL));
        memcpy(a + 1, sig1 + i * stride + off, (full - 1) * sizeof(REAL));
        memcpy(b + 1, sig2 + i * stride + off, (full - 1) * sizeof(REAL));
        for (uint64_t k = 0; k < full; ++k) o1[k] = o2[k] = (REAL)0;
        for (uint64_t n = 0; n <= degree; ++n) {            /* level of the left word u */
            const uint64_t cn = li[n + 1] - li[n];
            for (uint64_t m = 0; n + m <= degree; ++m) {    /* level of the right word v */
                if (n + m == 0) continue;
                const uint64_t cm = li[m + 1] - li[m];
                for (uint64_t u = 0; u < cn; ++u)
                    for (uint64_t v = 0; v < cm; ++v) {
                        const REAL g = ds[li[n + m] + u * cm + v];
                        o1[li[n] + u] = FMA(g, b[li[m] + v], o1[li[n] + u]);
                        o2[li[m] + v] = FMA(g, a[li[n] + u], o2[li[m] + v]);
                    }
            }
        }
        o1[0] = o2[0] = (REAL)0;
        memcpy(d1 + i * stride, o1 + (scalar_term ? 0 : 1), stride * sizeof(REAL));
        memcpy(d2 + i * stride, o2 + (scalar_term ? 0 : 1), stride * sizeof(REAL));
    }
    free(li);
    free(buf);
    return 0;
}

#undef FN
#undef CAT
#undef CAT_
