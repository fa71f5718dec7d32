/*
 * Timing build of the CPU oracle: TEST / BENCHMARK INFRASTRUCTURE ONLY.
 *
 * The checker (libsig_oracle.so) is compiled -O2 -ffp-contract=off so that its rounding
 * follows the reference operation by operation.  A CPU baseline timed beside the GPU should
 * instead be compiled the way a release build of the reference's CPU library is, so this
 * file rebuilds the same sources with -O3 -march=native (see the Makefile) into
 * libsig_oracle_timing.so, and adds the one forward variant the reference's dispatcher
 * would pick that the checker does not need:
 *
 *   oracle_signature_batch_simd_{f,d}   SIMD across paths, restating
 *       siglib/cpsig/cp_signature.h:605-717 (signature_horner_batch_): one vector holds the
 *       same coefficient of LANES paths (4 doubles / 8 floats: one AVX2 register, the width
 *       the reference's vec_batch_lanes gives on x86-64), increments pre-scaled by 1/level
 *       once per step (:670-673), work levels built with plain multiplies, the target level
 *       with multiply-add.  The reference's dispatcher takes this variant for augmented
 *       dimension <= 4, at most 8192 coefficients, length >= 16 and batch >= LANES
 *       (cp_signature.h:786-804); bench.py uses it for exactly those shapes.
 *
 * Only bench.py's CPU-baseline legs load this library; tests/test_oracle_timing.py holds it
 * to the checker's results.
 */
#include "sig_oracle.c"

#define BATCH_IMPL(REAL, SUF, LANES)                                                                   \
    typedef struct {                                                                                   \
        const REAL* path; REAL* out;                                                                   \
        uint64_t batch, d, L, degree, group_begin, group_end;                                          \
        int scalar_term, rc;                                                                           \
    } batch_job_##SUF;                                                                                 \
                                                                                                       \
    static int batch_group_##SUF(const batch_job_##SUF* j, uint64_t group) {                           \
        const uint64_t d = j->d, L = j->L, degree = j->degree, flat = d * L;                           \
        const uint64_t start = group * LANES;                                                          \
        const uint64_t valid = j->batch - start < LANES ? j->batch - start : LANES;                    \
        uint64_t* li = (uint64_t*)malloc((degree + 2) * sizeof(uint64_t));                             \
        if (!li) return 1;                                                                             \
        populate_level_index(li, d, degree + 2);                                                       \
        const uint64_t sig_len = li[degree + 1];                                                       \
        const uint64_t stride = j->scalar_term ? sig_len : sig_len - 1;                                \
        REAL(*sig)[LANES] = aligned_alloc(64, (sig_len + li[degree] + d * degree) * LANES * sizeof(REAL)); \
        if (!sig) { free(li); return 1; }                                                              \
        REAL(*work)[LANES] = sig + sig_len;                                                            \
        REAL(*inc)[LANES] = work + li[degree];                                                         \
        memset(sig, 0, (sig_len + li[degree] + d * degree) * LANES * sizeof(REAL));                    \
        for (uint64_t l = 0; l < LANES; ++l) sig[0][l] = (REAL)1;                                      \
        const REAL* base = j->path + start * flat;                                                     \
        for (uint64_t time = 1; time < L; ++time) {                                                    \
            for (uint64_t c = 0; c < d; ++c)                                                           \
                for (uint64_t l = 0; l < valid; ++l) {                                                 \
                    const REAL* point = base + l * flat + time * d;                                    \
                    inc[c][l] = point[c] - (point - d)[c];                                             \
                }                                                                                      \
            for (uint64_t level = 2; level <= degree; ++level) {                                       \
                const REAL r = (REAL)1 / (REAL)level;                                                  \
                for (uint64_t c = 0; c < d; ++c)                                                       \
                    for (uint64_t l = 0; l < LANES; ++l) inc[(level - 1) * d + c][l] = inc[c][l] * r;  \
            }                                                                                          \
            for (uint64_t target = degree; target > 1; --target) {                                     \
                for (uint64_t c = 0; c < d; ++c)                                                       \
                    for (uint64_t l = 0; l < LANES; ++l) work[1 + c][l] = inc[(target - 1) * d + c][l]; \
                for (uint64_t level = 1; level + 1 < target; ++level) {                                \
                    const uint64_t ls = li[level], ns = li[level + 1], count = ns - ls;                \
                    const uint64_t off = (target - level - 1) * d;                                     \
                    for (uint64_t w = 0; w < count; ++w) {                                             \
                        REAL sum[LANES];                                                               \
                        for (uint64_t l = 0; l < LANES; ++l) sum[l] = work[ls + w][l] + sig[ls + w][l]; \
                        for (uint64_t c = 0; c < d; ++c)                                               \
                            for (uint64_t l = 0; l < LANES; ++l)                                       \
                                work[ns + w * d + c][l] = sum[l] * inc[off + c][l];                    \
                    }                                                                                  \
                }                                                                                      \
                const uint64_t ts = li[target], ps = li[target - 1], count = ts - ps;                  \
                for (uint64_t w = 0; w < count; ++w) {                                                 \
                    REAL sum[LANES];                                                                   \
                    for (uint64_t l = 0; l < LANES; ++l) sum[l] = work[ps + w][l] + sig[ps + w][l];    \
                    for (uint64_t c = 0; c < d; ++c)                                                   \
                        for (uint64_t l = 0; l < LANES; ++l)                                           \
                            sig[ts + w * d + c][l] += sum[l] * inc[c][l];                              \
                }                                                                                      \
            }                                                                                          \
            for (uint64_t c = 0; c < d; ++c)                                                           \
                for (uint64_t l = 0; l < LANES; ++l) sig[1 + c][l] += inc[c][l];                       \
        }                                                                                              \
        for (uint64_t l = 0; l < valid; ++l) {                                                         \
            REAL* result = j->out + (start + l) * stride;                                              \
            for (uint64_t w = 0; w < stride; ++w) result[w] = sig[w + (j->scalar_term ? 0 : 1)][l];    \
        }                                                                                              \
        free(sig);                                                                                     \
        free(li);                                                                                      \
        return 0;                                                                                      \
    }                                                                                                  \
                                                                                                       \
    static void* batch_worker_##SUF(void* arg) {                                                       \
        batch_job_##SUF* j = (batch_job_##SUF*)arg;                                                    \
        for (uint64_t g = j->group_begin; g < j->group_end && !j->rc; ++g) j->rc = batch_group_##SUF(j, g); \
        return NULL;                                                                                   \
    }                                                                                                  \
                                                                                                       \
    /* static contiguous chunks of lane groups over the threads (multithreading.cpp:66-78) */          \
    int oracle_signature_batch_simd_##SUF(const REAL* path, REAL* out, uint64_t batch, uint64_t d, uint64_t L, \
                                          uint64_t degree, int scalar_term, int n_threads) {           \
        if (d == 0 || d > 4 || degree < 2 || L < 2) return 2;                                          \
        const uint64_t groups = (batch + LANES - 1) / LANES;                                           \
        uint64_t nt = n_threads < 1 ? 1 : (uint64_t)n_threads;                                         \
        if (nt > groups) nt = groups ? groups : 1;                                                     \
        batch_job_##SUF* jobs = (batch_job_##SUF*)calloc(nt, sizeof(batch_job_##SUF));                 \
        pthread_t* th = (pthread_t*)malloc(nt * sizeof(pthread_t));                                    \
        if (!jobs || !th) { free(jobs); free(th); return 1; }                                          \
        const uint64_t chunk = groups / nt, rem = groups % nt;                                         \
        uint64_t begin = 0;                                                                            \
        for (uint64_t t = 0; t < nt; ++t) {                                                            \
            batch_job_##SUF proto = {path, out, batch, d, L, degree, begin, begin + chunk + (t < rem ? 1 : 0), \
                                     scalar_term, 0};                                                  \
            jobs[t] = proto;                                                                           \
            begin = jobs[t].group_end;                                                                 \
            pthread_create(&th[t], NULL, batch_worker_##SUF, &jobs[t]);                                \
        }                                                                                              \
        int rc = 0;                                                                                    \
        for (uint64_t t = 0; t < nt; ++t) {                                                            \
            pthread_join(th[t], NULL);                                                                 \
            if (jobs[t].rc) rc = jobs[t].rc;                                                           \
        }                                                                                              \
        free(jobs);                                                                                    \
        free(th);                                                                                      \
        return rc;                                                                                     \
    }

BATCH_IMPL(float, f, 8)
BATCH_IMPL(double, d, 4)
