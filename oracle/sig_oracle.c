/*
 * CPU oracle for sig / sig_backprop: TEST INFRASTRUCTURE ONLY (see
 * sig_oracle_impl.h for what it restates and how it is pinned).  Only the test
 * suite, the smoke check and the benchmark's cpu-baseline leg may load the
 * library built from this file; the product never does.
 *
 * Build: make -C oracle   (gcc -O2 -ffp-contract=off, see Makefile)
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* siglib/cpsig/cp_utils.cpp:37-47: level_index[i] = level_index[i-1] * d + 1 */
static void populate_level_index(uint64_t* li, uint64_t dim, uint64_t n) {
    li[0] = 0;
    for (uint64_t i = 1; i < n; ++i) li[i] = li[i - 1] * dim + 1;
}

/* siglib/cpsig/cp_utils.cpp:91-105: number of coefficients including the scalar term;
 * 0 signals overflow */
uint64_t oracle_sig_length(uint64_t dim, uint64_t degree) {
    if (dim == 0) return 1;
    if (dim == 1) return degree + 1;
    uint64_t total = 1, level = 1;
    for (uint64_t k = 1; k <= degree; ++k) {
        if (level > UINT64_MAX / dim) return 0;
        level *= dim;
        if (total > UINT64_MAX - level) return 0;
        total += level;
    }
    return total;
}

#define REAL float
#define SUF f
#define FMA(a, b, c) fmaf((a), (b), (c))
#include "sig_oracle_impl.h"
#include "sig_oracle_algebra.h"
#include "sig_oracle_log.h"
#include "sig_oracle_coef.h"
#undef REAL
#undef SUF
#undef FMA

#define REAL double
#define SUF d
#define FMA(a, b, c) fma((a), (b), (c))
#include "sig_oracle_impl.h"
#include "sig_oracle_algebra.h"
#include "sig_oracle_log.h"
#include "sig_oracle_coef.h"
#undef REAL
#undef SUF
#undef FMA
