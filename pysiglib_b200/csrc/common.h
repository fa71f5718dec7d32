// Shared host-side declarations of the sm_100a signature library: error codes,
// exception -> code translation, checked size arithmetic, signature layout.
//
// Error convention of the C ABI (the reference's, siglib/cusig/cu_macros.h:27-89):
// 0 ok, 1 bad_alloc, 2 invalid_argument, 3 out_of_range, 10 runtime_error,
// 11 unknown, 100000 + cudaError_t for CUDA failures.  The detail text is kept
// per thread and returned by cusig_last_error_message().
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <new>
#include <stdexcept>
#include <string>

namespace sigb200 {

struct CudaFailure : std::runtime_error {
    cudaError_t code;
    CudaFailure(cudaError_t c, const std::string& what) : std::runtime_error(what), code(c) {}
};

void set_last_error(const char* text) noexcept;
void clear_last_error() noexcept;
const char* last_error() noexcept;

#define SIG_CUDA_CHECK(expr)                                                                   \
    do {                                                                                       \
        cudaError_t err__ = (expr);                                                            \
        if (err__ != cudaSuccess) {                                                            \
            (void)cudaGetLastError();                                                          \
            throw ::sigb200::CudaFailure(err__, std::string("CUDA Error (") +                  \
                std::to_string(static_cast<int>(err__)) + "): " + cudaGetErrorString(err__) +  \
                " at " #expr);                                                                 \
        }                                                                                      \
    } while (0)

// Runs `body` (a statement list) and converts any exception into the ABI's int code.
#define SIG_SAFE_CALL(body)                                                    \
    ::sigb200::clear_last_error();                                             \
    try {                                                                      \
        body;                                                                  \
        return 0;                                                              \
    } catch (const ::sigb200::CudaFailure& e) {                                \
        ::sigb200::set_last_error(e.what());                                   \
        return 100000 + static_cast<int>(e.code);                              \
    } catch (const std::bad_alloc& e) {                                        \
        ::sigb200::set_last_error(e.what());                                   \
        return 1;                                                              \
    } catch (const std::invalid_argument& e) {                                 \
        ::sigb200::set_last_error(e.what());                                   \
        return 2;                                                              \
    } catch (const std::out_of_range& e) {                                     \
        ::sigb200::set_last_error(e.what());                                   \
        return 3;                                                              \
    } catch (const std::runtime_error& e) {                                    \
        ::sigb200::set_last_error(e.what());                                   \
        return 10;                                                             \
    } catch (...) {                                                            \
        ::sigb200::set_last_error("unknown exception");                        \
        return 11;                                                             \
    }

inline uint64_t checked_mul(uint64_t a, uint64_t b, const char* what) {
    if (a != 0 && b > UINT64_MAX / a) throw std::out_of_range(std::string(what) + ": size overflow");
    return a * b;
}

inline uint64_t checked_add(uint64_t a, uint64_t b, const char* what) {
    if (a > UINT64_MAX - b) throw std::out_of_range(std::string(what) + ": size overflow");
    return a + b;
}

// d^k with overflow detection (0 = overflow).
inline uint64_t ipow(uint64_t d, uint64_t k) {
    uint64_t r = 1;
    for (uint64_t i = 0; i < k; ++i) {
        if (d != 0 && r > UINT64_MAX / d) return 0;
        r *= d;
    }
    return r;
}

// Number of coefficients of a degree-N signature in dimension d, scalar term
// included (reference: siglib/cpsig/cp_utils.cpp:91-105).  Throws on overflow.
inline uint64_t sig_length_full(uint64_t d, uint64_t degree) {
    if (d == 0) return 1;
    if (d == 1) return degree + 1;
    uint64_t total = 1, level = 1;
    for (uint64_t k = 1; k <= degree; ++k) {
        level = checked_mul(level, d, "signature length");
        total = checked_add(total, level, "signature length");
    }
    return total;
}

// Shape of one call after the flags are applied.
struct SigShape {
    uint64_t batch, data_dim, data_len, degree;
    bool time_aug, lead_lag, scalar_term;
    uint64_t dim;       // augmented dimension d'
    uint64_t len;       // augmented length L'
    uint64_t full_len;  // coefficients including the scalar term
    uint64_t stride;    // coefficients per path in the caller's buffers
};

inline SigShape make_shape(uint64_t batch, uint64_t d, uint64_t L, uint64_t degree, bool time_aug,
                           bool lead_lag, bool scalar_term) {
    SigShape s{};
    s.batch = batch; s.data_dim = d; s.data_len = L; s.degree = degree;
    s.time_aug = time_aug; s.lead_lag = lead_lag; s.scalar_term = scalar_term;
    s.dim = checked_add(lead_lag ? checked_mul(2, d, "dimension") : d, time_aug ? 1 : 0, "dimension");
    s.len = lead_lag ? (L == 0 ? 0 : 2 * L - 1) : L;
    s.full_len = sig_length_full(s.dim, degree);
    s.stride = scalar_term ? s.full_len : s.full_len - 1;
    return s;
}

}  // namespace sigb200
