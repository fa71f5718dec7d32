// Signature -> log signature on sm_100a: the tensor logarithm in Horner form,
//     log(1 + x) = x - x (x) (x/2 - x (x) (x/3 - ... )),
// optionally read out at the Lyndon words, and its backward pass.
//
// With R_{N+1} = 0 and R_k = x/k - x (x) R_{k+1} (k = N..2, kept on levels <= 1+N-k, the only ones
// that can reach level N), the result is y = x - x (x) R_2.  Every phase is one kernel with one
// thread per coefficient (arithmetic in algebra_math.h), signatures along grid.y, so the whole GPU
// works whatever the batch size; there is no synchronisation inside a kernel.  The backward keeps
// R_2..R_N, seeds the adjoint of y and walks the recursion up: N kernels, each producing the
// adjoint of the next R and accumulating into dLoss/d sig.
//
// Same values as siglib/cpsig/cp_tensor_log.h:47-122 (forward) and the derivative of that map
// (the reference evaluates it as cp_tensor_log.h:176-235); replaces sig_to_log_sig_cuda_ and
// sig_to_log_sig_backprop_cuda_ of siglib/cusig/cu_log_signature.cu for methods 0 and 1.
#include <map>
#include <mutex>
#include <tuple>

#include "algebra.h"
#include "algebra_host.h"
#include "algebra_math.h"
#include "kernels.h"
#include "runtime.h"

namespace sigb200 {

namespace {

// R_new = x / k - x (x) R_old on levels <= max_level, zero above.  R_old == nullptr: R_old = 0.
template <typename T>
__global__ void log_horner_kernel(const T* __restrict__ x, uint64_t x_stride, const T* __restrict__ r_old,
                                  T* __restrict__ r_new, Levels lv, uint64_t batch, uint32_t k, uint32_t max_level) {
    const uint32_t S = lv.total();
    const uint32_t j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= S) return;
    const uint32_t t = lv.level_of(j), w = j - lv.off[t];
    const T constant = T(1) / static_cast<T>(k);
    for (uint64_t b = blockIdx.y; b < batch; b += gridDim.y) {
        const T* xb = x + b * x_stride;
        T value = T(0);
        if (t <= max_level) {
            value = constant * xb[j];
            if (r_old) value -= nonunital_product_coeff(xb, r_old + b * S, lv, t, w);
        }
        r_new[b * S + j] = value;
    }
}

// out[i] = y[j(i)] with y = x - x (x) R_2; j(i) = i (expanded) or the position of the i-th Lyndon word.
template <typename T>
__global__ void log_final_kernel(const T* __restrict__ x, uint64_t x_stride, const T* __restrict__ r2,
                                 T* __restrict__ out, uint64_t out_stride, Levels lv, uint64_t batch,
                                 const uint32_t* __restrict__ lyndon, uint32_t count, bool write_zero_scalar) {
    const uint32_t S = lv.total();
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const uint32_t j = lyndon ? lyndon[i] : i;
    const uint32_t t = lv.level_of(j), w = j - lv.off[t];
    for (uint64_t b = blockIdx.y; b < batch; b += gridDim.y) {
        const T* xb = x + b * x_stride;
        T value = xb[j];
        if (r2 && t >= 2) value -= nonunital_product_coeff(xb, r2 + b * S, lv, t, w);
        out[b * out_stride + i] = value;
        if (write_zero_scalar && i == 0) out[b * out_stride - 1] = T(0);
    }
}

// Seeds the backward: D (batch, S) = dLoss/dy in expanded layout (scattered from the Lyndon
// coordinates for method 1), and dsig = D.
template <typename T>
__global__ void log_seed_kernel(const T* __restrict__ derivs, uint64_t derivs_stride, T* __restrict__ D,
                                T* __restrict__ dsig, uint64_t dsig_stride, Levels lv, uint64_t batch,
                                const uint32_t* __restrict__ lyndon, bool zero_scalar) {
    const uint32_t S = lv.total();
    const uint32_t j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= S) return;
    for (uint64_t b = blockIdx.y; b < batch; b += gridDim.y) {
        const T value = lyndon ? T(0) : derivs[b * derivs_stride + j];
        D[b * S + j] = value;
        dsig[b * dsig_stride + j] = value;
        if (zero_scalar && j == 0) dsig[b * dsig_stride - 1] = T(0);
    }
}

template <typename T>
__global__ void log_scatter_kernel(const T* __restrict__ derivs, uint64_t derivs_stride, T* __restrict__ D,
                                   T* __restrict__ dsig, uint64_t dsig_stride, uint32_t S, uint64_t batch,
                                   const uint32_t* __restrict__ lyndon, uint32_t count) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const uint32_t j = lyndon[i];
    for (uint64_t b = blockIdx.y; b < batch; b += gridDim.y) {
        const T value = derivs[b * derivs_stride + i];
        D[b * S + j] = value;
        dsig[b * dsig_stride + j] = value;
    }
}

// One step up the recursion.  Q = adjoint of the product's left operand chain at this step:
//   first step (k = 1): Q = dLoss/dy, the product is x (x) R_2 entering with a minus sign;
//   later steps (k >= 2): Q = dLoss/dR_k, R_k = x/k - x (x) R_{k+1}.
// Writes q_new = dLoss/dR_{k+1} = -(sum_u Q[u v] x[u]) and accumulates
//   dsig += Q/k (k >= 2 only) - sum_v Q[u v] R_{k+1}[v]   (r_next == nullptr: R_{k+1} = 0).
template <typename T>
__global__ void log_adjoint_kernel(const T* __restrict__ x, uint64_t x_stride, const T* __restrict__ q,
                                   const T* __restrict__ r_next, T* __restrict__ q_new, T* __restrict__ dsig,
                                   uint64_t dsig_stride, Levels lv, uint64_t batch, uint32_t k) {
    const uint32_t S = lv.total();
    const uint32_t j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= S) return;
    const uint32_t t = lv.level_of(j), w = j - lv.off[t];
    const T constant = T(1) / static_cast<T>(k);
    for (uint64_t b = blockIdx.y; b < batch; b += gridDim.y) {
        const T* xb = x + b * x_stride;
        const T* qb = q + b * S;
        T add = k >= 2 ? qb[j] * constant : T(0);
        if (r_next) add -= nonunital_left_adjoint_coeff(qb, r_next + b * S, lv, t, w);
        dsig[b * dsig_stride + j] += add;
        if (q_new) q_new[b * S + j] = -nonunital_right_adjoint_coeff(qb, xb, lv, t, w);
    }
}

dim3 coeff_grid(uint32_t count, uint64_t batch) { return batched_grid(count, batch, kThreads); }

// The adjoint sums are long for the few low-level coefficients (d^(N-1) terms for a letter) and
// empty for the top level: give every signature its own CTAs so that the long threads of different
// signatures run side by side instead of one after another.
dim3 adjoint_grid(uint32_t count, uint64_t batch) {
    return dim3(grid_1d(count, kThreads), static_cast<unsigned>(std::min<uint64_t>(batch, 65535)));
}

// ----- Lyndon words ----------------------------------------------------------------------------

// Positions (inside a scalar-free signature) of the Lyndon words of length 1..degree over `dim`
// letters, by length then lexicographically (Duval's algorithm), the order the reference uses
// (siglib/shared/preparation/log_sig/lyndon_words.cpp:25-112).
std::vector<uint32_t> lyndon_positions(uint64_t dim, uint64_t degree) {
    std::vector<uint32_t> out;
    std::vector<uint64_t> w;
    for (uint64_t n = 1; n <= degree; ++n) {
        w.assign(1, 0);
        while (!w.empty()) {
            const size_t m = w.size();
            if (m == n) {
                uint64_t idx = 0;
                for (uint64_t letter : w) idx = idx * dim + letter + 1;
                out.push_back(static_cast<uint32_t>(idx - 1));
            }
            while (w.size() < n) w.push_back(w[w.size() - m]);
            while (!w.empty() && w.back() == dim - 1) w.pop_back();
            if (!w.empty()) ++w.back();
        }
    }
    return out;
}

struct LyndonTable {
    uint32_t* device = nullptr;
    uint32_t count = 0;
};
std::mutex g_tables_mu;
std::map<std::tuple<int, uint64_t, uint64_t>, LyndonTable> g_tables;

LyndonTable lyndon_table(uint64_t dim, uint64_t degree) {
    const int device = current_device();
    std::lock_guard<std::mutex> lock(g_tables_mu);
    const auto key = std::make_tuple(device, dim, degree);
    auto it = g_tables.find(key);
    if (it != g_tables.end()) return it->second;
    const std::vector<uint32_t> host = lyndon_positions(dim, degree);
    LyndonTable table;
    table.count = static_cast<uint32_t>(host.size());
    SIG_CUDA_CHECK(cudaMalloc(&table.device, std::max<size_t>(host.size(), 1) * sizeof(uint32_t)));
    SIG_CUDA_CHECK(cudaMemcpy(table.device, host.data(), host.size() * sizeof(uint32_t), cudaMemcpyHostToDevice));
    g_tables.emplace(key, table);
    return table;
}

void check_method(int method, const char* who) {
    if (method == 0 || method == 1) return;
    if (method == 2 || method == 3)
        throw std::invalid_argument(std::string(who) + ": log-signature method " + std::to_string(method) +
                                    " is not part of this build of libcusig (methods 0 and 1 are)");
    throw std::invalid_argument(std::string(who) + ": method must be one of 0, 1 or 2");
}

constexpr uint64_t kLogScratchBudget = 8ull << 30;

// R_k for k = N..2 into `keep` (N-1 vectors of batch*S, R_k at keep + (k-2) * batch * S) when keep_all,
// else ping-pong in the first two; returns R_2 (nullptr when degree == 1).
template <typename T>
const T* run_horner(const T* x, uint64_t x_stride, T* keep, bool keep_all, const Levels& lv, uint64_t batch,
                    cudaStream_t st) {
    const uint32_t N = lv.degree;
    const uint64_t vec = batch * lv.total();
    const T* r_old = nullptr;
    for (uint32_t k = N; k >= 2; --k) {
        T* r_new = keep + (keep_all ? uint64_t(k - 2) : uint64_t(k & 1)) * vec;
        log_horner_kernel<T><<<coeff_grid(lv.total(), batch), kThreads, 0, st>>>(x, x_stride, r_old, r_new, lv, batch, k,
                                                                               1 + N - k);
        check_launch("tensor log kernel");
        r_old = r_new;
    }
    return r_old;
}

}  // namespace

uint64_t log_sig_length_host(uint64_t dimension, uint64_t degree) {
    return lyndon_positions(dimension, degree).size();
}

void release_log_sig_tables() noexcept {
    std::lock_guard<std::mutex> lock(g_tables_mu);
    for (auto& kv : g_tables) {
        int prev = -1;
        if (cudaGetDevice(&prev) != cudaSuccess) { (void)cudaGetLastError(); continue; }
        if (cudaSetDevice(std::get<0>(kv.first)) == cudaSuccess) (void)cudaFree(kv.second.device);
        (void)cudaSetDevice(prev);
        (void)cudaGetLastError();
    }
    g_tables.clear();
}

void prepare_log_sig_entry(uint64_t dimension, uint64_t degree, int method) {
    if (dimension == 0) throw std::invalid_argument("prepare_log_sig_cuda received dimension 0");
    check_method(method, "prepare_log_sig_cuda");
    if (method == 0) return;
    (void)checked_levels(dimension, degree, "prepare_log_sig_cuda");
    (void)lyndon_table(dimension, degree);
}

template <typename T>
void sig_to_log_sig_entry(const T* sig, T* out, uint64_t batch, uint64_t dimension, uint64_t degree, int method,
                          bool scalar_term, const CallOptions& opt) {
    if (dimension == 0) throw std::invalid_argument("signature received dimension 0");
    if (degree == 0) throw std::invalid_argument("log signature received degree 0");
    check_method(method, "sig_to_log_sig_cuda");
    if (batch == 0) return;
    if (!sig || !out) throw std::invalid_argument("sig_to_log_sig_cuda received a null pointer");
    const Levels lv = checked_levels(dimension, degree, "sig_to_log_sig_cuda");
    const uint64_t S = lv.total();
    const uint64_t in_stride = S + (scalar_term ? 1 : 0);
    const uint64_t shift = scalar_term ? 1 : 0;

    auto run = [&](const T* a, T* o, cudaStream_t st) {
        LyndonTable table;
        if (method == 1) table = lyndon_table(dimension, degree);
        const uint64_t out_stride = method == 1 ? table.count : in_stride;
        const uint64_t per_sig = 2 * S * sizeof(T);
        const uint64_t chunk = std::max<uint64_t>(1, std::min<uint64_t>(batch, kLogScratchBudget / per_sig));
        Scratch ws(degree >= 2 ? chunk * per_sig : 0, st);
        for (uint64_t b0 = 0; b0 < batch; b0 += chunk) {
            const uint64_t count = std::min(chunk, batch - b0);
            const T* x = a + b0 * in_stride + shift;
            const T* r2 = degree >= 2 ? run_horner<T>(x, in_stride, ws.as<T>(), false, lv, count, st) : nullptr;
            if (method == 1) {
                log_final_kernel<T><<<coeff_grid(table.count, count), kThreads, 0, st>>>(
                    x, in_stride, r2, o + b0 * out_stride, out_stride, lv, count, table.device, table.count, false);
            } else {
                log_final_kernel<T><<<coeff_grid(lv.total(), count), kThreads, 0, st>>>(
                    x, in_stride, r2, o + b0 * out_stride + shift, out_stride, lv, count, nullptr, lv.total(),
                    scalar_term);
            }
            check_launch("tensor log kernel");
        }
    };
    int device = -1;
    if (all_on_device({sig, out}, "sig_to_log_sig_cuda", &device)) {
        DeviceGuard guard(device);
        run(sig, out, opt.stream);
        if (opt.synchronize) SIG_CUDA_CHECK(cudaStreamSynchronize(opt.stream));
        return;
    }
    const uint64_t out_len = method == 1 ? log_sig_length_host(dimension, degree) : in_stride;
    run_staged({{sig, nullptr, batch * in_stride * sizeof(T)}, {nullptr, out, batch * out_len * sizeof(T)}}, opt.device,
               [&](const std::vector<void*>& d, cudaStream_t st) {
                   run(static_cast<const T*>(d[0]), static_cast<T*>(d[1]), st);
               });
}

template <typename T>
void sig_to_log_sig_backprop_entry(const T* sig, T* out, const T* log_sig_derivs, uint64_t batch, uint64_t dimension,
                                   uint64_t degree, int method, bool scalar_term, const CallOptions& opt) {
    if (dimension == 0) throw std::invalid_argument("sig_backprop received path of dimension 0");
    if (degree == 0) throw std::invalid_argument("log signature received degree 0");
    check_method(method, "sig_to_log_sig_backprop_cuda");
    if (batch == 0) return;
    if (!sig || !out || !log_sig_derivs) throw std::invalid_argument("sig_to_log_sig_backprop_cuda received a null pointer");
    const Levels lv = checked_levels(dimension, degree, "sig_to_log_sig_backprop_cuda");
    const uint64_t S = lv.total();
    const uint32_t N = lv.degree;
    const uint64_t stride = S + (scalar_term ? 1 : 0);
    const uint64_t shift = scalar_term ? 1 : 0;

    auto run = [&](const T* a, T* o, const T* g, cudaStream_t st) {
        LyndonTable table;
        if (method == 1) table = lyndon_table(dimension, degree);
        const uint64_t g_stride = method == 1 ? table.count : stride;
        const uint64_t vectors = 3 + (N >= 2 ? N - 1 : 0);  // D, two adjoint buffers, R_2..R_N
        const uint64_t per_sig = vectors * S * sizeof(T);
        const uint64_t chunk = std::max<uint64_t>(1, std::min<uint64_t>(batch, kLogScratchBudget / per_sig));
        Scratch ws(chunk * per_sig, st);
        for (uint64_t b0 = 0; b0 < batch; b0 += chunk) {
            const uint64_t count = std::min(chunk, batch - b0);
            const uint64_t vec = count * S;
            T* D = ws.as<T>();
            T* qa = D + vec;
            T* qb = qa + vec;
            T* keep = qb + vec;
            const T* x = a + b0 * stride + shift;
            T* dsig = o + b0 * stride + shift;
            log_seed_kernel<T><<<coeff_grid(lv.total(), count), kThreads, 0, st>>>(
                g + b0 * g_stride + (method == 1 ? 0 : shift), g_stride, D, dsig, stride, lv, count,
                method == 1 ? table.device : nullptr, scalar_term);
            check_launch("tensor log backward kernel");
            if (method == 1) {
                log_scatter_kernel<T><<<coeff_grid(table.count, count), kThreads, 0, st>>>(
                    g + b0 * g_stride, g_stride, D, dsig, stride, lv.total(), count, table.device, table.count);
                check_launch("tensor log backward kernel");
            }
            if (N < 2) continue;
            run_horner<T>(x, stride, keep, true, lv, count, st);
            const T* q = D;
            T* q_new = qa;
            for (uint32_t k = 1; k <= N; ++k) {
                // the product at this step has right operand R_{k+1} (none for k == N)
                const T* r_next = k < N ? keep + uint64_t(k - 1) * vec : nullptr;
                log_adjoint_kernel<T><<<adjoint_grid(lv.total(), count), kThreads, 0, st>>>(
                    x, stride, q, r_next, k < N ? q_new : nullptr, dsig, stride, lv, count, k);
                check_launch("tensor log backward kernel");
                q = q_new;
                q_new = q_new == qa ? qb : qa;
            }
        }
    };
    int device = -1;
    if (all_on_device({sig, out, log_sig_derivs}, "sig_to_log_sig_backprop_cuda", &device)) {
        DeviceGuard guard(device);
        run(sig, out, log_sig_derivs, opt.stream);
        if (opt.synchronize) SIG_CUDA_CHECK(cudaStreamSynchronize(opt.stream));
        return;
    }
    const uint64_t g_len = method == 1 ? log_sig_length_host(dimension, degree) : stride;
    run_staged({{sig, nullptr, batch * stride * sizeof(T)}, {nullptr, out, batch * stride * sizeof(T)},
                {log_sig_derivs, nullptr, batch * g_len * sizeof(T)}},
               opt.device, [&](const std::vector<void*>& d, cudaStream_t st) {
                   run(static_cast<const T*>(d[0]), static_cast<T*>(d[1]), static_cast<const T*>(d[2]), st);
               });
}

#define INSTANTIATE(T)                                                                                           \
    template void sig_to_log_sig_entry<T>(const T*, T*, uint64_t, uint64_t, uint64_t, int, bool, const CallOptions&); \
    template void sig_to_log_sig_backprop_entry<T>(const T*, T*, const T*, uint64_t, uint64_t, uint64_t, int, bool, \
                                                   const CallOptions&);
INSTANTIATE(float)
INSTANTIATE(double)
#undef INSTANTIATE

}  // namespace sigb200
