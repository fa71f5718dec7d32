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
// sig_to_log_sig_backprop_cuda_ of siglib/cusig/cu_log_signature.cu for methods 0, 1 and 2.
#include <map>
#include <mutex>
#include <tuple>

#include "algebra.h"
#include "algebra_host.h"
#include "algebra_math.h"
#include "dispatch.h"
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
    // Q = dLoss/dR_k lives on the levels of R_k (<= 1 + N - k; all levels for the seed, k = 1)
    const uint32_t top = k == 1 ? lv.degree : 1 + lv.degree - k;
    for (uint64_t b = blockIdx.y; b < batch; b += gridDim.y) {
        const T* xb = x + b * x_stride;
        const T* qb = q + b * S;
        T add = (k >= 2 && t <= top) ? qb[j] * constant : T(0);
        if (r_next) add -= nonunital_left_adjoint_coeff(qb, r_next + b * S, lv, t, w, top);
        if (t <= top) dsig[b * dsig_stride + j] += add;
        if (q_new) q_new[b * S + j] = -nonunital_right_adjoint_coeff(qb, xb, lv, t, w, top);
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

// Inverse of the Lyndon-position table for the fused sweep: rank[p] = index of the Lyndon word that
// sits at scalar-free position p, -1 for every other word.
struct LyndonRank {
    int32_t* device = nullptr;
    uint32_t count = 0;
};
std::map<std::tuple<int, uint64_t, uint64_t>, LyndonRank> g_ranks;

LyndonRank lyndon_rank_table(uint64_t dim, uint64_t degree) {
    const int device = current_device();
    std::lock_guard<std::mutex> lock(g_tables_mu);
    const auto key = std::make_tuple(device, dim, degree);
    auto it = g_ranks.find(key);
    if (it != g_ranks.end()) return it->second;
    const std::vector<uint32_t> positions = lyndon_positions(dim, degree);
    std::vector<int32_t> host(sig_length_full(dim, degree) - 1, -1);
    for (size_t i = 0; i < positions.size(); ++i) host[positions[i]] = static_cast<int32_t>(i);
    LyndonRank table;
    table.count = static_cast<uint32_t>(positions.size());
    SIG_CUDA_CHECK(cudaMalloc(&table.device, std::max<size_t>(host.size(), 1) * sizeof(int32_t)));
    SIG_CUDA_CHECK(cudaMemcpy(table.device, host.data(), host.size() * sizeof(int32_t), cudaMemcpyHostToDevice));
    g_ranks.emplace(key, table);
    return table;
}

// ----- Lyndon basis (method 2) --------------------------------------------------------------------
//
// The log signature is a Lie element: log S = sum_j b_j [w_j] over the Lyndon words w_j, where the
// bracket [w] = [[u],[v]] follows the standard factorisation w = u v (v the longest proper Lyndon
// suffix) and [a] = a for a letter.  Expanding a bracket gives w itself plus lexicographically larger
// words, so the matrix P[i][j] = coefficient of the word w_i in [w_j] is unit lower triangular and
// block diagonal by word length; the Lyndon-word coordinates a of method 1 are a = P b, hence
// b = P^-1 a.  As in the reference (siglib/shared/preparation/log_sig/lyndon_words.cpp:150-252,
// log_sig_cache.cpp:33-46) the inverse is built once per (dimension, degree) and applied as a sparse
// matrix; here both it and its transpose live on the device in CSR form.
struct CsrHost {
    std::vector<uint32_t> row_ptr, col;
    std::vector<double> val;
};

void rows_to_csr(const std::vector<std::map<uint32_t, double>>& rows, CsrHost& out) {
    out.row_ptr.assign(1, 0);
    for (const auto& row : rows) {
        for (const auto& kv : row)
            if (kv.second != 0.0) { out.col.push_back(kv.first); out.val.push_back(kv.second); }
        out.row_ptr.push_back(static_cast<uint32_t>(out.col.size()));
    }
}

void build_basis_inverse(uint64_t dim, uint64_t degree, CsrHost& inv, CsrHost& inv_t) {
    using Word = std::vector<uint32_t>;
    // Lyndon words in the table's order, their flat codes (code(uv) = code(u) dim^|v| + code(v))
    std::vector<Word> words;
    {
        Word w;
        for (uint64_t n = 1; n <= degree; ++n) {
            w.assign(1, 0);
            while (!w.empty()) {
                const size_t m = w.size();
                if (m == n) words.push_back(w);
                while (w.size() < n) w.push_back(w[w.size() - m]);
                while (!w.empty() && w.back() == dim - 1) w.pop_back();
                if (!w.empty()) ++w.back();
            }
        }
    }
    const uint32_t M = static_cast<uint32_t>(words.size());
    auto code_of = [&](const Word& w) {
        uint64_t c = 0;
        for (uint32_t letter : w) c = c * dim + letter + 1;
        return c;
    };
    std::map<Word, uint32_t> index_of;
    std::map<uint64_t, uint32_t> lyndon_by_code;
    for (uint32_t i = 0; i < M; ++i) {
        index_of[words[i]] = i;
        lyndon_by_code[code_of(words[i])] = i;
    }
    std::vector<uint64_t> dim_pow(degree + 1, 1);
    for (uint64_t k = 1; k <= degree; ++k) dim_pow[k] = dim_pow[k - 1] * dim;

    // bracket expansions: word code -> integer coefficient
    std::vector<std::map<uint64_t, double>> expansion(M);
    std::vector<std::map<uint32_t, double>> P(M);  // P[i][j]
    for (uint32_t j = 0; j < M; ++j) {
        const Word& w = words[j];
        if (w.size() == 1) {
            expansion[j][code_of(w)] = 1.0;
        } else {
            size_t cut = 1;
            for (; cut < w.size(); ++cut)
                if (index_of.count(Word(w.begin() + cut, w.end()))) break;  // longest proper Lyndon suffix
            const uint32_t ju = index_of.at(Word(w.begin(), w.begin() + cut));
            const uint32_t jv = index_of.at(Word(w.begin() + cut, w.end()));
            const size_t lu = cut, lv = w.size() - cut;
            for (const auto& eu : expansion[ju])
                for (const auto& ev : expansion[jv]) {
                    const double c = eu.second * ev.second;
                    expansion[j][eu.first * dim_pow[lv] + ev.first] += c;
                    expansion[j][ev.first * dim_pow[lu] + eu.first] -= c;
                }
        }
        for (const auto& term : expansion[j]) {
            if (term.second == 0.0) continue;
            const auto it = lyndon_by_code.find(term.first);
            if (it != lyndon_by_code.end()) P[it->second][j] = term.second;
        }
    }
    // forward substitution: row i of P^-1 = e_i - sum_{j < i} P[i][j] * (row j of P^-1)
    std::vector<std::map<uint32_t, double>> inverse(M), transpose(M);
    for (uint32_t i = 0; i < M; ++i) {
        if (P[i].count(i) == 0 || P[i][i] != 1.0)
            throw std::runtime_error("Lyndon projection matrix is not unit triangular");
        std::map<uint32_t, double>& row = inverse[i];
        row[i] = 1.0;
        for (const auto& kv : P[i]) {
            const uint32_t j = kv.first;
            if (j == i) continue;
            if (j > i) throw std::runtime_error("Lyndon projection matrix is not lower triangular");
            for (const auto& r : inverse[j]) row[r.first] -= kv.second * r.second;
        }
        for (const auto& r : row)
            if (r.second != 0.0) transpose[r.first][i] = r.second;
    }
    rows_to_csr(inverse, inv);
    rows_to_csr(transpose, inv_t);
}

struct BasisTable {
    uint32_t rows = 0;
    uint32_t *row_ptr = nullptr, *col = nullptr, *t_row_ptr = nullptr, *t_col = nullptr;
    double *val = nullptr, *t_val = nullptr;
};
std::map<std::tuple<int, uint64_t, uint64_t>, BasisTable> g_basis;

template <typename V>
V* upload(const std::vector<V>& host) {
    V* dev = nullptr;
    SIG_CUDA_CHECK(cudaMalloc(&dev, std::max<size_t>(host.size(), 1) * sizeof(V)));
    SIG_CUDA_CHECK(cudaMemcpy(dev, host.data(), host.size() * sizeof(V), cudaMemcpyHostToDevice));
    return dev;
}

BasisTable basis_table(uint64_t dim, uint64_t degree) {
    const int device = current_device();
    std::lock_guard<std::mutex> lock(g_tables_mu);
    const auto key = std::make_tuple(device, dim, degree);
    auto it = g_basis.find(key);
    if (it != g_basis.end()) return it->second;
    CsrHost inv, inv_t;
    build_basis_inverse(dim, degree, inv, inv_t);
    BasisTable t;
    t.rows = static_cast<uint32_t>(inv.row_ptr.size() - 1);
    t.row_ptr = upload(inv.row_ptr);
    t.col = upload(inv.col);
    t.val = upload(inv.val);
    t.t_row_ptr = upload(inv_t.row_ptr);
    t.t_col = upload(inv_t.col);
    t.t_val = upload(inv_t.val);
    g_basis.emplace(key, t);
    return t;
}

// out[b][i] = sum_k val[k] * in[b][col[k]] over row i of a CSR matrix; one thread per row.
template <typename T>
__global__ void basis_spmv_kernel(const T* __restrict__ in, uint64_t in_stride, T* __restrict__ out,
                                  uint64_t out_stride, const uint32_t* __restrict__ row_ptr,
                                  const uint32_t* __restrict__ col, const double* __restrict__ val, uint32_t rows,
                                  uint64_t batch) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows) return;
    const uint32_t begin = row_ptr[i], end = row_ptr[i + 1];
    for (uint64_t b = blockIdx.y; b < batch; b += gridDim.y) {
        const T* x = in + b * in_stride;
        T acc = T(0);
        for (uint32_t k = begin; k < end; ++k) acc = alg_fma(static_cast<T>(val[k]), x[col[k]], acc);
        out[b * out_stride + i] = acc;
    }
}

void check_method(int method, const char* who) {
    if (method == 0 || method == 1 || method == 2) return;
    if (method == 3)
        throw std::invalid_argument(std::string(who) + ": log-signature method 3 is not part of this build of "
                                    "libcusig (methods 0, 1 and 2 are)");
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
    {
        std::lock_guard<std::mutex> lock(g_tables_mu);
        for (auto& kv : g_ranks) {
            int prev = -1;
            if (cudaGetDevice(&prev) != cudaSuccess) { (void)cudaGetLastError(); continue; }
            if (cudaSetDevice(std::get<0>(kv.first)) == cudaSuccess && kv.second.device) (void)cudaFree(kv.second.device);
            (void)cudaSetDevice(prev);
            (void)cudaGetLastError();
        }
        g_ranks.clear();
    }
    std::lock_guard<std::mutex> lock(g_tables_mu);
    for (auto& kv : g_tables) {
        int prev = -1;
        if (cudaGetDevice(&prev) != cudaSuccess) { (void)cudaGetLastError(); continue; }
        if (cudaSetDevice(std::get<0>(kv.first)) == cudaSuccess) (void)cudaFree(kv.second.device);
        (void)cudaSetDevice(prev);
        (void)cudaGetLastError();
    }
    g_tables.clear();
    for (auto& kv : g_basis) {
        int prev = -1;
        if (cudaGetDevice(&prev) != cudaSuccess) { (void)cudaGetLastError(); continue; }
        if (cudaSetDevice(std::get<0>(kv.first)) == cudaSuccess) {
            BasisTable& t = kv.second;
            (void)cudaFree(t.row_ptr); (void)cudaFree(t.col); (void)cudaFree(t.val);
            (void)cudaFree(t.t_row_ptr); (void)cudaFree(t.t_col); (void)cudaFree(t.t_val);
        }
        (void)cudaSetDevice(prev);
        (void)cudaGetLastError();
    }
    g_basis.clear();
}

void prepare_log_sig_entry(uint64_t dimension, uint64_t degree, int method) {
    if (dimension == 0) throw std::invalid_argument("prepare_log_sig_cuda received dimension 0");
    check_method(method, "prepare_log_sig_cuda");
    if (method == 0) return;
    (void)checked_levels(dimension, degree, "prepare_log_sig_cuda");
    (void)lyndon_table(dimension, degree);
    if (method == 2) (void)basis_table(dimension, degree);
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
        BasisTable basis;
        if (method >= 1) table = lyndon_table(dimension, degree);
        if (method == 2) basis = basis_table(dimension, degree);
        const uint64_t out_stride = method >= 1 ? table.count : in_stride;
        const uint64_t per_sig = (2 * S + (method == 2 ? table.count : 0)) * sizeof(T);
        const uint64_t chunk = std::max<uint64_t>(1, std::min<uint64_t>(batch, kLogScratchBudget / per_sig));
        Scratch ws(chunk * per_sig, st);
        for (uint64_t b0 = 0; b0 < batch; b0 += chunk) {
            const uint64_t count = std::min(chunk, batch - b0);
            const T* x = a + b0 * in_stride + shift;
            // big batches: one kernel, one CTA per signature, the recursion in shared memory
            {
                T* target = method == 2 ? ws.as<T>() + 2 * chunk * S
                                        : o + b0 * out_stride + (method == 0 ? shift : 0);
                if (launch_log_forward_streamed<T>(x, in_stride, target, out_stride, method >= 1 ? table.device : nullptr,
                                                   method >= 1 ? table.count : static_cast<uint32_t>(S),
                                                   method == 0 && scalar_term, count, dimension, degree, st)) {
                    if (method == 2) {
                        basis_spmv_kernel<T><<<coeff_grid(basis.rows, count), kThreads, 0, st>>>(
                            target, out_stride, o + b0 * out_stride, out_stride, basis.row_ptr, basis.col, basis.val,
                            basis.rows, count);
                        check_launch("tensor log kernel");
                    }
                    continue;
                }
            }
            const T* r2 = degree >= 2 ? run_horner<T>(x, in_stride, ws.as<T>(), false, lv, count, st) : nullptr;
            if (method >= 1) {
                // Lyndon-word coordinates, straight into the result (method 1) or into scratch (method 2)
                T* words = method == 2 ? ws.as<T>() + 2 * chunk * S : o + b0 * out_stride;
                log_final_kernel<T><<<coeff_grid(table.count, count), kThreads, 0, st>>>(
                    x, in_stride, r2, words, out_stride, lv, count, table.device, table.count, false);
                if (method == 2) {
                    check_launch("tensor log kernel");
                    basis_spmv_kernel<T><<<coeff_grid(basis.rows, count), kThreads, 0, st>>>(
                        words, out_stride, o + b0 * out_stride, out_stride, basis.row_ptr, basis.col, basis.val,
                        basis.rows, count);
                }
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
    const uint64_t out_len = method >= 1 ? log_sig_length_host(dimension, degree) : in_stride;
    run_staged({{sig, nullptr, batch * in_stride * sizeof(T)}, {nullptr, out, batch * out_len * sizeof(T)}}, opt.device,
               [&](const std::vector<void*>& d, cudaStream_t st) {
                   run(static_cast<const T*>(d[0]), static_cast<T*>(d[1]), st);
               });
}

// Log signature straight from the path (methods 0, 1, 2).  Replaces the reference's Python-level
// composition sig -> sig_to_log_sig (pysiglib/log_sig.py:457) by one native call in which the
// signature never becomes a caller-visible array: when the shape has a fused sweep
// (launch_tile_forward_log) it never leaves the SMs at all; otherwise it is computed into pooled
// scratch, one batch chunk at a time, and fed to the kernels of sig_to_log_sig.
template <typename T>
void log_sig_entry(const T* path, T* out, uint64_t batch, uint64_t dimension, uint64_t length, uint64_t degree,
                   bool time_aug, bool lead_lag, T end_time, int method, bool scalar_term, const CallOptions& opt) {
    if (dimension == 0) throw std::invalid_argument("log_sig received path of dimension 0");
    if (degree == 0) throw std::invalid_argument("log signature received degree 0");
    check_method(method, "log_sig");
    if (opt.nonfinite) *opt.nonfinite = 0;
    if (batch == 0) return;
    if (!path || !out) throw std::invalid_argument("log_sig received a null pointer");
    const SigShape s = make_shape(batch, dimension, length, degree, time_aug, lead_lag, method == 0 && scalar_term);
    const Levels lv = checked_levels(s.dim, degree, "log_sig");
    const uint64_t S = lv.total();
    const uint64_t out_len = method >= 1 ? log_sig_length_host(s.dim, degree) : s.stride;

    auto run = [&](const T* dpath, T* dout, cudaStream_t st, int* flag) {
        LyndonRank rank;
        BasisTable basis;
        if (method >= 1) rank = lyndon_rank_table(s.dim, degree);
        if (method == 2) basis = basis_table(s.dim, degree);
        // method 2: Lyndon-word coordinates into scratch, then the sparse change of basis
        Scratch words(method == 2 ? batch * out_len * sizeof(T) : 0, st);
        T* target = method == 2 ? words.as<T>() : dout;
        const uint32_t shift = method == 0 && scalar_term ? 1 : 0;
        // tile preference 1 ("always the biggest tile", a test hook) also forces the fused sweep
        bool fused = kernel_policy() == 0 &&
                     launch_tile_forward_log<T>(dpath, target, s, end_time, static_cast<uint32_t>(out_len), shift,
                                                method >= 1 ? rank.device : nullptr, flag, st, tile_preference() == 1);
        if (!fused) {
            // signature of a batch chunk into scratch (scalar-free), then the tensor-logarithm kernels
            SigShape cs = make_shape(batch, dimension, length, degree, time_aug, lead_lag, false);
            const uint64_t per_path = 3 * S * sizeof(T);
            const uint64_t chunk = std::max<uint64_t>(1, std::min<uint64_t>(batch, kLogScratchBudget / per_path));
            Scratch ws(chunk * per_path, st);
            LyndonTable table;
            if (method >= 1) table = lyndon_table(s.dim, degree);
            for (uint64_t b0 = 0; b0 < batch; b0 += chunk) {
                const uint64_t count = std::min(chunk, batch - b0);
                cs.batch = count;
                T* sig = ws.as<T>() + 2 * chunk * S;
                forward_on_device<T>(dpath + b0 * length * dimension, sig, cs, end_time, st, flag);
                if (launch_log_forward_streamed<T>(sig, S, target + b0 * out_len + (method == 0 ? shift : 0), out_len,
                                                   method >= 1 ? table.device : nullptr,
                                                   method >= 1 ? table.count : static_cast<uint32_t>(S), shift != 0, count,
                                                   s.dim, degree, st))
                    continue;
                const T* r2 = degree >= 2 ? run_horner<T>(sig, S, ws.as<T>(), false, lv, count, st) : nullptr;
                if (method >= 1) {
                    log_final_kernel<T><<<coeff_grid(table.count, count), kThreads, 0, st>>>(
                        sig, S, r2, target + b0 * out_len, out_len, lv, count, table.device, table.count, false);
                } else {
                    log_final_kernel<T><<<coeff_grid(lv.total(), count), kThreads, 0, st>>>(
                        sig, S, r2, target + b0 * out_len + shift, out_len, lv, count, nullptr, lv.total(), shift != 0);
                }
                check_launch("tensor log kernel");
            }
        }
        if (method == 2) {
            basis_spmv_kernel<T><<<coeff_grid(basis.rows, batch), kThreads, 0, st>>>(
                target, out_len, dout, out_len, basis.row_ptr, basis.col, basis.val, basis.rows, batch);
            check_launch("tensor log kernel");
        }
    };
    auto with_flag = [&](const T* dpath, T* dout, cudaStream_t st, bool synchronize) {
        if (opt.nonfinite) {
            Scratch flag(sizeof(int), st);
            SIG_CUDA_CHECK(cudaMemsetAsync(flag.get(), 0, sizeof(int), st));
            run(dpath, dout, st, flag.as<int>());
            SIG_CUDA_CHECK(cudaMemcpyAsync(opt.nonfinite, flag.get(), sizeof(int), cudaMemcpyDeviceToHost, st));
            SIG_CUDA_CHECK(cudaStreamSynchronize(st));
        } else {
            run(dpath, dout, st, nullptr);
            if (synchronize) SIG_CUDA_CHECK(cudaStreamSynchronize(st));
        }
    };
    int device = -1;
    if (all_on_device({path, out}, "log_sig", &device)) {
        DeviceGuard guard(device);
        with_flag(path, out, opt.stream, opt.synchronize);
        return;
    }
    run_staged({{path, nullptr, batch * length * dimension * sizeof(T)}, {nullptr, out, batch * out_len * sizeof(T)}},
               opt.device, [&](const std::vector<void*>& d, cudaStream_t st) {
                   with_flag(static_cast<const T*>(d[0]), static_cast<T*>(d[1]), st, false);
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
        BasisTable basis;
        LyndonRank rank;
        if (method >= 1) table = lyndon_table(dimension, degree);
        if (method >= 1) rank = lyndon_rank_table(dimension, degree);
        if (method == 2) basis = basis_table(dimension, degree);
        const uint64_t g_stride = method >= 1 ? table.count : stride;
        const uint64_t vectors = 3 + (N >= 2 ? N - 1 : 0);  // D, two adjoint buffers, R_2..R_N
        const uint64_t per_sig = (vectors * S + (method == 2 ? table.count : 0)) * sizeof(T);
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
            const T* gw = g + b0 * g_stride + (method >= 1 ? 0 : shift);  // adjoint of the Lyndon-word coordinates
            if (method == 2) {
                // the forward applied P^-1 to the Lyndon-word coordinates: pull back through its transpose
                T* pulled = ws.as<T>() + chunk * vectors * S;
                basis_spmv_kernel<T><<<coeff_grid(basis.rows, count), kThreads, 0, st>>>(
                    gw, g_stride, pulled, g_stride, basis.t_row_ptr, basis.t_col, basis.t_val, basis.rows, count);
                check_launch("tensor log backward kernel");
                gw = pulled;
            }
            // big batches of power-of-two dimension: the whole backward in one kernel, one CTA per
            // signature, with the recursion in shared memory (sig_log_stream.cu)
            if (launch_log_adjoint_streamed<T>(x, stride, gw, g_stride, method >= 1 ? rank.device : nullptr, dsig, stride,
                                               scalar_term, count, dimension, degree, st))
                continue;
            log_seed_kernel<T><<<coeff_grid(lv.total(), count), kThreads, 0, st>>>(
                gw, g_stride, D, dsig, stride, lv, count, method >= 1 ? table.device : nullptr, scalar_term);
            check_launch("tensor log backward kernel");
            if (method >= 1) {
                log_scatter_kernel<T><<<coeff_grid(table.count, count), kThreads, 0, st>>>(
                    gw, g_stride, D, dsig, stride, lv.total(), count, table.device, table.count);
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
    const uint64_t g_len = method >= 1 ? log_sig_length_host(dimension, degree) : stride;
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
template void log_sig_entry<float>(const float*, float*, uint64_t, uint64_t, uint64_t, uint64_t, bool, bool, float, int,
                                   bool, const CallOptions&);
template void log_sig_entry<double>(const double*, double*, uint64_t, uint64_t, uint64_t, uint64_t, bool, bool, double,
                                    int, bool, const CallOptions&);
#undef INSTANTIATE

}  // namespace sigb200
