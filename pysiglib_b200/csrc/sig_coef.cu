// Individual signature coefficients (sig_coef) and their backward pass on sm_100a.
//
// One thread per (path, word): the thread carries the chain of prefix coefficients
// c_0 = 1, c_1, .., c_k of its word and applies Chen's identity for one increment per step,
//     c_i += sum_{m < i} c_m * (dx[w_{m+1}] .. dx[w_i]) / (i - m)!      (i = k .. 1),
// evaluated in Horner form.  The backward rewinds the chain with the signed factorials and pulls
// the adjoints of all prefixes back through each step, adding the increment gradients to the two
// end points of the segment with atomics (words of one path share channels).  Same recurrences as
// siglib/cpsig/cp_sig_coef_impl.cpp:36-80, 354-486; replaces sig_coef_cuda_ and
// sig_coef_backprop_cuda_ of siglib/cusig/cu_sig_coef.cu (no time_aug / lead_lag here either:
// the caller transforms the path first, as the reference's Python does for CUDA tensors).
#include <vector>

#include "algebra.h"
#include "algebra_host.h"
#include "kernels.h"
#include "runtime.h"

namespace sigb200 {

namespace {

constexpr int kMaxWord = 32;  // longest supported word

template <typename T>
__global__ void sig_coef_kernel(const T* __restrict__ path, T* __restrict__ out, const uint32_t* __restrict__ letters,
                                const uint32_t* __restrict__ word_off, const uint32_t* __restrict__ out_off,
                                uint32_t num, uint64_t batch, uint32_t d, uint32_t L, uint32_t out_stride,
                                bool prefixes) {
    const uint64_t gid = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (gid >= batch * num) return;
    const uint64_t b = gid / num;
    const uint32_t i = uint32_t(gid - b * num);
    const uint32_t k = word_off[i + 1] - word_off[i];
    T* o = out + b * out_stride + out_off[i];
    if (k == 0) { *o = T(1); return; }
    if (L <= 1) {
        for (uint32_t q = 0; q < (prefixes ? k : 1u); ++q) o[q] = T(0);
        return;
    }
    uint32_t w[kMaxWord];
    T c[kMaxWord + 1], inc[kMaxWord], f[kMaxWord + 1];
    f[0] = T(1);
    for (uint32_t q = 0; q < k; ++q) {
        w[q] = letters[word_off[i] + q];
        f[q + 1] = f[q] / static_cast<T>(q + 1);
    }
    const T* x = path + b * uint64_t(L) * d;
    c[0] = T(1);
    T product = T(1);
    for (uint32_t q = 0; q < k; ++q) {
        product *= x[d + w[q]] - x[w[q]];
        c[q + 1] = product * f[q + 1];
    }
    for (uint32_t t = 1; t + 1 < L; ++t) {
        const T* x0 = x + uint64_t(t) * d;
        for (uint32_t q = 0; q < k; ++q) inc[q] = x0[d + w[q]] - x0[w[q]];
        for (uint32_t n = k; n > 0; --n) {
            T acc = f[n];
            for (uint32_t j = 0; j + 1 < n; ++j) acc = acc * inc[j] + c[j + 1] * f[n - j - 1];
            c[n] += acc * inc[n - 1];
        }
    }
    if (!prefixes) *o = c[k];
    else for (uint32_t q = 0; q < k; ++q) o[q] = c[q + 1];
}

template <typename T>
__global__ void sig_coef_backprop_kernel(const T* __restrict__ path, T* __restrict__ out, const T* __restrict__ coefs,
                                         const T* __restrict__ derivs, const uint32_t* __restrict__ letters,
                                         const uint32_t* __restrict__ word_off, const uint32_t* __restrict__ out_off,
                                         uint32_t num, uint64_t batch, uint32_t d, uint32_t L, uint32_t coefs_stride) {
    const uint64_t gid = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (gid >= batch * num) return;
    const uint64_t b = gid / num;
    const uint32_t i = uint32_t(gid - b * num);
    const uint32_t k = word_off[i + 1] - word_off[i];
    if (k == 0 || L <= 1) return;
    uint32_t w[kMaxWord];
    T c[kMaxWord + 1], dc[kMaxWord], inc[kMaxWord], f[kMaxWord + 1], states[kMaxWord], ginc[kMaxWord];
    f[0] = T(1);
    c[0] = T(1);
    for (uint32_t q = 0; q < k; ++q) {
        w[q] = letters[word_off[i] + q];
        f[q + 1] = f[q] / static_cast<T>(q + 1);
        c[q + 1] = coefs[b * coefs_stride + out_off[i] + q];
        dc[q] = derivs[b * coefs_stride + out_off[i] + q];
    }
    const T* x = path + b * uint64_t(L) * d;
    T* g = out + b * uint64_t(L) * d;
    for (uint32_t t = L - 1; t-- > 0;) {
        const T* x0 = x + uint64_t(t) * d;
        for (uint32_t q = 0; q < k; ++q) inc[q] = x0[d + w[q]] - x0[w[q]];
        if (t == 0) {
            for (uint32_t q = 1; q <= k; ++q) c[q] = T(0);
        } else {  // chain at the start of this segment: multiply by the inverse increment
            for (uint32_t n = k; n > 0; --n) {
                T acc = (n & 1) ? -f[n] : f[n];
                for (uint32_t j = 0; j + 1 < n; ++j) {
                    const uint32_t r = n - j - 1;
                    acc = acc * inc[j] + c[j + 1] * ((r & 1) ? -f[r] : f[r]);
                }
                c[n] += acc * inc[n - 1];
            }
        }
        for (uint32_t q = 0; q < k; ++q) ginc[q] = T(0);
        for (uint32_t n = 1; n <= k; ++n) {
            states[0] = f[n];
            for (uint32_t j = 0; j + 1 < n; ++j) states[j + 1] = states[j] * inc[j] + c[j + 1] * f[n - j - 1];
            const T output_deriv = dc[n - 1];
            ginc[n - 1] += output_deriv * states[n - 1];
            T state_deriv = output_deriv * inc[n - 1];
            for (uint32_t j = n - 1; j-- > 0;) {
                ginc[j] += state_deriv * states[j];
                dc[j] += state_deriv * f[n - j - 1];
                state_deriv *= inc[j];
            }
        }
        T* g0 = g + uint64_t(t) * d;
        for (uint32_t q = 0; q < k; ++q) {
            atomicAdd(&g0[d + w[q]], ginc[q]);
            atomicAdd(&g0[w[q]], -ginc[q]);
        }
    }
}

// Word table on the device: letters, start of each word, start of each word's slot(s) in a result row.
struct WordTable {
    std::vector<uint32_t> host;  // letters | word_off (num + 1) | out_off (num + 1)
    uint32_t num = 0, total = 0, row = 0;
};

WordTable make_word_table(const uint64_t* multi_idx, uint64_t num, const uint64_t* degrees, uint64_t dimension,
                          bool prefixes, const char* who) {
    if (num > 0x7fffffffull) throw std::invalid_argument(std::string(who) + ": too many words");
    std::vector<uint64_t> deg(num);
    if (num) SIG_CUDA_CHECK(cudaMemcpy(deg.data(), degrees, num * sizeof(uint64_t), cudaMemcpyDefault));
    uint64_t total = 0;
    for (uint64_t k : deg) {
        if (k > kMaxWord)
            throw std::invalid_argument(std::string(who) + ": words longer than 32 letters are not supported");
        total += k;
    }
    std::vector<uint64_t> idx(total);
    if (total) SIG_CUDA_CHECK(cudaMemcpy(idx.data(), multi_idx, total * sizeof(uint64_t), cudaMemcpyDefault));
    for (uint64_t v : idx)
        if (v >= dimension) throw std::invalid_argument(std::string(who) + ": multi_idx element out of range");
    WordTable t;
    t.num = static_cast<uint32_t>(num);
    t.total = static_cast<uint32_t>(total);
    t.host.resize(total + 2 * (num + 1));
    for (uint64_t q = 0; q < total; ++q) t.host[q] = static_cast<uint32_t>(idx[q]);
    uint32_t* word_off = t.host.data() + total;
    uint32_t* out_off = word_off + num + 1;
    uint32_t wo = 0, oo = 0;
    for (uint64_t i = 0; i < num; ++i) {
        word_off[i] = wo;
        out_off[i] = oo;
        wo += static_cast<uint32_t>(deg[i]);
        oo += (prefixes && deg[i]) ? static_cast<uint32_t>(deg[i]) : 1u;
    }
    word_off[num] = wo;
    out_off[num] = oo;
    t.row = oo;
    return t;
}

}  // namespace

template <typename T>
void sig_coef_entry(const T* path, T* out, const uint64_t* multi_idx, uint64_t num, const uint64_t* degrees,
                    uint64_t batch, uint64_t dimension, uint64_t length, bool prefixes, const CallOptions& opt) {
    if (dimension == 0) throw std::invalid_argument("sig_coef received path of dimension 0");
    if (batch == 0 || num == 0) return;
    if (!out || !degrees || (!path && length * dimension != 0))
        throw std::invalid_argument("sig_coef_cuda received a null pointer");
    if (dimension >= (1ull << 31) || length >= (1ull << 31)) throw std::invalid_argument("sig_coef_cuda: path too large");
    int device = -1;
    const bool on_device = all_on_device({path, out}, "sig_coef_cuda", &device);
    DeviceGuard guard(on_device ? device : (opt.device >= 0 ? opt.device : current_device()));
    const WordTable table = make_word_table(multi_idx, num, degrees, dimension, prefixes, "sig_coef");
    auto run = [&](const T* p, T* o, cudaStream_t st) {
        Scratch tab(table.host.size() * sizeof(uint32_t), st);
        SIG_CUDA_CHECK(cudaMemcpyAsync(tab.get(), table.host.data(), table.host.size() * sizeof(uint32_t),
                                       cudaMemcpyHostToDevice, st));
        const uint32_t* letters = tab.as<uint32_t>();
        const uint32_t* word_off = letters + table.total;
        sig_coef_kernel<T><<<grid_1d(batch * num, 128), 128, 0, st>>>(
            p, o, letters, word_off, word_off + num + 1, table.num, batch, uint32_t(dimension), uint32_t(length),
            table.row, prefixes);
        check_launch("sig_coef kernel");
        SIG_CUDA_CHECK(cudaStreamSynchronize(st));  // the table's host copy must outlive the upload
    };
    if (on_device) {
        run(path, out, opt.stream);
        return;
    }
    run_staged({{path, nullptr, batch * length * dimension * sizeof(T)}, {nullptr, out, batch * table.row * sizeof(T)}},
               opt.device, [&](const std::vector<void*>& dv, cudaStream_t st) {
                   run(static_cast<const T*>(dv[0]), static_cast<T*>(dv[1]), st);
               });
}

template <typename T>
void sig_coef_backprop_entry(const T* path, T* out, const T* coefs, const T* derivs, const uint64_t* multi_idx,
                             uint64_t num, const uint64_t* degrees, uint64_t batch, uint64_t dimension,
                             uint64_t length, const CallOptions& opt) {
    if (dimension == 0) throw std::invalid_argument("sig_coef_backprop received path of dimension 0");
    if (batch == 0 || length == 0) return;
    if (!out || !path) throw std::invalid_argument("sig_coef_backprop_cuda received a null pointer");
    if (dimension >= (1ull << 31) || length >= (1ull << 31))
        throw std::invalid_argument("sig_coef_backprop_cuda: path too large");
    int device = -1;
    const bool on_device = all_on_device({path, out, coefs, derivs}, "sig_coef_backprop_cuda", &device);
    DeviceGuard guard(on_device ? device : (opt.device >= 0 ? opt.device : current_device()));
    WordTable table;
    if (num) {
        if (!degrees || !coefs || !derivs) throw std::invalid_argument("sig_coef_backprop_cuda received a null pointer");
        table = make_word_table(multi_idx, num, degrees, dimension, true, "sig_coef_backprop");
    }
    const uint64_t n_path = batch * length * dimension;
    auto run = [&](const T* p, T* o, const T* c, const T* g, cudaStream_t st) {
        SIG_CUDA_CHECK(cudaMemsetAsync(o, 0, n_path * sizeof(T), st));
        if (num == 0 || length <= 1) return;
        Scratch tab(table.host.size() * sizeof(uint32_t), st);
        SIG_CUDA_CHECK(cudaMemcpyAsync(tab.get(), table.host.data(), table.host.size() * sizeof(uint32_t),
                                       cudaMemcpyHostToDevice, st));
        const uint32_t* letters = tab.as<uint32_t>();
        const uint32_t* word_off = letters + table.total;
        sig_coef_backprop_kernel<T><<<grid_1d(batch * num, 128), 128, 0, st>>>(
            p, o, c, g, letters, word_off, word_off + num + 1, table.num, batch, uint32_t(dimension), uint32_t(length),
            table.row);
        check_launch("sig_coef backward kernel");
        SIG_CUDA_CHECK(cudaStreamSynchronize(st));
    };
    if (on_device) {
        run(path, out, coefs, derivs, opt.stream);
        if (opt.synchronize) SIG_CUDA_CHECK(cudaStreamSynchronize(opt.stream));
        return;
    }
    const size_t cb = batch * table.row * sizeof(T);
    run_staged({{path, nullptr, n_path * sizeof(T)}, {nullptr, out, n_path * sizeof(T)}, {coefs, nullptr, cb},
                {derivs, nullptr, cb}},
               opt.device, [&](const std::vector<void*>& dv, cudaStream_t st) {
                   run(static_cast<const T*>(dv[0]), static_cast<T*>(dv[1]), static_cast<const T*>(dv[2]),
                       static_cast<const T*>(dv[3]), st);
               });
}

#define INSTANTIATE(T)                                                                                              \
    template void sig_coef_entry<T>(const T*, T*, const uint64_t*, uint64_t, const uint64_t*, uint64_t, uint64_t,   \
                                    uint64_t, bool, const CallOptions&);                                            \
    template void sig_coef_backprop_entry<T>(const T*, T*, const T*, const T*, const uint64_t*, uint64_t,           \
                                             const uint64_t*, uint64_t, uint64_t, uint64_t, const CallOptions&);
INSTANTIATE(float)
INSTANTIATE(double)
#undef INSTANTIATE

}  // namespace sigb200
