// Host dispatch behind the C ABI: argument validation, closed-form cases, kernel
// family choice, scratch memory, and the pipelined path for calls that pass host
// memory (NumPy arrays) instead of device pointers.
//
// Replaces siglib/cusig/cu_signature.cu:2592-2657 (signature_cuda_),
// :2467-2590 (signature_cuda_core_), :3417-3488 (sig_backprop_cuda_) and the
// algorithm chooser :2980-3415 of the reference.  Differences kept deliberate:
//   * the device is taken from the pointer, not from cudaGetDevice();
//   * flags never materialise a transformed path (increments are synthesised in
//     the kernels), forward and backward;
//   * horner=false computes the same signature with the Horner kernels;
//   * host pointers are accepted: the batch is cut into chunks that are copied
//     in, computed and copied out on three streams so the copies overlap compute.
#include "dispatch.h"
#include "algebra.h"

#include <algorithm>
#include <cmath>
#include <memory>
#include <vector>

#include "kernels.h"
#include "runtime.h"

namespace sigb200 {

namespace {

// Number of correction values reachable from the base pointer for `batch` paths of `segments` segments.
template <typename T>
uint64_t corrected_elems(const CorrectionView<T>& c, uint64_t batch, uint64_t segments) {
    return (batch - 1) * c.batch_stride + (segments - 1) * c.segment_stride + c.len;
}

unsigned generic_ctas(const SigShape& s, int sm_count, uint64_t bytes_per_cta) {
    uint64_t ctas = std::min<uint64_t>(s.batch, uint64_t(sm_count) * 4);
    // keep the fallback's scratch under 4 GiB
    const uint64_t cap = std::max<uint64_t>(1, (4ull << 30) / std::max<uint64_t>(bytes_per_cta, 1));
    ctas = std::max<uint64_t>(1, std::min(ctas, cap));
    return static_cast<unsigned>(ctas);
}

int sm_count_of_current_device() {
    return device_context(current_device()).sm_count;
}

// One pipelined pass over the batch for host-resident operands.
struct HostOperand {
    const void* host;
    uint64_t bytes_per_path;
};

// Calls run(begin, count) over [0, batch) in pieces, halving the piece after every
// std::bad_alloc until a single path fails too (the reference's recovery from
// cudaErrorMemoryAllocation, siglib/cusig/cu_runtime_utils.h:212-235).  run() must take its
// scratch before it enqueues work that cannot be repeated.
template <typename Run>
void with_batch_backoff(uint64_t batch, Run&& run) {
    uint64_t piece = batch, begin = 0;
    while (begin < batch) {
        const uint64_t count = std::min(piece, batch - begin);
        try {
            run(begin, count);
            begin += count;
        } catch (const std::bad_alloc&) {
            if (piece <= 1) throw;
            piece = (piece + 1) / 2;
        }
    }
}

// Pipelined pass over the batch for host-resident operands: the batch is cut into chunks that
// are copied in, computed and copied out on three streams through two staging slots, so that
// the copies of one chunk overlap the kernels of its neighbours.  `wave_paths` is the number of
// paths that fill the GPU exactly once with the kernels compute() will launch (0 = unknown);
// chunks are whole multiples of it so that no chunk ends in a partly filled wave.
template <typename Compute>
void run_host_pipeline(uint64_t batch, const std::vector<HostOperand>& inputs, void* host_out,
                       uint64_t out_bytes_per_path, uint64_t wave_paths, Compute&& compute) {
    DeviceContext& ctx = device_context(current_device());
    std::lock_guard<std::mutex> lock(ctx.mu);

    auto aligned = [](uint64_t bytes) { return (bytes + 255) / 256 * 256; };
    uint64_t per_path = out_bytes_per_path;
    for (const auto& in : inputs) per_path += in.bytes_per_path;
    per_path = std::max<uint64_t>(per_path, 1);
    // The first chunk's copy-in and the last chunk's copy-out are not hidden behind any kernel, and every
    // chunk boundary drains the GPU once (the kernels of the next chunk start when the last CTA of this
    // one is done).  So the chunks ramp: one unit first, then 2, 4, ... up to 16 units in the middle, and
    // down again at the end; a unit is about 8 MiB of staged operands, rounded to whole waves of the
    // kernels compute() launches, and no chunk exceeds 2 GiB.
    const uint64_t total_bytes = per_path * batch;
    const uint64_t n_target = std::min<uint64_t>(64, std::max<uint64_t>(1, total_bytes / (8ull << 20)));
    uint64_t unit = (batch + n_target - 1) / n_target;
    if (wave_paths > 0 && n_target > 1) unit = std::max<uint64_t>(1, (unit + wave_paths / 2) / wave_paths) * wave_paths;
    unit = std::min<uint64_t>(unit, std::max<uint64_t>(1, (2ull << 30) / per_path));
    unit = std::max<uint64_t>(std::min(unit, batch), 1);
    const uint64_t cap = std::max<uint64_t>(unit, std::min<uint64_t>(16 * unit, std::max<uint64_t>(1, (2ull << 30) / per_path)));

    // staging slots: kept between calls, grown on demand; on out-of-memory the largest chunk is halved
    uint64_t chunk = cap;                                  // largest chunk = capacity of a slot, in paths
    std::vector<uint64_t> sizes;
    uint64_t slot_bytes = 0;
    int n_buf = 1;
    for (;;) {
        // up-ramp from the front, down-ramp from the back, the middle in chunks of `chunk`
        sizes.clear();
        std::vector<uint64_t> tail;
        uint64_t left = batch, step = std::min(unit, chunk);
        while (left > 0) {
            const uint64_t front = std::min(step, left);
            sizes.push_back(front);
            left -= front;
            if (left == 0) break;
            if (step < chunk) {
                const uint64_t back = std::min(step, left);
                tail.push_back(back);
                left -= back;
                step = std::min(2 * step, chunk);
            }
        }
        sizes.insert(sizes.end(), tail.rbegin(), tail.rend());
        slot_bytes = aligned(std::max<uint64_t>(out_bytes_per_path * chunk, 16));
        for (const auto& in : inputs) slot_bytes += aligned(std::max<uint64_t>(in.bytes_per_path * chunk, 16));
        n_buf = sizes.size() > 1 ? 2 : 1;
        try {
            reserve_staging(ctx, slot_bytes, n_buf);
            break;
        } catch (const std::bad_alloc&) {
            if (chunk <= 1) throw;
            chunk = (chunk + 1) / 2;
        }
    }
    const uint64_t n_chunks = sizes.size();

    auto drain = [&]() {
        (void)cudaStreamSynchronize(ctx.copy_in);
        (void)cudaStreamSynchronize(ctx.compute);
        (void)cudaStreamSynchronize(ctx.copy_out);
    };
    try {
        SIG_CUDA_CHECK(cudaEventRecord(ctx.ready, ctx.compute));
        SIG_CUDA_CHECK(cudaStreamWaitEvent(ctx.copy_in, ctx.ready, 0));
        SIG_CUDA_CHECK(cudaStreamWaitEvent(ctx.copy_out, ctx.ready, 0));
        std::vector<void*> din(inputs.size());
        uint64_t begin = 0;
        for (uint64_t c = 0; c < n_chunks; begin += sizes[c], ++c) {
            StagingSlot& sl = ctx.slots[c % n_buf];
            const uint64_t count = sizes[c];
            unsigned char* cursor = static_cast<unsigned char*>(sl.buffer);
            void* dout = cursor;
            cursor += aligned(std::max<uint64_t>(out_bytes_per_path * chunk, 16));
            for (size_t i = 0; i < inputs.size(); ++i) {
                din[i] = cursor;
                cursor += aligned(std::max<uint64_t>(inputs[i].bytes_per_path * chunk, 16));
            }
            if (c >= uint64_t(n_buf)) {
                // the slot's previous occupant must have been consumed before it is overwritten
                SIG_CUDA_CHECK(cudaStreamWaitEvent(ctx.copy_in, sl.computed, 0));
                SIG_CUDA_CHECK(cudaStreamWaitEvent(ctx.compute, sl.copied_out, 0));
            }
            for (size_t i = 0; i < inputs.size(); ++i) {
                const uint64_t bpp = inputs[i].bytes_per_path;
                if (bpp == 0) continue;
                SIG_CUDA_CHECK(cudaMemcpyAsync(din[i], static_cast<const char*>(inputs[i].host) + begin * bpp,
                                               count * bpp, cudaMemcpyHostToDevice, ctx.copy_in));
            }
            SIG_CUDA_CHECK(cudaEventRecord(sl.copied_in, ctx.copy_in));
            SIG_CUDA_CHECK(cudaStreamWaitEvent(ctx.compute, sl.copied_in, 0));
            compute(din, dout, count, ctx.compute);
            SIG_CUDA_CHECK(cudaEventRecord(sl.computed, ctx.compute));
            SIG_CUDA_CHECK(cudaStreamWaitEvent(ctx.copy_out, sl.computed, 0));
            if (out_bytes_per_path)
                SIG_CUDA_CHECK(cudaMemcpyAsync(static_cast<char*>(host_out) + begin * out_bytes_per_path, dout,
                                               count * out_bytes_per_path, cudaMemcpyDeviceToHost, ctx.copy_out));
            SIG_CUDA_CHECK(cudaEventRecord(sl.copied_out, ctx.copy_out));
        }
        SIG_CUDA_CHECK(cudaStreamSynchronize(ctx.copy_in));
        SIG_CUDA_CHECK(cudaStreamSynchronize(ctx.compute));
        SIG_CUDA_CHECK(cudaStreamSynchronize(ctx.copy_out));
    } catch (...) {
        drain();
        throw;
    }
}

// Device-side "output holds NaN / Inf" flag of one forward call: an int in scratch that the
// kernels set, read back once at the end of the call.
struct NonfiniteFlag {
    Scratch mem;
    cudaStream_t stream;
    NonfiniteFlag(cudaStream_t st) : mem(sizeof(int), st), stream(st) {
        SIG_CUDA_CHECK(cudaMemsetAsync(mem.get(), 0, sizeof(int), st));
    }
    int* device() const { return mem.as<int>(); }
    // copies the flag to `host` and waits for the stream
    void fetch(int* host) {
        SIG_CUDA_CHECK(cudaMemcpyAsync(host, mem.get(), sizeof(int), cudaMemcpyDeviceToHost, stream));
        SIG_CUDA_CHECK(cudaStreamSynchronize(stream));
    }
};

}  // namespace

// One piece of a forward call; takes its scratch before it launches anything.
template <typename T>
void forward_piece(const T* path, T* out, const SigShape& s, T end_time, cudaStream_t stream, int* nonfinite) {
    if (s.len <= 1 || s.degree <= 1 || s.dim == 1) {
        launch_trivial_forward<T>(path, out, s, end_time, stream);
        if (nonfinite) launch_nonfinite_scan<T>(out, s.batch * s.stride, nonfinite, stream);
        return;
    }
    // the register-tile sweep checks its own results as it stores them (no extra pass over the output)
    bool flag_done = false;
    if (kernel_policy() == 0 && launch_tile_forward<T>(path, out, s, end_time, stream, nonfinite, &flag_done)) {
        if (nonfinite && !flag_done) launch_nonfinite_scan<T>(out, s.batch * s.stride, nonfinite, stream);
        return;
    }
    const uint64_t elems = generic_forward_scratch_elems(s);
    const unsigned ctas = generic_ctas(s, sm_count_of_current_device(), elems * sizeof(T));
    Scratch scratch(checked_mul(checked_mul(elems, ctas, "scratch"), sizeof(T), "scratch"), stream);
    launch_generic_forward<T>(path, out, s, end_time, scratch.as<T>(), ctas, stream);
    if (nonfinite) launch_nonfinite_scan<T>(out, s.batch * s.stride, nonfinite, stream);
}

template <typename T>
void forward_on_device(const T* path, T* out, const SigShape& s, T end_time, cudaStream_t stream, int* nonfinite) {
    if (s.batch == 0 || s.stride == 0) return;
    with_batch_backoff(s.batch, [&](uint64_t begin, uint64_t count) {
        SigShape piece = s;
        piece.batch = count;
        forward_piece<T>(path + begin * s.data_len * s.data_dim, out + begin * s.stride, piece, end_time, stream,
                         nonfinite);
    });
}

template <typename T>
void backward_piece(const T* path, T* out, const T* sig_derivs, const T* sig, const SigShape& s, T end_time,
                    cudaStream_t stream) {
    if (kernel_policy() == 0 && tile_backward_available<T>(s)) {
        const uint64_t g_elems = checked_mul(s.batch, checked_mul(s.data_len - 1, s.data_dim, "scratch"), "scratch");
        Scratch incr(checked_mul(g_elems, sizeof(T), "scratch"), stream);
        if (launch_tile_backward<T>(path, out, sig_derivs, sig, s, end_time, incr.as<T>(), stream)) return;
    }
    const uint64_t elems = generic_backward_scratch_elems(s);
    const unsigned ctas = generic_ctas(s, sm_count_of_current_device(), elems * sizeof(T));
    Scratch scratch(checked_mul(checked_mul(elems, ctas, "scratch"), sizeof(T), "scratch"), stream);
    launch_generic_backward<T>(path, out, sig_derivs, sig, s, end_time, scratch.as<T>(), ctas, stream);
}

template <typename T>
void backward_on_device(const T* path, T* out, const T* sig_derivs, const T* sig, const SigShape& s,
                        T end_time, cudaStream_t stream) {
    const uint64_t out_elems = checked_mul(s.batch, checked_mul(s.data_len, s.data_dim, "path gradient"),
                                           "path gradient");
    if (out_elems == 0) return;
    if (s.len <= 1 || s.degree == 0) {
        launch_fill<T>(out, out_elems, T(0), stream);
        return;
    }
    if (s.degree == 1) {
        launch_degree_one_backward<T>(path, out, sig_derivs, s, end_time, stream);
        return;
    }
    if (s.degree > kMaxDegree)
        throw std::invalid_argument("sig_backprop on CUDA requires degree <= 64. Reduce the truncation level.");
    with_batch_backoff(s.batch, [&](uint64_t begin, uint64_t count) {
        SigShape piece = s;
        piece.batch = count;
        const uint64_t p_off = begin * s.data_len * s.data_dim, s_off = begin * s.stride;
        backward_piece<T>(path + p_off, out + p_off, sig_derivs + s_off, sig + s_off, piece, end_time, stream);
    });
}

template <typename T>
void signature_entry(const T* path, T* out, uint64_t batch, uint64_t dimension, uint64_t length,
                     uint64_t degree, bool time_aug, bool lead_lag, T end_time, bool /*horner*/,
                     bool scalar_term, const T* correction, uint64_t correction_len, const CallOptions& opt,
                     uint64_t correction_batch_stride, uint64_t correction_segment_stride) {
    if (dimension == 0) throw std::invalid_argument("signature_cuda received path of dimension 0");
    validate_correction(correction, correction_len, dimension, degree, lead_lag);
    if (opt.nonfinite) *opt.nonfinite = 0;
    if (batch == 0) return;
    const SigShape s = make_shape(batch, dimension, length, degree, time_aug, lead_lag, scalar_term);
    if (s.stride == 0) return;
    if (out == nullptr || (path == nullptr && length * dimension != 0))
        throw std::invalid_argument("signature_cuda received a null pointer");
    if (correction_len != 0 && s.len > 1) {
        // segment signatures exp(increment + correction): siglib/cusig/cu_signature.cu:2503-2531
        const CorrectionView<T> cv{correction, correction_len, correction_batch_stride, correction_segment_stride};
        const uint64_t corr_elems = corrected_elems(cv, batch, s.len - 1);
        const PointerInfo po = classify_pointer(out);
        if (po.on_device) {
            require_on_device({path, correction}, po.device, "signature_cuda");
            DeviceGuard guard(po.device);
            correction_forward_on_device<T>(path, out, s, end_time, cv, opt.stream);
            if (opt.nonfinite) {
                NonfiniteFlag flag(opt.stream);
                launch_nonfinite_scan<T>(out, s.batch * s.stride, flag.device(), opt.stream);
                flag.fetch(opt.nonfinite);
            } else if (opt.synchronize) {
                SIG_CUDA_CHECK(cudaStreamSynchronize(opt.stream));
            }
            return;
        }
        if (classify_pointer(path).on_device || classify_pointer(correction).on_device)
            throw std::invalid_argument("signature_cuda: path, correction and out must all be device pointers or all host pointers");
        // host buffers: one staged round trip (corrected signatures are small next to the headline workloads)
        DeviceGuard guard(opt.device >= 0 ? opt.device : current_device());
        DeviceContext& ctx = device_context(current_device());
        std::lock_guard<std::mutex> lock(ctx.mu);
        cudaStream_t st = ctx.compute;
        const uint64_t np = batch * length * dimension, no = batch * s.stride;
        Scratch buf((np + no + corr_elems) * sizeof(T), st);
        T* dp = buf.as<T>();
        T* dout = dp + np;
        T* dc = dout + no;
        SIG_CUDA_CHECK(cudaMemcpyAsync(dp, path, np * sizeof(T), cudaMemcpyHostToDevice, st));
        SIG_CUDA_CHECK(cudaMemcpyAsync(dc, correction, corr_elems * sizeof(T), cudaMemcpyHostToDevice, st));
        CorrectionView<T> dcv = cv;
        dcv.ptr = dc;
        correction_forward_on_device<T>(dp, dout, s, end_time, dcv, st);
        SIG_CUDA_CHECK(cudaMemcpyAsync(out, dout, no * sizeof(T), cudaMemcpyDeviceToHost, st));
        if (opt.nonfinite) {
            NonfiniteFlag flag(st);
            launch_nonfinite_scan<T>(dout, no, flag.device(), st);
            flag.fetch(opt.nonfinite);
        }
        SIG_CUDA_CHECK(cudaStreamSynchronize(st));
        return;
    }

    const PointerInfo pin = classify_pointer(path), pout = classify_pointer(out);
    const bool host_call = !pout.on_device;
    if (length * dimension != 0 && pin.on_device != pout.on_device)
        throw std::invalid_argument("signature_cuda: path and out must both be device pointers or both host pointers");

    if (!host_call) {
        if (length * dimension != 0) require_on_device({path}, pout.device, "signature_cuda");
        DeviceGuard guard(pout.device);
        if (opt.nonfinite) {
            NonfiniteFlag flag(opt.stream);
            forward_on_device<T>(path, out, s, end_time, opt.stream, flag.device());
            flag.fetch(opt.nonfinite);
        } else {
            forward_on_device<T>(path, out, s, end_time, opt.stream, nullptr);
            if (opt.synchronize) SIG_CUDA_CHECK(cudaStreamSynchronize(opt.stream));
        }
        return;
    }

    // host operands: stage through the device selected by the caller (current device)
    DeviceGuard guard(opt.device >= 0 ? opt.device : current_device());
    std::vector<HostOperand> ins{{path, s.data_len * s.data_dim * sizeof(T)}};
    // the check for NaN / Inf runs on the device while the chunks are there; only the flag comes back
    std::unique_ptr<NonfiniteFlag> flag;
    if (opt.nonfinite) flag.reset(new NonfiniteFlag(device_context(current_device()).compute));
    run_host_pipeline(batch, ins, out, s.stride * sizeof(T), tile_wave_paths<T>(s, false),
        [&](const std::vector<void*>& din, void* dout, uint64_t count, cudaStream_t stream) {
            SigShape cs = s;
            cs.batch = count;
            forward_on_device<T>(static_cast<const T*>(din[0]), static_cast<T*>(dout), cs, end_time, stream,
                                 flag ? flag->device() : nullptr);
        });
    if (flag) flag->fetch(opt.nonfinite);
}

template <typename T>
void sig_backprop_entry(const T* path, T* out, const T* sig_derivs, const T* sig, uint64_t batch,
                        uint64_t dimension, uint64_t length, uint64_t degree, bool time_aug, bool lead_lag,
                        T end_time, bool scalar_term, const T* correction, uint64_t correction_len,
                        const CallOptions& opt, uint64_t correction_batch_stride,
                        uint64_t correction_segment_stride) {
    if (dimension == 0) throw std::invalid_argument("sig_backprop_cuda received path of dimension 0");
    validate_correction(correction, correction_len, dimension, degree, lead_lag);
    if (batch == 0) return;
    const SigShape s = make_shape(batch, dimension, length, degree, time_aug, lead_lag, scalar_term);
    if (length == 0) return;
    if (out == nullptr || path == nullptr) throw std::invalid_argument("sig_backprop_cuda received a null pointer");
    const bool needs_sig = !(s.len <= 1 || s.degree == 0) && s.stride != 0;
    if (needs_sig && (sig == nullptr || sig_derivs == nullptr))
        throw std::invalid_argument("sig_backprop_cuda received a null pointer");
    if (correction_len != 0 && s.len > 1) {
        // reverse sweep through exp(increment + correction): siglib/cusig/cu_signature.cu:2936-2966
        const CorrectionView<T> cv{correction, correction_len, correction_batch_stride, correction_segment_stride};
        const uint64_t corr_elems = corrected_elems(cv, batch, s.len - 1);
        const PointerInfo po = classify_pointer(out);
        const bool others_on_device = classify_pointer(path).on_device && classify_pointer(sig).on_device &&
                                      classify_pointer(sig_derivs).on_device && classify_pointer(correction).on_device;
        const bool others_on_host = !classify_pointer(path).on_device && !classify_pointer(sig).on_device &&
                                    !classify_pointer(sig_derivs).on_device && !classify_pointer(correction).on_device;
        if (po.on_device ? !others_on_device : !others_on_host)
            throw std::invalid_argument("sig_backprop_cuda: all buffers must be device pointers or all host pointers");
        if (po.on_device) {
            require_on_device({path, sig, sig_derivs, correction}, po.device, "sig_backprop_cuda");
            DeviceGuard guard(po.device);
            correction_backward_on_device<T>(path, out, sig_derivs, sig, s, end_time, cv, opt.stream);
            if (opt.synchronize) SIG_CUDA_CHECK(cudaStreamSynchronize(opt.stream));
            return;
        }
        DeviceGuard guard(opt.device >= 0 ? opt.device : current_device());
        DeviceContext& ctx = device_context(current_device());
        std::lock_guard<std::mutex> lock(ctx.mu);
        cudaStream_t st = ctx.compute;
        const uint64_t np = batch * length * dimension, ns = batch * s.stride;
        Scratch buf((2 * np + 2 * ns + corr_elems) * sizeof(T), st);
        T* dp = buf.as<T>();
        T* dout = dp + np;
        T* dg = dout + np;
        T* dsig = dg + ns;
        T* dc = dsig + ns;
        SIG_CUDA_CHECK(cudaMemcpyAsync(dp, path, np * sizeof(T), cudaMemcpyHostToDevice, st));
        SIG_CUDA_CHECK(cudaMemcpyAsync(dg, sig_derivs, ns * sizeof(T), cudaMemcpyHostToDevice, st));
        SIG_CUDA_CHECK(cudaMemcpyAsync(dsig, sig, ns * sizeof(T), cudaMemcpyHostToDevice, st));
        SIG_CUDA_CHECK(cudaMemcpyAsync(dc, correction, corr_elems * sizeof(T), cudaMemcpyHostToDevice, st));
        CorrectionView<T> dcv = cv;
        dcv.ptr = dc;
        correction_backward_on_device<T>(dp, dout, dg, dsig, s, end_time, dcv, st);
        SIG_CUDA_CHECK(cudaMemcpyAsync(out, dout, np * sizeof(T), cudaMemcpyDeviceToHost, st));
        SIG_CUDA_CHECK(cudaStreamSynchronize(st));
        return;
    }

    const PointerInfo pout = classify_pointer(out);
    if (pout.on_device) {
        require_on_device({path}, pout.device, "sig_backprop_cuda");
        if (needs_sig) require_on_device({sig, sig_derivs}, pout.device, "sig_backprop_cuda");
        DeviceGuard guard(pout.device);
        backward_on_device<T>(path, out, sig_derivs, sig, s, end_time, opt.stream);
        if (opt.synchronize) SIG_CUDA_CHECK(cudaStreamSynchronize(opt.stream));
        return;
    }

    DeviceGuard guard(opt.device >= 0 ? opt.device : current_device());
    const uint64_t sig_bytes = needs_sig ? s.stride * sizeof(T) : 0;
    std::vector<HostOperand> ins{{path, s.data_len * s.data_dim * sizeof(T)}, {sig_derivs, sig_bytes}, {sig, sig_bytes}};
    run_host_pipeline(batch, ins, out, s.data_len * s.data_dim * sizeof(T), tile_wave_paths<T>(s, true),
        [&](const std::vector<void*>& din, void* dout, uint64_t count, cudaStream_t stream) {
            SigShape cs = s;
            cs.batch = count;
            backward_on_device<T>(static_cast<const T*>(din[0]), static_cast<T*>(dout),
                                  static_cast<const T*>(din[1]), static_cast<const T*>(din[2]), cs, end_time, stream);
        });
}

// Chen product of two batches of signatures.  Replaces siglib/cusig/cu_sig_combine.cu
// (sig_combine_cuda_): same buffers and layout; one thread per output coefficient.
template <typename T>
void sig_combine_entry(const T* sig1, const T* sig2, T* out, uint64_t batch, uint64_t dimension, uint64_t degree,
                       bool scalar_term, const CallOptions& opt) {
    if (dimension == 0) throw std::invalid_argument("sig_combine_cuda received dimension 0");
    if (batch == 0) return;
    const SigShape s = make_shape(batch, dimension, 2, degree, false, false, scalar_term);
    if (s.stride == 0) return;
    if (sig1 == nullptr || sig2 == nullptr || out == nullptr)
        throw std::invalid_argument("sig_combine_cuda received a null pointer");
    const uint64_t shift = scalar_term ? 1 : 0;
    auto run = [&](const T* a, const T* b, T* c, uint64_t count, cudaStream_t stream) {
        SigShape cs = s;
        cs.batch = count;
        if (degree == 0) launch_fill<T>(c, count * s.stride, T(1), stream);  // only the scalar term
        else launch_chen_product<T>(a + shift, s.stride, b + shift, s.stride, c + shift, s.stride, cs, stream, scalar_term);
    };
    const PointerInfo pout = classify_pointer(out);
    if (pout.on_device) {
        require_on_device({sig1, sig2}, pout.device, "sig_combine_cuda");
        DeviceGuard guard(pout.device);
        run(sig1, sig2, out, batch, opt.stream);
        if (opt.synchronize) SIG_CUDA_CHECK(cudaStreamSynchronize(opt.stream));
        return;
    }
    DeviceGuard guard(opt.device >= 0 ? opt.device : current_device());
    std::vector<HostOperand> ins{{sig1, s.stride * sizeof(T)}, {sig2, s.stride * sizeof(T)}};
    run_host_pipeline(batch, ins, out, s.stride * sizeof(T), 0,
        [&](const std::vector<void*>& din, void* dout, uint64_t count, cudaStream_t stream) {
            run(static_cast<const T*>(din[0]), static_cast<const T*>(din[1]), static_cast<T*>(dout), count, stream);
        });
}

// Backward of the Chen product.  Replaces siglib/cusig/cu_sig_combine.cu (sig_combine_backprop_cuda_):
// d sig1[u] = sum_v deriv[u v] sig2[v],  d sig2[v] = sum_u deriv[u v] sig1[u]; scalar slots get 0.
template <typename T>
void sig_combine_backprop_entry(const T* deriv, T* sig1_deriv, T* sig2_deriv, const T* sig1, const T* sig2,
                                uint64_t batch, uint64_t dimension, uint64_t degree, bool scalar_term,
                                const CallOptions& opt) {
    if (dimension == 0) throw std::invalid_argument("sig_combine_backprop_cuda received dimension 0");
    if (batch == 0) return;
    const SigShape s = make_shape(batch, dimension, 2, degree, false, false, scalar_term);
    if (s.stride == 0) return;
    if (!deriv || !sig1_deriv || !sig2_deriv || !sig1 || !sig2)
        throw std::invalid_argument("sig_combine_backprop_cuda received a null pointer");
    const uint64_t shift = scalar_term ? 1 : 0;
    const uint64_t n = batch * s.stride;
    auto run = [&](const T* dS, T* d1, T* d2, const T* a, const T* b, cudaStream_t stream) {
        if (scalar_term) {  // also clears the scalar slots; the kernels overwrite everything else
            SIG_CUDA_CHECK(cudaMemsetAsync(d1, 0, n * sizeof(T), stream));
            SIG_CUDA_CHECK(cudaMemsetAsync(d2, 0, n * sizeof(T), stream));
        }
        if (degree == 0) return;
        // big batches: both adjoints in one pass over the incoming gradient (sig_chen.cu)
        if (launch_chen_adjoints_streamed<T>(dS + shift, s.stride, a + shift, s.stride, b + shift, s.stride, d1 + shift,
                                             s.stride, d2 + shift, s.stride, s, stream))
            return;
        launch_chen_left_adjoint<T>(dS + shift, s.stride, b + shift, s.stride, d1 + shift, s.stride, s, stream);
        launch_chen_right_adjoint<T>(dS + shift, s.stride, a + shift, s.stride, d2 + shift, s.stride, s, stream);
    };
    const PointerInfo pout = classify_pointer(sig1_deriv);
    if (pout.on_device) {
        require_on_device({deriv, sig2_deriv, sig1, sig2}, pout.device, "sig_combine_backprop_cuda");
        DeviceGuard guard(pout.device);
        run(deriv, sig1_deriv, sig2_deriv, sig1, sig2, opt.stream);
        if (opt.synchronize) SIG_CUDA_CHECK(cudaStreamSynchronize(opt.stream));
        return;
    }
    // host buffers: these arrays are small next to a path batch, so one staged round trip
    DeviceGuard guard(opt.device >= 0 ? opt.device : current_device());
    DeviceContext& ctx = device_context(current_device());
    std::lock_guard<std::mutex> lock(ctx.mu);
    cudaStream_t st = ctx.compute;
    Scratch buf(5 * n * sizeof(T), st);
    T* d = buf.as<T>();
    SIG_CUDA_CHECK(cudaMemcpyAsync(d, deriv, n * sizeof(T), cudaMemcpyHostToDevice, st));
    SIG_CUDA_CHECK(cudaMemcpyAsync(d + n, sig1, n * sizeof(T), cudaMemcpyHostToDevice, st));
    SIG_CUDA_CHECK(cudaMemcpyAsync(d + 2 * n, sig2, n * sizeof(T), cudaMemcpyHostToDevice, st));
    run(d, d + 3 * n, d + 4 * n, d + n, d + 2 * n, st);
    SIG_CUDA_CHECK(cudaMemcpyAsync(sig1_deriv, d + 3 * n, n * sizeof(T), cudaMemcpyDeviceToHost, st));
    SIG_CUDA_CHECK(cudaMemcpyAsync(sig2_deriv, d + 4 * n, n * sizeof(T), cudaMemcpyDeviceToHost, st));
    SIG_CUDA_CHECK(cudaStreamSynchronize(st));
}

#define INSTANTIATE(T)                                                                                    \
    template void sig_combine_backprop_entry<T>(const T*, T*, T*, const T*, const T*, uint64_t, uint64_t, uint64_t, \
                                                bool, const CallOptions&);                                \
    template void sig_combine_entry<T>(const T*, const T*, T*, uint64_t, uint64_t, uint64_t, bool, const CallOptions&); \
    template void forward_on_device<T>(const T*, T*, const SigShape&, T, cudaStream_t, int*);             \
    template void backward_on_device<T>(const T*, T*, const T*, const T*, const SigShape&, T, cudaStream_t); \
    template void signature_entry<T>(const T*, T*, uint64_t, uint64_t, uint64_t, uint64_t, bool, bool, T, bool, \
                                     bool, const T*, uint64_t, const CallOptions&, uint64_t, uint64_t);   \
    template void sig_backprop_entry<T>(const T*, T*, const T*, const T*, uint64_t, uint64_t, uint64_t, uint64_t, \
                                        bool, bool, T, bool, const T*, uint64_t, const CallOptions&, uint64_t,    \
                                        uint64_t);
INSTANTIATE(float)
INSTANTIATE(double)
#undef INSTANTIATE

}  // namespace sigb200
