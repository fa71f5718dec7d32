// Register-resident FMA loop used by the benchmark to measure the FP32 / FP64 FMA-pipe
// peak of the device it runs on (the denominator of the roofline of this FMA-bound path).
// Built into its own small library (libsigb200_bench.so) that only bench.py loads; it is not
// part of libcusig.so.
#include <cuda_runtime.h>

namespace sigb200_bench {
namespace {

template <typename T>
__global__ void __launch_bounds__(256) fma_peak_kernel(T* sink, int iters, T a, T b) {
    T acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = T(threadIdx.x + i);
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[i] = acc[i] * a + b;
        }
    }
    T s = T(0);
#pragma unroll
    for (int i = 0; i < 16; ++i) s += acc[i];
    if (s == T(-1.2345)) sink[0] = s;  // never true; keeps the loop alive
}

// Same loop with the packed two-wide FP32 FMA of sm_100 (fma.rn.f32x2): one instruction
// performs two FMAs on a pair of registers.
__global__ void __launch_bounds__(256) fma2_peak_kernel(float* sink, int iters, float a, float b) {
    unsigned long long acc[8];
    unsigned long long aa, bb;
    asm("mov.b64 %0, {%1, %1};" : "=l"(aa) : "f"(a));
    asm("mov.b64 %0, {%1, %1};" : "=l"(bb) : "f"(b));
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float lo = float(threadIdx.x + i), hi = float(threadIdx.x + i + 8);
        asm("mov.b64 %0, {%1, %2};" : "=l"(acc[i]) : "f"(lo), "f"(hi));
    }
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                asm volatile("fma.rn.f32x2 %0, %0, %1, %2;" : "+l"(acc[i]) : "l"(aa), "l"(bb));
        }
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float lo, hi;
        asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(acc[i]));
        s += lo + hi;
    }
    if (s == -1.2345f) sink[0] = s;
}

}  // namespace
}  // namespace sigb200_bench

// Launches `blocks` CTAs of 256 threads, each thread issuing iters * 64 dependent-free
// FMAs (16 independent chains): FMAs per launch = blocks * 256 * iters * 64.
// mode 0: scalar float, 1: double, 2: packed float (same FMA count: 8 pair accumulators).
// `sink` is any 8-byte device buffer.  Asynchronous on `stream`; returns the cudaError_t of the launch.
extern "C" __attribute__((visibility("default")))
int sigb200_bench_fma_peak(int mode, void* sink, int blocks, int iters, void* stream) {
    using namespace sigb200_bench;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (mode == 2) fma2_peak_kernel<<<blocks, 256, 0, st>>>(static_cast<float*>(sink), iters, 0.999f, 0.001f);
    else if (mode == 1) fma_peak_kernel<double><<<blocks, 256, 0, st>>>(static_cast<double*>(sink), iters, 0.999, 0.001);
    else fma_peak_kernel<float><<<blocks, 256, 0, st>>>(static_cast<float*>(sink), iters, 0.999f, 0.001f);
    return static_cast<int>(cudaGetLastError());
}
