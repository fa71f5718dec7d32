// Register-resident FMA loop used by the benchmark to measure the FP32 / FP64 FMA-pipe
// peak of the device it runs on (the denominator of the roofline of this FMA-bound path).
#include "../../include/cusig_b200.h"
#include "common.h"
#include "runtime.h"

namespace sigb200 {
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

template <typename T>
void run_fma_peak(void* sink, int blocks, int iters, cudaStream_t stream) {
    fma_peak_kernel<T><<<blocks, 256, 0, stream>>>(static_cast<T*>(sink), iters, T(0.999), T(0.001));
    SIG_CUDA_CHECK(cudaGetLastError());
    count_launch();
}

// packed f32x2 variant: same FMA count per thread (8 pair accumulators x 4 x iters x 2)
void run_fma2_peak(void* sink, int blocks, int iters, cudaStream_t stream) {
    fma2_peak_kernel<<<blocks, 256, 0, stream>>>(static_cast<float*>(sink), iters, 0.999f, 0.001f);
    SIG_CUDA_CHECK(cudaGetLastError());
    count_launch();
}

}  // namespace
}  // namespace sigb200

// Launches `blocks` CTAs of 256 threads, each thread issuing iters * 64 dependent-free
// FMAs (16 independent chains).  FMAs per launch = blocks * 256 * iters * 64.
extern "C" __attribute__((visibility("default")))
int sigb200_fma_peak(int is_double, void* sink, int blocks, int iters, void* stream) {
    SIG_SAFE_CALL(
        if (is_double == 2) sigb200::run_fma2_peak(sink, blocks, iters, static_cast<cudaStream_t>(stream));
        else if (is_double) sigb200::run_fma_peak<double>(sink, blocks, iters, static_cast<cudaStream_t>(stream));
        else sigb200::run_fma_peak<float>(sink, blocks, iters, static_cast<cudaStream_t>(stream)));
}
