// Throughput of the packed FP32 FMA (fma.rn.f32x2) and of the scalar FMA under the operand
// patterns of the register-tile kernels, in SM cycles read with clock64 inside the kernel.
// Part of the benchmark helper library (libsigb200_bench.so), used by `bench.py --op fma_patterns`;
// not part of libcusig.so.
//
// Every thread keeps an 8 x 16 tile of accumulators (64 packed pairs), 16 "increment" values z and
// 8 "row factors" v in registers and repeats acc[j][c] += z[c] * v[j], the update of the deepest
// tile level of a forward sweep.  Patterns:
//   0  every instruction uses the same z pair and the same v pair (one register-fresh operand);
//   1  row by row, as the kernels do it (v reused over a row, z and the accumulator fresh);
//   2  column by column (z reused, v and the accumulator fresh);
//   3  no operand reused by consecutive instructions;
//   4  pattern 1 with scalar fma.rn.f32 (128 instructions instead of 64).
#include <cuda_runtime.h>

namespace sigb200_bench {
namespace {

typedef unsigned long long u64;
__device__ __forceinline__ u64 pack2(float a, float b) {
    u64 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ float sum2(u64 v) {
    float a, b;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
    return a + b;
}
#define SIGB200_FMA2(d, a, b) asm volatile("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(d) : "l"(a), "l"(b))

template <int MODE>
__global__ void __launch_bounds__(128, 1) pattern_kernel(float* sink, int iters, float a, float b, long long* cycles) {
    const long long t0 = clock64();
    float s = 0.f;
    if (MODE == 4) {
        float acc[8][16], z[16], v[8];
#pragma unroll
        for (int c = 0; c < 16; ++c) z[c] = a + c * 1e-3f + threadIdx.x * 1e-6f;
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = b + j * 1e-3f;
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int c = 0; c < 16; ++c) acc[j][c] = float(j + c);
        for (int it = 0; it < iters; ++it) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int c = 0; c < 16; ++c) asm volatile("fma.rn.f32 %0, %1, %2, %0;" : "+f"(acc[j][c]) : "f"(z[c]), "f"(v[j]));
        }
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int c = 0; c < 16; ++c) s += acc[j][c];
    } else {
        u64 acc[8][8], z[8], vv[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) z[c] = pack2(a + c * 1e-3f + threadIdx.x * 1e-6f, a - c * 1e-3f);
#pragma unroll
        for (int j = 0; j < 8; ++j) vv[j] = pack2(b + j * 1e-3f, b + j * 1e-3f);
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int c = 0; c < 8; ++c) acc[j][c] = pack2(float(j), float(c));
        for (int it = 0; it < iters; ++it) {
            if (MODE == 0) {
#pragma unroll
                for (int j = 0; j < 8; ++j)
#pragma unroll
                    for (int c = 0; c < 8; ++c) SIGB200_FMA2(acc[j][c], z[0], vv[0]);
            } else if (MODE == 1) {
#pragma unroll
                for (int j = 0; j < 8; ++j)
#pragma unroll
                    for (int c = 0; c < 8; ++c) SIGB200_FMA2(acc[j][c], z[c], vv[j]);
            } else if (MODE == 2) {
#pragma unroll
                for (int c = 0; c < 8; ++c)
#pragma unroll
                    for (int j = 0; j < 8; ++j) SIGB200_FMA2(acc[j][c], z[c], vv[j]);
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j)
#pragma unroll
                    for (int c = 0; c < 8; ++c) SIGB200_FMA2(acc[j][c], z[(c + j) % 8], vv[(j + c) % 8]);
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int c = 0; c < 8; ++c) s += sum2(acc[j][c]);
    }
    if (s == -1.2345f) sink[0] = s;  // never true; keeps the loop alive
    if (threadIdx.x == 0) cycles[blockIdx.x] = clock64() - t0;
}

}  // namespace
}  // namespace sigb200_bench

// Runs pattern `mode` with `blocks` CTAs of 128 threads (one warp per SM scheduler and CTA), each
// thread issuing iters * 128 FMAs; `cycles` receives one clock64 duration per CTA (device buffer of
// `blocks` long longs), `sink` is any 8-byte device buffer.  Returns the cudaError_t of the launch.
extern "C" __attribute__((visibility("default")))
int sigb200_bench_fma_pattern(int mode, void* sink, int blocks, int iters, long long* cycles, void* stream) {
    using namespace sigb200_bench;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    float* out = static_cast<float*>(sink);
    switch (mode) {
        case 0: pattern_kernel<0><<<blocks, 128, 0, st>>>(out, iters, 0.5f, 1e-4f, cycles); break;
        case 1: pattern_kernel<1><<<blocks, 128, 0, st>>>(out, iters, 0.5f, 1e-4f, cycles); break;
        case 2: pattern_kernel<2><<<blocks, 128, 0, st>>>(out, iters, 0.5f, 1e-4f, cycles); break;
        case 3: pattern_kernel<3><<<blocks, 128, 0, st>>>(out, iters, 0.5f, 1e-4f, cycles); break;
        default: pattern_kernel<4><<<blocks, 128, 0, st>>>(out, iters, 0.5f, 1e-4f, cycles); break;
    }
    return static_cast<int>(cudaGetLastError());
}
