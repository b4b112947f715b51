// Register-resident micro-benchmarks of the two pipes that bound the Palimpsa kernels on sm_100a:
// FP32 FMA (scalar and packed f32x2 issue) and the MUFU reciprocal.  Built into its own small
// library (libpalimpsa_microbench.so); the benchmark driver uses it to measure the compute
// ceilings on the GPU it runs on, because the driver-provided peak file only has HBM and bf16
// tensor figures.  Not part of the operator's ABI.
#include <cuda_runtime.h>

namespace {

constexpr int CH = 8;  // independent dependency chains per thread

__global__ void k_fma_scalar(float* sink, int iters) {
    float a[CH], m = 1.0000001f, c = 1e-9f;
#pragma unroll
    for (int i = 0; i < CH; ++i) a[i] = threadIdx.x * 1e-6f + i;
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int i = 0; i < CH; ++i) a[i] = fmaf(a[i], m, c);
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < CH; ++i) s += a[i];
    if (s == 123.456f) sink[0] = s;
}

__global__ void k_fma_packed(float* sink, int iters) {
    float2 a[CH], m = make_float2(1.0000001f, 0.9999999f), c = make_float2(1e-9f, 2e-9f);
#pragma unroll
    for (int i = 0; i < CH; ++i) a[i] = make_float2(threadIdx.x * 1e-6f + i, i);
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int i = 0; i < CH; ++i) a[i] = __ffma2_rn(a[i], m, c);
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < CH; ++i) s += a[i].x + a[i].y;
    if (s == 123.456f) sink[0] = s;
}

__device__ __forceinline__ float rcpa(float x) {
    float r;
    asm volatile("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

__global__ void k_rcp(float* sink, int iters) {
    float a[CH];
#pragma unroll
    for (int i = 0; i < CH; ++i) a[i] = 1.5f + threadIdx.x * 1e-3f + i;
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int i = 0; i < CH; ++i) a[i] = rcpa(a[i] + 0.25f);  // the add keeps the chain from collapsing
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < CH; ++i) s += a[i];
    if (s == 123.456f) sink[0] = s;
}

// The forward kernel's instruction mix per pair of state elements: 6 packed FP32 + 2 reciprocals.
__global__ void k_fwd_mix(float* sink, int iters) {
    float2 M[CH], I[CH], acc = make_float2(0.f, 0.f);
    const float2 f = make_float2(0.999f, 0.999f), vk = make_float2(1e-3f, 2e-3f), b = make_float2(0.5f, 0.5f),
                 kk = make_float2(1e-3f, 1e-3f), c = make_float2(1e-3f, 1e-3f), q = make_float2(0.1f, 0.2f);
#pragma unroll
    for (int i = 0; i < CH; ++i) {
        M[i] = make_float2(threadIdx.x * 1e-6f, i);
        I[i] = make_float2(1.f + i, 2.f);
    }
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int i = 0; i < CH; ++i) {
            M[i] = __ffma2_rn(f, M[i], __fmul2_rn(vk, q));
            I[i] = __ffma2_rn(f, I[i], __ffma2_rn(b, kk, c));
            const float2 r = make_float2(rcpa(I[i].x), rcpa(I[i].y));
            acc = __ffma2_rn(__fmul2_rn(M[i], r), q, acc);
        }
    }
    if (acc.x + acc.y == 123.456f) sink[0] = acc.x;
}

}  // namespace

// kind: 0 scalar FMA, 1 packed FMA, 2 reciprocal, 3 forward mix.  Runs `reps` launches of
// blocks x 256 threads and returns the best launch time in milliseconds through *ms; *ops gets the
// per-launch operation count (FMA lane-ops for 0/1, reciprocals for 2, state-element updates for 3).
extern "C" int palimpsa_microbench(int kind, int blocks, int iters, int reps, float* sink, float* ms, double* ops) {
    cudaEvent_t e0, e1;
    if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return -1;
    float best = 1e30f;
    for (int r = 0; r < reps + 1; ++r) {
        cudaEventRecord(e0);
        switch (kind) {
            case 0: k_fma_scalar<<<blocks, 256>>>(sink, iters); break;
            case 1: k_fma_packed<<<blocks, 256>>>(sink, iters); break;
            case 2: k_rcp<<<blocks, 256>>>(sink, iters); break;
            default: k_fwd_mix<<<blocks, 256>>>(sink, iters); break;
        }
        if (cudaGetLastError() != cudaSuccess) return -3;
        cudaEventRecord(e1);
        if (cudaEventSynchronize(e1) != cudaSuccess) return -2;
        float t;
        cudaEventElapsedTime(&t, e0, e1);
        if (r > 0 && t < best) best = t;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    const double thr = (double)blocks * 256.0 * iters * CH;
    *ops = kind == 0 ? thr : kind == 1 ? 2.0 * thr : kind == 2 ? thr : 2.0 * thr;
    *ms = best;
    return 0;
}
