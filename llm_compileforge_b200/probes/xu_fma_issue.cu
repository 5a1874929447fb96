// Stand-alone micro-measurements behind the prefill kernel's softmax design (sm_100a):
//   1. cycles per warp instruction of ex2.approx.f32 / ex2.approx.f16x2 / ex2.approx.ftz.bf16x2
//   2. how many independent FFMA issue in the shadow of one ex2 (1 ex2 + K fma per step)
//   3. the softmax second-pass body (FFMA2, 2 x ex2, FADD2, bf16x2 pack per pair of scores) on register data
// each with 1, 2 and 4 warps per SM sub-partition, 148 thread blocks, clock64 around the loop of block 0.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o xu_fma_issue llm_compileforge_b200/probes/xu_fma_issue.cu
//   ./xu_fma_issue
//
// Not part of libsfb.so; nothing in the package calls it.

#include <cstdint>
#include <cstdio>
#include <cuda_runtime.h>

__device__ __forceinline__ float ex2f(float x) { float r; asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x)); return r; }
__device__ __forceinline__ float ex2f_pure(float x) { float r; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x)); return r; }
__device__ __forceinline__ uint32_t ex2h2(uint32_t x) { uint32_t r; asm volatile("ex2.approx.f16x2 %0, %1;" : "=r"(r) : "r"(x)); return r; }
__device__ __forceinline__ uint32_t ex2b2(uint32_t x) { uint32_t r; asm volatile("ex2.approx.ftz.bf16x2 %0, %1;" : "=r"(r) : "r"(x)); return r; }
__device__ __forceinline__ uint32_t packbf(float lo, float hi) { uint32_t r; asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo)); return r; }

constexpr int kIters = 200;

// MODE 0..2: one kind of ex2 per step.  MODE 10 + K: 1 ex2.f32 + K independent FFMA per step.
template <int MODE>
__global__ void step_kernel(float* out, long long* cyc, float a, float b) {
    float v[32], w[32];
    uint32_t u[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) { v[i] = a * (threadIdx.x + i); w[i] = b * (threadIdx.x + 2 * i); u[i] = threadIdx.x * 77 + i; }
    __syncthreads();
    const long long t0 = clock64();
    for (int it = 0; it < kIters; ++it) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            if (MODE == 0 || MODE >= 10) v[i] = ex2f(v[i]);
            if (MODE == 1) u[i] = ex2h2(u[i]);
            if (MODE == 2) u[i] = ex2b2(u[i]);
#pragma unroll
            for (int j = 0; j < (MODE >= 10 ? MODE - 10 : 0); ++j) w[(i + j * 5) & 31] = fmaf(w[(i + j * 5) & 31], a, b);
        }
    }
    const long long t1 = clock64();
    float s = 0;
#pragma unroll
    for (int i = 0; i < 32; ++i) s += v[i] + w[i] + __uint_as_float(u[i]);
    out[blockIdx.x * blockDim.x + threadIdx.x] = s;
    if (threadIdx.x == 0 && blockIdx.x == 0) *cyc = t1 - t0;
}

// The second pass of the prefill softmax over 64 scores per thread, fed by its own results.
__global__ void softmax_body_kernel(float* out, long long* cyc, float sl2, float negm) {
    float v[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) v[i] = 0.01f * i + 0.001f * (threadIdx.x & 31);
    float acc = 0.f;
    uint32_t sink = 0;
    __syncthreads();
    const long long t0 = clock64();
    for (int it = 0; it < kIters; ++it) {
        const float2 s2 = make_float2(sl2, sl2), nm = make_float2(negm, negm);
        float2 a0 = make_float2(0, 0), a1 = make_float2(0, 0);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const float2 x = __ffma2_rn(make_float2(v[2 * i], v[2 * i + 1]), s2, nm);
            const float2 p = make_float2(ex2f_pure(x.x), ex2f_pure(x.y));
            if (i & 1) a1 = __fadd2_rn(a1, p);
            else a0 = __fadd2_rn(a0, p);
            sink ^= packbf(p.x, p.y);
            v[2 * i] = p.x;
            v[2 * i + 1] = p.y;
        }
        acc += a0.x + a0.y + a1.x + a1.y;
    }
    const long long t1 = clock64();
    out[blockIdx.x * blockDim.x + threadIdx.x] = acc + __uint_as_float(sink);
    if (threadIdx.x == 0 && blockIdx.x == 0) *cyc = t1 - t0;
}

template <typename Launch>
static double cycles(Launch launch, long long* cyc) {
    launch();
    cudaDeviceSynchronize();
    launch();
    cudaDeviceSynchronize();
    long long c = 0;
    cudaMemcpy(&c, cyc, 8, cudaMemcpyDeviceToHost);
    return (double)c;
}

template <int MODE>
static void run_step(const char* name, float* out, long long* cyc) {
    for (int warps : {4, 8, 16}) {
        const double c = cycles([&] { step_kernel<MODE><<<148, warps * 32>>>(out, cyc, 0.999f, 0.001f); }, cyc);
        printf("%-34s %d warp(s) per sub-partition: %6.2f clk per step per warp slot\n", name, warps / 4, c / kIters / 32 / (warps / 4));
    }
}

int main() {
    float* out;
    long long* cyc;
    cudaMalloc(&out, 148 * 512 * 4);
    cudaMalloc(&cyc, 8);
    run_step<0>("ex2.approx.ftz.f32", out, cyc);
    run_step<1>("ex2.approx.f16x2", out, cyc);
    run_step<2>("ex2.approx.ftz.bf16x2", out, cyc);
    run_step<12>("1 ex2 + 2 fma", out, cyc);
    run_step<14>("1 ex2 + 4 fma", out, cyc);
    run_step<16>("1 ex2 + 6 fma", out, cyc);
    run_step<18>("1 ex2 + 8 fma", out, cyc);
    for (int warps : {4, 8, 16}) {
        const double c = cycles([&] { softmax_body_kernel<<<148, warps * 32>>>(out, cyc, 0.127f, -3.f); }, cyc);
        printf("softmax second-pass body, %d warp(s) per sub-partition: %.0f clk per 64 scores per thread = %.0f per 128 ex2 warp instructions (XU floor 1024)\n",
               warps / 4, c / kIters, c / kIters / (warps / 4) * 2);
    }
    printf("status %s\n", cudaGetErrorString(cudaDeviceSynchronize()));
    return 0;
}
