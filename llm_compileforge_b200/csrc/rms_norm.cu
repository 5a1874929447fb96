// RMSNorm, optionally fused with a residual add.
//
// Restates the HAL operator `rms_norm`
// (python_runtime/hal/pytorch_backend/_ops_norm.py:30-45 of the reference) and
// the fused form kernels/rms_norm.py:26-29: s = x (+ residual);
// out = s * rsqrt(mean(s^2) + eps) * weight, float32 arithmetic, one rounding to
// the storage dtype at the end.
//
// One thread block per row.  The row is read once with 128-bit loads, held in
// registers across the reduction and written once: algorithmic traffic only
// (rows*hidden*(in+out) + hidden for the weight, which stays in L2).  Rows longer
// than the register budget, or not 16-byte tileable, take a two-pass scalar path.
// Bound: HBM bandwidth.

#include <type_traits>

#include "sfb_common.cuh"

namespace sfb {
namespace {

constexpr int kThreads = 128;   // small blocks: many rows resident per SM keeps more loads in flight
constexpr int kMaxChunks = 16;  // 16-byte chunks per thread held in registers (template-selected)

template <typename T>
struct Pack;  // 16 bytes of T
template <>
struct Pack<float> {
    static constexpr int N = 4;
    __device__ static void unpack(const uint4& r, float* o) {
        o[0] = __uint_as_float(r.x); o[1] = __uint_as_float(r.y); o[2] = __uint_as_float(r.z); o[3] = __uint_as_float(r.w);
    }
    __device__ static uint4 pack(const float* o) {
        return make_uint4(__float_as_uint(o[0]), __float_as_uint(o[1]), __float_as_uint(o[2]), __float_as_uint(o[3]));
    }
};
template <>
struct Pack<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ static void unpack(const uint4& r, float* o) {
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) { o[2 * i] = __uint_as_float(w[i] << 16); o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
    }
    __device__ static uint4 pack(const float* o) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 p = __floats2bfloat162_rn(o[2 * i], o[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&p);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
};
template <>
struct Pack<__half> {
    static constexpr int N = 8;
    __device__ static void unpack(const uint4& r, float* o) {
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            o[2 * i] = f.x; o[2 * i + 1] = f.y;
        }
    }
    __device__ static uint4 pack(const float* o) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __half2 p = __floats2half2_rn(o[2 * i], o[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&p);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
};

__device__ __forceinline__ float block_sum(float v, float* scratch) {
    v = warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = lane < (kThreads / 32) ? scratch[lane] : 0.f;
    t = warp_sum(t);
    __syncthreads();
    return t;
}

template <typename T, bool RES, int CH>
__global__ void __launch_bounds__(kThreads) rms_norm_vec_kernel(NormArgs a) {
    constexpr int N = Pack<T>::N;
    __shared__ float scratch[kThreads / 32];
    const int64_t row = blockIdx.x;
    const T* x = reinterpret_cast<const T*>(a.x) + row * a.x_stride;
    const T* res = RES ? reinterpret_cast<const T*>(a.residual) + row * a.res_stride : nullptr;
    T* out = reinterpret_cast<T*>(a.out) + row * a.out_stride;
    const T* w = reinterpret_cast<const T*>(a.weight);
    const int n_chunks = (int)(a.hidden / N);
    // The row stays in registers as the raw 16-byte words (and the residual's, when there is one): half the registers
    // of the unpacked floats, so more rows are in flight per SM; unpacking twice costs a few ALU instructions.
    uint4 raw[CH], rraw[RES ? CH : 1];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < CH; ++j) {
        const int c = threadIdx.x + j * kThreads;
        if (c < n_chunks) {
            raw[j] = ldg_stream(x + (int64_t)c * N);
            if (RES) rraw[j] = ldg_stream(res + (int64_t)c * N);
        }
    }
#pragma unroll
    for (int j = 0; j < CH; ++j) {
        const int c = threadIdx.x + j * kThreads;
        if (c < n_chunks) {
            float v[N];
            Pack<T>::unpack(raw[j], v);
            if (RES) {
                float r[N];
                Pack<T>::unpack(rraw[j], r);
#pragma unroll
                for (int e = 0; e < N; ++e) v[e] += r[e];
            }
#pragma unroll
            for (int e = 0; e < N; ++e) ss = fmaf(v[e], v[e], ss);
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = __frcp_rn(__fsqrt_rn(__fdiv_rn(ss, (float)a.hidden) + a.eps));  // torch: 1 / sqrt(mean + eps)
#pragma unroll
    for (int j = 0; j < CH; ++j) {
        const int c = threadIdx.x + j * kThreads;
        if (c < n_chunks) {
            float v[N], o[N];
            Pack<T>::unpack(raw[j], v);
            if (RES) {
                float r[N];
                Pack<T>::unpack(rraw[j], r);
#pragma unroll
                for (int e = 0; e < N; ++e) v[e] += r[e];
            }
            if (w) {
                float wv[N];
                uint4 wr = *reinterpret_cast<const uint4*>(w + (int64_t)c * N);
                Pack<T>::unpack(wr, wv);
#pragma unroll
                for (int e = 0; e < N; ++e) o[e] = v[e] * inv * wv[e];
            } else {
#pragma unroll
                for (int e = 0; e < N; ++e) o[e] = v[e] * inv;
            }
            *reinterpret_cast<uint4*>(out + (int64_t)c * N) = Pack<T>::pack(o);
        }
    }
}

template <typename T, bool RES>
__global__ void __launch_bounds__(kThreads) rms_norm_scalar_kernel(NormArgs a) {
    __shared__ float scratch[kThreads / 32];
    const int64_t row = blockIdx.x;
    const T* x = reinterpret_cast<const T*>(a.x) + row * a.x_stride;
    const T* res = RES ? reinterpret_cast<const T*>(a.residual) + row * a.res_stride : nullptr;
    T* out = reinterpret_cast<T*>(a.out) + row * a.out_stride;
    const T* w = reinterpret_cast<const T*>(a.weight);
    float ss = 0.f;
    for (int64_t i = threadIdx.x; i < a.hidden; i += kThreads) {
        float v = to_float(x[i]);
        if (RES) v += to_float(res[i]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = __frcp_rn(__fsqrt_rn(__fdiv_rn(ss, (float)a.hidden) + a.eps));  // torch: 1 / sqrt(mean + eps)
    for (int64_t i = threadIdx.x; i < a.hidden; i += kThreads) {
        float v = to_float(x[i]);
        if (RES) v += to_float(res[i]);
        v *= inv;
        if (w) v *= to_float(w[i]);
        out[i] = from_float<T>(v);
    }
}

template <typename T>
int launch_t(const NormArgs& a, cudaStream_t stream) {
    constexpr int N = Pack<T>::N;
    auto al = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    const int64_t eb = sizeof(T);
    bool vec = a.hidden % N == 0 && a.hidden / N <= (int64_t)kThreads * kMaxChunks && al(a.x) && al(a.out) &&
               (a.x_stride * eb) % 16 == 0 && (a.out_stride * eb) % 16 == 0 && (!a.weight || al(a.weight)) &&
               (!a.residual || (al(a.residual) && (a.res_stride * eb) % 16 == 0));
    if (a.rows > 0x7fffffffLL) return fail(SFB_ERR_UNSUPPORTED, "rms_norm: too many rows");
    dim3 grid((unsigned)a.rows);
    if (vec) {
        const int ch = (int)ceil_div(a.hidden / N, kThreads);
        auto go = [&](auto ch_c) {
            constexpr int CH = decltype(ch_c)::value;
            if (a.residual) rms_norm_vec_kernel<T, true, CH><<<grid, kThreads, 0, stream>>>(a);
            else rms_norm_vec_kernel<T, false, CH><<<grid, kThreads, 0, stream>>>(a);
        };
        if (ch <= 1) go(std::integral_constant<int, 1>{});
        else if (ch <= 2) go(std::integral_constant<int, 2>{});
        else if (ch <= 4) go(std::integral_constant<int, 4>{});
        else if (ch <= 8) go(std::integral_constant<int, 8>{});
        else go(std::integral_constant<int, 16>{});
    } else {
        if (a.residual) rms_norm_scalar_kernel<T, true><<<grid, kThreads, 0, stream>>>(a);
        else rms_norm_scalar_kernel<T, false><<<grid, kThreads, 0, stream>>>(a);
    }
    SFB_CUDA_CHECK(cudaGetLastError());
    return SFB_OK;
}

}  // namespace

int launch_rms_norm(const NormArgs& a, cudaStream_t stream) {
    switch (a.dtype) {
        case SFB_F32: return launch_t<float>(a, stream);
        case SFB_BF16: return launch_t<__nv_bfloat16>(a, stream);
        case SFB_F16: return launch_t<__half>(a, stream);
    }
    return fail(SFB_ERR_INVALID_ARG, "rms_norm: dtype %d", a.dtype);
}

}  // namespace sfb
