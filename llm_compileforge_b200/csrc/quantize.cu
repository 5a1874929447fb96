// Stand-alone FP8-e4m3 quantise / dequantise of a whole tensor.
//
// Restates FP8KVCacheQuantizer.quantize_block / dequantize_block
// (compiler/quantize/fp8_kv_cache.py:66-105 of the reference): one scale per
// group, scale = amax/448 (1.0 when amax == 0, at least 1e-12), codes =
// e4m3(x.float() / scale), dequantised value = code.float() * scale.  A group is
// the whole tensor (the reference's only granularity) or one x[b, :, h, :] slice
// of a [NB, bs, Hkv, D] pool.  The serving path quantises inside the cache write
// (kv_append.cu); these kernels serve the `quantize` / `dequantize` operators.

#include "sfb_common.cuh"

namespace sfb {
namespace {

struct V4 {
    char* base;
    int64_t size[4];
    int64_t stride[4];
};

V4 pack(const View& v) {
    V4 o;
    o.base = v.base;
    for (int i = 0; i < 4; ++i) { o.size[i] = v.size[i]; o.stride[i] = v.stride[i]; }
    return o;
}

__device__ __forceinline__ float scale_rule(float amax, bool has_nan) {
    if (has_nan) return __int_as_float(0x7fc00000);
    if (amax == 0.f) return 1.0f;
    return fmaxf(__fdiv_rn(amax, 448.0f), 1e-12f);
}

__device__ __forceinline__ uint8_t encode1(float x, float scale) {
    return (uint8_t)(float2_to_e4m3x2(__fdiv_rn(x, scale), 0.f) & 0xff);
}

// one warp per (b, h) slice: rows = size[1], cols = size[3]
template <typename T>
__global__ void quantize_slices_kernel(V4 x, V4 codes, V4 scales) {
    const int64_t slice = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (slice >= x.size[0] * x.size[2]) return;
    const int64_t b = slice / x.size[2], h = slice - b * x.size[2];
    const T* src = reinterpret_cast<const T*>(x.base) + b * x.stride[0] + h * x.stride[2];
    uint8_t* dst = reinterpret_cast<uint8_t*>(codes.base) + b * codes.stride[0] + h * codes.stride[2];
    const int64_t rows = x.size[1], cols = x.size[3];
    float amax = 0.f;
    bool has_nan = false;
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t c = lane; c < cols; c += 32) {
            float v = fabsf(to_float(src[r * x.stride[1] + c]));
            amax = fmaxf(amax, v);
            has_nan |= (v != v);
        }
    amax = warp_max(amax);
    has_nan = __any_sync(0xffffffffu, has_nan);
    const float scale = scale_rule(amax, has_nan);
    if (lane == 0) reinterpret_cast<float*>(scales.base)[b * scales.stride[2] + h * scales.stride[3]] = scale;
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t c = lane; c < cols; c += 32)
            dst[r * codes.stride[1] + c] = encode1(to_float(src[r * x.stride[1] + c]), scale);
}

// whole-tensor amax: non-negative floats order like their bit patterns
template <typename T>
__global__ void tensor_amax_kernel(V4 x, unsigned int* amax_bits) {
    const int64_t n = x.size[0] * x.size[1] * x.size[2] * x.size[3];
    float amax = 0.f;
    bool has_nan = false;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t c = i % x.size[3], t = i / x.size[3];
        int64_t h = t % x.size[2]; t /= x.size[2];
        int64_t r = t % x.size[1], b = t / x.size[1];
        float v = fabsf(to_float(reinterpret_cast<const T*>(x.base)[b * x.stride[0] + r * x.stride[1] + h * x.stride[2] + c]));
        amax = fmaxf(amax, v);
        has_nan |= (v != v);
    }
    amax = warp_max(amax);
    has_nan = __any_sync(0xffffffffu, has_nan);
    if ((threadIdx.x & 31) == 0) atomicMax(amax_bits, has_nan ? 0x7fc00000u : __float_as_uint(amax));
}

template <typename T>
__global__ void tensor_encode_kernel(V4 x, V4 codes, const unsigned int* amax_bits) {
    const int64_t n = x.size[0] * x.size[1] * x.size[2] * x.size[3];
    const unsigned int bits = *amax_bits;
    const float scale = scale_rule(__uint_as_float(bits), bits > 0x7f800000u);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t c = i % x.size[3], t = i / x.size[3];
        int64_t h = t % x.size[2]; t /= x.size[2];
        int64_t r = t % x.size[1], b = t / x.size[1];
        float v = to_float(reinterpret_cast<const T*>(x.base)[b * x.stride[0] + r * x.stride[1] + h * x.stride[2] + c]);
        reinterpret_cast<uint8_t*>(codes.base)[b * codes.stride[0] + r * codes.stride[1] + h * codes.stride[2] + c] = encode1(v, scale);
    }
}

__global__ void amax_to_scale_kernel(float* slot) {
    const unsigned int bits = __float_as_uint(*slot);
    *slot = scale_rule(__uint_as_float(bits), bits > 0x7f800000u);
}

template <typename T>
__global__ void dequantize_kernel(V4 codes, V4 scales, V4 out, int per_slice) {
    const int64_t n = out.size[0] * out.size[1] * out.size[2] * out.size[3];
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t c = i % out.size[3], t = i / out.size[3];
        int64_t h = t % out.size[2]; t /= out.size[2];
        int64_t r = t % out.size[1], b = t / out.size[1];
        const float s = per_slice ? reinterpret_cast<const float*>(scales.base)[b * scales.stride[2] + h * scales.stride[3]]
                                  : reinterpret_cast<const float*>(scales.base)[0];
        const uint8_t code = reinterpret_cast<const uint8_t*>(codes.base)[b * codes.stride[0] + r * codes.stride[1] + h * codes.stride[2] + c];
        reinterpret_cast<T*>(out.base)[b * out.stride[0] + r * out.stride[1] + h * out.stride[2] + c] =
            from_float<T>(e4m3_to_float(code) * s);
    }
}

int grid_for(int64_t n, int threads) {
    int64_t blocks = (n + threads - 1) / threads;
    const int64_t cap = 148 * 16;
    return (int)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

template <typename T>
int quantize_t(const View& x, const View& codes, const View& scales, int granularity, cudaStream_t stream) {
    V4 vx = pack(x), vc = pack(codes), vs = pack(scales);
    if (granularity == SFB_QUANT_PER_BLOCK_HEAD) {
        const int64_t slices = x.size[0] * x.size[2];
        const int warps = 4;
        quantize_slices_kernel<T><<<(unsigned)ceil_div(slices, warps), warps * 32, 0, stream>>>(vx, vc, vs);
    } else {
        unsigned int* slot = reinterpret_cast<unsigned int*>(scales.base);
        SFB_CUDA_CHECK(cudaMemsetAsync(slot, 0, 4, stream));
        const int g = grid_for(x.numel(), 256);
        tensor_amax_kernel<T><<<g, 256, 0, stream>>>(vx, slot);
        tensor_encode_kernel<T><<<g, 256, 0, stream>>>(vx, vc, slot);
        amax_to_scale_kernel<<<1, 1, 0, stream>>>(reinterpret_cast<float*>(slot));
    }
    SFB_CUDA_CHECK(cudaGetLastError());
    return SFB_OK;
}

template <typename T>
int dequantize_t(const View& codes, const View& scales, const View& out, int granularity, cudaStream_t stream) {
    dequantize_kernel<T><<<grid_for(out.numel(), 256), 256, 0, stream>>>(pack(codes), pack(scales), pack(out),
                                                                         granularity == SFB_QUANT_PER_BLOCK_HEAD);
    SFB_CUDA_CHECK(cudaGetLastError());
    return SFB_OK;
}

}  // namespace

int launch_quantize(const View& x, const View& codes, const View& scales, int x_dtype, int granularity, cudaStream_t stream) {
    switch (x_dtype) {
        case SFB_F32: return quantize_t<float>(x, codes, scales, granularity, stream);
        case SFB_BF16: return quantize_t<__nv_bfloat16>(x, codes, scales, granularity, stream);
        case SFB_F16: return quantize_t<__half>(x, codes, scales, granularity, stream);
    }
    return fail(SFB_ERR_INVALID_ARG, "quantize: dtype %d", x_dtype);
}

int launch_dequantize(const View& codes, const View& scales, const View& out, int out_dtype, int granularity,
                      cudaStream_t stream) {
    switch (out_dtype) {
        case SFB_F32: return dequantize_t<float>(codes, scales, out, granularity, stream);
        case SFB_BF16: return dequantize_t<__nv_bfloat16>(codes, scales, out, granularity, stream);
        case SFB_F16: return dequantize_t<__half>(codes, scales, out, granularity, stream);
    }
    return fail(SFB_ERR_INVALID_ARG, "dequantize: dtype %d", out_dtype);
}

}  // namespace sfb
