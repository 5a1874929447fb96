// KV cache write and FP8 quantise-on-append.
//
// Slot rule restated from python_runtime/engine/cache_manager.py:154-159 of the
// reference: token at position p of a request goes to (table[p / bs], p % bs).
// Quantiser restated from compiler/quantize/fp8_kv_cache.py:81-89, applied to
// every touched (block, kv_head) slice: amax over the slice (unwritten slots
// count as zero), scale = amax/448 (1.0 when amax == 0, at least 1e-12),
// codes = e4m3(x / scale) with an IEEE division.
//
// One warp owns one (block, kv_head) slice: it pulls the slice's rows with
// 128-bit loads (rows that precede this call's tokens come from the request's
// unquantised tail copy, rows after them are zero), keeps them in registers,
// reduces |x| with shuffles, then writes codes, scale and - while the block is
// still open - the refreshed tail copy.  Single pass over the source; bound:
// HBM bandwidth.

#include "sfb_common.cuh"

namespace sfb {
namespace {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;

template <typename T>
struct Src;  // 16-byte chunk of the source dtype
template <>
struct Src<float> {
    static constexpr int N = 4;
    __device__ static void unpack(const uint4& r, float* o) {
        o[0] = __uint_as_float(r.x); o[1] = __uint_as_float(r.y);
        o[2] = __uint_as_float(r.z); o[3] = __uint_as_float(r.w);
    }
};
template <>
struct Src<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ static void unpack(const uint4& r, float* o) {
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            o[2 * i] = __uint_as_float(w[i] << 16);
            o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};
template <>
struct Src<__half> {
    static constexpr int N = 8;
    __device__ static void unpack(const uint4& r, float* o) {
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            o[2 * i] = f.x; o[2 * i + 1] = f.y;
        }
    }
};

// scale rule of fp8_kv_cache.py:81-86 (NaN in the slice makes the scale NaN,
// as torch's max / clamp do)
__device__ __forceinline__ float scale_from_amax(float amax, bool has_nan) {
    if (has_nan) return __int_as_float(0x7fc00000);
    if (amax == 0.f) return 1.0f;
    return fmaxf(__fdiv_rn(amax, 448.0f), 1e-12f);
}

// N source values -> N codes packed little-endian into 32-bit words
template <int N>
__device__ __forceinline__ void encode(const float* x, float scale, uint32_t* words) {
#pragma unroll
    for (int i = 0; i < N / 4; ++i) {
        uint16_t lo = float2_to_e4m3x2(__fdiv_rn(x[4 * i], scale), __fdiv_rn(x[4 * i + 1], scale));
        uint16_t hi = float2_to_e4m3x2(__fdiv_rn(x[4 * i + 2], scale), __fdiv_rn(x[4 * i + 3], scale));
        words[i] = (uint32_t)lo | ((uint32_t)hi << 16);
    }
}

// CPL = 16-byte source chunks each lane keeps; a slice has bs * D / N chunks.
template <typename ST, int CPL, bool FP8>
__global__ void __launch_bounds__(kThreads) cache_write_kernel(AppendArgs a, int blk_offset) {
    constexpr int N = Src<ST>::N;
    const int req = blockIdx.y, which = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bs = a.block_size, dim = a.head_dim;
    const int n_new = a.cu_tokens[req + 1] - a.cu_tokens[req];
    if (n_new <= 0) return;
    const int start = a.start_pos[req], end = start + n_new;
    const int blk = start / bs + blk_offset + blockIdx.x;
    if (blk > (end - 1) / bs || blk >= a.max_blocks) return;
    const int64_t phys = a.tables[(int64_t)req * a.table_stride + blk];
    if (phys < 0 || phys >= a.n_pool_blocks) return;
    const int lo = blk * bs;

    const ST* src = reinterpret_cast<const ST*>(which ? a.v_new : a.k_new) + (int64_t)a.cu_tokens[req] * (which ? a.vnew_stride[0] : a.new_stride[0]);
    const int64_t src_tok = which ? a.vnew_stride[0] : a.new_stride[0];
    const int64_t src_head = which ? a.vnew_stride[1] : a.new_stride[1];
    const int64_t* ps = which ? a.v_stride : a.k_stride;
    const int cpr = dim / N;            // chunks per row
    const int n_chunks = bs * cpr;

    if constexpr (!FP8) {
        ST* pool = reinterpret_cast<ST*>(which ? a.v_cache : a.k_cache) + phys * ps[0];
        for (int h = warp; h < a.n_kv_heads; h += kWarps)
            for (int i = lane; i < n_chunks; i += 32) {
                int t = i / cpr, c = i - t * cpr, p = lo + t;
                if (p >= start && p < end) {
                    uint4 v = *reinterpret_cast<const uint4*>(src + (int64_t)(p - start) * src_tok + h * src_head + c * N);
                    *reinterpret_cast<uint4*>(pool + t * ps[1] + h * ps[2] + c * N) = v;
                }
            }
        return;
    } else {
        uint8_t* pool = reinterpret_cast<uint8_t*>(which ? a.v_cache : a.k_cache) + phys * ps[0];
        float* scales = which ? a.v_scale : a.k_scale;
        const int64_t* ss = which ? a.vs_stride : a.ks_stride;
        ST* tail = reinterpret_cast<ST*>(which ? a.v_tail : a.k_tail);
        const int64_t* ts = which ? a.vt_stride : a.kt_stride;
        tail += (int64_t)req * ts[0];
        const bool still_open = end < lo + bs;  // this block keeps free slots after the call

        for (int h = warp; h < a.n_kv_heads; h += kWarps) {
            uint4 raw[CPL];
            float amax = 0.f;
            bool has_nan = false;
#pragma unroll
            for (int j = 0; j < CPL; ++j) {
                const int i = lane + 32 * j;
                raw[j] = make_uint4(0, 0, 0, 0);
                if (i < n_chunks) {
                    int t = i / cpr, c = i - t * cpr, p = lo + t;
                    if (p < start) raw[j] = *reinterpret_cast<const uint4*>(tail + t * ts[1] + h * ts[2] + c * N);
                    else if (p < end) raw[j] = ldg_stream(src + (int64_t)(p - start) * src_tok + h * src_head + c * N);
                    float x[N];
                    Src<ST>::unpack(raw[j], x);
#pragma unroll
                    for (int e = 0; e < N; ++e) {
                        float v = fabsf(x[e]);
                        amax = fmaxf(amax, v);
                        has_nan |= (v != v);
                    }
                }
            }
            amax = warp_max(amax);
            has_nan = __any_sync(0xffffffffu, has_nan);
            const float scale = scale_from_amax(amax, has_nan);
            if (lane == 0) scales[phys * ss[0] + h * ss[1]] = scale;
#pragma unroll
            for (int j = 0; j < CPL; ++j) {
                const int i = lane + 32 * j;
                if (i < n_chunks) {
                    int t = i / cpr, c = i - t * cpr;
                    float x[N];
                    Src<ST>::unpack(raw[j], x);
                    uint32_t words[N / 4];
                    encode<N>(x, scale, words);
                    uint8_t* dst = pool + t * ps[1] + h * ps[2] + c * N;
                    if constexpr (N == 8) *reinterpret_cast<uint2*>(dst) = make_uint2(words[0], words[1]);
                    else *reinterpret_cast<uint32_t*>(dst) = words[0];
                    if (still_open) *reinterpret_cast<uint4*>(tail + t * ts[1] + h * ts[2] + c * N) = raw[j];
                }
            }
        }
    }
}

template <typename ST, bool FP8>
int launch_t(const AppendArgs& a, cudaStream_t stream) {
    constexpr int N = Src<ST>::N;
    const int n_chunks = a.block_size * a.head_dim / N;
    const int cpl = (n_chunks + 31) / 32;
    // a request that appends n tokens starting mid-block touches at most this many blocks
    const int touched = (a.max_new_tokens + a.block_size - 2) / a.block_size + 1;
    if (a.batch > 65535) return fail(SFB_ERR_UNSUPPORTED, "cache_write: batch %d exceeds the grid limit 65535", a.batch);
    if (cpl > 32) return fail(SFB_ERR_UNSUPPORTED, "cache_write: a (block, head) slice of %d x %d elements is too large", a.block_size, a.head_dim);
    // Two launches: the first touched block of every request reads the tail copy,
    // the last one rewrites it; stream order keeps the read before the write when
    // an append spans several blocks.
    for (int pass = 0; pass < 2; ++pass) {
        const int count = pass == 0 ? 1 : touched - 1;
        if (count <= 0) continue;
        dim3 grid((unsigned)count, (unsigned)a.batch, 2);
        if (!FP8 || cpl <= 4) cache_write_kernel<ST, 4, FP8><<<grid, kThreads, 0, stream>>>(a, pass);
        else if (cpl <= 8) cache_write_kernel<ST, 8, FP8><<<grid, kThreads, 0, stream>>>(a, pass);
        else if (cpl <= 16) cache_write_kernel<ST, 16, FP8><<<grid, kThreads, 0, stream>>>(a, pass);
        else cache_write_kernel<ST, 32, FP8><<<grid, kThreads, 0, stream>>>(a, pass);
        SFB_CUDA_CHECK(cudaGetLastError());
    }
    return SFB_OK;
}

}  // namespace

int launch_cache_write(const AppendArgs& a, cudaStream_t stream) {
    const bool fp8 = a.kv_dtype == SFB_F8E4M3;
    switch (a.src_dtype) {
        case SFB_F32: return fp8 ? launch_t<float, true>(a, stream) : launch_t<float, false>(a, stream);
        case SFB_BF16: return fp8 ? launch_t<__nv_bfloat16, true>(a, stream) : launch_t<__nv_bfloat16, false>(a, stream);
        case SFB_F16: return fp8 ? launch_t<__half, true>(a, stream) : launch_t<__half, false>(a, stream);
    }
    return fail(SFB_ERR_INVALID_ARG, "cache_write: source dtype %d", a.src_dtype);
}

}  // namespace sfb
