// Paged-attention decode, shape-generic CUDA-core kernel (template body; the
// decode_generic_*.cu files instantiate it per dtype pair to build in parallel).
//
// This kernel takes every supported dtype / head_dim / GQA ratio / stride
// pattern.  It is the path for float32 pools (config "opt-125m fp32", where the
// 1e-5 tolerance needs true float32 products) and the fallback for shapes the
// TMA + tensor-core kernel (decode_tma.cu) does not cover.
//
// Algorithm restated from kernels/paged_attention.py:36-71 of the reference as
// a split-K online softmax: thread block = (chunk of the KV length, kv head,
// request); each warp walks whole 16-token blocks of its chunk through the
// block table, stages K and V as float32 in shared memory with 128-bit loads,
// and keeps a running (max, denominator, numerator) per query head of the GQA
// group.  Bound: HBM bandwidth.

#pragma once
#include "sfb_common.cuh"

namespace sfb {
namespace generic {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kMaxGroup = 16;   // query heads per kv head
constexpr int kMaxDimSlots = 8; // head_dim <= 256 (32 columns per slot)
constexpr float kLog2e = 1.4426950408889634f;

template <typename T>
struct Vec16;  // 16-byte vector of T -> floats
template <>
struct Vec16<float> {
    static constexpr int N = 4;
    __device__ static void unpack(const uint4& r, float* o) {
        o[0] = __uint_as_float(r.x); o[1] = __uint_as_float(r.y);
        o[2] = __uint_as_float(r.z); o[3] = __uint_as_float(r.w);
    }
};
template <>
struct Vec16<__nv_bfloat16> {
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
struct Vec16<__half> {
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
template <>
struct Vec16<uint8_t> {  // e4m3 codes
    static constexpr int N = 16;
    __device__ static void unpack(const uint4& r, float* o) {
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)((w[i] >> (16 * j)) & 0xffffu), __NV_E4M3);
                float2 f = __half22float2(*reinterpret_cast<__half2*>(&h));
                o[4 * i + 2 * j] = f.x; o[4 * i + 2 * j + 1] = f.y;
            }
        }
    }
};

template <typename QT>
__device__ __forceinline__ float load_q(const void* p, int64_t i) { return to_float(reinterpret_cast<const QT*>(p)[i]); }

// Stage one [bs, D] tile (row stride `tok_stride` elements) as float32 rows of
// `ld` floats.  Rows >= n_valid are zero-filled.
template <typename KV>
__device__ __forceinline__ void stage_tile(const KV* src, int64_t tok_stride, int bs, int n_valid, int dim, float* dst,
                                           int ld, int lane) {
    constexpr int N = Vec16<KV>::N;
    const int vec_per_row = dim / N;
    const int total = bs * vec_per_row;
    for (int i = lane; i < total; i += 32) {
        int row = i / vec_per_row, c = i - row * vec_per_row;
        float vals[N];
        if (row < n_valid) {
            uint4 raw = ldg_stream(src + row * tok_stride + c * N);
            Vec16<KV>::unpack(raw, vals);
        } else {
#pragma unroll
            for (int j = 0; j < N; ++j) vals[j] = 0.f;
        }
        float* d = dst + row * ld + c * N;
#pragma unroll
        for (int j = 0; j < N; ++j) d[j] = vals[j];
    }
}

template <typename QT, typename KV, int GMAX, int DSLOTS>
__global__ void __launch_bounds__(kThreads) decode_generic_kernel(DecodeArgs a) {
    extern __shared__ float smem[];
    const int chunk = blockIdx.x, kvh = blockIdx.y, req = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int dim = a.head_dim, bs = a.block_size;
    const int group = a.n_heads / a.n_kv_heads;
    const int n_chunks = (int)a.split.n_chunks;
    int* status = a.workspace ? reinterpret_cast<int*>(a.workspace) : nullptr;

    int len = a.seq_lens[req];
    const int cap = a.max_blocks * bs;
    if (len > cap) len = cap;
    const int h0 = kvh * group;
    QT* out = reinterpret_cast<QT*>(a.out);

    if (len <= 0) {
        if (chunk == 0) {
            if (status && threadIdx.x == 0) atomicOr(status, SFB_STATUS_EMPTY_REQUEST);
            for (int i = threadIdx.x; i < group * dim; i += kThreads)
                out[req * a.out_stride[0] + (h0 + i / dim) * a.out_stride[1] + i % dim] = from_float<QT>(0.f);
        }
        return;
    }
    const int tok_begin = chunk * (int)a.split.chunk_tokens;
    if (tok_begin >= len) return;
    const int tok_end = min(len, tok_begin + (int)a.split.chunk_tokens);
    const int blk_begin = tok_begin / bs, blk_end = (tok_end + bs - 1) / bs;

    // shared memory carve-up
    const int ldk = dim + 1;
    float* q_s = smem;                                   // [group][dim], pre-multiplied by scale*log2e
    float* warp_base = q_s + group * dim;
    const int per_warp = bs * ldk + bs * dim + group * bs + 2 * group;
    float* k_s = warp_base + warp * per_warp;            // [bs][ldk]
    float* v_s = k_s + bs * ldk;                         // [bs][dim]
    float* p_s = v_s + bs * dim;                         // [group][bs]
    float* corr_s = p_s + group * bs;                    // [group]

    const float qscale = a.scale * kLog2e;
    for (int i = threadIdx.x; i < group * dim; i += kThreads) {
        int g = i / dim, d = i - g * dim;
        q_s[i] = load_q<QT>(a.q, req * a.q_stride[0] + (h0 + g) * a.q_stride[1] + d) * qscale;
    }
    __syncthreads();

    // per-warp running state: lanes g < group own (m, l) of query head g
    float m_run = -INFINITY, l_run = 0.f;
    float acc[GMAX][DSLOTS];
#pragma unroll
    for (int g = 0; g < GMAX; ++g)
#pragma unroll
        for (int i = 0; i < DSLOTS; ++i) acc[g][i] = 0.f;

    const int32_t* table = a.tables + decode_table_row(a, req, status) * a.table_stride;
    const KV* kbase = reinterpret_cast<const KV*>(a.k);
    const KV* vbase = reinterpret_cast<const KV*>(a.v);

    for (int blk = blk_begin + warp; blk < blk_end; blk += kWarps) {
        const int64_t phys = table[blk];
        if (phys < 0 || phys >= a.n_pool_blocks) {
            if (status && lane == 0) atomicOr(status, SFB_STATUS_BAD_BLOCK_ID);
            continue;
        }
        const int n_valid = min(bs, tok_end - blk * bs);
        stage_tile<KV>(kbase + phys * a.k_stride[0] + kvh * a.k_stride[2], a.k_stride[1], bs, n_valid, dim, k_s, ldk, lane);
        stage_tile<KV>(vbase + phys * a.v_stride[0] + kvh * a.v_stride[2], a.v_stride[1], bs, n_valid, dim, v_s, dim, lane);
        float ksc = 1.f, vsc = 1.f;
        if (a.k_scale) {
            ksc = a.k_scale[phys * a.ks_stride[0] + kvh * a.ks_stride[1]];
            vsc = a.v_scale[phys * a.vs_stride[0] + kvh * a.vs_stride[1]];
        }
        __syncwarp();

        // scores: (g, t) pairs, bs*group of them, 32 per pass
        for (int base = 0; base < group * bs; base += 32) {
            int idx = base + lane;
            int g = idx / bs, t = idx - g * bs;
            float s = -INFINITY;
            if (g < group && t < n_valid) {
                const float* kr = k_s + t * ldk;
                const float* qr = q_s + g * dim;
                float sum = 0.f;
                for (int d = 0; d < dim; ++d) sum = fmaf(qr[d], kr[d], sum);
                s = sum * ksc;
            }
            if (g < group) p_s[g * bs + t] = s;
        }
        __syncwarp();
        // online softmax per query head: lane g owns head g
        if (lane < group) {
            float mx = m_run;
            for (int t = 0; t < n_valid; ++t) mx = fmaxf(mx, p_s[lane * bs + t]);
            float corr = exp2f(m_run - mx);  // m_run = -inf on the first tile gives 0
            float sum = 0.f;
            for (int t = 0; t < bs; ++t) {
                float p = t < n_valid ? exp2f(p_s[lane * bs + t] - mx) : 0.f;
                sum += p;
                p_s[lane * bs + t] = p * vsc;
            }
            l_run = l_run * corr + sum;
            m_run = mx;
            corr_s[lane] = corr;
        }
        __syncwarp();
        // numerator: lane owns columns lane, lane+32, ...
#pragma unroll
        for (int g = 0; g < GMAX; ++g) {
            if (g < group) {
                const float corr = corr_s[g];
#pragma unroll
                for (int i = 0; i < DSLOTS; ++i) {
                    int d = lane + 32 * i;
                    if (d < dim) {
                        float s = acc[g][i] * corr;
                        for (int t = 0; t < n_valid; ++t) s = fmaf(p_s[g * bs + t], v_s[t * dim + d], s);
                        acc[g][i] = s;
                    }
                }
            }
        }
        __syncwarp();
    }

    // merge the warps of this block through shared memory (reuse the staging area)
    __syncthreads();
    float* red_o = warp_base;                        // [kWarps][group][dim]
    float* red_ml = red_o + kWarps * group * dim;    // [kWarps][group][2]
#pragma unroll
    for (int g = 0; g < GMAX; ++g)
        if (g < group)
#pragma unroll
            for (int i = 0; i < DSLOTS; ++i) {
                int d = lane + 32 * i;
                if (d < dim) red_o[(warp * group + g) * dim + d] = acc[g][i];
            }
    if (lane < group) {
        red_ml[(warp * group + lane) * 2] = m_run;
        red_ml[(warp * group + lane) * 2 + 1] = l_run;
    }
    __syncthreads();
    float* part_ml = reinterpret_cast<float*>(a.workspace + a.split.ml_offset);
    float* part_o = reinterpret_cast<float*>(a.workspace + a.split.o_offset);
    for (int i = threadIdx.x; i < group * dim; i += kThreads) {
        int g = i / dim, d = i - g * dim;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) m = fmaxf(m, red_ml[(w * group + g) * 2]);
        float l = 0.f, o = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            float mw = red_ml[(w * group + g) * 2];
            float f = mw == -INFINITY ? 0.f : exp2f(mw - m);
            l += red_ml[(w * group + g) * 2 + 1] * f;
            o += red_o[(w * group + g) * dim + d] * f;
        }
        if (n_chunks == 1) {
            out[req * a.out_stride[0] + (h0 + g) * a.out_stride[1] + d] = from_float<QT>(l > 0.f ? o / l : 0.f);
        } else {
            int64_t slot = ((int64_t)req * n_chunks + chunk) * a.n_heads + h0 + g;
            part_o[slot * dim + d] = o;
            if (d == 0) { part_ml[slot * 2] = m; part_ml[slot * 2 + 1] = l; }
        }
    }
}

template <typename QT, typename KV, int GMAX, int DSLOTS>
int launch_generic_gd(const DecodeArgs& a, cudaStream_t stream) {
    const int group = a.n_heads / a.n_kv_heads;
    const int per_warp = a.block_size * (a.head_dim + 1) + a.block_size * a.head_dim + group * a.block_size + 2 * group;
    int64_t floats = (int64_t)group * a.head_dim + (int64_t)kWarps * per_warp;
    int64_t red = (int64_t)kWarps * group * a.head_dim + kWarps * group * 2;
    if (red > (int64_t)kWarps * per_warp) floats = (int64_t)group * a.head_dim + red;
    size_t smem = (size_t)floats * 4;
    if (smem > 200 * 1024) return fail(SFB_ERR_UNSUPPORTED, "decode: shared memory need %zu B exceeds the limit", smem);
    auto kern = decode_generic_kernel<QT, KV, GMAX, DSLOTS>;
    SFB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((unsigned)a.split.n_chunks, (unsigned)a.n_kv_heads, (unsigned)a.batch);
    kern<<<grid, kThreads, smem, stream>>>(a);
    SFB_CUDA_CHECK(cudaGetLastError());
    return SFB_OK;
}

template <typename QT, typename KV, int GMAX>
int launch_generic_g(const DecodeArgs& a, cudaStream_t stream) {
    if (a.head_dim <= 128) return launch_generic_gd<QT, KV, GMAX, 4>(a, stream);
    return launch_generic_gd<QT, KV, GMAX, 8>(a, stream);
}

template <typename QT, typename KV>
int launch_generic_t(const DecodeArgs& a, cudaStream_t stream) {
    const int group = a.n_heads / a.n_kv_heads;
    if (group <= 1) return launch_generic_g<QT, KV, 1>(a, stream);
    if (group <= 4) return launch_generic_g<QT, KV, 4>(a, stream);
    if (group <= 8) return launch_generic_g<QT, KV, 8>(a, stream);
    return launch_generic_g<QT, KV, 16>(a, stream);
}

}  // namespace generic

// one definition per dtype pair, each in its own translation unit
int launch_decode_generic_f32(const DecodeArgs& a, cudaStream_t stream);
int launch_decode_generic_bf16(const DecodeArgs& a, cudaStream_t stream);
int launch_decode_generic_f16(const DecodeArgs& a, cudaStream_t stream);
int launch_decode_generic_bf16_e4m3(const DecodeArgs& a, cudaStream_t stream);
int launch_decode_generic_f16_e4m3(const DecodeArgs& a, cudaStream_t stream);

}  // namespace sfb
