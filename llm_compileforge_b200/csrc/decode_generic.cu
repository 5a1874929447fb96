// Paged-attention decode: dispatch of the shape-generic kernel and the split
// combine kernel shared by both decode kernels.
#include "decode_generic.cuh"

namespace sfb {
namespace {

// One thread block per (request, query head): merges the chunk partials.
template <typename QT>
__global__ void decode_combine_kernel(DecodeArgs a) {
    const int req = blockIdx.x / a.n_heads, h = blockIdx.x % a.n_heads;
    const int n_chunks = (int)a.split.n_chunks;
    int len = a.seq_lens[req];
    const int cap = a.max_blocks * a.block_size;
    if (len > cap) len = cap;
    if (len <= 0) return;  // the decode kernel already zero-filled the row
    const int used = (len + (int)a.split.chunk_tokens - 1) / (int)a.split.chunk_tokens;
    const float* part_ml = reinterpret_cast<const float*>(a.workspace + a.split.ml_offset);
    const float* part_o = reinterpret_cast<const float*>(a.workspace + a.split.o_offset);
    const int64_t slot0 = ((int64_t)req * n_chunks) * a.n_heads + h;
    float m = -INFINITY;
    for (int c = 0; c < used; ++c) m = fmaxf(m, part_ml[(slot0 + (int64_t)c * a.n_heads) * 2]);
    float l = 0.f;
    for (int c = 0; c < used; ++c) {
        const float* ml = part_ml + (slot0 + (int64_t)c * a.n_heads) * 2;
        l += ml[0] == -INFINITY ? 0.f : ml[1] * exp2f(ml[0] - m);
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    QT* out = reinterpret_cast<QT*>(a.out) + req * a.out_stride[0] + h * a.out_stride[1];
    for (int d = threadIdx.x; d < a.head_dim; d += blockDim.x) {
        float o = 0.f;
        for (int c = 0; c < used; ++c) {
            int64_t slot = slot0 + (int64_t)c * a.n_heads;
            float mc = part_ml[slot * 2];
            if (mc != -INFINITY) o += part_o[slot * a.head_dim + d] * exp2f(mc - m);
        }
        out[d] = from_float<QT>(o * inv);
    }
}

// Packed prefill tokens -> one decode row each: token i of request r sits at position
// ctx_len - n_q + i and attends to position + 1 tokens through request r's table row
// (or to its own `row_limits` entry of tokens, when those are given).
__global__ void prefill_expand_kernel(const int32_t* cu_q, const int32_t* ctx_lens, const int32_t* row_limits, int n_requests,
                                      int max_tokens_cap, int causal, int32_t* rows_out, int32_t* lens_out) {
    const int req = blockIdx.y;
    const int begin = cu_q[req], n_q = cu_q[req + 1] - begin;
    int ctx = ctx_lens[req];
    if (ctx > max_tokens_cap) ctx = max_tokens_cap;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_q; i += gridDim.x * blockDim.x) {
        rows_out[begin + i] = req;
        // <= 0 (inconsistent request, or a row that may see nothing) is flagged by the decode kernel and gives a zero row
        lens_out[begin + i] = row_limits ? min(row_limits[begin + i], ctx) : causal ? ctx - n_q + i + 1 : ctx;
    }
}

}  // namespace

int launch_prefill_expand(const int32_t* cu_q, const int32_t* ctx_lens, const int32_t* row_limits, int n_requests, int64_t total_q,
                          int max_blocks, int block_size, int causal, int32_t* rows_out, int32_t* lens_out, cudaStream_t stream) {
    (void)total_q;
    dim3 grid(8, (unsigned)n_requests);
    prefill_expand_kernel<<<grid, 256, 0, stream>>>(cu_q, ctx_lens, row_limits, n_requests, max_blocks * block_size, causal, rows_out, lens_out);
    SFB_CUDA_CHECK(cudaGetLastError());
    return SFB_OK;
}

int launch_decode_generic(const DecodeArgs& a, cudaStream_t stream) {
    const int group = a.n_heads / a.n_kv_heads;
    if (group > generic::kMaxGroup) return fail(SFB_ERR_UNSUPPORTED, "decode: %d query heads per kv head (max %d)", group, generic::kMaxGroup);
    if (a.head_dim > 32 * generic::kMaxDimSlots) return fail(SFB_ERR_UNSUPPORTED, "decode: head_dim %d > %d", a.head_dim, 32 * generic::kMaxDimSlots);
    if (a.block_size > 32) return fail(SFB_ERR_UNSUPPORTED, "decode: block_size %d > 32", a.block_size);
    if (a.n_kv_heads > 65535 || a.batch > 65535)
        return fail(SFB_ERR_UNSUPPORTED, "decode: batch %d / kv heads %d exceed the grid limit 65535", a.batch, a.n_kv_heads);
    switch (a.kv_dtype) {
        case SFB_F32: return launch_decode_generic_f32(a, stream);
        case SFB_BF16: return launch_decode_generic_bf16(a, stream);
        case SFB_F16: return launch_decode_generic_f16(a, stream);
        case SFB_F8E4M3:
            if (a.q_dtype == SFB_BF16) return launch_decode_generic_bf16_e4m3(a, stream);
            if (a.q_dtype == SFB_F16) return launch_decode_generic_f16_e4m3(a, stream);
            return fail(SFB_ERR_UNSUPPORTED, "decode: e4m3 pools need a bf16 or fp16 query");
    }
    return fail(SFB_ERR_INVALID_ARG, "decode: kv dtype %d", a.kv_dtype);
}
int launch_decode_combine(const DecodeArgs& a, cudaStream_t stream) {
    if (a.split.n_chunks <= 1) return SFB_OK;
    dim3 grid((unsigned)(a.batch * a.n_heads));
    int threads = a.head_dim <= 64 ? 64 : 128;
    switch (a.q_dtype) {
        case SFB_F32: decode_combine_kernel<float><<<grid, threads, 0, stream>>>(a); break;
        case SFB_BF16: decode_combine_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>(a); break;
        case SFB_F16: decode_combine_kernel<__half><<<grid, threads, 0, stream>>>(a); break;
        default: return fail(SFB_ERR_INVALID_ARG, "decode: q dtype %d", a.q_dtype);
    }
    SFB_CUDA_CHECK(cudaGetLastError());
    return SFB_OK;
}

}  // namespace sfb
