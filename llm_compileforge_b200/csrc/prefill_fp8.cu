// Chunked prefill over an e4m3 KV pool.
//
// The pool keeps FP8 codes with one fp32 scale per (block, kv head) (compiler/quantize/fp8_kv_cache.py:66-140 of the
// reference, applied per slice); a prompt's later chunks attend to earlier ones that are already stored that way.  The
// tensor-core prefill kernel wants 16-bit operands, so the blocks a batch attends to are first expanded into a compact
// scratch pool [R * max_blocks, 16, Hkv, D] of the query's 16-bit type (value = code * scale, one rounding; every e4m3
// value is exact in bf16 and fp16, the scale multiplication is what rounds) with identity tables, and the ordinary
// prefill runs on that.  One pass of 1 byte read + 2 bytes written per attended element, small beside the attention
// itself; blocks that a request shares with request 0 at the same table position (a common prompt prefix) are expanded
// once.  Bad block ids are flagged and expand to zeros.

#include "sfb_common.cuh"

namespace sfb {
namespace {

struct ExpandArgs {
    const uint8_t* codes[2];   // K, V pools
    const float* scales[2];
    void* scratch[2];
    const int32_t* tables;
    const int32_t* ctx_lens;
    int32_t* tables_out;       // identity tables over the scratch pool
    int64_t table_stride;
    int64_t pool_stride[3];    // block, token, head (bytes = elements)
    int64_t scale_stride[2];   // block, head
    int max_blocks, n_kv_heads, head_dim;
    int64_t n_pool_blocks;
    int* status;
};

template <typename T>
__global__ void __launch_bounds__(256) expand_fp8_blocks_kernel(ExpandArgs a) {
    const int b = blockIdx.x, r = blockIdx.y, which = blockIdx.z;
    int ctx = a.ctx_lens[r];
    if (ctx > a.max_blocks * 16) ctx = a.max_blocks * 16;
    const int used = (ctx + 15) >> 4;
    const int64_t slot = (int64_t)r * a.max_blocks + b;
    const int64_t phys = b < used ? (int64_t)a.tables[(int64_t)r * a.table_stride + b] : -1;
    // A block that request 0 holds at the same table position (a radix-shared prefix, runtime/src/cache/block.rs:214-232:
    // the same physical ids head every table) is expanded once, by request 0; the other requests' tables point at its copy.
    bool shared = false;
    if (r > 0 && b < used) {
        int ctx0 = a.ctx_lens[0];
        if (ctx0 > a.max_blocks * 16) ctx0 = a.max_blocks * 16;
        shared = b < ((ctx0 + 15) >> 4) && a.tables[b] == phys;
    }
    if (which == 0 && threadIdx.x == 0) a.tables_out[slot] = shared ? b : (int32_t)slot;
    if (b >= used || shared) return;  // never read by the attention / already there
    const bool ok = phys >= 0 && phys < a.n_pool_blocks;
    if (!ok && a.status && threadIdx.x == 0) atomicOr(a.status, SFB_STATUS_BAD_BLOCK_ID);
    const int cpr = a.head_dim / 16;                 // 16-code pieces per (token, head) row
    const int pieces = 16 * a.n_kv_heads * cpr;
    T* dst = reinterpret_cast<T*>(a.scratch[which]) + slot * 16 * a.n_kv_heads * a.head_dim;
    for (int i = threadIdx.x; i < pieces; i += blockDim.x) {
        const int c = i % cpr, h = (i / cpr) % a.n_kv_heads, t = i / (cpr * a.n_kv_heads);
        uint4 out0 = make_uint4(0, 0, 0, 0), out1 = out0;
        if (ok) {
            const uint4 raw = *reinterpret_cast<const uint4*>(a.codes[which] + phys * a.pool_stride[0] + t * a.pool_stride[1] + h * a.pool_stride[2] + c * 16);
            const float s = a.scales[which][phys * a.scale_stride[0] + h * a.scale_stride[1]];
            const uint8_t* code = reinterpret_cast<const uint8_t*>(&raw);
            T* o0 = reinterpret_cast<T*>(&out0);
            T* o1 = reinterpret_cast<T*>(&out1);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                o0[j] = from_float<T>(e4m3_to_float(code[j]) * s);
                o1[j] = from_float<T>(e4m3_to_float(code[8 + j]) * s);
            }
        }
        uint4* p = reinterpret_cast<uint4*>(dst + ((int64_t)t * a.n_kv_heads + h) * a.head_dim + c * 16);
        p[0] = out0;
        p[1] = out1;
    }
}

}  // namespace

int launch_expand_fp8_blocks(const void* k_codes, const void* v_codes, const float* k_scale, const float* v_scale, void* k_scratch,
                             void* v_scratch, const int32_t* tables, int64_t table_stride, const int32_t* ctx_lens, int32_t* tables_out,
                             const int64_t* pool_stride, const int64_t* scale_stride, int n_requests, int max_blocks, int n_kv_heads,
                             int head_dim, int64_t n_pool_blocks, int dtype, int* status, cudaStream_t stream) {
    ExpandArgs a{};
    a.codes[0] = static_cast<const uint8_t*>(k_codes); a.codes[1] = static_cast<const uint8_t*>(v_codes);
    a.scales[0] = k_scale; a.scales[1] = v_scale;
    a.scratch[0] = k_scratch; a.scratch[1] = v_scratch;
    a.tables = tables; a.ctx_lens = ctx_lens; a.tables_out = tables_out; a.table_stride = table_stride;
    for (int i = 0; i < 3; ++i) a.pool_stride[i] = pool_stride[i];
    a.scale_stride[0] = scale_stride[0]; a.scale_stride[1] = scale_stride[1];
    a.max_blocks = max_blocks; a.n_kv_heads = n_kv_heads; a.head_dim = head_dim; a.n_pool_blocks = n_pool_blocks; a.status = status;
    const dim3 grid((unsigned)max_blocks, (unsigned)n_requests, 2);
    if (dtype == SFB_BF16) expand_fp8_blocks_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(a);
    else expand_fp8_blocks_kernel<__half><<<grid, 256, 0, stream>>>(a);
    SFB_CUDA_CHECK(cudaGetLastError());
    return SFB_OK;
}

}  // namespace sfb
