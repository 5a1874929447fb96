// Paged-attention decode for callers that cannot hand over a workspace.
//
// Some hosts of this library have no way to allocate device memory when they
// reach the decode call: a serving runtime that gave every free byte of HBM to
// its KV block pool at start-up has nothing left for cudaMalloc to return, and a
// thin dlopen-style host (the reference's Rust HAL passes through only the
// buffers the compiled model declares) has no allocator binding at all.  For
// them the split-K scratch lives in this library's own image: a fixed
// file-scope device array that every GPU loading the library carries until the
// process exits.

#include <mutex>

#include "sfb_common.cuh"

namespace {

// Split-K partials + status word of sfb_paged_attention_decode_static.
static __device__ __align__(256) unsigned char g_static_scratch[SFB_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_ptr[kMaxDevices] = {};

// The array's name is only a host-side handle; kernels need its device address,
// which differs per GPU.  Looked up once per device, with that device current.
int scratch_for_current_device(void** out) {
    int dev = -1;
    SFB_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return sfb::fail(SFB_ERR_UNSUPPORTED, "decode_static: device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_ptr[dev]) {
        void* ptr = nullptr;
        SFB_CUDA_CHECK(cudaGetSymbolAddress(&ptr, g_static_scratch));
        if (!ptr) return sfb::fail(SFB_ERR_CUDA, "decode_static: cudaGetSymbolAddress returned a null address");
        g_scratch_ptr[dev] = ptr;
    }
    *out = g_scratch_ptr[dev];
    return SFB_OK;
}

}  // namespace

extern "C" int sfb_paged_attention_decode_static(const SFBTensor* q, const SFBTensor* k_cache, const SFBTensor* v_cache,
                                                 const SFBTensor* k_scale, const SFBTensor* v_scale,
                                                 const SFBTensor* block_tables, const SFBTensor* seq_lens, const SFBTensor* table_rows,
                                                 SFBTensor* out, int q_dtype, int kv_dtype, float scale, int64_t chunk_tokens,
                                                 void* stream) {
    if (!q || !k_cache || !block_tables) return sfb::fail(SFB_ERR_INVALID_ARG, "decode_static: q, k_cache and block_tables are required");
    if (q->rank != 3 || k_cache->rank != 4 || block_tables->rank != 2)
        return sfb::fail(SFB_ERR_INVALID_ARG, "decode_static: q must be rank 3, k_cache rank 4, block_tables rank 2");
    const int64_t need = sfb_paged_attention_workspace_bytes(q->r3.sizes[0], q->r3.sizes[1], q->r3.sizes[2],
                                                             block_tables->r2.sizes[1], k_cache->r4.sizes[1], chunk_tokens);
    if (need < 0) return sfb::fail(SFB_ERR_INVALID_ARG, "decode_static: invalid shapes");
    if (need > (int64_t)SFB_STATIC_SCRATCH_BYTES)
        return sfb::fail(SFB_ERR_WORKSPACE,
                         "decode_static: this call needs %lld B of split scratch but the built-in array holds %lld B; "
                         "use sfb_paged_attention_decode with a caller workspace, or a larger chunk_tokens",
                         (long long)need, (long long)SFB_STATIC_SCRATCH_BYTES);
    void* scratch = nullptr;
    int rc = scratch_for_current_device(&scratch);
    if (rc) return rc;
    // The regular entry point zeroes the status word (the only part of the scratch
    // that must start clean; partials are fully overwritten before they are read).
    return sfb_paged_attention_decode(q, k_cache, v_cache, k_scale, v_scale, block_tables, seq_lens, table_rows, out, q_dtype, kv_dtype,
                                      scale, chunk_tokens, scratch, SFB_STATIC_SCRATCH_BYTES, stream);
}

extern "C" int sfb_read_status_static(int32_t* bits, void* stream) {
    void* scratch = nullptr;
    int rc = scratch_for_current_device(&scratch);
    if (rc) return rc;
    return sfb_read_status(scratch, bits, stream);
}
