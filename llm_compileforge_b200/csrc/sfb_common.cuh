// Shared host/device helpers for libsfb.so (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/sfb.h"

namespace sfb {

// ---------------------------------------------------------------------------
// Host side: error text per calling thread, descriptor views.
// ---------------------------------------------------------------------------
void set_error(const char* fmt, ...);
int fail(int status, const char* fmt, ...);

#define SFB_CUDA_CHECK(expr)                                                          \
    do {                                                                              \
        cudaError_t err__ = (expr);                                                   \
        if (err__ != cudaSuccess)                                                     \
            return ::sfb::fail(SFB_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(err__)); \
    } while (0)

// Opt-in to more than 48 KB of dynamic shared memory for `kernel` on the calling thread's current device.  The
// attribute is per kernel AND device, so it is made on a kernel's first launch on each device (not once per
// process, which breaks the second device of a multi-device host; not on every call either).
int allow_shared_memory_once(const void* kernel, int smem_bytes);

// A descriptor flattened to rank 4 (leading dimensions of size 1, stride 0).
struct View {
    char* base = nullptr;  // element 0
    int rank = 0;
    int elem = 0;
    int64_t size[4] = {1, 1, 1, 1};
    int64_t stride[4] = {0, 0, 0, 0};  // elements
    int64_t numel() const { return size[0] * size[1] * size[2] * size[3]; }
};

// Fills `v` from `t`; checks device, rank range and element size.  `what` names
// the argument in the error text.
int make_view(const SFBTensor* t, const char* what, int min_rank, int max_rank, int elem_size, View* v);

inline int dtype_size(int dt) {
    switch (dt) {
        case SFB_F32: return 4;
        case SFB_BF16: return 2;
        case SFB_F16: return 2;
        case SFB_F8E4M3: return 1;
        default: return 0;
    }
}

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// One stderr line per operator call when the environment has SFB_TRACE=1 (host time of the call: validation and
// enqueue) or SFB_TRACE=2 (the stream is synchronised first, so the time covers the kernels too - it serialises the
// stream, for debugging only).  The counterpart of the reference's per-step ledger (SERVEFORGE_ACCOUNT,
// runtime/src/engine/account.rs:1-60) at the granularity this library has: one operator.
int trace_level();
struct TraceScope {
    const char* op;
    cudaStream_t stream;
    char what[96];
    double t0;
    TraceScope(const char* op_name, void* st, const char* fmt, ...);
    ~TraceScope();
};
#define SFB_TRACE_OP(name, stream, ...) ::sfb::TraceScope sfb_trace_scope__(name, stream, __VA_ARGS__)

// ---------------------------------------------------------------------------
// Workspace layout of the decode path (shared by the kernels and the size query):
//   [0, 256)                     status word + padding
//   done    [B][Hkv]             int32 arrival counters (chunks finished per request and kv-head group)
//   part_ml [B][n_chunks][H][2]  float32 (running max in log2 units, denominator)
//   part_o  [B][n_chunks][H][D]  float32 (unnormalised numerator)
// ---------------------------------------------------------------------------
constexpr int64_t kWorkspaceHeader = 256;
constexpr int64_t kDefaultChunkTokens = 512;

struct DecodeSplit {
    int64_t chunk_tokens;
    int64_t n_chunks;
    int64_t cnt_offset;
    int64_t ml_offset;
    int64_t o_offset;
    int64_t work_offset;  // [0]: number of work items, [64..): (request << 16 | chunk) sorted largest first (split decode only)
    int64_t total_bytes;
};

inline DecodeSplit decode_split(int64_t batch, int64_t n_heads, int64_t head_dim, int64_t max_blocks,
                                int64_t block_size, int64_t chunk_tokens, int64_t extra_chunks = 0) {
    DecodeSplit s;
    if (chunk_tokens <= 0) chunk_tokens = kDefaultChunkTokens;
    chunk_tokens = ceil_div(chunk_tokens, block_size) * block_size;
    s.chunk_tokens = chunk_tokens;
    s.n_chunks = ceil_div(max_blocks * block_size, chunk_tokens);
    if (s.n_chunks < 1) s.n_chunks = 1;
    s.n_chunks += extra_chunks;  // e.g. one slot per request for a shared-prefix partial
    s.cnt_offset = kWorkspaceHeader;
    s.ml_offset = s.cnt_offset + ceil_div(batch * n_heads * 4, 256) * 256;  // n_heads >= kv-head groups
    int64_t ml_bytes = batch * s.n_chunks * n_heads * 2 * 4;
    s.o_offset = s.ml_offset + ceil_div(ml_bytes, 256) * 256;
    s.work_offset = s.o_offset + ceil_div(batch * s.n_chunks * n_heads * head_dim * 4, 256) * 256;
    s.total_bytes = s.work_offset + 256 + batch * s.n_chunks * 4;
    if (s.n_chunks == 1) s.total_bytes = kWorkspaceHeader;
    return s;
}

// ---------------------------------------------------------------------------
// Device helpers
// ---------------------------------------------------------------------------
#ifdef __CUDACC__

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_float(__half v) { return __half2float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }

// e4m3 code -> float.  Exact (every e4m3 value is a float16 value).
__device__ __forceinline__ float e4m3_to_float(uint8_t c) {
    __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)c, __NV_E4M3);
    return __half2float(*reinterpret_cast<__half*>(&h));
}

// Two floats -> two e4m3 codes (low byte = a).  Round to nearest even,
// subnormals kept; magnitudes above 448 clamp to 448 (never reached by
// x / (amax/448)), NaN stays NaN.
__device__ __forceinline__ uint16_t float2_to_e4m3x2(float a, float b) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(b), "f"(a));
    return r;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// 16-byte global load that does not allocate in L1 (streamed KV data).
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

#endif  // __CUDACC__

// ---------------------------------------------------------------------------
// Kernel launchers (one per .cu file), called from abi.cu after validation.
// ---------------------------------------------------------------------------
struct DecodeArgs {
    const void* q;
    const void* k;
    const void* v;
    const float* k_scale;
    const float* v_scale;
    const int32_t* tables;
    const int32_t* table_rows;  // optional: query row r uses table row table_rows[r] (prefill tokens share a row)
    const uint32_t* work;       // split decode with many items: thread block x takes item work[x] = request << 16 | chunk ...
    const int* n_work;          // ... of *n_work items, largest first; nullptr: blockIdx (x, z) = (chunk, request)
    void* peer_out[8];          // n_peers > 0: every output store goes to the same offset in each of these buffers
    int n_peers;                // (head-partitioned multi-GPU decode: each GPU writes its heads into every GPU's copy)
    int64_t n_table_rows;       // rows of `tables`; a table_rows entry outside [0, n) is flagged and row 0 is read
    const int32_t* seq_lens;
    void* out;
    int q_dtype, kv_dtype;
    int batch, n_heads, n_kv_heads, head_dim, block_size, max_blocks;
    int64_t n_pool_blocks;
    int64_t q_stride[2];    // request, head (elements)
    int64_t out_stride[2];  // request, head
    int64_t k_stride[3];    // block, token, head (elements)
    int64_t v_stride[3];
    int64_t ks_stride[2];  // block, head
    int64_t vs_stride[2];
    int64_t table_stride;  // elements between rows
    float scale;
    DecodeSplit split;
    char* workspace;  // may be null when split.n_chunks == 1
    // Shared-prefix mode: the first prefix_tokens tokens of every request were attended by another kernel
    // whose partial sits in the chunk slot right after the request's own chunks; this launch covers the rest.
    int prefix_tokens;
};

// Table row of batch position `req`: the position itself, or table_rows[req] when the caller
// maps positions onto rows of a larger (device-resident) table.  A row outside the table is
// flagged like a bad block id and row 0 is read instead, so no address leaves the table.
__device__ __forceinline__ int64_t decode_table_row(const DecodeArgs& a, int req, int* status) {
    if (!a.table_rows) return req;
    int64_t row = a.table_rows[req];
    if (row < 0 || row >= a.n_table_rows) {
        if (status && threadIdx.x == 0) atomicOr(status, SFB_STATUS_BAD_BLOCK_ID);
        row = 0;
    }
    return row;
}

int launch_decode_generic(const DecodeArgs& a, cudaStream_t stream);
int launch_decode_combine(const DecodeArgs& a, cudaStream_t stream);
// Returns SFB_ERR_UNSUPPORTED (leaving the error text alone) when the shape is
// outside what the TMA + tensor-core kernel covers; the caller then falls back
// to the generic kernel.
int launch_decode_tma(const DecodeArgs& a, cudaStream_t stream);

struct AppendArgs {
    const void* k_new;
    const void* v_new;
    const int32_t* cu_tokens;
    const int32_t* start_pos;
    const int32_t* tables;
    int64_t table_stride;
    int max_blocks;
    void* k_cache;
    void* v_cache;
    float* k_scale;
    float* v_scale;
    void* k_tail;
    void* v_tail;
    const int32_t* tail_rows;  // optional: request r's tail copy lives in row tail_rows[r] (stable slot across steps)
    const int32_t* table_rows; // optional: request r's block table is row table_rows[r] of `tables`
    int64_t n_table_rows, n_tail_rows;
    int src_dtype, kv_dtype;
    int batch, n_kv_heads, head_dim, block_size, max_new_tokens;
    int64_t n_pool_blocks;
    int64_t new_stride[2];   // token, head (elements)
    int64_t vnew_stride[2];
    int64_t k_stride[3];     // block, token, head
    int64_t v_stride[3];
    int64_t ks_stride[2];
    int64_t vs_stride[2];
    int64_t kt_stride[3];    // request, token, head
    int64_t vt_stride[3];
};
int launch_cache_write(const AppendArgs& a, cudaStream_t stream);

int launch_quantize(const View& x, const View& codes, const View& scales, int x_dtype, int granularity, cudaStream_t stream);
int launch_dequantize(const View& codes, const View& scales, const View& out, int out_dtype, int granularity,
                      cudaStream_t stream);

struct PrefillLaunch {
    const void* q;
    const void* k;
    const void* v;
    void* out;
    const int32_t* cu_q;
    const int32_t* ctx_lens;
    const int32_t* row_limits;  // optional [total_q]: query row r attends to positions 0 .. row_limits[r] - 1 (replaces `causal`)
    const int32_t* tables;
    int64_t table_stride;
    int max_blocks, block_size, head_dim;
    int n_requests, n_heads, n_kv_heads;
    int64_t n_pool_blocks, total_q, max_q_tokens;
    int64_t q_stride[2];    // token, head (elements)
    int64_t out_stride[2];
    int64_t k_stride[3];    // block, token, head
    int64_t v_stride[3];
    float scale;
    int dtype;
    int causal;
    int* status;
    int* ticket;  // optional zeroed int: the resident thread blocks draw their work items from it
    // Shared-prefix mode (cu_q == nullptr): one pseudo-request of fixed_nq rows (row i = decode request i) over
    // fixed_ctx cached tokens; results go out as split partials, not as rows of `out`.
    int fixed_nq, fixed_ctx;
    float* part_o;
    float* part_ml;
    const int32_t* part_seq_lens;
    int part_n_chunks, part_chunk_tokens, part_max_tokens;
};
int launch_prefill_tcgen05(const PrefillLaunch& p, cudaStream_t stream);
// token r of the packed query batch -> (table row, attended length) for the decode-kernel route
int launch_prefill_expand(const int32_t* cu_q, const int32_t* ctx_lens, const int32_t* row_limits, int n_requests, int64_t total_q,
                          int max_blocks, int block_size, int causal, int32_t* rows_out, int32_t* lens_out, cudaStream_t stream);

struct NormArgs {
    const void* x;
    const void* residual;
    const void* weight;
    void* out;
    int64_t rows, hidden;
    int64_t x_stride, out_stride, res_stride;
    int dtype;
    float eps;
};
int launch_rms_norm(const NormArgs& a, cudaStream_t stream);

// prefill_fp8.cu: e4m3 blocks of a batch's contexts -> compact 16-bit scratch pool with identity tables
int launch_expand_fp8_blocks(const void* k_codes, const void* v_codes, const float* k_scale, const float* v_scale, void* k_scratch,
                             void* v_scratch, const int32_t* tables, int64_t table_stride, const int32_t* ctx_lens, int32_t* tables_out,
                             const int64_t* pool_stride, const int64_t* scale_stride, int n_requests, int max_blocks, int n_kv_heads,
                             int head_dim, int64_t n_pool_blocks, int dtype, int* status, cudaStream_t stream);

// norm_matmul_tcgen05.cu: Wg = diag(g) W, and y = rstd(x) * (x @ Wg) on the tensor cores (strides in elements)
int launch_fold_norm_weight(const void* g, const void* w, void* out, int64_t K, int64_t N, int64_t w_stride, int64_t out_stride,
                            int dtype, cudaStream_t stream);
// Tile shape the fused norm-matmul launcher picks for a problem (see plan_norm_matmul in norm_matmul_tcgen05.cu).
struct NormMatmulPlan {
    int pair;               // 1: clusters of two thread blocks on 256 x 256 tiles; 0: one thread block per 128 x tile_n tile
    int tile_n;             // tile width
    int stages;             // pipeline stages
    int k_steps_per_stage;  // 64-wide K steps behind one pair of barriers
    int prepass;            // 1: row statistics from the pre-pass kernel
    int x_box_rows;         // rows of x one TMA box brings in
};
NormMatmulPlan plan_norm_matmul(int64_t M, int64_t N, int sms, int clusters, bool has_scratch);
int launch_norm_matmul(const void* x, int64_t x_stride, const void* wg, int64_t wg_stride, void* out, int64_t out_stride, int64_t M,
                       int64_t N, int64_t K, float eps, int dtype, int* status, float* rstd_scratch, cudaStream_t stream);

}  // namespace sfb
