// C-ABI entry points of libsfb.so: descriptor validation, error text, dispatch.
// The kernels live in the sibling .cu files; nothing here touches device data.

#include <cstdlib>
#include <cstring>
#include <ctime>
#include <mutex>
#include <utility>
#include <vector>

#include "sfb_common.cuh"

namespace sfb {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int fail(int status, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return status;
}

int trace_level() {
    static const int level = [] {
        const char* v = getenv("SFB_TRACE");
        return v ? atoi(v) : 0;
    }();
    return level;
}

static double now_us() {
    timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return ts.tv_sec * 1e6 + ts.tv_nsec * 1e-3;
}

TraceScope::TraceScope(const char* op_name, void* st, const char* fmt, ...) : op(op_name), stream(static_cast<cudaStream_t>(st)), t0(0.0) {
    what[0] = 0;
    if (trace_level() <= 0) return;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(what, sizeof(what), fmt, ap);
    va_end(ap);
    t0 = now_us();
}

TraceScope::~TraceScope() {
    if (trace_level() <= 0) return;
    const bool synced = trace_level() >= 2 && cudaStreamSynchronize(stream) == cudaSuccess;
    fprintf(stderr, "[sfb] %-28s %-56s %9.1f us%s\n", op, what, now_us() - t0, synced ? " (stream synchronised)" : " (enqueue)");
}

int allow_shared_memory_once(const void* kernel, int smem_bytes) {
    static std::mutex mu;
    static std::vector<std::pair<const void*, int>> done;
    int dev = 0;
    SFB_CUDA_CHECK(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mu);
    for (const auto& e : done)
        if (e.first == kernel && e.second == dev) return SFB_OK;
    SFB_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    done.emplace_back(kernel, dev);
    return SFB_OK;
}

int make_view(const SFBTensor* t, const char* what, int min_rank, int max_rank, int elem_size, View* v) {
    if (!t) return fail(SFB_ERR_INVALID_ARG, "%s: descriptor is NULL", what);
    if (t->device != SFB_DEVICE_CUDA)
        return fail(SFB_ERR_INVALID_ARG, "%s: device %d is not SFB_DEVICE_CUDA (no CPU path exists)", what, t->device);
    if (t->rank < min_rank || t->rank > max_rank)
        return fail(SFB_ERR_INVALID_ARG, "%s: rank %d outside [%d, %d]", what, t->rank, min_rank, max_rank);
    if (elem_size > 0 && t->elem_size != elem_size)
        return fail(SFB_ERR_INVALID_ARG, "%s: elem_size %d, expected %d", what, t->elem_size, elem_size);
    // Every per-rank layout starts {allocated, aligned, offset, sizes[R], strides[R]}.
    const int64_t* tail = t->r4.sizes;  // same address for every rank
    const int r = t->rank;
    const int64_t* sizes = tail;
    const int64_t* strides = tail + r;
    v->rank = r;
    v->elem = t->elem_size;
    for (int i = 0; i < 4; ++i) { v->size[i] = 1; v->stride[i] = 0; }
    for (int i = 0; i < r; ++i) {
        if (sizes[i] < 0) return fail(SFB_ERR_INVALID_ARG, "%s: negative size", what);
        v->size[4 - r + i] = sizes[i];
        v->stride[4 - r + i] = strides[i];
    }
    if (v->numel() > 0 && !t->r1.aligned) return fail(SFB_ERR_INVALID_ARG, "%s: data pointer is NULL", what);
    if (v->size[3] > 1 && v->stride[3] != 1)
        return fail(SFB_ERR_INVALID_ARG, "%s: innermost dimension must be contiguous (stride %lld)", what,
                    (long long)v->stride[3]);
    v->base = static_cast<char*>(t->r1.aligned) + t->r1.offset * (int64_t)t->elem_size;
    return SFB_OK;
}

static bool aligned16(const View& v, int first_dim) {
    if (reinterpret_cast<uintptr_t>(v.base) % 16) return false;
    for (int i = first_dim; i < 3; ++i)
        if (v.size[i] > 1 && (v.stride[i] * v.elem) % 16) return false;
    return true;
}

}  // namespace sfb

using namespace sfb;

extern "C" {

int sfb_abi_version(void) { return SFB_ABI_VERSION; }

const char* sfb_last_error(void) { return g_error; }

const char* sfb_status_string(int status) {
    switch (status) {
        case SFB_OK: return "ok";
        case SFB_ERR_INVALID_ARG: return "invalid argument";
        case SFB_ERR_UNSUPPORTED: return "unsupported configuration";
        case SFB_ERR_WORKSPACE: return "workspace missing or too small";
        case SFB_ERR_CUDA: return "CUDA call failed";
        case SFB_ERR_DEVICE_STATUS: return "kernel flagged bad data";
        case SFB_ERR_OUT_OF_BLOCKS: return "block pool or table rows exhausted";
        default: return "unknown status";
    }
}

int64_t sfb_paged_attention_workspace_bytes(int64_t batch, int64_t n_heads, int64_t head_dim, int64_t max_blocks,
                                            int64_t block_size, int64_t chunk_tokens) {
    if (batch < 0 || n_heads <= 0 || head_dim <= 0 || max_blocks < 0 || block_size <= 0) return SFB_ERR_INVALID_ARG;
    return decode_split(batch, n_heads, head_dim, max_blocks, block_size, chunk_tokens).total_bytes;
}

// `world` > 0: `out` is this GPU's copy of the whole [B, H * world, D] output and peer_out[0..world) are the base
// addresses of every GPU's copy (this GPU's own included); the heads computed here are written into all of them.
static int decode_impl(const SFBTensor* q, const SFBTensor* k_cache, const SFBTensor* v_cache, const SFBTensor* k_scale,
                       const SFBTensor* v_scale, const SFBTensor* block_tables, const SFBTensor* seq_lens,
                       const SFBTensor* table_rows, SFBTensor* out, int q_dtype, int kv_dtype, float scale, int64_t chunk_tokens,
                       void* workspace, int64_t workspace_bytes, void* stream, void* const* peer_out, int world, int rank) {
    SFB_TRACE_OP(world > 0 ? "paged_attention_decode_gather" : "paged_attention_decode", stream, "kv dtype %d chunk %lld", kv_dtype, (long long)chunk_tokens);
    const int qe = dtype_size(q_dtype), kve = dtype_size(kv_dtype);
    if (!qe || q_dtype == SFB_F8E4M3) return fail(SFB_ERR_INVALID_ARG, "decode: q dtype %d", q_dtype);
    if (!kve) return fail(SFB_ERR_INVALID_ARG, "decode: kv dtype %d", kv_dtype);
    if (kv_dtype != SFB_F8E4M3 && kv_dtype != q_dtype)
        return fail(SFB_ERR_INVALID_ARG, "decode: kv dtype %d must equal q dtype %d (or be e4m3)", kv_dtype, q_dtype);
    if (kv_dtype == SFB_F8E4M3 && q_dtype == SFB_F32)
        return fail(SFB_ERR_UNSUPPORTED, "decode: e4m3 pools need a bf16 or fp16 query");
    View vq, vk, vv, vks, vvs, vt, vl, vo;
    int rc;
    if ((rc = make_view(q, "q", 3, 3, qe, &vq))) return rc;
    if ((rc = make_view(out, "out", 3, 3, qe, &vo))) return rc;
    if ((rc = make_view(k_cache, "k_cache", 4, 4, kve, &vk))) return rc;
    if ((rc = make_view(v_cache, "v_cache", 4, 4, kve, &vv))) return rc;
    if ((rc = make_view(block_tables, "block_tables", 2, 2, 4, &vt))) return rc;
    if ((rc = make_view(seq_lens, "seq_lens", 1, 1, 4, &vl))) return rc;
    const int64_t B = vq.size[1], H = vq.size[2], D = vq.size[3];
    const int64_t NB = vk.size[0], bs = vk.size[1], Hkv = vk.size[2];
    if (vk.size[3] != D || vv.size[3] != D) return fail(SFB_ERR_INVALID_ARG, "decode: head_dim of q (%lld) and pools differ", (long long)D);
    for (int i = 0; i < 4; ++i)
        if (vk.size[i] != vv.size[i]) return fail(SFB_ERR_INVALID_ARG, "decode: k_cache and v_cache shapes differ");
    const int64_t out_heads = world > 0 ? H * world : H;
    if (vo.size[1] != B || vo.size[2] != out_heads || vo.size[3] != D)
        return fail(SFB_ERR_INVALID_ARG, "decode: out must be [%lld, %lld, %lld]", (long long)B, (long long)out_heads, (long long)D);
    if (Hkv <= 0 || H % Hkv) return fail(SFB_ERR_INVALID_ARG, "decode: %lld query heads not a multiple of %lld kv heads", (long long)H, (long long)Hkv);
    View vr;
    if (table_rows) {
        if ((rc = make_view(table_rows, "table_rows", 1, 1, 4, &vr))) return rc;
        if (vr.size[3] != B) return fail(SFB_ERR_INVALID_ARG, "decode: table_rows must have one entry per request");
    } else if (vt.size[2] != B) {
        return fail(SFB_ERR_INVALID_ARG, "decode: block_tables rows != batch %lld", (long long)B);
    }
    if (vl.size[3] != B) return fail(SFB_ERR_INVALID_ARG, "decode: seq_lens rows != batch %lld", (long long)B);
    if (vl.size[3] > 1 && vl.stride[3] != 1) return fail(SFB_ERR_INVALID_ARG, "decode: seq_lens must be contiguous");
    if (bs <= 0 || (D * kve) % 16) return fail(SFB_ERR_UNSUPPORTED, "decode: head_dim*elem (%lld B) must be a multiple of 16", (long long)(D * kve));
    if (!aligned16(vk, 0) || !aligned16(vv, 0)) return fail(SFB_ERR_UNSUPPORTED, "decode: pool base and strides must be 16-byte aligned");
    const int64_t max_blocks = vt.size[3];
    if (B == 0) return SFB_OK;

    DecodeArgs a{};
    a.q = vq.base; a.k = vk.base; a.v = vv.base; a.out = vo.base;
    a.tables = reinterpret_cast<const int32_t*>(vt.base);
    a.seq_lens = reinterpret_cast<const int32_t*>(vl.base);
    a.table_rows = table_rows ? reinterpret_cast<const int32_t*>(vr.base) : nullptr;
    a.n_table_rows = vt.size[2];
    a.q_dtype = q_dtype; a.kv_dtype = kv_dtype;
    a.batch = (int)B; a.n_heads = (int)H; a.n_kv_heads = (int)Hkv; a.head_dim = (int)D;
    a.block_size = (int)bs; a.max_blocks = (int)max_blocks; a.n_pool_blocks = NB;
    a.q_stride[0] = vq.stride[1]; a.q_stride[1] = vq.stride[2];
    a.out_stride[0] = vo.stride[1]; a.out_stride[1] = vo.stride[2];
    if (world > 0) {
        // this GPU's heads start at head rank * H of every copy; all copies share the local copy's strides
        const int64_t head_off = (int64_t)rank * H * vo.stride[2] * qe;
        const int64_t local_off = static_cast<const char*>(vo.base) - static_cast<const char*>(peer_out[rank]);
        a.out = static_cast<char*>(vo.base) + head_off;
        a.n_peers = world;
        for (int p = 0; p < world; ++p) a.peer_out[p] = static_cast<char*>(peer_out[p]) + local_off + head_off;
    }
    for (int i = 0; i < 3; ++i) { a.k_stride[i] = vk.stride[i]; a.v_stride[i] = vv.stride[i]; }
    a.table_stride = vt.stride[2];
    a.scale = scale > 0.f ? scale : 1.0f / sqrtf((float)D);
    if (kv_dtype == SFB_F8E4M3) {
        if ((rc = make_view(k_scale, "k_scale", 2, 2, 4, &vks))) return rc;
        if ((rc = make_view(v_scale, "v_scale", 2, 2, 4, &vvs))) return rc;
        if (vks.size[2] != NB || vks.size[3] != Hkv || vvs.size[2] != NB || vvs.size[3] != Hkv)
            return fail(SFB_ERR_INVALID_ARG, "decode: scales must be [NB, Hkv]");
        a.k_scale = reinterpret_cast<const float*>(vks.base);
        a.v_scale = reinterpret_cast<const float*>(vvs.base);
        a.ks_stride[0] = vks.stride[2]; a.ks_stride[1] = vks.stride[3];
        a.vs_stride[0] = vvs.stride[2]; a.vs_stride[1] = vvs.stride[3];
    } else if (k_scale || v_scale) {
        return fail(SFB_ERR_INVALID_ARG, "decode: scales given for a non-e4m3 pool");
    }
    a.split = decode_split(B, H, D, max_blocks, bs, chunk_tokens);
    if (a.split.n_chunks > 1) {
        if (!workspace || workspace_bytes < a.split.total_bytes)
            return fail(SFB_ERR_WORKSPACE, "decode: workspace of %lld B needed, %lld given", (long long)a.split.total_bytes,
                        (long long)(workspace ? workspace_bytes : 0));
    } else if (workspace && workspace_bytes < kWorkspaceHeader) {
        workspace = nullptr;
    }
    a.workspace = static_cast<char*>(workspace);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (a.workspace)  // status word, and the arrival counters when the split is active
        SFB_CUDA_CHECK(cudaMemsetAsync(a.workspace, 0, a.split.n_chunks > 1 ? a.split.ml_offset : 4, st));
    if (max_blocks == 0) {
        // every request is empty: zero rows, flag it
        return fail(SFB_ERR_INVALID_ARG, "decode: block_tables has zero columns");
    }
    rc = launch_decode_tma(a, st);  // merges its own partials; SFB_ERR_UNSUPPORTED when the shape is not covered
    if (rc != SFB_ERR_UNSUPPORTED) return rc;
    if (world > 0) return fail(SFB_ERR_UNSUPPORTED, "decode_gather: only shapes of the TMA decode kernel (16-bit query, block 16, 16-byte aligned rows)");
    if ((rc = launch_decode_generic(a, st))) return rc;
    return launch_decode_combine(a, st);
}

int sfb_paged_attention_decode(const SFBTensor* q, const SFBTensor* k_cache, const SFBTensor* v_cache,
                               const SFBTensor* k_scale, const SFBTensor* v_scale, const SFBTensor* block_tables,
                               const SFBTensor* seq_lens, const SFBTensor* table_rows, SFBTensor* out, int q_dtype,
                               int kv_dtype, float scale, int64_t chunk_tokens, void* workspace, int64_t workspace_bytes,
                               void* stream) {
    return decode_impl(q, k_cache, v_cache, k_scale, v_scale, block_tables, seq_lens, table_rows, out, q_dtype, kv_dtype, scale,
                       chunk_tokens, workspace, workspace_bytes, stream, nullptr, 0, 0);
}

int sfb_paged_attention_decode_gather(const SFBTensor* q, const SFBTensor* k_cache, const SFBTensor* v_cache,
                                      const SFBTensor* k_scale, const SFBTensor* v_scale, const SFBTensor* block_tables,
                                      const SFBTensor* seq_lens, const SFBTensor* table_rows, SFBTensor* out_all,
                                      void* const* peer_out, int world, int rank, int q_dtype, int kv_dtype, float scale,
                                      int64_t chunk_tokens, void* workspace, int64_t workspace_bytes, void* stream) {
    if (world < 1 || world > 8 || rank < 0 || rank >= world || !peer_out)
        return fail(SFB_ERR_INVALID_ARG, "decode_gather: world must be 1..8, rank inside it, peer_out given");
    for (int p = 0; p < world; ++p)
        if (!peer_out[p] || reinterpret_cast<uintptr_t>(peer_out[p]) % 16) return fail(SFB_ERR_INVALID_ARG, "decode_gather: peer_out[%d] is null or not 16-byte aligned", p);
    return decode_impl(q, k_cache, v_cache, k_scale, v_scale, block_tables, seq_lens, table_rows, out_all, q_dtype, kv_dtype, scale,
                       chunk_tokens, workspace, workspace_bytes, stream, peer_out, world, rank);
}

int64_t sfb_prefill_workspace_bytes(int64_t total_q_tokens) {
    if (total_q_tokens < 0) return SFB_ERR_INVALID_ARG;
    return kWorkspaceHeader + ceil_div(total_q_tokens * 8, 256) * 256;
}

static int prefill_impl(const SFBTensor* q, const SFBTensor* k_cache, const SFBTensor* v_cache, const SFBTensor* block_tables,
                        const SFBTensor* cu_q, const SFBTensor* ctx_lens, SFBTensor* out, int dtype, float scale, int causal,
                        int64_t max_q_tokens, void* workspace, int64_t workspace_bytes, void* stream, bool clear_status,
                        const SFBTensor* row_limits = nullptr) {
    SFB_TRACE_OP(row_limits ? "prefill_paged_rows" : "prefill_paged", stream, "dtype %d causal %d max_q %lld", dtype, causal, (long long)max_q_tokens);
    const int e = dtype_size(dtype);
    if (!e || dtype == SFB_F8E4M3) return fail(SFB_ERR_INVALID_ARG, "prefill: dtype %d", dtype);
    View vq, vk, vv, vt, vc, vl, vo;
    int rc;
    if ((rc = make_view(q, "q", 3, 3, e, &vq))) return rc;
    if ((rc = make_view(out, "out", 3, 3, e, &vo))) return rc;
    if ((rc = make_view(k_cache, "k_cache", 4, 4, e, &vk))) return rc;
    if ((rc = make_view(v_cache, "v_cache", 4, 4, e, &vv))) return rc;
    if ((rc = make_view(block_tables, "block_tables", 2, 2, 4, &vt))) return rc;
    if ((rc = make_view(cu_q, "cu_q", 1, 1, 4, &vc))) return rc;
    if ((rc = make_view(ctx_lens, "ctx_lens", 1, 1, 4, &vl))) return rc;
    const int64_t T = vq.size[1], H = vq.size[2], D = vq.size[3], R = vl.size[3];
    const int64_t NB = vk.size[0], bs = vk.size[1], Hkv = vk.size[2];
    if (vc.size[3] != R + 1 || vt.size[2] != R) return fail(SFB_ERR_INVALID_ARG, "prefill: cu_q needs R+1 and block_tables R rows (R = %lld)", (long long)R);
    if (vk.size[3] != D || vv.size[3] != D) return fail(SFB_ERR_INVALID_ARG, "prefill: head_dim of q and pools differ");
    for (int i = 0; i < 4; ++i)
        if (vk.size[i] != vv.size[i]) return fail(SFB_ERR_INVALID_ARG, "prefill: k_cache and v_cache shapes differ");
    if (vo.size[1] != T || vo.size[2] != H || vo.size[3] != D) return fail(SFB_ERR_INVALID_ARG, "prefill: out shape differs from q");
    if (Hkv <= 0 || H % Hkv) return fail(SFB_ERR_INVALID_ARG, "prefill: query heads not a multiple of kv heads");
    if ((D * e) % 16 || !aligned16(vk, 0) || !aligned16(vv, 0)) return fail(SFB_ERR_UNSUPPORTED, "prefill: pools must be 16-byte aligned");
    View vr;
    if (row_limits) {
        if ((rc = make_view(row_limits, "row_limits", 1, 1, 4, &vr))) return rc;
        if (vr.size[3] != T || (T > 1 && vr.stride[3] != 1)) return fail(SFB_ERR_INVALID_ARG, "prefill: row_limits must be a contiguous int32 [T]");
    }
    if (T == 0 || R == 0 || max_q_tokens <= 0) return SFB_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (workspace && workspace_bytes < kWorkspaceHeader) workspace = nullptr;
    // word 0: status bits; word 4: the ticket the tensor-core kernel's thread blocks draw their work items from
    if (workspace && clear_status) SFB_CUDA_CHECK(cudaMemsetAsync(workspace, 0, 32, st));
    else if (workspace) SFB_CUDA_CHECK(cudaMemsetAsync(static_cast<char*>(workspace) + 16, 0, 4, st));
    const float sc = scale > 0.f ? scale : 1.0f / sqrtf((float)D);

    PrefillLaunch p{};
    p.row_limits = row_limits ? reinterpret_cast<const int32_t*>(vr.base) : nullptr;
    p.q = vq.base; p.k = vk.base; p.v = vv.base; p.out = vo.base;
    p.cu_q = reinterpret_cast<const int32_t*>(vc.base);
    p.ctx_lens = reinterpret_cast<const int32_t*>(vl.base);
    p.tables = reinterpret_cast<const int32_t*>(vt.base);
    p.table_stride = vt.stride[2]; p.max_blocks = (int)vt.size[3]; p.block_size = (int)bs; p.head_dim = (int)D;
    p.n_requests = (int)R; p.n_heads = (int)H; p.n_kv_heads = (int)Hkv; p.n_pool_blocks = NB;
    p.total_q = T; p.max_q_tokens = max_q_tokens;
    p.q_stride[0] = vq.stride[1]; p.q_stride[1] = vq.stride[2];
    p.out_stride[0] = vo.stride[1]; p.out_stride[1] = vo.stride[2];
    for (int i = 0; i < 3; ++i) { p.k_stride[i] = vk.stride[i]; p.v_stride[i] = vv.stride[i]; }
    p.scale = sc; p.dtype = dtype; p.causal = causal != 0; p.status = static_cast<int*>(workspace);
    p.ticket = workspace ? static_cast<int*>(workspace) + 4 : nullptr;
    const bool q_tma_ok = reinterpret_cast<uintptr_t>(vq.base) % 16 == 0 && (vq.stride[1] * e) % 16 == 0 && (vq.stride[2] * e) % 16 == 0;
    rc = q_tma_ok ? launch_prefill_tcgen05(p, st) : SFB_ERR_UNSUPPORTED;
    if (rc != SFB_ERR_UNSUPPORTED) return rc;

    // every other shape: one decode row per query token, single pass over its whole context
    const int64_t need = sfb_prefill_workspace_bytes(T);
    if (!workspace || workspace_bytes < need)
        return fail(SFB_ERR_WORKSPACE, "prefill: workspace of %lld B needed for this shape, %lld given", (long long)need,
                    (long long)(workspace ? workspace_bytes : 0));
    int32_t* rows = reinterpret_cast<int32_t*>(static_cast<char*>(workspace) + kWorkspaceHeader);
    int32_t* lens = rows + T;
    if ((rc = launch_prefill_expand(p.cu_q, p.ctx_lens, p.row_limits, (int)R, T, p.max_blocks, (int)bs, causal != 0, rows, lens, st))) return rc;
    DecodeArgs a{};
    a.q = vq.base; a.k = vk.base; a.v = vv.base; a.out = vo.base;
    a.tables = p.tables; a.table_rows = rows; a.n_table_rows = R; a.seq_lens = lens;
    a.q_dtype = dtype; a.kv_dtype = dtype;
    a.batch = (int)T; a.n_heads = (int)H; a.n_kv_heads = (int)Hkv; a.head_dim = (int)D;
    a.block_size = (int)bs; a.max_blocks = p.max_blocks; a.n_pool_blocks = NB;
    a.q_stride[0] = vq.stride[1]; a.q_stride[1] = vq.stride[2];
    a.out_stride[0] = vo.stride[1]; a.out_stride[1] = vo.stride[2];
    for (int i = 0; i < 3; ++i) { a.k_stride[i] = vk.stride[i]; a.v_stride[i] = vv.stride[i]; }
    a.table_stride = vt.stride[2];
    a.scale = sc;
    a.split = decode_split(T, H, D, p.max_blocks, bs, (int64_t)p.max_blocks * bs);  // one chunk: no partials
    a.workspace = static_cast<char*>(workspace);
    if (T > 65535) return fail(SFB_ERR_UNSUPPORTED, "prefill: %lld query tokens exceed the generic route's limit 65535", (long long)T);
    rc = launch_decode_tma(a, st);
    if (rc == SFB_ERR_UNSUPPORTED) rc = launch_decode_generic(a, st);
    return rc;
}

int64_t sfb_shared_prefix_workspace_bytes(int64_t batch, int64_t n_heads, int64_t head_dim, int64_t max_blocks, int64_t block_size,
                                          int64_t chunk_tokens, int64_t shared_prefix_blocks) {
    if (batch < 0 || n_heads <= 0 || head_dim <= 0 || block_size <= 0 || shared_prefix_blocks < 0 || max_blocks < shared_prefix_blocks)
        return SFB_ERR_INVALID_ARG;
    return decode_split(batch, n_heads, head_dim, max_blocks - shared_prefix_blocks, block_size, chunk_tokens, 1).total_bytes;
}

int sfb_paged_attention_decode_shared_prefix(const SFBTensor* q, const SFBTensor* k_cache, const SFBTensor* v_cache,
                                             const SFBTensor* block_tables, const SFBTensor* seq_lens, SFBTensor* out, int dtype,
                                             float scale, int64_t shared_prefix_blocks, int64_t chunk_tokens, void* workspace,
                                             int64_t workspace_bytes, void* stream) {
    SFB_TRACE_OP("decode_shared_prefix", stream, "prefix blocks %lld chunk %lld", (long long)shared_prefix_blocks, (long long)chunk_tokens);
    const int e = dtype_size(dtype);
    if (dtype != SFB_BF16 && dtype != SFB_F16)
        return fail(SFB_ERR_UNSUPPORTED, "shared-prefix decode: bf16 / fp16 pools only (the prefix runs on the tcgen05 kernel)");
    View vq, vk, vv, vt, vl, vo;
    int rc;
    if ((rc = make_view(q, "q", 3, 3, e, &vq))) return rc;
    if ((rc = make_view(out, "out", 3, 3, e, &vo))) return rc;
    if ((rc = make_view(k_cache, "k_cache", 4, 4, e, &vk))) return rc;
    if ((rc = make_view(v_cache, "v_cache", 4, 4, e, &vv))) return rc;
    if ((rc = make_view(block_tables, "block_tables", 2, 2, 4, &vt))) return rc;
    if ((rc = make_view(seq_lens, "seq_lens", 1, 1, 4, &vl))) return rc;
    const int64_t B = vq.size[1], H = vq.size[2], D = vq.size[3];
    const int64_t NB = vk.size[0], bs = vk.size[1], Hkv = vk.size[2], max_blocks = vt.size[3];
    if (vk.size[3] != D || vv.size[3] != D) return fail(SFB_ERR_INVALID_ARG, "shared-prefix decode: head_dim of q and pools differ");
    for (int i = 0; i < 4; ++i)
        if (vk.size[i] != vv.size[i]) return fail(SFB_ERR_INVALID_ARG, "shared-prefix decode: k_cache and v_cache shapes differ");
    if (vo.size[1] != B || vo.size[2] != H || vo.size[3] != D) return fail(SFB_ERR_INVALID_ARG, "shared-prefix decode: out shape differs from q");
    if (Hkv <= 0 || H % Hkv) return fail(SFB_ERR_INVALID_ARG, "shared-prefix decode: query heads not a multiple of kv heads");
    if (vt.size[2] != B || vl.size[3] != B) return fail(SFB_ERR_INVALID_ARG, "shared-prefix decode: block_tables/seq_lens rows != batch");
    if (shared_prefix_blocks <= 0 || shared_prefix_blocks >= max_blocks)
        return fail(SFB_ERR_INVALID_ARG, "shared-prefix decode: shared_prefix_blocks must be in [1, max_blocks)");
    if (bs != 16 || D != 128) return fail(SFB_ERR_UNSUPPORTED, "shared-prefix decode: block_size 16 and head_dim 128 only");
    if (!aligned16(vk, 0) || !aligned16(vv, 0)) return fail(SFB_ERR_UNSUPPORTED, "shared-prefix decode: pools must be 16-byte aligned");
    if (B == 0) return SFB_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const float sc = scale > 0.f ? scale : 1.0f / sqrtf((float)D);

    DecodeArgs a{};
    a.q = vq.base; a.k = vk.base; a.v = vv.base; a.out = vo.base;
    a.tables = reinterpret_cast<const int32_t*>(vt.base);
    a.seq_lens = reinterpret_cast<const int32_t*>(vl.base);
    a.q_dtype = a.kv_dtype = dtype;
    a.batch = (int)B; a.n_heads = (int)H; a.n_kv_heads = (int)Hkv; a.head_dim = (int)D;
    a.block_size = (int)bs; a.max_blocks = (int)max_blocks; a.n_pool_blocks = NB;
    a.q_stride[0] = vq.stride[1]; a.q_stride[1] = vq.stride[2];
    a.out_stride[0] = vo.stride[1]; a.out_stride[1] = vo.stride[2];
    for (int i = 0; i < 3; ++i) { a.k_stride[i] = vk.stride[i]; a.v_stride[i] = vv.stride[i]; }
    a.table_stride = vt.stride[2];
    a.scale = sc;
    a.prefix_tokens = (int)(shared_prefix_blocks * bs);
    a.split = decode_split(B, H, D, max_blocks - shared_prefix_blocks, bs, chunk_tokens, 1);
    if (!workspace || workspace_bytes < a.split.total_bytes)
        return fail(SFB_ERR_WORKSPACE, "shared-prefix decode: workspace of %lld B needed, %lld given", (long long)a.split.total_bytes,
                    (long long)(workspace ? workspace_bytes : 0));
    a.workspace = static_cast<char*>(workspace);
    SFB_CUDA_CHECK(cudaMemsetAsync(a.workspace, 0, a.split.ml_offset, st));

    // (1) the shared prefix once for all requests: rows = requests, keys = the prefix blocks of table row 0
    PrefillLaunch p{};
    p.q = vq.base; p.k = vk.base; p.v = vv.base; p.out = nullptr;
    p.cu_q = nullptr; p.ctx_lens = nullptr;
    p.tables = a.tables; p.table_stride = vt.stride[2]; p.max_blocks = (int)max_blocks; p.block_size = (int)bs; p.head_dim = (int)D;
    p.n_requests = 1; p.n_heads = (int)H; p.n_kv_heads = (int)Hkv; p.n_pool_blocks = NB;
    p.total_q = B; p.max_q_tokens = B;
    p.q_stride[0] = vq.stride[1]; p.q_stride[1] = vq.stride[2];
    for (int i = 0; i < 3; ++i) { p.k_stride[i] = vk.stride[i]; p.v_stride[i] = vv.stride[i]; }
    p.scale = sc; p.dtype = dtype; p.causal = 0; p.status = reinterpret_cast<int*>(workspace);
    p.fixed_nq = (int)B; p.fixed_ctx = a.prefix_tokens;
    p.part_o = reinterpret_cast<float*>(a.workspace + a.split.o_offset);
    p.part_ml = reinterpret_cast<float*>(a.workspace + a.split.ml_offset);
    p.part_seq_lens = a.seq_lens; p.part_n_chunks = (int)a.split.n_chunks; p.part_chunk_tokens = (int)a.split.chunk_tokens;
    p.part_max_tokens = (int)(max_blocks * bs);
    if (reinterpret_cast<uintptr_t>(vq.base) % 16 || (vq.stride[1] * e) % 16 || (vq.stride[2] * e) % 16)
        return fail(SFB_ERR_UNSUPPORTED, "shared-prefix decode: q must be 16-byte aligned");
    rc = launch_prefill_tcgen05(p, st);
    if (rc == SFB_ERR_UNSUPPORTED) return fail(SFB_ERR_UNSUPPORTED, "shared-prefix decode: shape not covered by the tcgen05 kernel");
    if (rc) return rc;
    // (2) every request's own tokens, merged in-kernel with the prefix partial
    rc = launch_decode_tma(a, st);
    if (rc == SFB_ERR_UNSUPPORTED) return fail(SFB_ERR_UNSUPPORTED, "shared-prefix decode: shape not covered by the TMA decode kernel");
    return rc;
}

int sfb_read_status(const void* workspace, int32_t* bits, void* stream) {
    if (!workspace) return fail(SFB_ERR_INVALID_ARG, "read_status: workspace is NULL");
    int32_t host = 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    SFB_CUDA_CHECK(cudaMemcpyAsync(&host, workspace, 4, cudaMemcpyDeviceToHost, st));
    SFB_CUDA_CHECK(cudaStreamSynchronize(st));
    if (bits) *bits = host;
    if (host) return fail(SFB_ERR_DEVICE_STATUS, "device status bits 0x%x", host);
    return SFB_OK;
}

int sfb_cache_write(const SFBTensor* k_new, const SFBTensor* v_new, const SFBTensor* cu_tokens,
                    const SFBTensor* start_pos, const SFBTensor* block_tables, SFBTensor* k_cache, SFBTensor* v_cache,
                    SFBTensor* k_scale, SFBTensor* v_scale, SFBTensor* k_tail, SFBTensor* v_tail,
                    const SFBTensor* tail_rows, const SFBTensor* table_rows, int src_dtype, int kv_dtype,
                    int64_t max_new_tokens, void* stream) {
    SFB_TRACE_OP("cache_write", stream, "src dtype %d pool dtype %d max_new %lld", src_dtype, kv_dtype, (long long)max_new_tokens);
    const int se = dtype_size(src_dtype), kve = dtype_size(kv_dtype);
    if (!se || src_dtype == SFB_F8E4M3) return fail(SFB_ERR_INVALID_ARG, "cache_write: source dtype %d", src_dtype);
    if (!kve) return fail(SFB_ERR_INVALID_ARG, "cache_write: pool dtype %d", kv_dtype);
    const bool fp8 = kv_dtype == SFB_F8E4M3;
    if (!fp8 && kv_dtype != src_dtype) return fail(SFB_ERR_INVALID_ARG, "cache_write: pool dtype must equal the source dtype or be e4m3");
    View kn, vn, cu, sp, bt, kc, vc, ks, vs, kt, vt;
    int rc;
    if ((rc = make_view(k_new, "k_new", 3, 3, se, &kn))) return rc;
    if ((rc = make_view(v_new, "v_new", 3, 3, se, &vn))) return rc;
    if ((rc = make_view(cu_tokens, "cu_tokens", 1, 1, 4, &cu))) return rc;
    if ((rc = make_view(start_pos, "start_pos", 1, 1, 4, &sp))) return rc;
    if ((rc = make_view(block_tables, "block_tables", 2, 2, 4, &bt))) return rc;
    if ((rc = make_view(k_cache, "k_cache", 4, 4, kve, &kc))) return rc;
    if ((rc = make_view(v_cache, "v_cache", 4, 4, kve, &vc))) return rc;
    const int64_t B = sp.size[3], Hkv = kc.size[2], D = kc.size[3], bs = kc.size[1];
    if (cu.size[3] != B + 1) return fail(SFB_ERR_INVALID_ARG, "cache_write: cu_tokens must have batch+1 = %lld entries", (long long)(B + 1));
    View trw;
    if (table_rows) {
        if ((rc = make_view(table_rows, "table_rows", 1, 1, 4, &trw))) return rc;
        if (trw.size[3] != B) return fail(SFB_ERR_INVALID_ARG, "cache_write: table_rows must have one entry per request");
    } else if (bt.size[2] != B) {
        return fail(SFB_ERR_INVALID_ARG, "cache_write: block_tables rows != batch");
    }
    for (int i = 0; i < 4; ++i)
        if (kc.size[i] != vc.size[i]) return fail(SFB_ERR_INVALID_ARG, "cache_write: k_cache and v_cache shapes differ");
    if (kn.size[2] != Hkv || kn.size[3] != D || vn.size[2] != Hkv || vn.size[3] != D || vn.size[1] != kn.size[1])
        return fail(SFB_ERR_INVALID_ARG, "cache_write: k_new/v_new must be [T, %lld, %lld]", (long long)Hkv, (long long)D);
    if ((D * se) % 16 || (D * kve) % 16) return fail(SFB_ERR_UNSUPPORTED, "cache_write: head_dim rows must be multiples of 16 bytes");
    if (!aligned16(kn, 1) || !aligned16(vn, 1) || !aligned16(kc, 0) || !aligned16(vc, 0))
        return fail(SFB_ERR_UNSUPPORTED, "cache_write: tensors must be 16-byte aligned");
    if (B == 0 || max_new_tokens <= 0) return SFB_OK;

    AppendArgs a{};
    a.k_new = kn.base; a.v_new = vn.base;
    a.cu_tokens = reinterpret_cast<const int32_t*>(cu.base);
    a.start_pos = reinterpret_cast<const int32_t*>(sp.base);
    a.tables = reinterpret_cast<const int32_t*>(bt.base);
    a.table_stride = bt.stride[2];
    a.max_blocks = (int)bt.size[3];
    a.table_rows = table_rows ? reinterpret_cast<const int32_t*>(trw.base) : nullptr;
    a.n_table_rows = bt.size[2];
    a.k_cache = kc.base; a.v_cache = vc.base;
    a.src_dtype = src_dtype; a.kv_dtype = kv_dtype;
    a.batch = (int)B; a.n_kv_heads = (int)Hkv; a.head_dim = (int)D; a.block_size = (int)bs;
    a.n_pool_blocks = kc.size[0];
    a.max_new_tokens = (int)max_new_tokens;
    a.new_stride[0] = kn.stride[1]; a.new_stride[1] = kn.stride[2];
    a.vnew_stride[0] = vn.stride[1]; a.vnew_stride[1] = vn.stride[2];
    for (int i = 0; i < 3; ++i) { a.k_stride[i] = kc.stride[i]; a.v_stride[i] = vc.stride[i]; }
    if (fp8) {
        if ((rc = make_view(k_scale, "k_scale", 2, 2, 4, &ks))) return rc;
        if ((rc = make_view(v_scale, "v_scale", 2, 2, 4, &vs))) return rc;
        if ((rc = make_view(k_tail, "k_tail", 4, 4, se, &kt))) return rc;
        if ((rc = make_view(v_tail, "v_tail", 4, 4, se, &vt))) return rc;
        if (ks.size[2] != kc.size[0] || ks.size[3] != Hkv || vs.size[2] != kc.size[0] || vs.size[3] != Hkv)
            return fail(SFB_ERR_INVALID_ARG, "cache_write: scales must be [NB, Hkv]");
        View tr;
        if (tail_rows) {
            if ((rc = make_view(tail_rows, "tail_rows", 1, 1, 4, &tr))) return rc;
            if (tr.size[3] != B) return fail(SFB_ERR_INVALID_ARG, "cache_write: tail_rows must have one entry per request");
            a.tail_rows = reinterpret_cast<const int32_t*>(tr.base);
        }
        if ((!tail_rows && kt.size[0] < B) || kt.size[1] != bs || kt.size[2] != Hkv || kt.size[3] != D)
            return fail(SFB_ERR_INVALID_ARG, "cache_write: k_tail must be [>=batch, bs, Hkv, D]");
        for (int i = 0; i < 4; ++i)
            if (kt.size[i] != vt.size[i]) return fail(SFB_ERR_INVALID_ARG, "cache_write: k_tail and v_tail shapes differ");
        if (!aligned16(kt, 0) || !aligned16(vt, 0)) return fail(SFB_ERR_UNSUPPORTED, "cache_write: tails must be 16-byte aligned");
        a.k_scale = reinterpret_cast<float*>(ks.base); a.v_scale = reinterpret_cast<float*>(vs.base);
        a.ks_stride[0] = ks.stride[2]; a.ks_stride[1] = ks.stride[3];
        a.vs_stride[0] = vs.stride[2]; a.vs_stride[1] = vs.stride[3];
        a.k_tail = kt.base; a.v_tail = vt.base;
        a.n_tail_rows = kt.size[0];
        for (int i = 0; i < 3; ++i) { a.kt_stride[i] = kt.stride[i]; a.vt_stride[i] = vt.stride[i]; }
    }
    return launch_cache_write(a, static_cast<cudaStream_t>(stream));
}

int sfb_fold_norm_weight(const SFBTensor* rms_weight, const SFBTensor* mat_weight, SFBTensor* folded, int dtype, void* stream) {
    if (dtype != SFB_BF16 && dtype != SFB_F16) return fail(SFB_ERR_UNSUPPORTED, "fold_norm_weight: bf16 or fp16");
    View vg, vw, vf;
    int rc;
    if ((rc = make_view(rms_weight, "rms_weight", 1, 1, 2, &vg))) return rc;
    if ((rc = make_view(mat_weight, "mat_weight", 2, 2, 2, &vw))) return rc;
    if ((rc = make_view(folded, "folded", 2, 2, 2, &vf))) return rc;
    const int64_t K = vw.size[2], N = vw.size[3];
    if (vg.size[3] != K || vf.size[2] != K || vf.size[3] != N) return fail(SFB_ERR_INVALID_ARG, "fold_norm_weight: rms_weight [K], mat_weight and folded [K, N]");
    if (vg.stride[3] != 1 && K > 1) return fail(SFB_ERR_UNSUPPORTED, "fold_norm_weight: rms_weight must be contiguous");
    if (N % 8 || vw.stride[3] != 1 || vf.stride[3] != 1 || !aligned16(vw, 2) || !aligned16(vf, 2))
        return fail(SFB_ERR_UNSUPPORTED, "fold_norm_weight: N a multiple of 8, rows contiguous and 16-byte aligned");
    if (K == 0 || N == 0) return SFB_OK;
    return launch_fold_norm_weight(vg.base, vw.base, vf.base, K, N, vw.stride[2], vf.stride[2], dtype, static_cast<cudaStream_t>(stream));
}

int sfb_prefill_paged(const SFBTensor* q, const SFBTensor* k_cache, const SFBTensor* v_cache, const SFBTensor* block_tables,
                      const SFBTensor* cu_q, const SFBTensor* ctx_lens, SFBTensor* out, int dtype, float scale,
                      int causal, int64_t max_q_tokens, void* workspace, int64_t workspace_bytes, void* stream) {
    return prefill_impl(q, k_cache, v_cache, block_tables, cu_q, ctx_lens, out, dtype, scale, causal, max_q_tokens, workspace, workspace_bytes,
                        stream, true);
}

int sfb_prefill_paged_rows(const SFBTensor* q, const SFBTensor* k_cache, const SFBTensor* v_cache, const SFBTensor* block_tables,
                           const SFBTensor* cu_q, const SFBTensor* ctx_lens, const SFBTensor* row_limits, SFBTensor* out, int dtype,
                           float scale, int64_t max_q_tokens, void* workspace, int64_t workspace_bytes, void* stream) {
    if (!row_limits) return fail(SFB_ERR_INVALID_ARG, "prefill_rows: row_limits is NULL");
    return prefill_impl(q, k_cache, v_cache, block_tables, cu_q, ctx_lens, out, dtype, scale, 0, max_q_tokens, workspace, workspace_bytes,
                        stream, true, row_limits);
}

static SFBTensor device_tensor(void* base, int elem, int rank, const int64_t* sizes) {
    SFBTensor t{};
    t.device = SFB_DEVICE_CUDA; t.rank = rank; t.elem_size = elem;
    int64_t stride = 1;
    SFBMemRef4* m = &t.r4;  // the four layouts share their first fields; sizes / strides are written per rank below
    m->allocated = m->aligned = base; m->offset = 0;
    int64_t* sz = rank == 1 ? t.r1.sizes : rank == 2 ? t.r2.sizes : rank == 3 ? t.r3.sizes : t.r4.sizes;
    int64_t* st = rank == 1 ? t.r1.strides : rank == 2 ? t.r2.strides : rank == 3 ? t.r3.strides : t.r4.strides;
    for (int i = rank - 1; i >= 0; --i) { sz[i] = sizes[i]; st[i] = stride; stride *= sizes[i]; }
    return t;
}

int64_t sfb_prefill_fp8_workspace_bytes(int64_t total_q_tokens, int64_t n_requests, int64_t max_blocks, int64_t n_kv_heads, int64_t head_dim) {
    if (total_q_tokens < 0 || n_requests < 0 || max_blocks < 0 || n_kv_heads <= 0 || head_dim <= 0) return SFB_ERR_INVALID_ARG;
    const int64_t slots = n_requests * max_blocks;
    return sfb_prefill_workspace_bytes(total_q_tokens) + ceil_div(slots * 4, 256) * 256 + 2 * ceil_div(slots * 16 * n_kv_heads * head_dim * 2, 256) * 256;
}

int sfb_prefill_paged_fp8(const SFBTensor* q, const SFBTensor* k_cache, const SFBTensor* v_cache, const SFBTensor* k_scale,
                          const SFBTensor* v_scale, const SFBTensor* block_tables, const SFBTensor* cu_q, const SFBTensor* ctx_lens,
                          SFBTensor* out, int q_dtype, float scale, int causal, int64_t max_q_tokens, void* workspace,
                          int64_t workspace_bytes, void* stream) {
    SFB_TRACE_OP("prefill_paged_fp8", stream, "q dtype %d causal %d max_q %lld", q_dtype, causal, (long long)max_q_tokens);
    if (q_dtype != SFB_BF16 && q_dtype != SFB_F16) return fail(SFB_ERR_UNSUPPORTED, "prefill_fp8: bf16 or fp16 queries");
    View vq, vk, vv, vks, vvs, vt, vl;
    int rc;
    if ((rc = make_view(q, "q", 3, 3, 2, &vq))) return rc;
    if ((rc = make_view(k_cache, "k_cache", 4, 4, 1, &vk))) return rc;
    if ((rc = make_view(v_cache, "v_cache", 4, 4, 1, &vv))) return rc;
    if ((rc = make_view(k_scale, "k_scale", 2, 2, 4, &vks))) return rc;
    if ((rc = make_view(v_scale, "v_scale", 2, 2, 4, &vvs))) return rc;
    if ((rc = make_view(block_tables, "block_tables", 2, 2, 4, &vt))) return rc;
    if ((rc = make_view(ctx_lens, "ctx_lens", 1, 1, 4, &vl))) return rc;
    const int64_t T = vq.size[1], D = vq.size[3], R = vl.size[3];
    const int64_t NB = vk.size[0], bs = vk.size[1], Hkv = vk.size[2], max_blocks = vt.size[3];
    if (bs != 16 || vk.size[3] != D || D % 16) return fail(SFB_ERR_UNSUPPORTED, "prefill_fp8: block size 16, head_dim a multiple of 16 equal to q's");
    for (int i = 0; i < 4; ++i)
        if (vk.size[i] != vv.size[i] || (i < 3 && vk.stride[i] != vv.stride[i])) return fail(SFB_ERR_INVALID_ARG, "prefill_fp8: k_cache and v_cache layouts differ");
    if (vk.stride[3] != 1 || !aligned16(vk, 0) || !aligned16(vv, 0)) return fail(SFB_ERR_UNSUPPORTED, "prefill_fp8: pool rows must be contiguous and 16-byte aligned");
    if (vt.size[2] != R) return fail(SFB_ERR_INVALID_ARG, "prefill_fp8: block_tables rows != requests");
    if (vks.size[2] != NB || vks.size[3] != Hkv || vvs.size[2] != NB || vvs.size[3] != Hkv || vks.stride[2] != vvs.stride[2] || vks.stride[3] != vvs.stride[3])
        return fail(SFB_ERR_INVALID_ARG, "prefill_fp8: scales must be [NB, Hkv] with one layout for K and V");
    if (vl.size[3] > 1 && vl.stride[3] != 1) return fail(SFB_ERR_INVALID_ARG, "prefill_fp8: ctx_lens must be contiguous");
    if (T == 0 || R == 0 || max_q_tokens <= 0 || max_blocks == 0) return SFB_OK;
    const int64_t need = sfb_prefill_fp8_workspace_bytes(T, R, max_blocks, Hkv, D);
    if (!workspace || workspace_bytes < need)
        return fail(SFB_ERR_WORKSPACE, "prefill_fp8: workspace of %lld B needed, %lld given", (long long)need, (long long)(workspace ? workspace_bytes : 0));
    if (R * max_blocks > 0x7fffffffLL) return fail(SFB_ERR_UNSUPPORTED, "prefill_fp8: too many table entries");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    char* ws = static_cast<char*>(workspace);
    const int64_t inner = sfb_prefill_workspace_bytes(T), slots = R * max_blocks;
    int32_t* tables2 = reinterpret_cast<int32_t*>(ws + inner);
    char* k_scratch = ws + inner + ceil_div(slots * 4, 256) * 256;
    char* v_scratch = k_scratch + ceil_div(slots * 16 * Hkv * D * 2, 256) * 256;
    SFB_CUDA_CHECK(cudaMemsetAsync(ws, 0, 4, st));
    const int64_t ps[3] = {vk.stride[0], vk.stride[1], vk.stride[2]}, ss[2] = {vks.stride[2], vks.stride[3]};
    if ((rc = launch_expand_fp8_blocks(vk.base, vv.base, reinterpret_cast<const float*>(vks.base), reinterpret_cast<const float*>(vvs.base), k_scratch,
                                       v_scratch, reinterpret_cast<const int32_t*>(vt.base), vt.stride[2], reinterpret_cast<const int32_t*>(vl.base),
                                       tables2, ps, ss, (int)R, (int)max_blocks, (int)Hkv, (int)D, NB, q_dtype,
                                       reinterpret_cast<int*>(ws), st)))
        return rc;
    const int64_t pool_sizes[4] = {slots, 16, Hkv, D}, table_sizes[2] = {R, max_blocks};
    SFBTensor kt = device_tensor(k_scratch, 2, 4, pool_sizes), vt2 = device_tensor(v_scratch, 2, 4, pool_sizes);
    SFBTensor tt = device_tensor(tables2, 4, 2, table_sizes);
    return prefill_impl(q, &kt, &vt2, &tt, cu_q, ctx_lens, out, q_dtype, scale, causal, max_q_tokens, ws, inner, stream, false);
}

int64_t sfb_fused_rms_norm_matmul_workspace_bytes(int64_t rows) {
    if (rows < 0) return SFB_ERR_INVALID_ARG;
    return kWorkspaceHeader + ceil_div(rows * 4, 256) * 256;
}

int sfb_fused_rms_norm_matmul_plan(int64_t rows, int64_t cols, int sms, int clusters, int has_workspace, int32_t* plan6) {
    if (rows < 0 || cols < 0 || sms <= 0 || clusters < 0 || !plan6) return fail(SFB_ERR_INVALID_ARG, "fused_rms_norm_matmul_plan: bad argument");
    const NormMatmulPlan p = plan_norm_matmul(rows, cols, sms, clusters, has_workspace != 0);
    plan6[0] = p.pair; plan6[1] = p.tile_n; plan6[2] = p.stages; plan6[3] = p.k_steps_per_stage; plan6[4] = p.prepass; plan6[5] = p.x_box_rows;
    return SFB_OK;
}

int sfb_fused_rms_norm_matmul(const SFBTensor* x, const SFBTensor* folded_weight, SFBTensor* out, int dtype, float eps, void* workspace,
                              int64_t workspace_bytes, void* stream) {
    SFB_TRACE_OP("fused_rms_norm_matmul", stream, "dtype %d eps %g", dtype, (double)eps);
    if (dtype != SFB_BF16 && dtype != SFB_F16) return fail(SFB_ERR_UNSUPPORTED, "fused_rms_norm_matmul: bf16 or fp16 (other types go to the fallback executor)");
    View vx, vw, vo;
    int rc;
    if ((rc = make_view(x, "x", 2, 2, 2, &vx))) return rc;
    if ((rc = make_view(folded_weight, "folded_weight", 2, 2, 2, &vw))) return rc;
    if ((rc = make_view(out, "out", 2, 2, 2, &vo))) return rc;
    const int64_t M = vx.size[2], K = vx.size[3], N = vw.size[3];
    if (vw.size[2] != K || vo.size[2] != M || vo.size[3] != N) return fail(SFB_ERR_INVALID_ARG, "fused_rms_norm_matmul: x [M, K], weight [K, N], out [M, N]");
    if (K % 8 || N % 8 || vx.stride[3] != 1 || vw.stride[3] != 1 || vo.stride[3] != 1 || !aligned16(vx, 2) || !aligned16(vw, 2) || !aligned16(vo, 2))
        return fail(SFB_ERR_UNSUPPORTED, "fused_rms_norm_matmul: K and N multiples of 8, rows contiguous and 16-byte aligned");
    if (M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL) return fail(SFB_ERR_UNSUPPORTED, "fused_rms_norm_matmul: dimension too large");
    if (M == 0 || N == 0) return SFB_OK;
    if (K == 0) return fail(SFB_ERR_INVALID_ARG, "fused_rms_norm_matmul: K is zero");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int* status = nullptr;
    float* rstd = nullptr;
    if (workspace && workspace_bytes >= kWorkspaceHeader) {
        status = static_cast<int*>(workspace);
        SFB_CUDA_CHECK(cudaMemsetAsync(status, 0, 4, st));
        if (workspace_bytes >= sfb_fused_rms_norm_matmul_workspace_bytes(M)) rstd = reinterpret_cast<float*>(static_cast<char*>(workspace) + kWorkspaceHeader);
    }
    return launch_norm_matmul(vx.base, vx.stride[2], vw.base, vw.stride[2], vo.base, vo.stride[2], M, N, K, eps, dtype, status, rstd, st);
}

static int quant_views(const SFBTensor* x, const SFBTensor* codes, const SFBTensor* scales, int x_dtype, int granularity,
                       const char* op, View* vx, View* vc, View* vs) {
    const int xe = dtype_size(x_dtype);
    if (!xe || x_dtype == SFB_F8E4M3) return fail(SFB_ERR_INVALID_ARG, "%s: float dtype %d", op, x_dtype);
    int rc;
    if ((rc = make_view(x, "x", 1, 4, xe, vx))) return rc;
    if ((rc = make_view(codes, "codes", 1, 4, 1, vc))) return rc;
    for (int i = 0; i < 4; ++i)
        if (vx->size[i] != vc->size[i]) return fail(SFB_ERR_INVALID_ARG, "%s: float tensor and codes shapes differ", op);
    if (granularity == SFB_QUANT_PER_TENSOR) {
        if ((rc = make_view(scales, "scales", 1, 1, 4, vs))) return rc;
        if (vs->size[3] != 1) return fail(SFB_ERR_INVALID_ARG, "%s: per-tensor scale must have one element", op);
    } else if (granularity == SFB_QUANT_PER_BLOCK_HEAD) {
        if (vx->rank != 4) return fail(SFB_ERR_INVALID_ARG, "%s: per-(block, head) needs a rank-4 [NB, bs, Hkv, D] tensor", op);
        if ((rc = make_view(scales, "scales", 2, 2, 4, vs))) return rc;
        if (vs->size[2] != vx->size[0] || vs->size[3] != vx->size[2])
            return fail(SFB_ERR_INVALID_ARG, "%s: scales must be [NB, Hkv]", op);
    } else {
        return fail(SFB_ERR_INVALID_ARG, "%s: granularity %d", op, granularity);
    }
    return SFB_OK;
}

int sfb_quantize_fp8(const SFBTensor* x, SFBTensor* codes, SFBTensor* scales, int x_dtype, int granularity, void* stream) {
    SFB_TRACE_OP("quantize_fp8", stream, "dtype %d granularity %d", x_dtype, granularity);
    View vx, vc, vs;
    int rc = quant_views(x, codes, scales, x_dtype, granularity, "quantize", &vx, &vc, &vs);
    if (rc) return rc;
    if (vx.numel() == 0) return SFB_OK;
    return launch_quantize(vx, vc, vs, x_dtype, granularity, static_cast<cudaStream_t>(stream));
}

int sfb_dequantize_fp8(const SFBTensor* codes, const SFBTensor* scales, SFBTensor* out, int out_dtype, int granularity,
                       void* stream) {
    SFB_TRACE_OP("dequantize_fp8", stream, "dtype %d granularity %d", out_dtype, granularity);
    View vx, vc, vs;
    int rc = quant_views(out, codes, scales, out_dtype, granularity, "dequantize", &vx, &vc, &vs);
    if (rc) return rc;
    if (vx.numel() == 0) return SFB_OK;
    return launch_dequantize(vc, vs, vx, out_dtype, granularity, static_cast<cudaStream_t>(stream));
}

int sfb_rms_norm(const SFBTensor* x, const SFBTensor* residual, const SFBTensor* weight, SFBTensor* out, int dtype,
                 float eps, void* stream) {
    SFB_TRACE_OP("rms_norm", stream, "dtype %d residual %d", dtype, residual ? 1 : 0);
    const int e = dtype_size(dtype);
    if (!e || dtype == SFB_F8E4M3) return fail(SFB_ERR_INVALID_ARG, "rms_norm: dtype %d", dtype);
    View vx, vr, vw, vo;
    int rc;
    if ((rc = make_view(x, "x", 1, 2, e, &vx))) return rc;
    if ((rc = make_view(out, "out", 1, 2, e, &vo))) return rc;
    const int64_t rows = vx.size[2], hidden = vx.size[3];
    if (vo.size[2] != rows || vo.size[3] != hidden) return fail(SFB_ERR_INVALID_ARG, "rms_norm: out shape differs from x");
    if (residual) {
        if ((rc = make_view(residual, "residual", 1, 2, e, &vr))) return rc;
        if (vr.size[2] != rows || vr.size[3] != hidden) return fail(SFB_ERR_INVALID_ARG, "rms_norm: residual shape differs from x");
    }
    if (weight) {
        if ((rc = make_view(weight, "weight", 1, 1, e, &vw))) return rc;
        if (vw.size[3] != hidden) return fail(SFB_ERR_INVALID_ARG, "rms_norm: weight must have %lld elements", (long long)hidden);
    }
    if (rows == 0 || hidden == 0) return SFB_OK;
    NormArgs a{};
    a.x = vx.base; a.out = vo.base;
    a.residual = residual ? vr.base : nullptr;
    a.weight = weight ? vw.base : nullptr;
    a.rows = rows; a.hidden = hidden;
    a.x_stride = vx.stride[2]; a.out_stride = vo.stride[2]; a.res_stride = residual ? vr.stride[2] : 0;
    a.dtype = dtype; a.eps = eps;
    return launch_rms_norm(a, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
