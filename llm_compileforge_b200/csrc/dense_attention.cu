// Dense attention over [B, H, S, D] tensors and dense reads of the paged pool - the two operators the reference's
// hosts use when they are not speaking "paged":
//
//   sfb_attention_dense   python_runtime/hal/pytorch_backend/_ops_attention.py:13-53 (scaled_dot_product_attention with
//                         its positional-mask convention) and runtime/src/engine/kernels.rs:97-302 (the Rust runtime's
//                         fp32 attention_forward: head-major operands, top-left causal mask in prefill, none in decode)
//   sfb_cache_read        sf-dialect/include/Sf/HALOps.td:190-194 `cache_read`, python_runtime/engine/cache_manager.py:173-197
//                         read_paged: the dense [R, max_seq_len, Hkv, D] copy of what the block tables point at
//
// Dense attention does not get kernels of its own: q is repacked token-major, K / V are repacked as a private paged pool
// (16-token blocks, identity block tables) and the chunked-prefill kernels run over that with one visible length per
// query row - the tcgen05 kernel for bf16 / fp16 with D = 128, the decode kernels otherwise (fp32, other head sizes).
// Every mask the two references use is a prefix of keys per query row: none (all keys), top-left causal (row i sees
// keys 0..i), bottom-right causal (row i sees keys 0..Skv-Sq+i), positional (key j is visible to query i iff
// pos[i] >= pos[j], a prefix when the positions do not decrease; a decreasing pair is flagged, not guessed at).

#include <algorithm>

#include "sfb_common.cuh"

namespace sfb {
namespace {

struct Copy4 {
    const char* src;
    char* dst;
    int64_t size[3];        // outer sizes; the innermost run of `inner_vecs` 16-byte pieces is contiguous on both sides
    int64_t src_stride[3];  // bytes
    int64_t dst_stride[3];
    int inner_vecs;
};

// dst[a, b, c, :] = src[a, b, c, :] for two different stride sets; one 16-byte piece per thread and step.
__global__ void strided_copy_kernel(Copy4 c) {
    const int64_t rows = c.size[0] * c.size[1] * c.size[2];
    const int64_t total = rows * c.inner_vecs;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / c.inner_vecs;
        const int v = (int)(i - row * c.inner_vecs);
        const int64_t i2 = row % c.size[2], r1 = row / c.size[2];
        const int64_t i1 = r1 % c.size[1], i0 = r1 / c.size[1];
        const uint4 x = *reinterpret_cast<const uint4*>(c.src + i0 * c.src_stride[0] + i1 * c.src_stride[1] + i2 * c.src_stride[2] + v * 16);
        *reinterpret_cast<uint4*>(c.dst + i0 * c.dst_stride[0] + i1 * c.dst_stride[1] + i2 * c.dst_stride[2] + v * 16) = x;
    }
}

int launch_copy(const Copy4& c, cudaStream_t st) {
    const int64_t total = c.size[0] * c.size[1] * c.size[2] * c.inner_vecs;
    if (total == 0) return SFB_OK;
    const int64_t blocks = ceil_div(total, 256);
    strided_copy_kernel<<<(unsigned)(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0, st>>>(c);
    SFB_CUDA_CHECK(cudaGetLastError());
    return SFB_OK;
}

// Per batch entry: packed-query offsets, context lengths, identity block tables; per query row its visible length.
__global__ void dense_setup_kernel(int batch, int sq, int skv, int nblk, int mask_mode, const float* positions, int64_t pos_batch_stride,
                                   int32_t* cu_q, int32_t* ctx, int32_t* tables, int32_t* row_limits) {
    const int b = blockIdx.y;
    const int tid = blockIdx.x * blockDim.x + threadIdx.x, step = gridDim.x * blockDim.x;
    if (tid == 0) {
        cu_q[b] = b * sq;
        if (b == batch - 1) cu_q[batch] = batch * sq;
        ctx[b] = skv;
    }
    for (int j = tid; j < nblk; j += step) tables[(int64_t)b * nblk + j] = b * nblk + j;
    const float* pos = positions ? positions + b * pos_batch_stride : nullptr;
    for (int i = tid; i < sq; i += step) {
        int limit = skv;
        if (mask_mode == SFB_MASK_CAUSAL_TOP_LEFT) limit = min(i + 1, skv);
        if (mask_mode == SFB_MASK_CAUSAL_BOTTOM_RIGHT) limit = min(max(skv - sq + i + 1, 0), skv);
        if (mask_mode == SFB_MASK_POSITIONS) {  // number of keys with pos[j] <= pos[i]: upper bound in the non-decreasing row
            const float mine = pos[i];
            int lo = 0, hi = skv;
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if (pos[mid] <= mine) lo = mid + 1;
                else hi = mid;
            }
            limit = lo;
        }
        row_limits[(int64_t)b * sq + i] = limit;
    }
}

// Positions that decrease somewhere (or are NaN) do not describe a prefix per row: flag them.
__global__ void positions_check_kernel(int s, const float* positions, int64_t pos_batch_stride, int* status) {
    const float* pos = positions + blockIdx.y * pos_batch_stride;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x + 1; i < s; i += gridDim.x * blockDim.x)
        if (!(pos[i] >= pos[i - 1])) atomicOr(status, SFB_STATUS_UNSORTED_POSITIONS);
}

SFBTensor tensor_of(void* base, int elem, int rank, const int64_t* sizes) {
    SFBTensor t{};
    t.device = SFB_DEVICE_CUDA;
    t.rank = rank;
    t.elem_size = elem;
    t.r4.allocated = t.r4.aligned = base;
    t.r4.offset = 0;
    int64_t* sz = rank == 1 ? t.r1.sizes : rank == 2 ? t.r2.sizes : rank == 3 ? t.r3.sizes : t.r4.sizes;
    int64_t* st = rank == 1 ? t.r1.strides : rank == 2 ? t.r2.strides : rank == 3 ? t.r3.strides : t.r4.strides;
    int64_t stride = 1;
    for (int i = rank - 1; i >= 0; --i) { sz[i] = sizes[i]; st[i] = stride; stride *= sizes[i]; }
    return t;
}

int64_t round256(int64_t x) { return ceil_div(x, 256) * 256; }

struct DenseLayout {
    int64_t inner, limits, cu_q, ctx, tables, q_tok, k_pool, v_pool, out_tok, total;
    int64_t nblk;
};

DenseLayout dense_layout(int64_t B, int64_t H, int64_t Hkv, int64_t Sq, int64_t Skv, int64_t D, int e) {
    DenseLayout L{};
    L.nblk = ceil_div(Skv, 16);
    const int64_t T = B * Sq;
    int64_t off = 0;
    L.inner = off; off += sfb_prefill_workspace_bytes(T);  // status word first, then the decode route's per-row arrays
    L.limits = off; off += round256(T * 4);
    L.cu_q = off; off += round256((B + 1) * 4);
    L.ctx = off; off += round256(B * 4);
    L.tables = off; off += round256(B * L.nblk * 4);
    L.q_tok = off; off += round256(T * H * D * e);
    L.k_pool = off; off += round256(B * L.nblk * 16 * Hkv * D * e);
    L.v_pool = off; off += round256(B * L.nblk * 16 * Hkv * D * e);
    L.out_tok = off; off += round256(T * H * D * e);
    L.total = off;
    return L;
}

// out[r, t, h, :] = value of token t of request r (pool[table[r, t / bs], t % bs, h, :], times the block's scale for
// e4m3 codes), zero for t >= seq_lens[r].
template <typename OutT, bool FP8>
__global__ void cache_read_kernel(const char* pool, const float* scales, const int32_t* tables, int64_t table_stride, const int32_t* seq_lens,
                                  OutT* out, int max_seq_len, int n_kv_heads, int head_dim, int block_size, int max_blocks,
                                  int64_t n_pool_blocks, int64_t ps0, int64_t ps1, int64_t ps2, int64_t ss0, int64_t ss1, int pool_elem,
                                  int* status) {
    const int r = blockIdx.y;
    int len = seq_lens[r];
    if (len > max_blocks * block_size) len = max_blocks * block_size;
    const int vec = 16 / (int)sizeof(OutT);  // output elements per thread and step
    const int per_row = head_dim / vec;
    const int64_t total = (int64_t)max_seq_len * n_kv_heads * per_row;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int piece = (int)(i % per_row);
        const int64_t th = i / per_row;
        const int h = (int)(th % n_kv_heads), t = (int)(th / n_kv_heads);
        __align__(16) OutT vals[16 / sizeof(OutT)];
#pragma unroll
        for (int k = 0; k < vec; ++k) vals[k] = OutT(0.f);
        if (t < len) {
            const int64_t phys = tables[(int64_t)r * table_stride + t / block_size];
            if (phys < 0 || phys >= n_pool_blocks) {
                if (status) atomicOr(status, SFB_STATUS_BAD_BLOCK_ID);
            } else {
                const char* src = pool + (phys * ps0 + (int64_t)(t % block_size) * ps1 + (int64_t)h * ps2 + (int64_t)piece * vec) * pool_elem;
                if constexpr (FP8) {
                    const float sc = scales[phys * ss0 + h * ss1];
                    const __nv_fp8_storage_t* c = reinterpret_cast<const __nv_fp8_storage_t*>(src);
#pragma unroll
                    for (int k = 0; k < vec; ++k) vals[k] = OutT(__half2float(__half(__nv_cvt_fp8_to_halfraw(c[k], __NV_E4M3))) * sc);
                } else {
                    *reinterpret_cast<uint4*>(vals) = *reinterpret_cast<const uint4*>(src);
                }
            }
        }
        OutT* dst = out + (((int64_t)r * max_seq_len + t) * n_kv_heads + h) * head_dim + (int64_t)piece * vec;
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(vals);
    }
}

}  // namespace
}  // namespace sfb

using namespace sfb;

extern "C" {

int64_t sfb_attention_dense_workspace_bytes(int64_t batch, int64_t n_heads, int64_t n_kv_heads, int64_t q_len, int64_t kv_len,
                                            int64_t head_dim, int dtype) {
    const int e = dtype_size(dtype);
    if (batch < 0 || n_heads <= 0 || n_kv_heads <= 0 || q_len < 0 || kv_len < 0 || head_dim <= 0 || !e || dtype == SFB_F8E4M3)
        return SFB_ERR_INVALID_ARG;
    return dense_layout(batch, n_heads, n_kv_heads, q_len, kv_len, head_dim, e).total;
}

int sfb_attention_dense(const SFBTensor* q, const SFBTensor* k, const SFBTensor* v, const SFBTensor* positions, SFBTensor* out, int dtype,
                        float scale, int mask_mode, void* workspace, int64_t workspace_bytes, void* stream) {
    SFB_TRACE_OP("attention_dense", stream, "dtype %d mask %d", dtype, mask_mode);
    const int e = dtype_size(dtype);
    if (!e || dtype == SFB_F8E4M3) return fail(SFB_ERR_INVALID_ARG, "attention_dense: dtype %d", dtype);
    if (mask_mode < SFB_MASK_NONE || mask_mode > SFB_MASK_POSITIONS) return fail(SFB_ERR_INVALID_ARG, "attention_dense: mask mode %d", mask_mode);
    View vq, vk, vv, vo, vp;
    int rc;
    if ((rc = make_view(q, "q", 4, 4, e, &vq))) return rc;
    if ((rc = make_view(k, "k", 4, 4, e, &vk))) return rc;
    if ((rc = make_view(v, "v", 4, 4, e, &vv))) return rc;
    if ((rc = make_view(out, "out", 4, 4, e, &vo))) return rc;
    const int64_t B = vq.size[0], H = vq.size[1], Sq = vq.size[2], D = vq.size[3];
    const int64_t Hkv = vk.size[1], Skv = vk.size[2];
    for (int i = 0; i < 4; ++i) {
        if (vk.size[i] != vv.size[i]) return fail(SFB_ERR_INVALID_ARG, "attention_dense: k and v shapes differ");
        if (vo.size[i] != vq.size[i]) return fail(SFB_ERR_INVALID_ARG, "attention_dense: out shape differs from q");
    }
    if (vk.size[0] != B || vk.size[3] != D) return fail(SFB_ERR_INVALID_ARG, "attention_dense: batch / head_dim of q and k differ");
    if (Hkv <= 0 || H % Hkv) return fail(SFB_ERR_INVALID_ARG, "attention_dense: %lld query heads not a multiple of %lld kv heads", (long long)H, (long long)Hkv);
    if ((D * e) % 16) return fail(SFB_ERR_UNSUPPORTED, "attention_dense: head_dim * elem_size must be a multiple of 16 bytes");
    for (const View* w : {&vq, &vk, &vv, &vo}) {
        if (reinterpret_cast<uintptr_t>(w->base) % 16) return fail(SFB_ERR_UNSUPPORTED, "attention_dense: tensors must be 16-byte aligned");
        for (int i = 0; i < 3; ++i)
            if (w->size[i] > 1 && (w->stride[i] * e) % 16) return fail(SFB_ERR_UNSUPPORTED, "attention_dense: strides must be multiples of 16 bytes");
    }
    if (mask_mode == SFB_MASK_POSITIONS) {
        if (!positions) return fail(SFB_ERR_INVALID_ARG, "attention_dense: SFB_MASK_POSITIONS needs the positions tensor");
        if ((rc = make_view(positions, "positions", 2, 2, 4, &vp))) return rc;
        if (Sq != Skv || vp.size[3] != Sq || (vp.size[2] != B && vp.size[2] != 1))
            return fail(SFB_ERR_INVALID_ARG, "attention_dense: positions must be [B or 1, S] with S = q_len = kv_len");
    }
    if (B == 0 || Sq == 0) return SFB_OK;
    if (Skv == 0) return fail(SFB_ERR_INVALID_ARG, "attention_dense: no keys");
    if (B * Sq > 0x7fffffffLL || B * ceil_div(Skv, 16) > 0x7ffffffeLL) return fail(SFB_ERR_UNSUPPORTED, "attention_dense: too many rows or blocks");
    const DenseLayout L = dense_layout(B, H, Hkv, Sq, Skv, D, e);
    if (!workspace || workspace_bytes < L.total)
        return fail(SFB_ERR_WORKSPACE, "attention_dense: workspace of %lld B needed, %lld given", (long long)L.total, (long long)(workspace ? workspace_bytes : 0));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    char* ws = static_cast<char*>(workspace);
    const int64_t T = B * Sq, nblk = L.nblk;
    int32_t* limits = reinterpret_cast<int32_t*>(ws + L.limits);
    int32_t* cu_q = reinterpret_cast<int32_t*>(ws + L.cu_q);
    int32_t* ctx = reinterpret_cast<int32_t*>(ws + L.ctx);
    int32_t* tables = reinterpret_cast<int32_t*>(ws + L.tables);
    const float* pos = mask_mode == SFB_MASK_POSITIONS ? reinterpret_cast<const float*>(vp.base) : nullptr;
    const int64_t pos_stride = mask_mode == SFB_MASK_POSITIONS && vp.size[2] > 1 ? vp.stride[2] : 0;
    {
        dim3 grid((unsigned)std::min<int64_t>(ceil_div(std::max(Sq, nblk), 256), 64), (unsigned)B);
        if (B > 65535) return fail(SFB_ERR_UNSUPPORTED, "attention_dense: batch %lld exceeds 65535", (long long)B);
        dense_setup_kernel<<<grid, 256, 0, st>>>((int)B, (int)Sq, (int)Skv, (int)nblk, mask_mode, pos, pos_stride, cu_q, ctx, tables, limits);
        SFB_CUDA_CHECK(cudaGetLastError());
    }
    // repack: q token-major, K / V as a pool of 16-token blocks (rows past kv_len zero)
    if (Skv % 16) {
        SFB_CUDA_CHECK(cudaMemsetAsync(ws + L.k_pool, 0, (size_t)(B * nblk * 16 * Hkv * D * e), st));
        SFB_CUDA_CHECK(cudaMemsetAsync(ws + L.v_pool, 0, (size_t)(B * nblk * 16 * Hkv * D * e), st));
    }
    const int inner = (int)(D * e / 16);
    Copy4 cq{vq.base, ws + L.q_tok, {B, H, Sq}, {vq.stride[0] * e, vq.stride[1] * e, vq.stride[2] * e}, {Sq * H * D * e, D * e, H * D * e}, inner};
    if ((rc = launch_copy(cq, st))) return rc;
    Copy4 ck{vk.base, ws + L.k_pool, {B, Hkv, Skv}, {vk.stride[0] * e, vk.stride[1] * e, vk.stride[2] * e}, {nblk * 16 * Hkv * D * e, D * e, Hkv * D * e}, inner};
    if ((rc = launch_copy(ck, st))) return rc;
    Copy4 cv = ck;
    cv.src = vv.base; cv.dst = ws + L.v_pool;
    cv.src_stride[0] = vv.stride[0] * e; cv.src_stride[1] = vv.stride[1] * e; cv.src_stride[2] = vv.stride[2] * e;
    if ((rc = launch_copy(cv, st))) return rc;

    const int64_t qs[3] = {T, H, D}, ps[4] = {B * nblk, 16, Hkv, D}, ts[2] = {B, nblk}, cs[1] = {B + 1}, ls[1] = {B}, rs[1] = {T};
    SFBTensor tq = tensor_of(ws + L.q_tok, e, 3, qs), to = tensor_of(ws + L.out_tok, e, 3, qs);
    SFBTensor tk = tensor_of(ws + L.k_pool, e, 4, ps), tv = tensor_of(ws + L.v_pool, e, 4, ps);
    SFBTensor tt = tensor_of(tables, 4, 2, ts), tc = tensor_of(cu_q, 4, 1, cs), tl = tensor_of(ctx, 4, 1, ls), tr = tensor_of(limits, 4, 1, rs);
    if (mask_mode == SFB_MASK_NONE)
        rc = sfb_prefill_paged(&tq, &tk, &tv, &tt, &tc, &tl, &to, dtype, scale, 0, Sq, ws + L.inner, L.limits - L.inner, stream);
    else
        rc = sfb_prefill_paged_rows(&tq, &tk, &tv, &tt, &tc, &tl, &tr, &to, dtype, scale, Sq, ws + L.inner, L.limits - L.inner, stream);
    if (rc) return rc;
    if (mask_mode == SFB_MASK_POSITIONS && Sq > 1) {  // after the attention call, which clears the status word at its start
        dim3 grid((unsigned)std::min<int64_t>(ceil_div(Sq, 256), 64), (unsigned)(vp.size[2]));
        positions_check_kernel<<<grid, 256, 0, st>>>((int)Sq, pos, vp.size[2] > 1 ? vp.stride[2] : 0, reinterpret_cast<int*>(ws));
        SFB_CUDA_CHECK(cudaGetLastError());
    }
    Copy4 co{ws + L.out_tok, vo.base, {B, H, Sq}, {Sq * H * D * e, D * e, H * D * e}, {vo.stride[0] * e, vo.stride[1] * e, vo.stride[2] * e}, inner};
    return launch_copy(co, st);
}

int sfb_cache_read(const SFBTensor* cache, const SFBTensor* scale, const SFBTensor* block_tables, const SFBTensor* seq_lens, SFBTensor* out,
                   int cache_dtype, int out_dtype, void* status, void* stream) {
    SFB_TRACE_OP("cache_read", stream, "pool dtype %d -> %d", cache_dtype, out_dtype);
    const int ce = dtype_size(cache_dtype), oe = dtype_size(out_dtype);
    if (!ce || !oe || out_dtype == SFB_F8E4M3) return fail(SFB_ERR_INVALID_ARG, "cache_read: dtypes %d -> %d", cache_dtype, out_dtype);
    const bool fp8 = cache_dtype == SFB_F8E4M3;
    if (!fp8 && cache_dtype != out_dtype) return fail(SFB_ERR_INVALID_ARG, "cache_read: a pool that is not e4m3 is read in its own type");
    if (fp8 != (scale != nullptr)) return fail(SFB_ERR_INVALID_ARG, "cache_read: scales go with an e4m3 pool, and only with it");
    View vc, vs, vt, vl, vo;
    int rc;
    if ((rc = make_view(cache, "cache", 4, 4, ce, &vc))) return rc;
    if ((rc = make_view(block_tables, "block_tables", 2, 2, 4, &vt))) return rc;
    if ((rc = make_view(seq_lens, "seq_lens", 1, 1, 4, &vl))) return rc;
    if ((rc = make_view(out, "out", 4, 4, oe, &vo))) return rc;
    const int64_t NB = vc.size[0], bs = vc.size[1], Hkv = vc.size[2], D = vc.size[3];
    const int64_t R = vt.size[2], max_blocks = vt.size[3], max_len = vo.size[1];
    if (vo.size[0] != R || vo.size[2] != Hkv || vo.size[3] != D) return fail(SFB_ERR_INVALID_ARG, "cache_read: out must be [R, max_seq_len, Hkv, D]");
    if (vl.size[3] != R || (R > 1 && vl.stride[3] != 1)) return fail(SFB_ERR_INVALID_ARG, "cache_read: seq_lens must be a contiguous int32 [R]");
    if (vo.stride[3] != 1 || vo.stride[2] != D || vo.stride[1] != Hkv * D || (R > 1 && vo.stride[0] != max_len * Hkv * D))
        return fail(SFB_ERR_UNSUPPORTED, "cache_read: out must be contiguous");
    if (bs <= 0 || (D * oe) % 16 || (D * ce) % (fp8 ? 16 / oe : 16) || reinterpret_cast<uintptr_t>(vo.base) % 16 || reinterpret_cast<uintptr_t>(vc.base) % 16)
        return fail(SFB_ERR_UNSUPPORTED, "cache_read: rows must be whole 16-byte pieces and 16-byte aligned");
    if (!fp8)
        for (int i = 0; i < 3; ++i)
            if (vc.size[i] > 1 && (vc.stride[i] * ce) % 16) return fail(SFB_ERR_UNSUPPORTED, "cache_read: pool strides must be multiples of 16 bytes");
    if (fp8) {
        if ((rc = make_view(scale, "scale", 2, 2, 4, &vs))) return rc;
        if (vs.size[2] != NB || vs.size[3] != Hkv) return fail(SFB_ERR_INVALID_ARG, "cache_read: scales must be [NB, Hkv]");
    }
    if (R == 0 || max_len == 0) return SFB_OK;
    if (R > 65535 || max_len > 0x7fffffffLL || max_blocks * bs > 0x7fffffffLL) return fail(SFB_ERR_UNSUPPORTED, "cache_read: more than 65535 requests or 2^31 tokens");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t work = max_len * Hkv * (D * oe / 16);
    dim3 grid((unsigned)std::min<int64_t>(ceil_div(work, 256), 148 * 8), (unsigned)R);
    const char* pool = vc.base;
    const float* sc = fp8 ? reinterpret_cast<const float*>(vs.base) : nullptr;
    const int32_t* tb = reinterpret_cast<const int32_t*>(vt.base);
    const int32_t* ln = reinterpret_cast<const int32_t*>(vl.base);
    const int64_t ss0 = fp8 ? vs.stride[2] : 0, ss1 = fp8 ? vs.stride[3] : 0;
#define SFB_CACHE_READ(OutT, FP8)                                                                                                           \
    cache_read_kernel<OutT, FP8><<<grid, 256, 0, st>>>(pool, sc, tb, vt.stride[2], ln, reinterpret_cast<OutT*>(vo.base), (int)max_len, (int)Hkv, \
                                                       (int)D, (int)bs, (int)max_blocks, NB, vc.stride[0], vc.stride[1], vc.stride[2], ss0, \
                                                       ss1, ce, static_cast<int*>(status))
    if (out_dtype == SFB_F32) { if (fp8) SFB_CACHE_READ(float, true); else SFB_CACHE_READ(float, false); }
    else if (out_dtype == SFB_BF16) { if (fp8) SFB_CACHE_READ(__nv_bfloat16, true); else SFB_CACHE_READ(__nv_bfloat16, false); }
    else { if (fp8) SFB_CACHE_READ(__half, true); else SFB_CACHE_READ(__half, false); }
#undef SFB_CACHE_READ
    SFB_CUDA_CHECK(cudaGetLastError());
    return SFB_OK;
}

}  // extern "C"
