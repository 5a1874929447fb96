// `_mlir_ciface_*` entry points in the calling convention the reference's runtime uses
// for compiled kernels (runtime/src/hal/cpu/executable.rs:23-29,159-200 of the reference;
// known-answer twin tests/data/golden/rms_norm.c:35-75):
//
//     void _mlir_ciface_<name>(void* sret, const memref* in0, const memref* in1, ...)
//
// The callee allocates its outputs and writes one memref descriptor per output into
// `sret`; the caller copies the data out and releases `allocated` through the library's
// `serveforge_free` (runtime/src/hal/cpu/device.rs:94-109).  There is no error channel in
// this convention (void), so failures leave a NULL `allocated` pointer in the descriptor
// and the text in sfb_last_error().  Pointers are device pointers; work runs on the
// default stream and is synchronised before returning, as the CPU convention implies.

#include <cstring>

#include "sfb_common.cuh"

using namespace sfb;

namespace {

SFBTensor wrap2(const SFBMemRef2* m, int elem) {
    SFBTensor t{};
    t.device = SFB_DEVICE_CUDA;
    t.rank = 2;
    t.elem_size = elem;
    t.r2 = *m;
    return t;
}
SFBTensor wrap1(const SFBMemRef1* m, int elem) {
    SFBTensor t{};
    t.device = SFB_DEVICE_CUDA;
    t.rank = 1;
    t.elem_size = elem;
    t.r1 = *m;
    return t;
}

}  // namespace

extern "C" {

// y = x * rsqrt(mean(x^2) + 1e-5) * w; x [rows, hidden] f32, w [hidden] f32 -> y [rows, hidden] f32.
// Same signature and epsilon as the reference's golden kernel `_mlir_ciface_rms_norm_f32`.
SFB_API void _mlir_ciface_sfb_rms_norm_f32(void* sret, const SFBMemRef2* x, const SFBMemRef1* w) {
    SFBMemRef2* out = static_cast<SFBMemRef2*>(sret);
    out->allocated = out->aligned = nullptr;
    out->offset = 0;
    out->sizes[0] = x->sizes[0];
    out->sizes[1] = x->sizes[1];
    out->strides[0] = x->sizes[1];
    out->strides[1] = 1;
    void* buf = nullptr;
    const size_t bytes = (size_t)x->sizes[0] * (size_t)x->sizes[1] * 4;
    if (bytes == 0) return;
    if (cudaMalloc(&buf, bytes) != cudaSuccess) {
        set_error("ciface rms_norm: cudaMalloc of %zu B failed", bytes);
        return;
    }
    SFBMemRef2 om = *out;
    om.allocated = om.aligned = buf;
    SFBTensor tx = wrap2(x, 4), tw = wrap1(w, 4), to = wrap2(&om, 4);
    if (sfb_rms_norm(&tx, nullptr, &tw, &to, SFB_F32, 1e-5f, nullptr) != SFB_OK || cudaStreamSynchronize(nullptr) != cudaSuccess) {
        cudaFree(buf);
        return;
    }
    out->allocated = out->aligned = buf;
}

// ---- the attention operators in the same convention -------------------------------------------------------------
// One exported function per (operator, element type) through the macros at the end; the bodies below are shared.
// Outputs are contiguous; every output's `allocated` is NULL when the call failed (text in sfb_last_error()).
// Scratch the kernels need is allocated and released inside the call.

}  // extern "C"

namespace {

template <int R>
struct MemRefOf;
template <> struct MemRefOf<1> { using type = SFBMemRef1; };
template <> struct MemRefOf<2> { using type = SFBMemRef2; };
template <> struct MemRefOf<3> { using type = SFBMemRef3; };
template <> struct MemRefOf<4> { using type = SFBMemRef4; };

template <int R>
SFBTensor wrap(const typename MemRefOf<R>::type* m, int elem) {
    SFBTensor t{};
    t.device = SFB_DEVICE_CUDA;
    t.rank = R;
    t.elem_size = elem;
    memcpy(&t.r1, m, sizeof(*m));  // the union's members all start at the same address
    return t;
}

// Writes a contiguous rank-R descriptor of `sizes` at `slot`, allocates its buffer (NULL on failure or zero size).
template <int R>
typename MemRefOf<R>::type* make_output(void* slot, const int64_t (&sizes)[R], int elem) {
    auto* m = static_cast<typename MemRefOf<R>::type*>(slot);
    m->allocated = m->aligned = nullptr;
    m->offset = 0;
    int64_t n = 1;
    for (int i = R - 1; i >= 0; --i) { m->sizes[i] = sizes[i]; m->strides[i] = n; n *= sizes[i]; }
    if (n <= 0) return m;
    void* buf = nullptr;
    if (cudaMalloc(&buf, (size_t)n * elem) != cudaSuccess) {
        set_error("ciface: cudaMalloc of %lld B failed", (long long)n * elem);
        return m;
    }
    m->allocated = m->aligned = buf;
    return m;
}

template <class M>
void drop_output(M* m) {
    if (m->allocated) cudaFree(m->allocated);
    m->allocated = m->aligned = nullptr;
}

struct Scratch {
    void* p = nullptr;
    bool get(int64_t bytes) { return bytes <= 0 || cudaMalloc(&p, (size_t)bytes) == cudaSuccess; }
    ~Scratch() { if (p) cudaFree(p); }
};

bool finish(int rc) { return rc == SFB_OK && cudaStreamSynchronize(nullptr) == cudaSuccess; }

// paged_attention(query [B,H,D], key_cache, value_cache [NB,bs,Hkv,D], block_table [B,max_blocks] i32, seq_lens [B] i32) -> [B,H,D]
void ciface_paged_attention(void* sret, const SFBMemRef3* q, const SFBMemRef4* kc, const SFBMemRef4* vc, const SFBMemRef2* table,
                            const SFBMemRef1* lens, int dtype) {
    const int e = dtype_size(dtype);
    const int64_t sizes[3] = {q->sizes[0], q->sizes[1], q->sizes[2]};
    SFBMemRef3* out = make_output<3>(sret, sizes, e);
    if (!out->allocated) return;
    const int64_t wsb = sfb_paged_attention_workspace_bytes(sizes[0], sizes[1], sizes[2], table->sizes[1], kc->sizes[1], 0);
    Scratch ws;
    if (wsb < 0 || !ws.get(wsb)) { set_error("ciface paged_attention: workspace of %lld B", (long long)wsb); drop_output(out); return; }
    SFBTensor tq = wrap<3>(q, e), tk = wrap<4>(kc, e), tv = wrap<4>(vc, e), tt = wrap<2>(table, 4), tl = wrap<1>(lens, 4), to = wrap<3>(out, e);
    if (!finish(sfb_paged_attention_decode(&tq, &tk, &tv, nullptr, nullptr, &tt, &tl, nullptr, &to, dtype, dtype, 0.f, 0, ws.p, wsb, nullptr)))
        drop_output(out);
}

// cache_write(key, value [T,Hkv,D], cu_tokens [B+1] i32, start_pos [B] i32, block_table [B,max_blocks] i32, key_cache, value_cache): no result
void ciface_cache_write(const SFBMemRef3* k, const SFBMemRef3* v, const SFBMemRef1* cu, const SFBMemRef1* start, const SFBMemRef2* table,
                        const SFBMemRef4* kc, const SFBMemRef4* vc, int dtype) {
    const int e = dtype_size(dtype);
    SFBTensor tk = wrap<3>(k, e), tv = wrap<3>(v, e), tc = wrap<1>(cu, 4), ts = wrap<1>(start, 4), tt = wrap<2>(table, 4);
    SFBTensor tkc = wrap<4>(kc, e), tvc = wrap<4>(vc, e);
    finish(sfb_cache_write(&tk, &tv, &tc, &ts, &tt, &tkc, &tvc, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, dtype, dtype,
                           k->sizes[0] > 0 ? k->sizes[0] : 1, nullptr));
}

// cache_read(block_table [R,max_blocks] i32, seq_lens [R] i32, key_cache, value_cache) -> key, value [R, max_blocks*bs, Hkv, D]
void ciface_cache_read(void* sret, const SFBMemRef2* table, const SFBMemRef1* lens, const SFBMemRef4* kc, const SFBMemRef4* vc, int dtype) {
    const int e = dtype_size(dtype);
    const int64_t sizes[4] = {table->sizes[0], table->sizes[1] * kc->sizes[1], kc->sizes[2], kc->sizes[3]};
    SFBMemRef4* ko = make_output<4>(sret, sizes, e);
    SFBMemRef4* vo = make_output<4>(static_cast<char*>(sret) + sizeof(SFBMemRef4), sizes, e);
    bool ok = ko->allocated && vo->allocated;
    if (ok) {
        SFBTensor tt = wrap<2>(table, 4), tl = wrap<1>(lens, 4), tkc = wrap<4>(kc, e), tvc = wrap<4>(vc, e), tko = wrap<4>(ko, e), tvo = wrap<4>(vo, e);
        ok = sfb_cache_read(&tkc, nullptr, &tt, &tl, &tko, dtype, dtype, nullptr, nullptr) == SFB_OK &&
             finish(sfb_cache_read(&tvc, nullptr, &tt, &tl, &tvo, dtype, dtype, nullptr, nullptr));
    }
    if (!ok) { drop_output(ko); drop_output(vo); }
}

// quantize(input [NB,bs,Hkv,D]) -> codes [NB,bs,Hkv,D] u8 (e4m3), scales [NB,Hkv] f32 (one per block and kv head)
void ciface_quantize(void* sret, const SFBMemRef4* x, int dtype) {
    const int64_t cs[4] = {x->sizes[0], x->sizes[1], x->sizes[2], x->sizes[3]}, ss[2] = {x->sizes[0], x->sizes[2]};
    SFBMemRef4* codes = make_output<4>(sret, cs, 1);
    SFBMemRef2* scales = make_output<2>(static_cast<char*>(sret) + sizeof(SFBMemRef4), ss, 4);
    bool ok = codes->allocated && scales->allocated;
    if (ok) {
        SFBTensor tx = wrap<4>(x, dtype_size(dtype)), tc = wrap<4>(codes, 1), ts = wrap<2>(scales, 4);
        ok = finish(sfb_quantize_fp8(&tx, &tc, &ts, dtype, SFB_QUANT_PER_BLOCK_HEAD, nullptr));
    }
    if (!ok) { drop_output(codes); drop_output(scales); }
}

// dequantize(codes [NB,bs,Hkv,D] u8, scales [NB,Hkv] f32) -> [NB,bs,Hkv,D]
void ciface_dequantize(void* sret, const SFBMemRef4* codes, const SFBMemRef2* scales, int dtype) {
    const int64_t sizes[4] = {codes->sizes[0], codes->sizes[1], codes->sizes[2], codes->sizes[3]};
    SFBMemRef4* out = make_output<4>(sret, sizes, dtype_size(dtype));
    if (!out->allocated) return;
    SFBTensor tc = wrap<4>(codes, 1), ts = wrap<2>(scales, 4), to = wrap<4>(out, dtype_size(dtype));
    if (!finish(sfb_dequantize_fp8(&tc, &ts, &to, dtype, SFB_QUANT_PER_BLOCK_HEAD, nullptr))) drop_output(out);
}

// scaled_dot_product_attention(q [B,H,Sq,D], k, v [B,Hkv,Skv,D]) -> [B,H,Sq,D]; scale 1/sqrt(D)
void ciface_attention(void* sret, const SFBMemRef4* q, const SFBMemRef4* k, const SFBMemRef4* v, int dtype, int mask_mode) {
    const int e = dtype_size(dtype);
    const int64_t sizes[4] = {q->sizes[0], q->sizes[1], q->sizes[2], q->sizes[3]};
    SFBMemRef4* out = make_output<4>(sret, sizes, e);
    if (!out->allocated) return;
    const int64_t wsb = sfb_attention_dense_workspace_bytes(sizes[0], sizes[1], k->sizes[1], sizes[2], k->sizes[2], sizes[3], dtype);
    Scratch ws;
    if (wsb < 0 || !ws.get(wsb)) { set_error("ciface attention: workspace of %lld B", (long long)wsb); drop_output(out); return; }
    SFBTensor tq = wrap<4>(q, e), tk = wrap<4>(k, e), tv = wrap<4>(v, e), to = wrap<4>(out, e);
    if (!finish(sfb_attention_dense(&tq, &tk, &tv, nullptr, &to, dtype, 0.f, mask_mode, ws.p, wsb, nullptr))) drop_output(out);
}

}  // namespace

extern "C" {

#define SFB_CIFACE_SET(sfx, DT)                                                                                                             \
    SFB_API void _mlir_ciface_sfb_paged_attention_##sfx(void* sret, const SFBMemRef3* q, const SFBMemRef4* kc, const SFBMemRef4* vc,         \
                                                        const SFBMemRef2* table, const SFBMemRef1* lens) {                                   \
        ciface_paged_attention(sret, q, kc, vc, table, lens, DT);                                                                           \
    }                                                                                                                                       \
    SFB_API void _mlir_ciface_sfb_cache_write_##sfx(void* sret, const SFBMemRef3* k, const SFBMemRef3* v, const SFBMemRef1* cu,              \
                                                    const SFBMemRef1* start, const SFBMemRef2* table, const SFBMemRef4* kc,                 \
                                                    const SFBMemRef4* vc) {                                                                 \
        (void)sret;                                                                                                                         \
        ciface_cache_write(k, v, cu, start, table, kc, vc, DT);                                                                             \
    }                                                                                                                                       \
    SFB_API void _mlir_ciface_sfb_cache_read_##sfx(void* sret, const SFBMemRef2* table, const SFBMemRef1* lens, const SFBMemRef4* kc,        \
                                                   const SFBMemRef4* vc) {                                                                  \
        ciface_cache_read(sret, table, lens, kc, vc, DT);                                                                                   \
    }                                                                                                                                       \
    SFB_API void _mlir_ciface_sfb_quantize_##sfx(void* sret, const SFBMemRef4* x) { ciface_quantize(sret, x, DT); }                          \
    SFB_API void _mlir_ciface_sfb_dequantize_##sfx(void* sret, const SFBMemRef4* codes, const SFBMemRef2* scales) {                          \
        ciface_dequantize(sret, codes, scales, DT);                                                                                         \
    }                                                                                                                                       \
    SFB_API void _mlir_ciface_sfb_scaled_dot_product_attention_##sfx(void* sret, const SFBMemRef4* q, const SFBMemRef4* k,                   \
                                                                     const SFBMemRef4* v) {                                                 \
        ciface_attention(sret, q, k, v, DT, SFB_MASK_NONE);                                                                                 \
    }                                                                                                                                       \
    SFB_API void _mlir_ciface_sfb_causal_attention_##sfx(void* sret, const SFBMemRef4* q, const SFBMemRef4* k, const SFBMemRef4* v) {        \
        ciface_attention(sret, q, k, v, DT, SFB_MASK_CAUSAL_TOP_LEFT);                                                                      \
    }
SFB_CIFACE_SET(f32, SFB_F32)
SFB_CIFACE_SET(bf16, SFB_BF16)
#undef SFB_CIFACE_SET

// Releases a buffer handed out through an sret descriptor.
SFB_API void serveforge_free(void* ptr) {
    if (ptr) cudaFree(ptr);
}

}  // extern "C"
