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

// Releases a buffer handed out through an sret descriptor.
SFB_API void serveforge_free(void* ptr) {
    if (ptr) cudaFree(ptr);
}

}  // extern "C"
