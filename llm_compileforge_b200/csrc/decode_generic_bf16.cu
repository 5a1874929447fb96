// Instantiation of the shape-generic decode kernel for one dtype pair.
#include "decode_generic.cuh"

namespace sfb {
int launch_decode_generic_bf16(const DecodeArgs& a, cudaStream_t stream) {
    return generic::launch_generic_t<__nv_bfloat16, __nv_bfloat16>(a, stream);
}
}  // namespace sfb
