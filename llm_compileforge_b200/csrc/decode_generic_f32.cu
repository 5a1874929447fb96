// Instantiation of the shape-generic decode kernel for one dtype pair.
#include "decode_generic.cuh"

namespace sfb {
int launch_decode_generic_f32(const DecodeArgs& a, cudaStream_t stream) {
    return generic::launch_generic_t<float, float>(a, stream);
}
}  // namespace sfb
