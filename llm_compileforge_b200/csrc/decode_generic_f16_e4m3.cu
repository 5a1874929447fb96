// Instantiation of the shape-generic decode kernel for one dtype pair.
#include "decode_generic.cuh"

namespace sfb {
int launch_decode_generic_f16_e4m3(const DecodeArgs& a, cudaStream_t stream) {
    return generic::launch_generic_t<__half, uint8_t>(a, stream);
}
}  // namespace sfb
