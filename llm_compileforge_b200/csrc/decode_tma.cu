// Placeholder until the TMA + tensor-core decode kernel lands: every shape is
// reported as not covered, so the generic kernel runs.
#include "sfb_common.cuh"

namespace sfb {
int launch_decode_tma(const DecodeArgs&, cudaStream_t) { return SFB_ERR_UNSUPPORTED; }
}  // namespace sfb
