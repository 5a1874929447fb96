// Step signal between the GPUs of a head-partitioned decode.
//
// sfb_paged_attention_decode_gather stores each GPU's heads straight into every GPU's copy of the output.
// Kernel completion makes those stores visible; what is left is telling the peers.  This kernel, launched on
// the same stream right after the decode, writes `step` into slot `rank` of every peer's flag array (release,
// system scope) and then waits until all `world` slots of its own array have reached `step`.  The wait is
// bounded: after the limit it sets SFB_STATUS_WAIT_TIMEOUT in the caller's status word and returns, so a
// missing peer costs a status bit, never a hung device.  One launch per GPU per step; the kernels of different
// GPUs wait for one another, so they must run on different GPUs (never as several ranks on one device, except
// with the phases split - every rank's SFB_PEER_SIGNAL launch first, then every rank's SFB_PEER_WAIT launch -
// as the single-GPU test does).

#include "sfb_common.cuh"

namespace sfb {
namespace {

struct PeerFlags {
    uint32_t* flags[8];  // flags[p] = GPU p's array of `world` slots
};

constexpr uint32_t kSignalSpin = 1u << 22;  // polls ~0.25 us apart: gives up after about a second

__global__ void peer_signal_wait_kernel(PeerFlags pf, int world, int rank, uint32_t step, int phases, int* status) {
    const int p = threadIdx.x;
    if (p >= world) return;
    if (phases & SFB_PEER_SIGNAL) {
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(pf.flags[p] + rank), "r"(step) : "memory");
    }
    if (!(phases & SFB_PEER_WAIT)) return;
    const uint32_t* mine = pf.flags[rank] + p;
    uint32_t seen = 0;
    for (uint32_t i = 0; i < kSignalSpin; ++i) {
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
        if ((int32_t)(seen - step) >= 0) return;  // wrap-safe "reached step"
        __nanosleep(200);
    }
    if (status) atomicOr(status, SFB_STATUS_WAIT_TIMEOUT);
}

}  // namespace
}  // namespace sfb

using namespace sfb;

extern "C" int sfb_peer_signal_wait(void* const* peer_flags, int world, int rank, uint32_t step, int phases, void* status,
                                    void* stream) {
    if (world < 1 || world > 8 || rank < 0 || rank >= world || !peer_flags || phases < 1 || phases > 3)
        return fail(SFB_ERR_INVALID_ARG, "peer_signal_wait: world must be 1..8, rank inside it, peer_flags given");
    PeerFlags pf{};
    for (int p = 0; p < world; ++p) {
        if (!peer_flags[p] || reinterpret_cast<uintptr_t>(peer_flags[p]) % 4) return fail(SFB_ERR_INVALID_ARG, "peer_signal_wait: peer_flags[%d] is null or misaligned", p);
        pf.flags[p] = static_cast<uint32_t*>(peer_flags[p]);
    }
    peer_signal_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(pf, world, rank, step, phases, static_cast<int*>(status));
    SFB_CUDA_CHECK(cudaGetLastError());
    return SFB_OK;
}
