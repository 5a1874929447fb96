// RMSNorm fused into the matmul that follows it, on the sm_100a tensor cores.
//
// Replaces the reference's `fused_rms_norm_matmul`
// (python_runtime/hal/pytorch_backend/_ops_norm.py:47-65; sf-dialect SfPasses.td:91-92 fuses
// rms_norm -> matmul into it):   y = ( x * rsqrt(mean(x^2) + eps) * g ) @ W,   x [M, K], g [K], W [K, N].
//
// The row factor commutes with the contraction:  y[m, :] = rstd[m] * ( x[m, :] @ (diag(g) W) ).
// So the weight is folded once (fold_norm_weight_kernel: Wg = diag(g) W, weights are static in serving), the
// GEMM runs on the RAW activations straight out of HBM - the normalised activations are never written or
// re-read - and rstd scales the accumulators on their way out.  Where rstd comes from depends on M: for few rows
// (decode) the epilogue warps take each row's sum of squares from the very A tiles the tensor core consumes, while
// the MMAs run, so the operator stays one launch; those shared-memory reads cost the MMAs about a tenth of their
// operand bandwidth, so for many rows (prefill) a pre-pass (row_rstd_kernel, x read once) supplies rstd instead.
//
// Two kernels: one thread block per 128 x {256, 128, 64} tile (below), and a cluster of two thread blocks per
// 256 x 256 tile (cta_group::2, further down) for shapes with enough tiles and a workspace for the pre-pass; the
// launcher at the end of the file prices both by what an SM has to take in and runs the cheaper.
//
// Persistent thread blocks (one per SM) walk the tiles of y; the accumulator is double-buffered in tensor memory
// (2 x 256 columns), so tile i drains through the epilogue warps while tile i+1's MMAs run:
//   warp 4    TMA producer: per 64-wide K step a [128 rows x 128 B] box of x (K-major, 128B swizzle) and one
//             [64 k x 128 B] box of Wg (N-major) per 64 columns of the tile; four or six stages
//   warp 5    issues tcgen05.mma.cta_group::1.kind::f16, M 128, N = tile width, K 16, four per stage, accumulator =
//             tensor-memory columns of fp32 (two sets, alternating); tcgen05.commit frees the stage / publishes the
//             accumulator
//   warps 0-3 one thread per output row: reads its row of every A stage from shared memory (16-byte chunks in
//             a rotated order, so a quarter-warp never hits one bank twice; the swizzle only permutes chunks
//             inside the row, the sum does not care), then tcgen05.ld the accumulator row, times rstd, 16-bit
//             pack, 16-byte stores
// Every wait is bounded; a stuck pipeline sets SFB_STATUS_WAIT_TIMEOUT in *status and the block leaves
// through the common teardown, which releases tensor memory.
// Bound: 2*M*N*K flops on the tensor pipe.  What keeps the pipe from being busy all the time: the 48 KB a block takes
// in per K step (110 GB/s per SM), and the instruction chain of the one MMA-issuing thread between two K steps (see
// the note at mma_ss); the cluster kernel halves both.
// HBM traffic is x once per N tile (L2 keeps it) and Wg once per M tile.

#include <cuda.h>

#include <algorithm>
#include <mutex>
#include <type_traits>

#include "sfb_common.cuh"

namespace sfb {
namespace {

constexpr int kTileM = 128, kTileN = 256, kStepK = 64, kMaxStages = 8;
constexpr int kABytes = kTileM * kStepK * 2;       // 16 KB
constexpr int kBBlockBytes = kStepK * 128;         // one [64 k][64 n] block: 8 KB
constexpr int kThreads = 192;
constexpr uint32_t kSpin = 1u << 21;
constexpr int64_t kPrepassRows = 2048;  // from this many rows on, row statistics come from a pre-pass instead of the A tiles

enum { B_FULL = 0, B_EMPTY = kMaxStages, B_ACC_FULL = 2 * kMaxStages, B_ACC_EMPTY = 2 * kMaxStages + 2, B_COUNT = 2 * kMaxStages + 4 };
// Tile widths: 256 columns for large problems; 128 and 64 when 256-wide tiles would leave SMs without one (few rows).
// Pipeline depth per width: 192 KB of operands in flight per SM - four 48 KB stages (256), six 32 KB stages (128),
// four stages of TWO K steps each (64-wide tiles with an SM each: 2 x 24 KB per stage), or two resident thread blocks of
// four 24 KB stages when there are more 64-wide tiles than SMs.  With narrow tiles the MMAs are short (an N = 64 MMA
// occupies the pipe for about 50 cycles, four of them 200) and what the MMA warp's one thread executes between them
// - barrier wait about 80 cycles, commit 65, loop - is time the pipe idles: measured 630 cycles per K step with the
// first version of that loop, about 400 now (840 per two-step stage with the trace stamps in).
constexpr int smem_bytes(int tn, int stages, int ksub) { return stages * ksub * (kABytes + (tn / 64) * kBBlockBytes) + B_COUNT * 8 + 16 + 1024; }

struct GemmArgs {
    void* out;
    int64_t out_stride;  // elements between output rows
    int M, N, K;
    int tiles_n, tiles_total;
    int a_bytes;  // bytes one K step's box of x brings in: 128 per row, kABytes unless there are fewer than 128 rows in all
    float eps;
    int* status;
    const float* rstd;  // per-row rsqrt(mean(x^2) + eps) from the statistics pre-pass; nullptr: taken in this kernel from the A tiles
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kSpin; ++i) {
        uint32_t done;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// The MMA-issuing thread is alone in its warp and every instruction it runs between two MMAs is time the tensor pipe
// idles (an MMA issue returns when the pipe accepts it, i.e. when the one before has finished), so its loop is kept
// short: descriptors are a per-kernel constant plus the stage offset (low word: start address and leading offset in
// 16-byte units; high word: stride offset, version, swizzle mode), stage and phase are running counters.
__device__ __forceinline__ void mma_ss(uint32_t d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                       uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n .reg .b64 da, db;\n mov.b64 da, {%1, %2};\n mov.b64 db, {%3, %4};\n setp.ne.b32 p, %6, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n}\n"
        ::"r"(d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,"
        "%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// Shared-memory matrix descriptor (sm_100 format): start address, leading and stride byte offsets in
// 16-byte units, version 1, 128-byte swizzle.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3fff);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
__device__ __forceinline__ uint32_t desc_lo(uint32_t addr, uint32_t lbo_bytes) { return (uint32_t)smem_desc(addr, lbo_bytes, 0); }
__device__ __forceinline__ uint32_t desc_hi(uint32_t sbo_bytes) { return (uint32_t)(smem_desc(0, 0, sbo_bytes) >> 32); }
// Instruction descriptor for kind::f16: fp32 accumulate, 16-bit A/B, A K-major, B MN-major, M x N tile.
__host__ __device__ constexpr uint32_t instr_desc(bool bf16, int m, int n) {
    return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | (1u << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}
template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    uint32_t r;
    if constexpr (BF16) asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    else asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
template <bool BF16>
__device__ __forceinline__ float sumsq8(uint4 w) {  // sum of squares of eight 16-bit values
    float s = 0.f;
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float lo, hi;
        if constexpr (BF16) {
            lo = __uint_as_float(u[i] << 16);
            hi = __uint_as_float(u[i] & 0xffff0000u);
        } else {
            const __half2 h = *reinterpret_cast<const __half2*>(&u[i]);
            lo = __low2float(h);
            hi = __high2float(h);
        }
        s = fmaf(lo, lo, s);
        s = fmaf(hi, hi, s);
    }
    return s;
}

template <bool BF16, bool STATS, int TN, int kStages, int KSUB>
__global__ void __launch_bounds__(kThreads, 1)
norm_matmul_tcgen05_kernel(const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap bmap, const GemmArgs a) {
    extern __shared__ uint8_t smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int kSub = kABytes + (TN / 64) * kBBlockBytes;  // one 64-wide K step: a box of x and TN / 64 boxes of the weight
    constexpr int kStage = KSUB * kSub;                       // a pipeline stage = KSUB such steps behind one pair of barriers
    const int n_k = (a.K + kStepK * KSUB - 1) / (kStepK * KSUB);  // a ragged last step reads zeros (TMA fills what lies outside)

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    uint64_t* bars = reinterpret_cast<uint64_t*>(base_ptr + kStages * kStage);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + B_COUNT);
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    auto a_stage = [&](int s) { return base + (uint32_t)s * kStage; };
    auto b_stage = [&](int s) { return base + (uint32_t)s * kStage + kABytes; };

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar(B_FULL + s), 1);
            mbar_init(bar(B_EMPTY + s), STATS ? 5 : 1);  // the MMA warp's commit (+ the four row-statistics warps)
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar(B_ACC_FULL + i), 1);
            mbar_init(bar(B_ACC_EMPTY + i), 4);  // the four epilogue warps
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 5) tmem_alloc(smem_u32(tmem_slot), 2 * TN);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    bool timed_out = false;

    // Persistent: thread block b works on tiles b, b + gridDim.x, ...; tile index -> (row block, column block) with the
    // column block running fastest, so the blocks in flight share a few row blocks of x.  `it` counts this block's
    // tiles, g = it * n_k + kb its K steps: stage g % kStages, accumulator it & 1.
    if (warp == 4) {
        // ============================ TMA producer ============================
        // The whole warp waits for the stage; then lane l issues the l-th box of the stage (per K step one box of x and
        // TN / 64 boxes of the weight) in ONE warp instruction: the producer's chain per stage is a wait, the expect and a
        // single issue, whatever the number of boxes - it, too, is a single instruction stream whose length per stage
        // bounds the pipeline when the tiles are small.
        constexpr int kBoxesPerSub = 1 + TN / 64, kBoxes = KSUB * kBoxesPerSub;
        static_assert(kBoxes <= 32, "one lane per box");
        const int sub = lane / kBoxesPerSub, j = lane % kBoxesPerSub;  // lane's box: j == 0 the x box, else weight box j - 1
        const bool has_box = lane < kBoxes;
        const CUtensorMap* map = j == 0 ? &amap : &bmap;
        const uint32_t dst0 = base + (uint32_t)sub * kSub + (j == 0 ? 0u : (uint32_t)(kABytes + (j - 1) * kBBlockBytes));
        uint32_t s = 0, ephase = 1;
        for (int tile = blockIdx.x; tile < a.tiles_total && !timed_out; tile += gridDim.x) {
            const int m0 = (tile / a.tiles_n) * kTileM, n0 = (tile % a.tiles_n) * TN;
            for (int kb = 0; kb < n_k; ++kb) {
                if (!mbar_wait(bar0 + 8u * (B_EMPTY + s), ephase)) { timed_out = true; break; }
                const uint32_t full = bar0 + 8u * (B_FULL + s);
                if (lane == 0) mbar_expect_tx(full, KSUB * (a.a_bytes + (TN / 64) * kBBlockBytes));
                const int k0 = (kb * KSUB + sub) * kStepK;
                if (has_box) tma_load_2d(dst0 + s * kStage, map, full, j == 0 ? k0 : n0 + (j - 1) * 64, j == 0 ? m0 : k0);
                if (++s == kStages) { s = 0; ephase ^= 1; }
            }
        }
        timed_out = __any_sync(0xffffffffu, timed_out);
    } else if (warp == 5) {
        // ============================ MMA issuer ==============================
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(BF16, kTileM, TN);
            const uint32_t a_lo0 = desc_lo(a_stage(0), 16), b_lo0 = desc_lo(b_stage(0), kBBlockBytes), hi = desc_hi(1024);
            bool ok = true;
            uint32_t s = 0, phase = 0, off = 0;  // stage, its parity, its offset in 16-byte units
            int it = 0;
            for (int tile = blockIdx.x; tile < a.tiles_total && ok; tile += gridDim.x, ++it) {
                const int buf = it & 1;
                ok = mbar_wait(bar(B_ACC_EMPTY + buf), ((it >> 1) & 1) ^ 1);  // the epilogue has drained this accumulator
                if (!ok) break;
                tc_fence_after();
                const uint32_t d = tmem + buf * TN;
                for (int kb = 0; kb < n_k; ++kb) {
                    ok = mbar_wait(bar0 + 8u * (B_FULL + s), phase);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int sub = 0; sub < KSUB; ++sub) {
                        const uint32_t o = off + sub * (kSub >> 4);
                        mma_ss(d, a_lo0 + o, hi, b_lo0 + o, hi, idesc, sub > 0 || kb > 0);
                        mma_ss(d, a_lo0 + o + 2, hi, b_lo0 + o + 128, hi, idesc, 1);
                        mma_ss(d, a_lo0 + o + 4, hi, b_lo0 + o + 256, hi, idesc, 1);
                        mma_ss(d, a_lo0 + o + 6, hi, b_lo0 + o + 384, hi, idesc, 1);
                    }
                    tc_commit(bar0 + 8u * (B_EMPTY + s));
                    ++s;
                    off += kStage >> 4;
                    if (s == kStages) { s = 0; off = 0; phase ^= 1; }
                }
                if (ok) tc_commit(bar(B_ACC_FULL + buf));
            }
            timed_out = !ok;
        }
    } else {
        // ================= row statistics, then the epilogue ==================
        const int row = threadIdx.x;  // 0..127 = tensor-memory lane = row of the tile
        bool ok = true;
        int g = 0, it = 0;
        for (int tile = blockIdx.x; tile < a.tiles_total && ok; tile += gridDim.x, ++it) {
            const int m0 = (tile / a.tiles_n) * kTileM, n0 = (tile % a.tiles_n) * TN;
            const int buf = it & 1;
            float ss = 0.f;
            for (int kb = 0; STATS && kb < n_k && ok; ++kb, ++g) {
                const int s = g % kStages;
                ok = mbar_wait(bar(B_FULL + s), (g / kStages) & 1);
                if (!ok) break;
#pragma unroll
                for (int sub = 0; sub < KSUB; ++sub) {
                    const uint4* rowp = reinterpret_cast<const uint4*>(base_ptr + (size_t)s * kStage + (size_t)sub * kSub + (size_t)row * 128);
#pragma unroll
                    for (int c = 0; c < 8; ++c) ss += sumsq8<BF16>(rowp[(c + row) & 7]);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(B_EMPTY + s));
            }
            if (ok) ok = mbar_wait(bar(B_ACC_FULL + buf), (it >> 1) & 1);
            if (!ok) break;
            tc_fence_after();
            const bool row_ok = m0 + row < a.M;
            const float rstd = STATS ? rsqrtf(ss / (float)a.K + a.eps) : (row_ok ? a.rstd[m0 + row] : 0.f);
            const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16) + buf * TN;
            uint16_t* dst = reinterpret_cast<uint16_t*>(a.out) + (int64_t)(m0 + row) * a.out_stride + n0;
#pragma unroll 1
            for (int ch = 0; ch < TN / 32; ++ch) {
                float v[32];
                tmem_ld32(lane_base + ch * 32, v);
                if (row_ok) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        if (n0 + ch * 32 + i * 8 < a.N) {  // N is a multiple of 8: a 16-byte piece is inside or outside as a whole
                            uint4 w;
                            w.x = pack2<BF16>(v[8 * i] * rstd, v[8 * i + 1] * rstd);
                            w.y = pack2<BF16>(v[8 * i + 2] * rstd, v[8 * i + 3] * rstd);
                            w.z = pack2<BF16>(v[8 * i + 4] * rstd, v[8 * i + 5] * rstd);
                            w.w = pack2<BF16>(v[8 * i + 6] * rstd, v[8 * i + 7] * rstd);
                            *reinterpret_cast<uint4*>(dst + ch * 32 + i * 8) = w;
                        }
                    }
                }
            }
            // the accumulator goes back to the MMA warp: the next-but-one tile may overwrite it
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(B_ACC_EMPTY + buf));
        }
        timed_out = !ok;
    }
    if (timed_out && a.status && lane == 0) atomicOr(a.status, SFB_STATUS_WAIT_TIMEOUT);
    // ---- teardown: every warp arrives here; tensor memory is released before exit
    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem, 2 * TN);
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Two thread blocks on one 256 x 256 tile (a cluster of two, tcgen05 cta_group::2), for many rows.
//
// With one thread block per 128 x 256 tile every SM takes in 48 KB per K step (16 KB of x, 32 KB of the weight,
// about 110 GB/s per SM) and the issuing thread pays its wait / commit / loop chain once per four M 128 MMAs; the
// tensor pipe is 86 % busy.  Here the two thread blocks of a cluster share the weight tile, and an M 256 MMA is twice
// the work per issue (94 % busy): each loads its own 128 rows of x and HALF of the 256 weight
// columns (32 KB per step and SM), and the leader's MMA (M 256) reads the B operand out of both blocks' shared
// memory; each block's tensor memory receives its own 128 rows of the accumulator.
//   leader and peer, warp 4: wait for the local "stage empty" barrier, TMA into local shared memory, transaction
//                            bytes reported to the LEADER's "stage full" barrier (the cta_group::2 form of the load)
//   leader, warp 5:          waits on "stage full" (64 KB), issues the MMAs, tcgen05.commit with a cluster mask
//                            arrives on "stage empty" / "accumulator full" in both blocks
//   both, warps 0-3:         drain their 128 accumulator rows; all eight warps arrive on the leader's
//                            "accumulator empty" barrier
// Row statistics always come from the pre-pass here (a peer has no "stage full" barrier of its own to read tiles by).
// Waits are bounded as above; both blocks meet at a cluster barrier before tensor memory is released, so neither
// leaves while the other can still touch its shared memory.
constexpr int kPairStages = 6;
constexpr int kPairStage = kABytes + 2 * kBBlockBytes;  // per thread block and stage: 32 KB
constexpr int kPairTile = 256;
constexpr int pair_smem_bytes() { return kPairStages * kPairStage + B_COUNT * 8 + 16 + 1024; }
static_assert(kPairStages <= kMaxStages, "barrier slots");

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t leader_addr(uint32_t local) {  // the same shared-memory offset in the cluster's block 0
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(r) : "r"(local));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t cluster_bar, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(cluster_bar)
                 : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {  // arrives on this barrier in both thread blocks
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3)
                 : "memory");
}
__device__ __forceinline__ void mma_ss_pair(uint32_t d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n .reg .b64 da, db;\n mov.b64 da, {%1, %2};\n mov.b64 db, {%3, %4};\n setp.ne.b32 p, %6, 0;\n"
        " tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, p;\n}\n"
        ::"r"(d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}

template <bool BF16>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
norm_matmul_pair_kernel(const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap bmap, const GemmArgs a) {
    extern __shared__ uint8_t smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = (int)cluster_rank();
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int n_k = (a.K + kStepK - 1) / kStepK;

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    uint64_t* bars = reinterpret_cast<uint64_t*>(base_ptr + kPairStages * kPairStage);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + B_COUNT);
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    auto a_stage = [&](int s) { return base + (uint32_t)s * kPairStage; };
    auto b_stage = [&](int s) { return base + (uint32_t)s * kPairStage + kABytes; };

    if (threadIdx.x == 0) {
        for (int s = 0; s < kPairStages; ++s) {
            mbar_init(bar(B_FULL + s), 1);   // used in the leader only: its producer's arrive + both blocks' bytes
            mbar_init(bar(B_EMPTY + s), 1);  // the leader's commit, delivered to both blocks
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar(B_ACC_FULL + i), 1);
            mbar_init(bar(B_ACC_EMPTY + i), 8);  // used in the leader only: the epilogue warps of both blocks
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 5) tmem_alloc_pair(smem_u32(tmem_slot), 2 * kPairTile);
    tc_fence_before();
    __syncthreads();
    cluster_sync();  // the peer's barriers exist before anything is sent to them
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    bool timed_out = false;

    if (warp == 4) {
        // ===================== TMA producer (both thread blocks) ====================
        if (lane == 0) {
            int g = 0;
            for (int tile = pair; tile < a.tiles_total && !timed_out; tile += n_pairs) {
                const int m0 = (tile / a.tiles_n) * kPairTile + rank * kTileM;
                const int n0 = (tile % a.tiles_n) * kPairTile + rank * (kPairTile / 2);
                for (int kb = 0; kb < n_k; ++kb, ++g) {
                    const int s = g % kPairStages;
                    if (!mbar_wait(bar(B_EMPTY + s), ((g / kPairStages) & 1) ^ 1)) { timed_out = true; break; }
                    if (rank == 0) mbar_expect_tx(bar(B_FULL + s), 2 * kPairStage);
                    const uint32_t full = leader_addr(bar(B_FULL + s));
                    tma_load_2d_pair(a_stage(s), &amap, full, kb * kStepK, m0);
                    tma_load_2d_pair(b_stage(s), &bmap, full, n0, kb * kStepK);
                    tma_load_2d_pair(b_stage(s) + kBBlockBytes, &bmap, full, n0 + 64, kb * kStepK);
                }
            }
        }
    } else if (warp == 5) {
        // ========================= MMA issuer (leader only) =========================
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = instr_desc(BF16, 2 * kTileM, kPairTile);
            const uint32_t a_lo0 = desc_lo(a_stage(0), 16), b_lo0 = desc_lo(b_stage(0), kBBlockBytes), hi = desc_hi(1024);
            bool ok = true;
            uint32_t s = 0, phase = 0, off = 0;
            int it = 0;
            for (int tile = pair; tile < a.tiles_total && ok; tile += n_pairs, ++it) {
                const int buf = it & 1;
                ok = mbar_wait(bar(B_ACC_EMPTY + buf), ((it >> 1) & 1) ^ 1);  // both blocks have drained this accumulator
                if (!ok) break;
                tc_fence_after();
                const uint32_t d = tmem + buf * kPairTile;
                for (int kb = 0; kb < n_k; ++kb) {
                    ok = mbar_wait(bar0 + 8u * (B_FULL + s), phase);
                    if (!ok) break;
                    tc_fence_after();
                    mma_ss_pair(d, a_lo0 + off, hi, b_lo0 + off, hi, idesc, kb > 0);
                    mma_ss_pair(d, a_lo0 + off + 2, hi, b_lo0 + off + 128, hi, idesc, 1);
                    mma_ss_pair(d, a_lo0 + off + 4, hi, b_lo0 + off + 256, hi, idesc, 1);
                    mma_ss_pair(d, a_lo0 + off + 6, hi, b_lo0 + off + 384, hi, idesc, 1);
                    tc_commit_pair(bar0 + 8u * (B_EMPTY + s));
                    ++s;
                    off += kPairStage >> 4;
                    if (s == kPairStages) { s = 0; off = 0; phase ^= 1; }
                }
                if (ok) tc_commit_pair(bar(B_ACC_FULL + buf));
            }
            timed_out = !ok;
        }
    } else {
        // ===================== epilogue (both thread blocks) ========================
        const int row = threadIdx.x;
        bool ok = true;
        int it = 0;
        for (int tile = pair; tile < a.tiles_total && ok; tile += n_pairs, ++it) {
            const int m0 = (tile / a.tiles_n) * kPairTile + rank * kTileM, n0 = (tile % a.tiles_n) * kPairTile;
            const int buf = it & 1;
            ok = mbar_wait(bar(B_ACC_FULL + buf), (it >> 1) & 1);
            if (!ok) break;
            tc_fence_after();
            const bool row_ok = m0 + row < a.M;
            const float rstd = row_ok ? a.rstd[m0 + row] : 0.f;
            const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16) + buf * kPairTile;
            uint16_t* dst = reinterpret_cast<uint16_t*>(a.out) + (int64_t)(m0 + row) * a.out_stride + n0;
#pragma unroll 1
            for (int ch = 0; ch < kPairTile / 32; ++ch) {
                float v[32];
                tmem_ld32(lane_base + ch * 32, v);
                if (row_ok) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        if (n0 + ch * 32 + i * 8 < a.N) {
                            uint4 w;
                            w.x = pack2<BF16>(v[8 * i] * rstd, v[8 * i + 1] * rstd);
                            w.y = pack2<BF16>(v[8 * i + 2] * rstd, v[8 * i + 3] * rstd);
                            w.z = pack2<BF16>(v[8 * i + 4] * rstd, v[8 * i + 5] * rstd);
                            w.w = pack2<BF16>(v[8 * i + 6] * rstd, v[8 * i + 7] * rstd);
                            *reinterpret_cast<uint4*>(dst + ch * 32 + i * 8) = w;
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(leader_addr(bar(B_ACC_EMPTY + buf)));
        }
        timed_out = !ok;
    }
    if (timed_out && a.status && lane == 0) atomicOr(a.status, SFB_STATUS_WAIT_TIMEOUT);
    // ---- teardown: both thread blocks meet before tensor memory goes back
    tc_fence_before();
    __syncthreads();
    cluster_sync();
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc_pair(tmem, 2 * kPairTile);
    }
}

// One warp per row: rstd[m] = rsqrt(mean(x[m, :]^2) + eps), 16-byte loads.
template <bool BF16>
__global__ void row_rstd_kernel(const uint16_t* __restrict__ x, int64_t x_stride, int M, int K, float eps, float* __restrict__ rstd) {
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= M) return;
    const uint4* p = reinterpret_cast<const uint4*>(x + (int64_t)row * x_stride);
    float ss = 0.f;
    for (int i = lane; i < K / 8; i += 32) ss += sumsq8<BF16>(__ldg(p + i));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) rstd[row] = rsqrtf(ss / (float)K + eps);
}

template <typename T>
__global__ void fold_norm_weight_kernel(const T* __restrict__ g, const T* __restrict__ w, T* __restrict__ out, int64_t K, int64_t N,
                                        int64_t w_stride, int64_t out_stride) {
    const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;  // eight columns per thread
    if (i >= K * N) return;
    const int64_t k = i / N, n = i - k * N;  // N is a multiple of 8
    const float gk = to_float(g[k]);
    const uint4 raw = *reinterpret_cast<const uint4*>(w + k * w_stride + n);
    const T* x = reinterpret_cast<const T*>(&raw);
    uint4 res;
    T* y = reinterpret_cast<T*>(&res);
#pragma unroll
    for (int j = 0; j < 8; ++j) y[j] = from_float<T>(to_float(x[j]) * gk);
    *reinterpret_cast<uint4*>(out + k * out_stride + n) = res;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static std::once_flag once;
    static EncodeTiledFn fn = nullptr;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &res) == cudaSuccess &&
            res == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// 2-D map over a row-major 16-bit matrix [rows, cols] with a [box_rows x 64 columns] (128-byte wide) box.
bool encode_2d(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t row_stride_elems, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)row_stride_elems * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    const cuuint32_t es[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

int launch_fold_norm_weight(const void* g, const void* w, void* out, int64_t K, int64_t N, int64_t w_stride, int64_t out_stride,
                            int dtype, cudaStream_t stream) {
    const int64_t groups = K * N / 8;
    const unsigned blocks = (unsigned)ceil_div(groups, (int64_t)256);
    if (dtype == SFB_BF16)
        fold_norm_weight_kernel<<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(g), static_cast<const __nv_bfloat16*>(w),
                                                            static_cast<__nv_bfloat16*>(out), K, N, w_stride, out_stride);
    else
        fold_norm_weight_kernel<<<blocks, 256, 0, stream>>>(static_cast<const __half*>(g), static_cast<const __half*>(w),
                                                            static_cast<__half*>(out), K, N, w_stride, out_stride);
    SFB_CUDA_CHECK(cudaGetLastError());
    return SFB_OK;
}

namespace {

// How many clusters of two the pair kernel can have resident on this device (0: cannot run); asked once per device.
template <bool BF16>
int pair_clusters(int dev, int sms) {
    static std::mutex mu;
    static int cached[64];
    static bool known[64];
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < 64 && known[dev]) return cached[dev];
    auto kernel = norm_matmul_pair_kernel<BF16>;
    int clusters = 0;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, pair_smem_bytes()) == cudaSuccess) {
        cudaLaunchConfig_t cfg{};
        cudaLaunchAttribute attr{};
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
        cfg.gridDim = dim3((unsigned)(sms & ~1)); cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = pair_smem_bytes();
        cfg.attrs = &attr; cfg.numAttrs = 1;
        if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess) clusters = 0;
    }
    cudaGetLastError();  // a refusal above only means "not available"
    clusters = std::max(0, std::min(clusters, sms / 2));
    if (dev >= 0 && dev < 64) { cached[dev] = clusters; known[dev] = true; }
    return clusters;
}

}  // namespace

// Shape of the work (host arithmetic only).  Every candidate is priced by what the busiest SM has to take in: a
// 128-row panel of x plus its share of the weight columns per K step (kTileM + width rows of 128 bytes) x its rounds
// of tiles - a proxy that also orders the shapes by tensor work per SM - and the cheapest runs:
//   one thread block per 128 x {256, 128, 64} tile  (ties go to the wider tile: less traffic in total), or
//   a cluster of two on a 256 x 256 tile, each block taking in 128 + 128 rows - needs the statistics pre-pass,
//   so only with a workspace for it, and only when strictly cheaper.
//   With fewer than 128 rows in all, the box of x is cut to the rows there are (in eights): the MMA still reads 128
//   rows of shared memory, but what the rows past M hold only reaches accumulator rows that are never stored.
NormMatmulPlan plan_norm_matmul(int64_t M, int64_t N, int sms, int clusters, bool has_scratch) {
    NormMatmulPlan p{};
    sms = std::max(sms, 1);
    const int64_t m_tiles = ceil_div(M, (int64_t)kTileM);
    p.x_box_rows = M < kTileM ? (int)std::max<int64_t>(8, ceil_div(M, (int64_t)8) * 8) : kTileM;
    p.tile_n = kTileN;
    int64_t best = -1;
    for (int w : {256, 128, 64}) {
        const int64_t cost = ceil_div(m_tiles * ceil_div(N, (int64_t)w), (int64_t)sms) * (p.x_box_rows + w);
        if (best < 0 || cost < best) { best = cost; p.tile_n = w; }
    }
    const int64_t ptiles = ceil_div(N, (int64_t)kPairTile) * ceil_div(M, (int64_t)kPairTile);
    p.pair = has_scratch && clusters > 0 && ptiles <= 0x7fffffffLL &&
             ceil_div(ptiles, (int64_t)clusters) * (kTileM + kPairTile / 2) < best;
    p.prepass = has_scratch && (p.pair || M >= kPrepassRows);
    if (p.pair) {
        p.tile_n = kPairTile; p.x_box_rows = kTileM; p.stages = kPairStages; p.k_steps_per_stage = 1;
    } else {
        const int64_t tiles = m_tiles * ceil_div(N, (int64_t)p.tile_n);
        const bool deep64 = p.tile_n == 64 && tiles <= sms;  // every 64-wide tile has an SM to itself
        p.stages = p.tile_n == 128 ? 6 : 4;
        p.k_steps_per_stage = deep64 ? 2 : 1;
    }
    return p;
}

int launch_norm_matmul(const void* x, int64_t x_stride, const void* wg, int64_t wg_stride, void* out, int64_t out_stride, int64_t M,
                       int64_t N, int64_t K, float eps, int dtype, int* status, float* rstd_scratch, cudaStream_t stream) {
    const bool bf16 = dtype == SFB_BF16;
    int dev = 0, sms = 0;
    SFB_CUDA_CHECK(cudaGetDevice(&dev));
    SFB_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));

    const int64_t ptiles_n = ceil_div(N, (int64_t)kPairTile), ptiles = ptiles_n * ceil_div(M, (int64_t)kPairTile);
    int clusters = 0;
    if (rstd_scratch != nullptr && ptiles <= 0x7fffffffLL) clusters = bf16 ? pair_clusters<true>(dev, sms) : pair_clusters<false>(dev, sms);
    const NormMatmulPlan plan = plan_norm_matmul(M, N, sms, clusters, rstd_scratch != nullptr);
    const bool pair = plan.pair != 0;
    const int tn = plan.tile_n, a_rows = plan.x_box_rows;
    const int64_t m_tiles = ceil_div(M, (int64_t)kTileM);
    const bool prepass = plan.prepass != 0;
    if (prepass) {
        const unsigned blocks = (unsigned)ceil_div(M, (int64_t)8);
        if (bf16) row_rstd_kernel<true><<<blocks, 256, 0, stream>>>(static_cast<const uint16_t*>(x), x_stride, (int)M, (int)K, eps, rstd_scratch);
        else row_rstd_kernel<false><<<blocks, 256, 0, stream>>>(static_cast<const uint16_t*>(x), x_stride, (int)M, (int)K, eps, rstd_scratch);
        SFB_CUDA_CHECK(cudaGetLastError());
    }
    CUtensorMap amap, bmap;
    if (!encode_2d(&amap, x, M, K, x_stride, pair ? kTileM : a_rows) || !encode_2d(&bmap, wg, K, N, wg_stride, kStepK))
        return fail(SFB_ERR_UNSUPPORTED, "fused_rms_norm_matmul: tensor map encoding failed (16-byte aligned bases and row strides are required)");
    GemmArgs a{};
    a.out = out; a.out_stride = out_stride;
    a.M = (int)M; a.N = (int)N; a.K = (int)K;
    a.a_bytes = a_rows * kStepK * 2;
    a.eps = eps; a.status = status;
    a.rstd = prepass ? rstd_scratch : nullptr;
    if (pair) {
        a.tiles_n = (int)ptiles_n;
        a.tiles_total = (int)ptiles;
        const dim3 grid(2u * (unsigned)std::min<int64_t>(ptiles, clusters));
        if (bf16) norm_matmul_pair_kernel<true><<<grid, kThreads, pair_smem_bytes(), stream>>>(amap, bmap, a);
        else norm_matmul_pair_kernel<false><<<grid, kThreads, pair_smem_bytes(), stream>>>(amap, bmap, a);
        SFB_CUDA_CHECK(cudaGetLastError());
        return SFB_OK;
    }
    const int64_t tiles_n = ceil_div(N, (int64_t)tn), tiles = tiles_n * m_tiles;
    if (tiles > 0x7fffffffLL) return fail(SFB_ERR_UNSUPPORTED, "fused_rms_norm_matmul: too many tiles");
    a.tiles_n = (int)tiles_n;
    a.tiles_total = (int)tiles;
    // persistent thread blocks walk the tiles; with more 64-wide tiles than SMs two thread blocks of four stages share an SM
    const bool deep64 = plan.k_steps_per_stage == 2;
    const dim3 grid((unsigned)std::min<int64_t>(tiles, tn == 64 && !deep64 ? 2 * sms : sms));
    auto launch = [&](auto kernel, int smem) -> int {
        const int rc = allow_shared_memory_once(reinterpret_cast<const void*>(kernel), smem);
        if (rc != SFB_OK) return rc;
        kernel<<<grid, kThreads, smem, stream>>>(amap, bmap, a);
        SFB_CUDA_CHECK(cudaGetLastError());
        return SFB_OK;
    };
    auto pick = [&](auto width, auto stages, auto ksub) -> int {
        constexpr int W = decltype(width)::value, S = decltype(stages)::value, KS = decltype(ksub)::value;
        constexpr int sm = smem_bytes(W, S, KS);
        if (bf16) return prepass ? launch(norm_matmul_tcgen05_kernel<true, false, W, S, KS>, sm) : launch(norm_matmul_tcgen05_kernel<true, true, W, S, KS>, sm);
        return prepass ? launch(norm_matmul_tcgen05_kernel<false, false, W, S, KS>, sm) : launch(norm_matmul_tcgen05_kernel<false, true, W, S, KS>, sm);
    };
    using std::integral_constant;
    // 64-wide tiles with an SM each: four stages of two K steps (each wait / commit of the MMA warp covers eight MMAs)
    if (deep64) return pick(integral_constant<int, 64>{}, integral_constant<int, 4>{}, integral_constant<int, 2>{});
    if (tn == 64) return pick(integral_constant<int, 64>{}, integral_constant<int, 4>{}, integral_constant<int, 1>{});
    if (tn == 128) return pick(integral_constant<int, 128>{}, integral_constant<int, 6>{}, integral_constant<int, 1>{});
    return pick(integral_constant<int, 256>{}, integral_constant<int, 4>{}, integral_constant<int, 1>{});
}

}  // namespace sfb
