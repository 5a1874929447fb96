// Chunked-prefill attention over the paged KV pool on the 5th-generation tensor
// cores (tcgen05 MMA, accumulators in tensor memory, operands fed by TMA).
//
// Semantics restated from kernels/flash_attention.py:35-46 of the reference
// (dense causal softmax(Q K^T scale) V): the queries of a request's chunk sit at
// positions ctx_len - n_q .. ctx_len - 1 and see every cached token up to their
// own position; K/V come from the request's block table exactly like
// kernels/paged_attention.py:36-48, so a radix-shared prefix is simply the same
// physical blocks at the head of several tables.  GQA: query head h reads kv
// head h / (H / Hkv).
//
// One thread block = 256 query tokens (two 128-row tiles) of one (request, query head), five warpgroups:
//   warps 0-15 softmax, eight warps per query tile, two threads per query row (64 key columns each; a warp
//             can only reach its own 32 tensor-memory lanes, so warps w and w+4 share lanes and split the
//             columns).  With two warps per SM sub-partition on a tile, one warp's FMA / pack instructions
//             issue while the other's ex2 occupy the XU pipe.  A thread reads its 64 scores ONCE
//             (tcgen05.ld into registers; the softmax warpgroups raise their register allowance with
//             setmaxnreg, the fifth warpgroup lowers its own), swaps half-row maxima with its partner
//             through shared memory under a 64-thread named barrier, keeps running max / sum in log2
//             units, writes P as bf16/fp16 over its own S columns in two halves so that the P.V product
//             starts on the first half while the second is still being computed, rescales O in tensor
//             memory only when the max grew by more than 2^8 (the stale max stays exact in fp32), adds the
//             partial sums in the epilogue and writes O / l.
//   warp 16   TMA producer: both Q tiles once, then per 128-token KV tile sixteen
//             [16 tokens x 128 B] boxes for K and sixteen for V, two stages each
//   warp 17   issues tcgen05.mma: S_t = Q_t K^T (128x128x128, both operands K-major
//             in 128B-swizzled shared memory) and O_t += P_t V with P_t read from
//             tensor memory and V as an MN-major shared-memory operand, alternating
//             between the two query tiles so that one tile's MMAs run while the
//             other tile's rows are in the softmax warps
//   warp 18   clears the V rows past the context in the last KV tile (a pool that was never
//             zero-filled may hold NaN patterns there, and 0 * NaN would reach O)
// Tensor memory: per query tile S|P (128 columns) and O (128) = 512 columns in all.
// Bound: tensor pipe (4*D*Sq*Skv flops per head against ~1.4 PFLOP/s dense).

#include <cuda.h>

#include <mutex>
#include <type_traits>

#include "sfb_common.cuh"

namespace sfb {
namespace {

constexpr int kTileQ = 128;
constexpr int kTileKV = 128;
constexpr int kHeadDim = 128;
constexpr int kSubBytes = kTileKV * 128;     // one [128 rows][128 B] swizzled sub-tile
constexpr int kTileBytes = 2 * kSubBytes;    // D = 128 16-bit values = two sub-tiles
constexpr int kThreads = 640;  // 2 x 8 softmax warps (one group per query tile) + a warpgroup with the TMA, MMA and fix-up warps
constexpr int kMmaWarp = 0, kTmaWarp = 1, kTmaWarpV = 2, kFirstSoftmaxWarp = 4;
constexpr int kPParts = 1;  // P is handed to the MMA thread in this many parts per KV tile (1 or 2)
constexpr uint32_t kSpin = 1u << 21;  // bounded waits: a stuck pipeline gives up (status bit) within about a second
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f;    // log2 units

struct PrefillArgs {
    const void* q;
    void* out;
    const int32_t* cu_q;      // [R+1] packed query offsets
    const int32_t* ctx_lens;  // [R]   tokens cached after this chunk was written
    const int32_t* row_limits;  // optional [T]: query row r sees positions 0 .. row_limits[r] - 1 (instead of `causal`)
    const int32_t* tables;
    int64_t table_stride;
    int max_blocks;
    int n_requests, n_heads, n_kv_heads;
    int64_t n_pool_blocks;
    int64_t out_stride[2];  // token, head (elements)
    float scale;
    int bf16;               // 1 = bfloat16, 0 = float16
    int causal;             // 0: every query sees all ctx_len tokens
    int* status;
    int fixed_nq, fixed_ctx;  // used when cu_q == nullptr (shared-prefix mode)
    float* part_o;            // non-null: write split partials instead of normalised rows
    float* part_ml;
    const int32_t* part_seq_lens;
    int part_n_chunks, part_chunk_tokens, part_max_tokens;
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
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
        ::"r"(dst), "l"(map), "r"(0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c2, int c3, int c4) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
        ::"r"(dst), "l"(map), "r"(0), "r"(0), "r"(c2), "r"(c3), "r"(c4), "r"(bar)
        : "memory");
}
// ---- tensor memory and tcgen05 ------------------------------------------------
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
// D[tmem] (+)= A[smem desc] . B[smem desc]; descriptors as (low, high) words
__device__ __forceinline__ void mma_ss(uint32_t d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                       uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n .reg .b64 da, db;\n mov.b64 da, {%1, %2};\n mov.b64 db, {%3, %4};\n setp.ne.b32 p, %6, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n}\n"
        ::"r"(d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] . B[smem desc]
__device__ __forceinline__ void mma_ts(uint32_t d, uint32_t a, uint32_t b_lo, uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n .reg .b64 db;\n mov.b64 db, {%2, %3};\n setp.ne.b32 p, %5, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n}\n"
        ::"r"(d), "r"(a), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, float (&v)[32]) {
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
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    tmem_ld32_issue(taddr, v);
    tmem_wait_ld();
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    tmem_wait_ld();
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float fast_exp2(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    uint32_t r;
    if constexpr (BF16) asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    else asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// Shared-memory matrix descriptor (sm_100 format): start address, leading and
// stride byte offsets in 16-byte units, version 1, 128-byte swizzle.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3fff);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32;
    d |= (uint64_t)1 << 46;  // descriptor version for sm_100
    d |= (uint64_t)2 << 61;  // SWIZZLE_128B
    return d;
}
// Instruction descriptor for kind::f16: fp32 accumulate, 16-bit A/B, M x N tile.
__host__ __device__ constexpr uint32_t instr_desc(bool bf16, bool b_mn_major, int m, int n) {
    return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((b_mn_major ? 1u : 0u) << 16) |
           ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// barrier slots.  Ring slot j&1 of K holds K(j), of V holds V(j); the MMA step j needs V(j) and K(j+1), so one
// "full" / "empty" pair per step parity covers V slot j&1 together with K slot (j+1)&1.
enum {
    B_Q_FULL = 0,    // both Q tiles and K(0)
    B_KV_FULL = 1,   // +step parity: V(j) and K(j+1) have landed (one arrival per producer warp)
    B_KV_EMPTY = 3,  // +step parity: every MMA that read them is complete
    B_S_FULL = 5,    // +query tile
    B_P_FULL = 7,    // +2 * query tile + half: keys 0-31 of both column halves, then keys 32-63
    B_PV_DONE = 11,  // +query tile: the tile's last P.V product is complete
    B_V_FIXED = 13,  // the last KV tile's V rows past the context are cleared
    B_COUNT = 14
};
constexpr int kXchFloats = 2 * 2 * 2 * kTileQ;  // [step parity][query tile][column half][row]
constexpr int kSmemBytes = 6 * kTileBytes + B_COUNT * 8 + 16 + kXchFloats * 4 + 1024;  // 2 Q tiles, 2 K stages, 2 V stages

// Tensor-memory columns of query tile t: S (fp32, 128 columns) at t*256, with P (16-bit pairs,
// 64 columns) written over its first half once the row has been read; O (fp32) at t*256 + 128.
constexpr uint32_t kColTile = 256;
constexpr uint32_t kColO = 128;

// Register allowances after the role split (five warpgroups of 128 threads; the kernel is compiled for
// 65536 / 640 -> 96 registers per thread, and shared memory admits one thread block per SM, so the block may
// grow into the rest of the register file): 4 * 128 * kSoftmaxRegs + 128 * kOtherRegs <= 65536, and the first
// warpgroup lowers its allowance before the others can finish raising theirs.
constexpr int kSoftmaxRegs = 104;
constexpr int kOtherRegs = 64;

template <bool BF16>
__global__ void __launch_bounds__(kThreads, 1)
prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                       const __grid_constant__ CUtensorMap vmap, const PrefillArgs a) {
    extern __shared__ uint8_t smem_raw[];
    const int req = blockIdx.z, head = blockIdx.y;
    const int q_begin = a.cu_q ? a.cu_q[req] : 0, n_q = a.cu_q ? a.cu_q[req + 1] - q_begin : a.fixed_nq;
    // heaviest blocks (latest queries) first
    const int q_blocks = (n_q + 2 * kTileQ - 1) / (2 * kTileQ);
    const int qb = q_blocks - 1 - (int)blockIdx.x;
    if (qb < 0) return;
    int ctx = a.cu_q ? a.ctx_lens[req] : a.fixed_ctx;
    if (ctx > a.max_blocks * 16) ctx = a.max_blocks * 16;
    if ((a.causal && !a.row_limits && ctx < n_q) || n_q <= 0 || ctx <= 0) {  // inconsistent request: flag it, write nothing
        if (a.status && threadIdx.x == 0) atomicOr(a.status, SFB_STATUS_EMPTY_REQUEST);
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q0 = qb * 2 * kTileQ;                       // first query row of the block
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    uint64_t* bars = reinterpret_cast<uint64_t*>(base_ptr + 6 * kTileBytes);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + B_COUNT);
    int* limit_max = reinterpret_cast<int*>(tmem_slot + 1);  // [2]: with row limits, the largest limit of each query tile
    float* xch = reinterpret_cast<float*>(tmem_slot + 4);
    int my_limit = 0;
    if (a.row_limits) {  // one row per thread of the first eight warps; the tiles' maxima go through shared memory
        if (threadIdx.x < 2 * kTileQ) {
            if (q0 + (int)threadIdx.x < n_q) my_limit = min(max(a.row_limits[q_begin + q0 + threadIdx.x], 0), ctx);
            const int wmax = __reduce_max_sync(0xffffffffu, my_limit);
            if (lane == 0) reinterpret_cast<int*>(xch)[warp] = wmax;
        }
        __syncthreads();
        if (threadIdx.x < 2) {
            const int* w = reinterpret_cast<const int*>(xch) + 4 * threadIdx.x;
            limit_max[threadIdx.x] = max(max(w[0], w[1]), max(w[2], w[3]));
        }
        __syncthreads();
    }
    int rows_t[2], tiles_t[2];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        rows_t[t] = max(0, min(kTileQ, n_q - q0 - t * kTileQ));
        const int last_pos = a.row_limits ? max(limit_max[t], 1) - 1 : a.causal ? ctx - n_q + q0 + t * kTileQ + rows_t[t] - 1 : ctx - 1;
        tiles_t[t] = rows_t[t] > 0 ? last_pos / kTileKV + 1 : 0;
    }
    const int n_tiles = max(tiles_t[0], tiles_t[1]);
    const int used_blocks = (ctx + 15) >> 4;
    const int group = a.n_heads / a.n_kv_heads;
    const int kvh = head / group;
    // the KV tile that holds the last cached token may end inside a 16-token block: its V rows past the context are cleared
    const int fix_tile = (ctx - 1) / kTileKV;
    const bool fix_v = (ctx & 15) != 0 && fix_tile < n_tiles;

    const uint32_t q_s = base, k_s = base + 2 * kTileBytes, v_s = base + 4 * kTileBytes;
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };

    if (threadIdx.x == 0) {
        mbar_init(bar(B_Q_FULL), 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(bar(B_KV_FULL + s), 2);
            mbar_init(bar(B_KV_EMPTY + s), 1);
            mbar_init(bar(B_S_FULL + s), 1);
            mbar_init(bar(B_P_FULL + 2 * s), 8);
            mbar_init(bar(B_P_FULL + 2 * s + 1), 8);
            mbar_init(bar(B_PV_DONE + s), 1);
        }
        mbar_init(bar(B_V_FIXED), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == kMmaWarp) tmem_alloc(smem_u32(tmem_slot), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    bool timed_out = false;

    if (warp < kFirstSoftmaxWarp) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kOtherRegs));
        auto produce = [&](auto is_v_tag) {
            constexpr bool is_v = decltype(is_v_tag)::value;
            // ============================ TMA producers ===========================
            // Warp 1 feeds Q and K, warp 2 feeds V: the issue of one step's boxes (a few tens of clocks per box) is
            // shared between two warps.  For MMA step j the K warp loads K(j+1), the V warp V(j), both behind the
            // step's "empty" barrier and onto its "full" barrier.
            // K: lane = (block of the tile, 64-value half), a [16 tokens x 128 B] box each, laid out [half][128 tokens][128 B].
            // V: lane = block of the tile, one [2 halves x 16 tokens x 128 B] box each, laid out [block][half][16 tokens][128 B].
            const int blk = is_v ? (lane & 7) : ((lane & 15) >> 1), sub = lane & 1;
            const bool active = is_v ? lane < 8 : lane < 16;
            const uint32_t dst_off = is_v ? blk * 4096 : sub * kSubBytes + blk * 2048;
            const int32_t* table = a.tables + (int64_t)req * a.table_stride + blk;
            const int pool = (int)a.n_pool_blocks;  // the launcher keeps the pool below 2^31 blocks
            const int limit = min(n_tiles * 8, used_blocks) - blk;
            auto lookup = [&](int tile) -> int {
                if (tile * 8 >= limit) return pool;  // past the context -> an out-of-range block index, TMA fills zeros
                const int p = table[tile * 8];
                if ((unsigned)p >= (unsigned)pool) {
                    if (a.status && !is_v) atomicOr(a.status, SFB_STATUS_BAD_BLOCK_ID);
                    return pool;
                }
                return p;
            };
            const int first = is_v ? 0 : 1;  // KV tile of step 0
            int phys = lookup(first), phys1 = lookup(first + 1);
            if (!is_v) {
                const int phys0 = lookup(0);
                if (lane == 0) {
                    mbar_expect_tx(bar(B_Q_FULL), 3 * kTileBytes);
#pragma unroll
                    for (int t = 0; t < 2; ++t) {  // rows past the packed batch read as zeros
                        tma_load_4d(q_s + t * kTileBytes, &qmap, bar(B_Q_FULL), q_begin + q0 + t * kTileQ, 0, head);
                        tma_load_4d(q_s + t * kTileBytes + kSubBytes, &qmap, bar(B_Q_FULL), q_begin + q0 + t * kTileQ, 1, head);
                    }
                }
                __syncwarp();
                if (active) tma_load_5d(k_s + dst_off, &kmap, bar(B_Q_FULL), sub, kvh, phys0);  // K(0) into slot 0
            }
            for (int j = 0; j < n_tiles; ++j) {
                const int s = j & 1;
                // "empty" phases: parity 0 completes at the end of step 0 (pair 0) resp. once Q.K(0)^T is done (pair 1)
                const uint32_t par = s ? ((j >> 1) & 1) : (((j >> 1) & 1) ^ 1);
                const int phys2 = lookup(first + j + 2);  // table entries are fetched two tiles ahead of their use
                if (!mbar_wait(bar(B_KV_EMPTY + s), par)) { timed_out = true; break; }
                if (is_v) {
                    if (lane == 0) mbar_expect_tx(bar(B_KV_FULL + s), kTileBytes);
                    __syncwarp();
                    if (active) tma_load_5d(v_s + s * kTileBytes + dst_off, &vmap, bar(B_KV_FULL + s), 0, kvh, phys);
                } else if (j + 1 < n_tiles) {
                    if (lane == 0) mbar_expect_tx(bar(B_KV_FULL + s), kTileBytes);
                    __syncwarp();
                    if (active) tma_load_5d(k_s + (s ^ 1) * kTileBytes + dst_off, &kmap, bar(B_KV_FULL + s), sub, kvh, phys);
                } else if (lane == 0) {
                    mbar_arrive(bar(B_KV_FULL + s));  // no further K tile: the step's barrier still counts two arrivals
                }
                phys = phys1;
                phys1 = phys2;
            }
            if (is_v && fix_v && !timed_out) {
                // Clear the V rows past the context in the last KV tile.  A 128-byte row of a swizzled sub-tile is permuted
                // only inside itself, so whole rows can be cleared in place.
                const int s = fix_tile & 1;
                if (mbar_wait(bar(B_KV_FULL + s), (fix_tile >> 1) & 1)) {
                    const int fblk = ((ctx - 1) >> 4) & 7, first = ctx & 15;
                    uint8_t* v_tile = base_ptr + 4 * kTileBytes + s * kTileBytes + fblk * 4096;
                    for (int i = lane; i < (16 - first) * 16; i += 32) {  // (row, 64-value half, 16-byte piece)
                        const int r = first + (i >> 4), h = (i >> 3) & 1, piece = i & 7;
                        *reinterpret_cast<uint4*>(v_tile + h * 2048 + r * 128 + piece * 16) = make_uint4(0, 0, 0, 0);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar(B_V_FIXED));
                } else {
                    timed_out = true;
                }
            }
        };
        if (warp == kTmaWarp) {
            produce(std::false_type{});
        } else if (warp == kTmaWarpV) {
            produce(std::true_type{});
        } else if (warp == kMmaWarp) {
            // ============================ MMA issuer ==============================
            // One thread issues every MMA, in the order PV0(j), QK0(j+1), PV1(j), QK1(j+1): while one query tile's rows
            // are in the softmax warps, the tensor pipe works on the other tile (two issuing threads, one per tile, were
            // measured: the tiles then fall into step and the pipe idles while both are in their softmax).  An issue
            // returns when the pipe accepts the MMA, so whatever else this thread runs is time with nothing queued: per
            // step it waits once for the operands and once or twice per tile for P, and commits the S tiles and the
            // operand slots; descriptors are a constant plus a slot / K-step offset in the low word.
            if (lane == 0) {
                constexpr uint32_t idesc_qk = instr_desc(BF16, false, kTileQ, kTileKV);
                constexpr uint32_t idesc_pv = instr_desc(BF16, true, kTileQ, kHeadDim);
                const uint32_t hi = (uint32_t)(smem_desc(0, 0, 1024) >> 32);
                const uint32_t q_lo = (uint32_t)smem_desc(q_s, 16, 0);
                const uint32_t k_lo = (uint32_t)smem_desc(k_s, 16, 0), v_lo = (uint32_t)smem_desc(v_s, 2048, 0);
                auto issue_qk = [&](int t, int slot) {  // 16 head-dim values per instruction
                    const uint32_t qb_lo = q_lo + t * (kTileBytes >> 4), kb = k_lo + slot * (kTileBytes >> 4);
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks) {
                        const uint32_t off = ((ks >> 2) * kSubBytes + (ks & 3) * 32) >> 4;
                        mma_ss(tmem + t * kColTile, qb_lo + off, hi, kb + off, hi, idesc_qk, ks > 0);
                    }
                    tc_commit(bar(B_S_FULL + t));
                };
                auto issue_pv = [&](int t, int j) -> bool {
                    const uint32_t vb = v_lo + (j & 1) * (kTileBytes >> 4), s_tm = tmem + t * kColTile;
#pragma unroll
                    for (int part = 0; part < kPParts; ++part) {  // with two parts: keys {0-31, 64-95}, then {32-63, 96-127}
                        if (!mbar_wait(bar(B_P_FULL + 2 * t + part), j & 1)) return false;
                        tc_fence_after();
#pragma unroll
                        for (int i = 0; i < 8 / kPParts; ++i) {  // 16 KV tokens per instruction
                            const int ks = kPParts == 2 ? (i >> 1) * 4 + part * 2 + (i & 1) : i;
                            mma_ts(s_tm + kColO, s_tm + (ks >> 2) * 64 + (ks & 3) * 8, vb + ks * (4096 >> 4), hi, idesc_pv,
                                   (j > 0 || part > 0 || i > 0));
                        }
                    }
                    if (j + 1 == tiles_t[t]) tc_commit(bar(B_PV_DONE + t));  // the tile's last product: the epilogue waits for it
                    return true;
                };
                bool ok = mbar_wait(bar(B_Q_FULL), 0);
                if (ok) {
                    tc_fence_after();
                    if (tiles_t[0] > 0) issue_qk(0, 0);
                    if (tiles_t[1] > 0) issue_qk(1, 0);
                    tc_commit(bar(B_KV_EMPTY + 1));  // K slot 0 may take K(2) once these are done
                }
                for (int j = 0; ok && j < n_tiles; ++j) {
                    ok = mbar_wait(bar(B_KV_FULL + (j & 1)), (j >> 1) & 1);
                    if (ok && fix_v && j == fix_tile) ok = mbar_wait(bar(B_V_FIXED), 0);
#pragma unroll
                    for (int t = 0; t < 2; ++t) {
                        if (ok && j < tiles_t[t]) ok = issue_pv(t, j);
                        if (ok && j + 1 < tiles_t[t]) issue_qk(t, (j + 1) & 1);
                    }
                    if (ok && j + 2 < n_tiles) tc_commit(bar(B_KV_EMPTY + (j & 1)));  // the producers wait for it before step j + 2
                }
                timed_out = !ok;
            }
        }
    } else {
        // ======================= softmax / correction / epilogue ==============
        // Eight warps per query tile.  Warp w owns tensor-memory lanes 32*(w&3).. (its hardware window) and key
        // columns 64*((w>>2)&1).. of its tile: two threads share a query row, swap their half-row maxima through
        // shared memory (64-thread named barrier, slots alternate by step) and keep partial sums that are only
        // added up in the epilogue.
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kSoftmaxRegs));
        const int my_t = (warp - kFirstSoftmaxWarp) >> 3;  // query tile of this 8-warp group
        const int hf = ((warp - kFirstSoftmaxWarp) >> 2) & 1;
        const int row = threadIdx.x & 127;
        const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        const uint32_t pair_bar = 1 + my_t * 4 + (warp & 3);  // named barrier of the two warps that share a lane window
        const float sl2 = a.scale * kLog2e;
        float m_used = -INFINITY, l = 0.f;
        const int my_rows = my_t ? rows_t[1] : rows_t[0], my_tiles = my_t ? tiles_t[1] : tiles_t[0];
        // last visible position of this thread's row; padding rows see everything
        int pos = (row < my_rows && a.causal) ? ctx - n_q + q0 + my_t * kTileQ + row : ctx - 1;
        if (a.row_limits && row < my_rows) pos = min(max(a.row_limits[q_begin + q0 + my_t * kTileQ + row], 0), ctx) - 1;
        const uint32_t s_addr = lane_addr + my_t * kColTile + hf * 64;  // this thread's 64 score columns
        const uint32_t o_addr = lane_addr + my_t * kColTile + kColO + hf * 64;

        // both warps of a pair run the same waits in the same order, so they reach this barrier together or not at all
        auto exchange = [&](int step, float mine) -> float {
            float* slot = xch + ((step & 1) * 2 + my_t) * 2 * kTileQ;
            slot[hf * kTileQ + row] = mine;
            asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
            return slot[(hf ^ 1) * kTileQ + row];
        };

        auto softmax_tile = [&](int j) -> bool {
            if (!mbar_wait(bar(B_S_FULL + my_t), j & 1)) return false;
            tc_fence_after();
            const int kv0 = j * kTileKV + hf * 64;
            // tcgen05.ld / st are warp-collective: the masked / unmasked choice must be uniform across the warp
            const bool full = __all_sync(0xffffffffu, kv0 + 63 <= pos);
            float s[64];
            tmem_ld32_issue(s_addr, *reinterpret_cast<float(*)[32]>(s));
            tmem_ld32_issue(s_addr + 32, *reinterpret_cast<float(*)[32]>(s + 32));
            tmem_wait_ld();
            float mx0 = -INFINITY, mx1 = -INFINITY;
            if (full) {
#pragma unroll
                for (int i = 0; i < 64; i += 4) {
                    mx0 = max3(mx0, s[i], s[i + 1]);
                    mx1 = max3(mx1, s[i + 2], s[i + 3]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    if (kv0 + i > pos) s[i] = -INFINITY;  // exp2(-inf) = 0 below
                    mx0 = fmaxf(mx0, s[i]);
                }
            }
            const float mx = fmaxf(fmaxf(mx0, mx1), exchange(j, fmaxf(mx0, mx1)));
            const float m_new = fmaxf(m_used, mx * sl2);
            if (j == 0) {
                m_used = m_new;
            } else {
                const bool need = m_new > m_used + kRescaleThreshold;  // the same for both threads of a row
                if (__any_sync(0xffffffffu, need)) {
                    // O is only touched between P.V products.  The previous one is complete: this tile's S was committed by
                    // the same thread after it, and a commit covers everything that thread issued before.
                    const float f = need ? fast_exp2(m_used - m_new) : 1.f;
                    l *= f;
                    if (need) m_used = m_new;
#pragma unroll 1
                    for (int ch = 0; ch < 4; ++ch) {
                        float o[16];
                        tmem_ld16(o_addr + ch * 16, o);
#pragma unroll
                        for (int i = 0; i < 16; ++i) o[i] *= f;
                        tmem_st16(o_addr + ch * 16, *reinterpret_cast<uint32_t(*)[16]>(o));
                    }
                    tmem_wait_st();
                }
            }
            // P (16-bit pairs, 32 columns) goes over the first half of this thread's own score columns, in two halves
            // packed fp32 pairs: one FFMA2 scales and shifts two scores, one FADD2 adds two probabilities
            const float neg_m = m_used == -INFINITY ? 0.f : -m_used;  // a row that sees nothing yet: every score is -inf, P = 0
            const float2 sl2v = make_float2(sl2, sl2), nmv = make_float2(neg_m, neg_m);
            float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
#pragma unroll
            for (int ch = 0; ch < 2; ++ch) {
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float2 x = __ffma2_rn(make_float2(s[32 * ch + 2 * i], s[32 * ch + 2 * i + 1]), sl2v, nmv);
                    const float2 pr = make_float2(fast_exp2(x.x), fast_exp2(x.y));
                    if (i & 1) acc1 = __fadd2_rn(acc1, pr);
                    else acc0 = __fadd2_rn(acc0, pr);
                    pk[i] = pack2<BF16>(pr.x, pr.y);
                }
                tmem_st16(s_addr + ch * 16, pk);
                if (kPParts == 2 || ch == 1) {
                    tmem_wait_st();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar(B_P_FULL + 2 * my_t + (kPParts == 2 ? ch : 0)));
                }
            }
            l += (acc0.x + acc1.x) + (acc0.y + acc1.y);
            return true;
        };

        bool ok = true;
        for (int j = 0; j < my_tiles && ok; ++j) ok = softmax_tile(j);
        // ---- epilogue: O / l, each thread its 64 output columns
        if (ok && my_tiles > 0) ok = mbar_wait(bar(B_PV_DONE + my_t), 0);
        if (ok && my_tiles > 0) {
            tc_fence_after();
            const float l_row = l + exchange(my_tiles, l);
            const bool row_valid = row < my_rows;
            if (a.part_o) {
                // shared-prefix mode: this row is decode request `qrow`; its partial goes to the chunk slot right after
                // the request's own chunks, in the decode kernel's format (unnormalised O, max in log2 units, sum)
                const int qrow = q0 + my_t * kTileQ + row;
                int64_t pslot = 0;
                if (row_valid) {
                    int len = a.part_seq_lens[qrow];
                    if (len > a.part_max_tokens) len = a.part_max_tokens;
                    const int chunk = (max(0, len - ctx) + a.part_chunk_tokens - 1) / a.part_chunk_tokens;
                    pslot = ((int64_t)qrow * a.part_n_chunks + chunk) * a.n_heads + head;
                    if (hf == 0) {
                        a.part_ml[pslot * 2] = m_used;
                        a.part_ml[pslot * 2 + 1] = l_row;
                    }
                }
#pragma unroll 1
                for (int ch = 0; ch < 2; ++ch) {
                    float o[32];
                    tmem_ld32(o_addr + ch * 32, o);
                    if (row_valid) {
                        float* dst = a.part_o + pslot * kHeadDim + hf * 64 + ch * 32;
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            *reinterpret_cast<float4*>(dst + 4 * i) = make_float4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
                    }
                }
            } else {
                const float inv = l_row > 0.f ? 1.f / l_row : 0.f;
                uint16_t* dst = reinterpret_cast<uint16_t*>(a.out) + (int64_t)(q_begin + q0 + my_t * kTileQ + row) * a.out_stride[0] +
                                (int64_t)head * a.out_stride[1] + hf * 64;
#pragma unroll 1
                for (int ch = 0; ch < 2; ++ch) {
                    float o[32];
                    tmem_ld32(o_addr + ch * 32, o);
                    if (row_valid) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            uint4 w;
                            w.x = pack2<BF16>(o[8 * i] * inv, o[8 * i + 1] * inv);
                            w.y = pack2<BF16>(o[8 * i + 2] * inv, o[8 * i + 3] * inv);
                            w.z = pack2<BF16>(o[8 * i + 4] * inv, o[8 * i + 5] * inv);
                            w.w = pack2<BF16>(o[8 * i + 6] * inv, o[8 * i + 7] * inv);
                            *reinterpret_cast<uint4*>(dst + ch * 32 + i * 8) = w;
                        }
                    }
                }
            }
        }
        timed_out = !ok;
    }
    if (timed_out && a.status && lane == 0) atomicOr(a.status, SFB_STATUS_WAIT_TIMEOUT);
    // ---- teardown: every warp arrives here; tensor memory is released before exit
    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
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

bool encode(CUtensorMap* map, const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides, const cuuint32_t* box) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint32_t es[5] = {1, 1, 1, 1, 1};
    for (int i = 0; i < rank - 1; ++i)
        if (strides[i] % 16 || strides[i] >= (1ull << 40)) return false;
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, rank, const_cast<void*>(base), dims, strides, box, es,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

// Returns SFB_ERR_UNSUPPORTED when the shape is outside this kernel (the caller then takes the generic route).
int launch_prefill_tcgen05(const PrefillLaunch& p, cudaStream_t stream) {
    if (p.head_dim != kHeadDim || p.block_size != 16 || (p.dtype != SFB_BF16 && p.dtype != SFB_F16)) return SFB_ERR_UNSUPPORTED;
    if (p.n_heads % p.n_kv_heads || p.n_requests > 65535 || p.n_heads > 65535 || p.n_pool_blocks >= (1ll << 31) - 1) return SFB_ERR_UNSUPPORTED;
    if (!p.part_o && (reinterpret_cast<uintptr_t>(p.out) % 16 || p.out_stride[0] % 8 || p.out_stride[1] % 8)) return SFB_ERR_UNSUPPORTED;
    CUtensorMap qmap, kmap, vmap;
    {
        cuuint64_t dims[4] = {128, (cuuint64_t)p.total_q, 2, (cuuint64_t)p.n_heads};
        cuuint64_t strides[3] = {(cuuint64_t)p.q_stride[0] * 2, 128, (cuuint64_t)p.q_stride[1] * 2};
        cuuint32_t box[4] = {128, (cuuint32_t)kTileQ, 1, 1};
        if (!encode(&qmap, p.q, 4, dims, strides, box)) return SFB_ERR_UNSUPPORTED;
    }
    for (int which = 0; which < 2; ++which) {
        const int64_t* st = which ? p.v_stride : p.k_stride;
        cuuint64_t dims[5] = {128, 16, 2, (cuuint64_t)p.n_kv_heads, (cuuint64_t)p.n_pool_blocks};
        cuuint64_t strides[4] = {(cuuint64_t)st[1] * 2, 128, (cuuint64_t)st[2] * 2, (cuuint64_t)st[0] * 2};
        cuuint32_t box[5] = {128, 16, which ? 2u : 1u, 1, 1};  // V: both 64-value halves of a block in one box
        if (!encode(which ? &vmap : &kmap, which ? p.v : p.k, 5, dims, strides, box)) return SFB_ERR_UNSUPPORTED;
    }
    PrefillArgs a{};
    a.q = p.q; a.out = p.out; a.cu_q = p.cu_q; a.ctx_lens = p.ctx_lens; a.row_limits = p.row_limits; a.tables = p.tables;
    a.table_stride = p.table_stride; a.max_blocks = p.max_blocks; a.n_requests = p.n_requests;
    a.n_heads = p.n_heads; a.n_kv_heads = p.n_kv_heads; a.n_pool_blocks = p.n_pool_blocks;
    a.out_stride[0] = p.out_stride[0]; a.out_stride[1] = p.out_stride[1];
    a.scale = p.scale; a.bf16 = p.dtype == SFB_BF16; a.causal = p.causal; a.status = p.status;
    a.fixed_nq = p.fixed_nq; a.fixed_ctx = p.fixed_ctx; a.part_o = p.part_o; a.part_ml = p.part_ml;
    a.part_seq_lens = p.part_seq_lens; a.part_n_chunks = p.part_n_chunks; a.part_chunk_tokens = p.part_chunk_tokens;
    a.part_max_tokens = p.part_max_tokens;
    dim3 grid((unsigned)ceil_div(p.max_q_tokens, 2 * kTileQ), (unsigned)p.n_heads, (unsigned)p.n_requests);
    if (a.bf16) {
        if (const int rc = allow_shared_memory_once(reinterpret_cast<const void*>(prefill_tcgen05_kernel<true>), kSmemBytes)) return rc;
        prefill_tcgen05_kernel<true><<<grid, kThreads, kSmemBytes, stream>>>(qmap, kmap, vmap, a);
    } else {
        if (const int rc = allow_shared_memory_once(reinterpret_cast<const void*>(prefill_tcgen05_kernel<false>), kSmemBytes)) return rc;
        prefill_tcgen05_kernel<false><<<grid, kThreads, kSmemBytes, stream>>>(qmap, kmap, vmap, a);
    }
    SFB_CUDA_CHECK(cudaGetLastError());
    return SFB_OK;
}

}  // namespace sfb
