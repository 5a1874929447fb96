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
// A work item is 256 query tokens (two 128-row tiles) of one (request, query head).  The grid is one resident thread block per
// SM; a block takes items blockIdx.x, blockIdx.x + gridDim.x, ... of a list ordered heaviest first, and runs them as ONE
// pipeline: the K / V tiles of consecutive items form a single stream through the two-slot rings, the next item's Q tiles
// land as soon as the current item's last Q.K^T has read the old ones, and the next item's first Q.K^T is issued in the place
// of the step's usual next score tile - the tensor pipe keeps running while the softmax warps write an item's rows out.
// Twelve warps (three warpgroups):
//   warp 0    issues tcgen05.mma (one thread): S_t = Q_t K^T (128x128x128, both operands K-major in 128B-swizzled shared
//             memory) and O_t += P_t V with P_t read from tensor memory and V as an MN-major shared-memory operand,
//             alternating between the two query tiles so that one tile's MMAs run while the other's rows are in the softmax warps
//   warp 1    TMA producer for Q and K: per 128-token KV tile sixteen [16 tokens x 128 B] boxes (block table entries are
//             fetched two tiles ahead; entries past the context become an out-of-range block index, which TMA zero-fills)
//   warp 2    TMA producer for V: eight [2 halves x 16 tokens x 128 B] boxes per tile; it also clears the V rows past the
//             context in the last KV tile (a pool that was never zero-filled may hold NaN there, and 0 * NaN would reach O)
//   warp 3    scheduler: works out each item's geometry (request offsets and lengths from global memory) ahead of time and
//             hands it to the other warps through a four-slot ring in shared memory
//   warps 4-11 softmax, one warpgroup per query tile, one thread per query row (warp w owns tensor-memory lanes 32*(w&3)..,
//             its hardware window).  A thread reads its row's 128 scores ONCE (tcgen05.ld into registers; the softmax
//             warpgroups raise their register allowance to 208 with setmaxnreg, the first warpgroup lowers its own), keeps
//             running max / sum in log2 units - no exchange with other threads -, writes P as bf16/fp16 over the first half
//             of its own S columns, rescales O in tensor memory only when the max grew by more than 2^8 (the stale max
//             stays exact in fp32) and writes O / l at the end of the item.
// Tensor memory: per query tile S|P (128 columns) and O (128) = 512 columns in all.
// Bound: tensor pipe (4*D*Sq*Skv flops per head); every wait is bounded and reports SFB_STATUS_WAIT_TIMEOUT.

#include <cuda.h>

#include <algorithm>
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
constexpr int kThreads = 384;  // a warpgroup with the MMA, TMA and scheduler warps + one softmax warpgroup per query tile
constexpr int kMmaWarp = 0, kTmaWarp = 1, kTmaWarpV = 2, kSchedWarp = 3, kFirstSoftmaxWarp = 4;
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
    int q_blocks;             // 256-row query blocks of the longest chunk
    int n_items;              // q_blocks * n_heads * n_requests work items
    int out_vec8;             // output rows allow 32-byte stores
    int* ticket;              // optional: zeroed counter the thread blocks draw item numbers from
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

// barrier slots.  The KV tiles of all work items of a thread block form ONE stream of steps g = 0, 1, ...: ring slot g&1 of
// K holds K(g), of V holds V(g); step g needs V(g) and K(g+1) (the next tile's scores, or the first tile of the next item), so
// one "full" / "empty" pair per step parity covers V slot g&1 together with K slot (g+1)&1.
enum {
    B_Q_FULL = 0,    // +query tile: the tile's Q rows have landed (tile 0 of the first item: and K(0))
    B_Q_EMPTY = 2,   // +query tile: the item's last Q.K^T of the tile is complete, the next item's rows may land
    B_KV_FULL = 4,   // +step parity: V(g) and K(g+1) have landed (one arrival per producer warp)
    B_KV_EMPTY = 6,  // +step parity: every MMA that read them is complete
    B_S_FULL = 8,    // +query tile
    B_P_FULL = 10,   // +query tile: P is in tensor memory (four warps arrive)
    B_PV_DONE = 12,  // +query tile: the item's last P.V product of the tile is complete
    B_V_FIXED = 14,  // the last KV tile's V rows past the context are cleared
    B_FINAL = 15,    // every MMA and every commit of this thread block is complete
    B_ITEM_FULL = 16,   // +ring slot: the scheduler warp has written the item record
    B_ITEM_EMPTY = 20,  // +ring slot: all nineteen consumer warps have read it
    B_COUNT = 24
};
constexpr int kItemSlots = 4, kItemConsumers = 10;  // the K producer, the MMA issuer and eight softmax warps
constexpr int kSmemBytes = 6 * kTileBytes + B_COUNT * 8 + 16 + kItemSlots * 64 + 1024;  // 2 Q tiles, 2 K stages, 2 V stages

// Tensor-memory columns of query tile t: S (fp32, 128 columns) at t*256, with P (16-bit pairs,
// 64 columns) written over its first half once the row has been read; O (fp32) at t*256 + 128.
constexpr uint32_t kColTile = 256;
constexpr uint32_t kColO = 128;

// Register allowances after the role split (three warpgroups of 128 threads; the kernel is compiled for
// 65536 / 384 -> 168 registers per thread, and shared memory admits one thread block per SM):
// 2 * 128 * kSoftmaxRegs + 128 * kOtherRegs <= 384 * 168 - a split that asks for more than the block owned at
// launch never returns from setmaxnreg.inc.
static_assert(2 * 128 * 208 + 128 * 88 <= 384 * 168, "register split exceeds the launch allocation");
constexpr int kSoftmaxRegs = 208;
constexpr int kOtherRegs = 88;

// One work item: 256 query rows (two 128-row tiles) of one (request, query head) - or, where a request's query block has no
// second tile (a chunk of at most 128 rows, or its ragged end), the same 128 rows of two query heads that share a kv head:
// both tensor-memory tile slots, softmax warp groups and the ping-pong stay in use, and the K / V stream serves two heads.
struct Item {
    int req, head, q_begin, q0, n_q, ctx;
    int rows[2], tiles[2], n_tiles;
    bool valid;
    bool pair;  // the query block has at most 128 rows: tile 1 is the same rows of the NEXT query head (same kv head)
    __device__ __forceinline__ int row0(int t) const { return q0 + (pair ? 0 : t * kTileQ); }  // first chunk row of tile t
    __device__ __forceinline__ int head_of(int t) const { return head + (pair ? t : 0); }
};

// Items are numbered heaviest first (the last query block of every request, all heads, then the block before ...).  A thread
// block takes the next number from a ticket in the workspace (whichever block is free takes the heaviest item left: requests
// of very different lengths still end together), or - without a workspace - the numbers blockIdx.x, blockIdx.x + gridDim.x, ...
// `idx` moves on (through `next`) to the first item at or after it that has work.  Called by a whole warp: with per-row limits
// the tiles' lengths come from the largest limit of each tile's rows, a reduction over the warp.
template <typename Next>
__device__ __forceinline__ Item find_item(const PrefillArgs& a, int& idx, bool report, Next next) {
    Item it;
    it.valid = false;
    it.pair = false;
    const int per_rank = a.n_heads * a.n_requests;
    for (; idx < a.n_items; idx = next()) {
        const int rank = idx / per_rank, rem = idx - rank * per_rank;
        it.req = rem / a.n_heads;
        it.head = rem - it.req * a.n_heads;
        it.q_begin = a.cu_q ? a.cu_q[it.req] : 0;
        it.n_q = a.cu_q ? a.cu_q[it.req + 1] - it.q_begin : a.fixed_nq;
        const int qb = (it.n_q + 2 * kTileQ - 1) / (2 * kTileQ) - 1 - rank;
        if (qb < 0) continue;
        int ctx = a.cu_q ? a.ctx_lens[it.req] : a.fixed_ctx;
        if (ctx > a.max_blocks * 16) ctx = a.max_blocks * 16;
        if ((a.causal && !a.row_limits && ctx < it.n_q) || it.n_q <= 0 || ctx <= 0) {  // inconsistent request: flag it, write nothing
            if (report && a.status) atomicOr(a.status, SFB_STATUS_EMPTY_REQUEST);
            continue;
        }
        it.ctx = ctx;
        it.q0 = qb * 2 * kTileQ;
        it.pair = it.n_q - it.q0 <= kTileQ && (a.n_heads / a.n_kv_heads) % 2 == 0;
        if (it.pair && (it.head & 1)) continue;  // the even head before it takes this one along
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            it.rows[t] = max(0, min(kTileQ, it.n_q - it.row0(t)));
            int last_pos = a.causal ? ctx - it.n_q + it.row0(t) + it.rows[t] - 1 : ctx - 1;
            if (a.row_limits) {
                int longest = 0;
                for (int r = threadIdx.x & 31; r < it.rows[t]; r += 32) longest = max(longest, min(max(a.row_limits[it.q_begin + it.row0(t) + r], 0), ctx));
                last_pos = max(__reduce_max_sync(0xffffffffu, longest), 1) - 1;
            }
            it.tiles[t] = it.rows[t] > 0 ? last_pos / kTileKV + 1 : 0;
        }
        it.n_tiles = max(it.tiles[0], it.tiles[1]);
        it.valid = true;
        return it;
    }
    return it;
}

template <bool BF16>
__global__ void __launch_bounds__(kThreads, 1)
prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                       const __grid_constant__ CUtensorMap vmap, const PrefillArgs a) {
    extern __shared__ uint8_t smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    uint64_t* bars = reinterpret_cast<uint64_t*>(base_ptr + 6 * kTileBytes);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + B_COUNT);
    int* item_ring = reinterpret_cast<int*>(tmem_slot + 4);  // [kItemSlots][16]
    const uint32_t q_s = base, k_s = base + 2 * kTileBytes, v_s = base + 4 * kTileBytes;
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };

    if (threadIdx.x == 0) {
        for (int s = 0; s < 2; ++s) {
            mbar_init(bar(B_Q_FULL + s), 1);
            mbar_init(bar(B_Q_EMPTY + s), 1);
            mbar_init(bar(B_KV_FULL + s), 2);
            mbar_init(bar(B_KV_EMPTY + s), 1);
            mbar_init(bar(B_S_FULL + s), 1);
            mbar_init(bar(B_P_FULL + s), 4);
            mbar_init(bar(B_PV_DONE + s), 1);
        }
        mbar_init(bar(B_V_FIXED), 1);
        mbar_init(bar(B_FINAL), 1);
        for (int s = 0; s < kItemSlots; ++s) {
            mbar_init(bar(B_ITEM_FULL + s), 1);
            mbar_init(bar(B_ITEM_EMPTY + s), kItemConsumers);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == kMmaWarp) tmem_alloc(smem_u32(tmem_slot), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    bool timed_out = false;
    const int group = a.n_heads / a.n_kv_heads;
    const int pool = (int)a.n_pool_blocks;  // the launcher keeps the pool below 2^31 blocks
    // Items reach the other warps through a small ring in shared memory that the scheduler warp fills ahead of time, so that
    // nobody waits for the global loads behind an item's geometry (request offsets and lengths) at an item boundary.
    auto fetch_item = [&](uint32_t n, Item& it) -> bool {
        const int slot = n & (kItemSlots - 1);
        if (!mbar_wait(bar(B_ITEM_FULL + slot), (n / kItemSlots) & 1)) return false;
        const int4* r = reinterpret_cast<const int4*>(item_ring + slot * 16);
        const int4 r0 = r[0], r1 = r[1], r2 = r[2];
        it.req = r0.x; it.head = r0.y; it.q_begin = r0.z; it.q0 = r0.w;
        it.n_q = r1.x; it.ctx = r1.y; it.rows[0] = r1.z; it.rows[1] = r1.w;
        it.tiles[0] = r2.x; it.tiles[1] = r2.y; it.n_tiles = r2.z; it.valid = (r2.w & 1) != 0; it.pair = (r2.w & 2) != 0;
        return true;
    };
    auto release_item = [&](uint32_t n) { mbar_arrive(bar(B_ITEM_EMPTY + (n & (kItemSlots - 1)))); };  // one lane per consumer warp

    if (warp < kFirstSoftmaxWarp) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kOtherRegs));
        if (warp == kTmaWarp) {
            // ============================ TMA producer: Q and K ===================
            // lane = (block of the tile, 64-value half), a [16 tokens x 128 B] box each, laid out [half][128 tokens][128 B].
            // At step g it loads K(g+1): the item's next tile or, at the item's last step, the first tile of the next item.
            const int blk = (lane & 15) >> 1, sub = lane & 1;
            const bool active = lane < 16;
            const uint32_t dst_off = sub * kSubBytes + blk * 2048;
            auto lookup = [&](const Item& it, int tile) -> int {
                if (!it.valid || tile * 8 + blk >= min(it.n_tiles * 8, (it.ctx + 15) >> 4)) return pool;  // past the context: TMA fills zeros
                const int p = a.tables[(int64_t)it.req * a.table_stride + tile * 8 + blk];
                if ((unsigned)p >= (unsigned)pool) {
                    if (a.status) atomicOr(a.status, SFB_STATUS_BAD_BLOCK_ID);
                    return pool;
                }
                return p;
            };
            uint32_t q_loaded = 0, q_phase = 0;  // bit t: tile t has been loaded before / parity of its next "empty" wait
            auto load_q = [&](const Item& it, int t, bool with_k0) -> bool {  // rows past the packed batch read as zeros
                if ((q_loaded >> t) & 1) {
                    if (!mbar_wait(bar(B_Q_EMPTY + t), (q_phase >> t) & 1)) return false;
                    q_phase ^= 1u << t;
                }
                q_loaded |= 1u << t;
                if (lane == 0) {
                    mbar_expect_tx(bar(B_Q_FULL + t), (with_k0 ? 2 : 1) * kTileBytes);
                    tma_load_4d(q_s + t * kTileBytes, &qmap, bar(B_Q_FULL + t), it.q_begin + it.row0(t), 0, it.head_of(t));
                    tma_load_4d(q_s + t * kTileBytes + kSubBytes, &qmap, bar(B_Q_FULL + t), it.q_begin + it.row0(t), 1, it.head_of(t));
                }
                __syncwarp();
                return true;
            };
            int g = 0;
            uint32_t n = 0;
            Item cur, nxt;
            cur.valid = false;
            if (!fetch_item(0, cur)) timed_out = true;
            if (cur.valid) {
                const int phys0 = lookup(cur, 0);
                load_q(cur, 0, true);
                if (active) tma_load_5d(k_s + dst_off, &kmap, bar(B_Q_FULL), sub, cur.head / group, phys0);  // K(0) into slot 0
                if (cur.tiles[1] > 0) load_q(cur, 1, false);
            }
            while (cur.valid && !timed_out) {
                nxt.valid = false;
                if (!fetch_item(n + 1, nxt)) { timed_out = true; break; }
                const int kvh = cur.head / group;
                const int next_first = lookup(nxt, 0);
                int phys = lookup(cur, 1), phys1 = lookup(cur, 2);
                for (int j = 0; j < cur.n_tiles; ++j, ++g) {
#pragma unroll
                    for (int t = 0; t < 2; ++t)
                        if (nxt.valid && j == cur.tiles[t] && nxt.tiles[t] > 0 && !load_q(nxt, t, false)) timed_out = true;
                    const int s = g & 1;
                    const int phys2 = lookup(cur, j + 3);  // table entries are fetched two tiles ahead of their use
                    // "empty" phases: slot 0 completes at the end of steps 0, 2, ...; slot 1 once the first Q.K(0)^T is done, then at
                    // the end of steps 1, 3, ...
                    const uint32_t par = s ? ((g >> 1) & 1) : (((g >> 1) & 1) ^ 1);
                    if (timed_out || !mbar_wait(bar(B_KV_EMPTY + s), par)) { timed_out = true; break; }
                    if (j + 1 < cur.n_tiles || nxt.valid) {
                        const bool own = j + 1 < cur.n_tiles;
                        if (lane == 0) mbar_expect_tx(bar(B_KV_FULL + s), kTileBytes);
                        __syncwarp();
                        if (active)
                            tma_load_5d(k_s + (s ^ 1) * kTileBytes + dst_off, &kmap, bar(B_KV_FULL + s), sub, own ? kvh : nxt.head / group,
                                        own ? phys : next_first);
                    } else if (lane == 0) {
                        mbar_arrive(bar(B_KV_FULL + s));  // no further K tile: the step's barrier still counts two arrivals
                    }
                    phys = phys1;
                    phys1 = phys2;
                }
#pragma unroll
                for (int t = 0; t < 2; ++t)
                    if (!timed_out && nxt.valid && cur.tiles[t] == cur.n_tiles && nxt.tiles[t] > 0 && !load_q(nxt, t, false)) timed_out = true;
                __syncwarp();
                if (lane == 0) release_item(n);
                cur = nxt;
                ++n;
            }
        } else if (warp == kTmaWarpV) {
            // ============================ TMA producer: V =========================
            // lane = block of the tile, one [2 halves x 16 tokens x 128 B] box each, laid out [block][half][16 tokens][128 B].
            const int blk = lane & 7;
            const bool active = lane < 8;
            auto lookup = [&](const Item& it, int tile) -> int {  // bad ids are reported by the K warp
                if (tile * 8 + blk >= min(it.n_tiles * 8, (it.ctx + 15) >> 4)) return pool;
                const int p = a.tables[(int64_t)it.req * a.table_stride + tile * 8 + blk];
                return (unsigned)p >= (unsigned)pool ? pool : p;
            };
            int g = 0;
            uint32_t n = 0;
            Item cur;
            cur.valid = false;
            if (!fetch_item(0, cur)) timed_out = true;
            while (cur.valid && !timed_out) {
                const int kvh = cur.head / group, g0 = g;
                int phys = lookup(cur, 0), phys1 = lookup(cur, 1);
                for (int j = 0; j < cur.n_tiles; ++j, ++g) {
                    const int s = g & 1;
                    const int phys2 = lookup(cur, j + 2);
                    const uint32_t par = s ? ((g >> 1) & 1) : (((g >> 1) & 1) ^ 1);
                    if (!mbar_wait(bar(B_KV_EMPTY + s), par)) { timed_out = true; break; }
                    if (lane == 0) mbar_expect_tx(bar(B_KV_FULL + s), kTileBytes);
                    __syncwarp();
                    if (active) tma_load_5d(v_s + s * kTileBytes + blk * 4096, &vmap, bar(B_KV_FULL + s), 0, kvh, phys);
                    phys = phys1;
                    phys1 = phys2;
                }
                // The KV tile that holds the last cached token may end inside a 16-token block: its V rows past the context are
                // cleared (an unzeroed pool may hold NaN there, and 0 * NaN would reach O).  A 128-byte row of a swizzled sub-tile
                // is permuted only inside itself, so whole rows can be cleared in place.
                const int fix_tile = (cur.ctx - 1) / kTileKV;
                if (!timed_out && (cur.ctx & 15) != 0 && fix_tile < cur.n_tiles) {
                    const int gf = g0 + fix_tile, s = gf & 1;
                    if (mbar_wait(bar(B_KV_FULL + s), (gf >> 1) & 1)) {
                        const int fblk = ((cur.ctx - 1) >> 4) & 7, first = cur.ctx & 15;
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
                __syncwarp();
                if (lane == 0) release_item(n);
                ++n;
                cur.valid = false;
                if (!timed_out && !fetch_item(n, cur)) timed_out = true;
            }
        } else if (warp == kSchedWarp) {
            // ============================ item scheduler ==========================
            int strided = blockIdx.x;
            auto next = [&]() -> int {
                if (!a.ticket) return strided += gridDim.x;
                int v = 0;
                if (lane == 0) v = atomicAdd(a.ticket, 1);
                return __shfl_sync(0xffffffffu, v, 0);
            };
            int idx = a.ticket ? next() : strided;
            for (uint32_t n = 0;; ++n) {
                const int slot = n & (kItemSlots - 1);
                if (n >= kItemSlots && !mbar_wait(bar(B_ITEM_EMPTY + slot), (n / kItemSlots - 1) & 1)) { timed_out = true; break; }
                const Item it = find_item(a, idx, lane == 0, next);
                if (lane == 0) {
                    int4* r = reinterpret_cast<int4*>(item_ring + slot * 16);
                    r[0] = make_int4(it.req, it.head, it.q_begin, it.q0);
                    r[1] = make_int4(it.n_q, it.ctx, it.rows[0], it.rows[1]);
                    r[2] = make_int4(it.tiles[0], it.tiles[1], it.n_tiles, (it.valid ? 1 : 0) | (it.pair ? 2 : 0));
                    mbar_arrive(bar(B_ITEM_FULL + slot));
                }
                __syncwarp();
                if (!it.valid) break;  // the end-of-work record
                idx = next();
            }
        } else if (warp == kMmaWarp) {
            // ============================ MMA issuer ==============================
            // One thread issues every MMA, per step in the order PV0(j), QK0(j+1), PV1(j), QK1(j+1): while one query tile's rows
            // are in the softmax warps, the tensor pipe works on the other tile.  At an item's last step the place of QK_t(j+1)
            // is taken by the NEXT item's first Q_t.K(0)^T, so the pipe runs on while the softmax warps write the item's rows
            // out.  An issue returns when the pipe accepts the MMA; descriptors are a constant plus a slot / K-step offset in
            // the low word.
            if (lane == 0) {
                constexpr uint32_t idesc_qk = instr_desc(BF16, false, kTileQ, kTileKV);
                constexpr uint32_t idesc_pv = instr_desc(BF16, true, kTileQ, kHeadDim);
                const uint32_t hi = (uint32_t)(smem_desc(0, 0, 1024) >> 32);
                const uint32_t q_lo = (uint32_t)smem_desc(q_s, 16, 0);
                const uint32_t k_lo = (uint32_t)smem_desc(k_s, 16, 0), v_lo = (uint32_t)smem_desc(v_s, 2048, 0);
                uint32_t q_phase = 0, p_phase = 0, fix_waits = 0;  // bit t: parity of tile t's next wait
                bool ok = true;
                // Q_t . K(slot)^T, 16 head-dim values per instruction; `first` = the item's first score tile (its Q rows must
                // have landed), `last` = the item's last one (the tile's Q rows may be replaced afterwards)
                auto issue_qk = [&](int t, int slot, bool first, bool last) {
                    if (first) {
                        ok = mbar_wait(bar(B_Q_FULL + t), (q_phase >> t) & 1);
                        q_phase ^= 1u << t;
                        if (!ok) return;
                        tc_fence_after();
                    }
                    const uint32_t qb_lo = q_lo + t * (kTileBytes >> 4), kb = k_lo + slot * (kTileBytes >> 4);
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks) {
                        const uint32_t off = ((ks >> 2) * kSubBytes + (ks & 3) * 32) >> 4;
                        mma_ss(tmem + t * kColTile, qb_lo + off, hi, kb + off, hi, idesc_qk, ks > 0);
                    }
                    tc_commit(bar(B_S_FULL + t));
                    if (last) tc_commit(bar(B_Q_EMPTY + t));
                };
                auto issue_pv = [&](int t, int slot, bool first, bool last) {  // 16 KV tokens per instruction
                    ok = mbar_wait(bar(B_P_FULL + t), (p_phase >> t) & 1);
                    p_phase ^= 1u << t;
                    if (!ok) return;
                    tc_fence_after();
                    const uint32_t vb = v_lo + slot * (kTileBytes >> 4), s_tm = tmem + t * kColTile;
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks)
                        mma_ts(s_tm + kColO, s_tm + ks * 8, vb + ks * (4096 >> 4), hi, idesc_pv, !first || ks > 0);
                    if (last) tc_commit(bar(B_PV_DONE + t));  // the epilogue waits for it
                };
                int g = 0;
                uint32_t n = 0;
                Item cur, nxt;
                cur.valid = false;
                ok = fetch_item(0, cur);
                if (cur.valid) {
#pragma unroll
                    for (int t = 0; t < 2; ++t)
                        if (ok && cur.tiles[t] > 0) issue_qk(t, 0, true, cur.tiles[t] == 1);
                    if (ok) tc_commit(bar(B_KV_EMPTY + 1));  // K slot 0 may take K(2) once these are done
                }
                while (ok && cur.valid) {
                    nxt.valid = false;
                    ok = fetch_item(n + 1, nxt);
                    const int fix_tile = (cur.ctx - 1) / kTileKV;
                    const bool fix_v = (cur.ctx & 15) != 0 && fix_tile < cur.n_tiles;
                    for (int j = 0; ok && j < cur.n_tiles; ++j, ++g) {
                        ok = mbar_wait(bar(B_KV_FULL + (g & 1)), (g >> 1) & 1);
                        if (ok && fix_v && j == fix_tile) {
                            ok = mbar_wait(bar(B_V_FIXED), fix_waits & 1);
                            ++fix_waits;
                        }
                        const bool last_step = j + 1 == cur.n_tiles;
#pragma unroll
                        for (int t = 0; t < 2; ++t) {
                            if (ok && j < cur.tiles[t]) issue_pv(t, g & 1, j == 0, j + 1 == cur.tiles[t]);
                            if (ok && j + 1 < cur.tiles[t]) issue_qk(t, (g + 1) & 1, false, j + 2 == cur.tiles[t]);
                            else if (ok && last_step && nxt.valid && nxt.tiles[t] > 0) issue_qk(t, (g + 1) & 1, true, nxt.tiles[t] == 1);
                        }
                        if (ok) tc_commit(bar(B_KV_EMPTY + (g & 1)));  // the producers wait for it before step g + 2
                    }
                    release_item(n);
                    cur = nxt;
                    ++n;
                }
                // every commit above arrives on a barrier of this block's shared memory: all of them must have landed before exit
                tc_commit(bar(B_FINAL));
                if (!mbar_wait(bar(B_FINAL), 0)) ok = false;
                timed_out = !ok;
            }
        }
    } else {
        // ======================= softmax / correction / epilogue ==============
        // Four warps per query tile, one thread per query row.  Warp w owns tensor-memory lanes 32*(w&3).. (its hardware
        // window) and all 128 key columns of its rows.
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kSoftmaxRegs));
        const int my_t = (warp - kFirstSoftmaxWarp) >> 2;  // query tile of this 4-warp group
        const int row = threadIdx.x & 127;
        const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        const float sl2 = a.scale * kLog2e;
        const uint32_t s_addr = lane_addr + my_t * kColTile;  // this thread's row: 128 score columns
        const uint32_t o_addr = lane_addr + my_t * kColTile + kColO;
        uint32_t s_waits = 0, e_waits = 0;
        float m_used = -INFINITY, l = 0.f;
        int pos = 0;

        auto softmax_tile = [&](int j) -> bool {
            if (!mbar_wait(bar(B_S_FULL + my_t), s_waits & 1)) return false;
            ++s_waits;
            tc_fence_after();
            const int kv0 = j * kTileKV;
            // tcgen05.ld / st are warp-collective: the masked / unmasked choice must be uniform across the warp
            const bool full = __all_sync(0xffffffffu, kv0 + 127 <= pos);
            float s[128];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld32_issue(s_addr + 32 * c, *reinterpret_cast<float(*)[32]>(s + 32 * c));
            tmem_wait_ld();
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
            if (full) {
#pragma unroll
                for (int i = 0; i < 128; i += 8) {
                    mx0 = max3(mx0, s[i], s[i + 1]);
                    mx1 = max3(mx1, s[i + 2], s[i + 3]);
                    mx2 = max3(mx2, s[i + 4], s[i + 5]);
                    mx3 = max3(mx3, s[i + 6], s[i + 7]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 128; ++i) {
                    if (kv0 + i > pos) s[i] = -INFINITY;  // exp2(-inf) = 0 below
                    mx0 = fmaxf(mx0, s[i]);
                }
            }
            const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
            const float m_new = fmaxf(m_used, mx * sl2);
            if (j == 0) {
                m_used = m_new;
            } else {
                const bool need = m_new > m_used + kRescaleThreshold;
                if (__any_sync(0xffffffffu, need)) {
                    // O is only touched between P.V products.  The previous one is complete: this tile's S was committed by
                    // the same thread after it, and a commit covers everything that thread issued before.
                    const float f = need ? fast_exp2(m_used - m_new) : 1.f;
                    l *= f;
                    if (need) m_used = m_new;
#pragma unroll 1
                    for (int ch = 0; ch < 8; ++ch) {
                        float o[16];
                        tmem_ld16(o_addr + ch * 16, o);
#pragma unroll
                        for (int i = 0; i < 16; ++i) o[i] *= f;
                        tmem_st16(o_addr + ch * 16, *reinterpret_cast<uint32_t(*)[16]>(o));
                    }
                    tmem_wait_st();
                }
            }
            // P (16-bit pairs, 64 columns) goes over the first half of this thread's own score columns
            const float neg_m = m_used == -INFINITY ? 0.f : -m_used;  // a row that sees nothing yet: every score is -inf, P = 0
            const float2 sl2v = make_float2(sl2, sl2), nmv = make_float2(neg_m, neg_m);
            float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {
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
            }
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(B_P_FULL + my_t));
            l += (acc0.x + acc1.x) + (acc0.y + acc1.y);
            return true;
        };

        bool ok = true;
        uint32_t n = 0;
        Item cur;
        cur.valid = false;
        ok = fetch_item(0, cur);
        while (ok && cur.valid) {
            const int my_rows = my_t ? cur.rows[1] : cur.rows[0], my_tiles = my_t ? cur.tiles[1] : cur.tiles[0];
            if (my_tiles > 0) {
                // last visible position of this thread's row; padding rows see everything
                const int my_row = cur.row0(my_t) + row, my_head = cur.head_of(my_t);  // row of the request's chunk, query head
                pos = (row < my_rows && a.causal) ? cur.ctx - cur.n_q + my_row : cur.ctx - 1;
                if (a.row_limits && row < my_rows) pos = min(max(a.row_limits[cur.q_begin + my_row], 0), cur.ctx) - 1;
                m_used = -INFINITY;
                l = 0.f;
                for (int j = 0; j < my_tiles && ok; ++j) ok = softmax_tile(j);
                // ---- epilogue: O / l, each thread its 64 output columns
                if (ok) {
                    ok = mbar_wait(bar(B_PV_DONE + my_t), e_waits & 1);
                    ++e_waits;
                }
                if (ok) {
                    tc_fence_after();
                    const float l_row = l;
                    const bool row_valid = row < my_rows;
                    if (a.part_o) {
                        // shared-prefix mode: this row is decode request `qrow`; its partial goes to the chunk slot right after
                        // the request's own chunks, in the decode kernel's format (unnormalised O, max in log2 units, sum)
                        const int qrow = my_row;
                        int64_t pslot = 0;
                        if (row_valid) {
                            int len = a.part_seq_lens[qrow];
                            if (len > a.part_max_tokens) len = a.part_max_tokens;
                            const int chunk = (max(0, len - cur.ctx) + a.part_chunk_tokens - 1) / a.part_chunk_tokens;
                            pslot = ((int64_t)qrow * a.part_n_chunks + chunk) * a.n_heads + my_head;
                            a.part_ml[pslot * 2] = m_used;
                            a.part_ml[pslot * 2 + 1] = l_row;
                        }
#pragma unroll 1
                        for (int ch = 0; ch < 4; ++ch) {
                            float o[32];
                            tmem_ld32(o_addr + ch * 32, o);
                            if (row_valid) {
                                float* dst = a.part_o + pslot * kHeadDim + ch * 32;
#pragma unroll
                                for (int i = 0; i < 8; ++i)
                                    *reinterpret_cast<float4*>(dst + 4 * i) = make_float4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
                            }
                        }
                    } else {
                        const float inv = l_row > 0.f ? 1.f / l_row : 0.f;
                        uint16_t* dst = reinterpret_cast<uint16_t*>(a.out) + (int64_t)(cur.q_begin + my_row) * a.out_stride[0] +
                                        (int64_t)my_head * a.out_stride[1];
#pragma unroll 1
                        for (int ch = 0; ch < 4; ++ch) {
                            float o[32];
                            tmem_ld32(o_addr + ch * 32, o);
                            if (row_valid) {
#pragma unroll
                                for (int i = 0; i < 2; ++i) {
                                    uint32_t w[8];
#pragma unroll
                                    for (int k = 0; k < 8; ++k) w[k] = pack2<BF16>(o[16 * i + 2 * k] * inv, o[16 * i + 2 * k + 1] * inv);
                                    uint16_t* p = dst + ch * 32 + i * 16;
                                    if (a.out_vec8) {
                                        asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]),
                                                     "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                                                     : "memory");
                                    } else {
                                        *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
                                        *reinterpret_cast<uint4*>(p + 8) = make_uint4(w[4], w[5], w[6], w[7]);
                                    }
                                }
                            }
                        }
                    }
                    // the next item's first P.V overwrites O: it waits for this warp's next P, which follows these loads in program
                    // order (tcgen05.wait::ld above), so nothing else has to say that O has been read
                    tc_fence_before();
                }
            }
            __syncwarp();
            if (lane == 0) release_item(n);
            ++n;
            cur.valid = false;
            ok = ok && fetch_item(n, cur);
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

int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0) n = v;
        else return 148;
    }
    return n;
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
    // Work items (256 query rows of one head of one request) are spread over one resident thread block per SM.
    a.q_blocks = (int)ceil_div(p.max_q_tokens, 2 * kTileQ);
    const int64_t n_items = (int64_t)a.q_blocks * p.n_heads * p.n_requests;
    if (n_items <= 0) return SFB_OK;
    if (n_items > 0x7fffffffLL) return SFB_ERR_UNSUPPORTED;
    a.n_items = (int)n_items;
    a.out_vec8 = !p.part_o && reinterpret_cast<uintptr_t>(p.out) % 32 == 0 && p.out_stride[0] % 16 == 0 && p.out_stride[1] % 16 == 0;
    a.ticket = p.ticket;
    const dim3 grid((unsigned)std::min<int64_t>(n_items, sm_count()));
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
