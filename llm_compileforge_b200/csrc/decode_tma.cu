// Paged-attention decode, TMA + tensor-core kernel for sm_100a.
//
// Same algorithm as decode_generic.cuh (kernels/paged_attention.py:36-71 of the
// reference restated as split-K online softmax) for the shapes that matter at
// scale: block_size 16, K/V rows of 128 or 256 bytes (e4m3 D 128/256, bf16/fp16
// D 64/128), up to 8 query heads per kv head.
//
// Data movement: one producer warp walks the request's block table and, per
// 16-token KV block, issues one tiled TMA load for K and one for V
// (cp.async.bulk.tensor.5d, 128-byte swizzle) that land all kv heads of the
// thread block's head group in shared memory as [head][16 tokens][128 B] tiles;
// the per-(block, kv_head) FP8 scales ride along with 4-byte cp.async copies
// that arrive on the same mbarrier.  A ring of STAGES such buffers keeps
// 100-200 KB per SM in flight.
//
// Math: one consumer warp per (kv head, block slot).  S^T = K . Q^T runs as
// mma.sync.m16n8k16 with the 16 tokens of the block on the M axis and the (up
// to 8) query heads of the GQA group on the N axis, so the tile has no padding;
// O^T = V^T . P^T likewise with head_dim on M.  e4m3 codes are widened to fp16
// in registers (exact); the K scale multiplies the fp32 logit, the V scale is
// folded into the softmax exponent (weights exp2(s + log2 v_scale - m) feed
// the PV product, the denominator divides it back out), so dequantisation
// costs no extra pass.  With 8 query heads per kv head and 1-byte KV the fp32
// pipes could not keep up with HBM (2048 multiply-adds per 256 bytes); the
// tensor pipe runs this at a few percent utilisation.  Bound: HBM bandwidth.

#include <cuda.h>

#include <mutex>
#include <type_traits>

#include "sfb_common.cuh"

namespace sfb {
namespace {

constexpr float kLog2e = 1.4426950408889634f;
constexpr int kTileBytes = 2048;      // one [16 tokens][128 B] sub-tile
constexpr int kMaxChunkBlocks = 256;  // block-table entries cached per thread block
constexpr uint32_t kSpinLimit = 1u << 21;  // bounded waits: a stuck pipeline gives up (status bit) within about a second

enum KvKind { KV_E4M3 = 0, KV_BF16 = 1, KV_F16 = 2 };

// ---------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------
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
// Bounded wait: false when the phase did not complete within the spin limit.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
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
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c3, int c4) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
        ::"r"(dst), "l"(map), "r"(0), "r"(0), "r"(0), "r"(c3), "r"(c4), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint16_t v) {
    uint32_t r;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(v));
    return r;
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t v) {
    uint32_t r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(v));
    return r;
}
template <bool BF16>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if constexpr (BF16) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    } else {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
}
template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    uint32_t r;
    if constexpr (BF16) asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    else asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ float fast_exp2(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

// Row / chunk permutation that keeps the 128-bit shared loads conflict-free
// under the 128-byte TMA swizzle: consecutive lane groups alternate between the
// lower and upper half of the swizzle pattern.
__device__ __forceinline__ int perm8(int g) { return (g >> 1) | ((g & 1) << 2); }

__device__ __forceinline__ uint32_t word(const uint4& v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

template <int KV, int NSUB, int HB, int BPS, int STAGES>
struct Cfg {
    static constexpr bool kFp8 = KV == KV_E4M3;
    static constexpr bool kBf16 = KV == KV_BF16;       // MMA operand type: bf16, else fp16
    static constexpr int EPC = kFp8 ? 16 : 8;          // elements per 16-byte chunk
    static constexpr int EPR = 8 * EPC;                // elements per 128-byte sub-row
    static constexpr int D = NSUB * EPR;
    static constexpr int KSTEPS = D / 16;
    static constexpr int MTILES = D / 16;
    static constexpr int CONSUMERS = HB * BPS;
    static constexpr int THREADS = (CONSUMERS + 1) * 32;
    static constexpr int TILE = NSUB * kTileBytes;     // one (block, head) K or V tile
    static constexpr int KV_STAGE_BYTES = CONSUMERS * TILE;
    static constexpr int STAGE_BYTES = 2 * KV_STAGE_BYTES;
    static constexpr int SCALE_FLOATS = 2 * CONSUMERS;  // per stage: [K|V][BPS][HB]
    static constexpr int MERGE_FLOATS = MTILES * 4 + 4;  // per thread: O fragment + m0, m1, l0, l1
    static constexpr int AUX_BYTES = STAGES * SCALE_FLOATS * 4 + STAGES * BPS * 4 + kMaxChunkBlocks * 4 + 2 * STAGES * 8;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + AUX_BYTES + 1024;  // + alignment slack
    static constexpr int MIN_BLOCKS = (2 * SMEM_BYTES <= 227 * 1024) ? 2 : 1;  // co-resident thread blocks aimed for
    static_assert((BPS - 1) * HB * MERGE_FLOATS * 32 * 4 <= STAGES * STAGE_BYTES, "merge buffer must fit the ring");
};

// Running softmax state of one consumer warp: two query-head columns per thread.
template <int MTILES>
struct State {
    float o[MTILES][4];
    float m[2];
    float l[2];
};

// Output store: into `out`, or - when the heads of a batch are split over GPUs and every GPU wants the whole
// output - to the same element offset of every peer's buffer (plain stores over NVLink; this GPU's own buffer is
// one of the peers).  The peers learn that the data has landed from the signal kernel that follows on the stream.
template <typename QT, typename V>
__device__ __forceinline__ void store_out(const DecodeArgs& a, QT* out, int64_t off, V v) {
    if (a.n_peers == 0) {
        *reinterpret_cast<V*>(out + off) = v;
        return;
    }
#pragma unroll
    for (int p = 0; p < 8; ++p)
        if (p < a.n_peers) *reinterpret_cast<V*>(reinterpret_cast<QT*>(a.peer_out[p]) + off) = v;
}

template <int KV, int NSUB, int HB, int BPS, int STAGES, bool QBF16>
__global__ void __launch_bounds__(Cfg<KV, NSUB, HB, BPS, STAGES>::THREADS, Cfg<KV, NSUB, HB, BPS, STAGES>::MIN_BLOCKS)
decode_tma_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap, const DecodeArgs a) {
    using C = Cfg<KV, NSUB, HB, BPS, STAGES>;
    constexpr bool FP8 = C::kFp8, BF = C::kBf16;
    extern __shared__ uint8_t smem_raw[];
    int chunk = blockIdx.x, req = blockIdx.z;
    const int hg = blockIdx.y;
    if (a.work) {  // work list: largest items first, so the last wave is made of the small ones
        if ((int)blockIdx.x >= *a.n_work) return;
        const uint32_t item = a.work[blockIdx.x];
        req = (int)(item >> 16);
        chunk = (int)(item & 0xffffu);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = a.n_heads / a.n_kv_heads;
    const int n_chunks = (int)a.split.n_chunks;
    int* status = a.workspace ? reinterpret_cast<int*>(a.workspace) : nullptr;
    using QT = typename std::conditional<QBF16, __nv_bfloat16, __half>::type;
    QT* out = reinterpret_cast<QT*>(a.out);

    int len = a.seq_lens[req];
    if (len > a.max_blocks * 16) len = a.max_blocks * 16;
    len -= a.prefix_tokens;  // shared-prefix mode: this launch covers the tokens after the prefix
    if (len <= 0) {
        if (chunk == 0) {
            if (status && threadIdx.x == 0 && hg == 0) atomicOr(status, SFB_STATUS_EMPTY_REQUEST);
            for (int i = threadIdx.x; i < HB * group * C::D; i += C::THREADS)
                store_out(a, out, req * a.out_stride[0] + (hg * HB * group + i / C::D) * a.out_stride[1] + i % C::D, from_float<QT>(0.f));
        }
        return;
    }
    const int tok_begin = chunk * (int)a.split.chunk_tokens;
    if (tok_begin >= len) return;
    const int tok_end = min(len, tok_begin + (int)a.split.chunk_tokens);
    const int blk_begin = tok_begin >> 4;
    const int nblk = ((tok_end + 15) >> 4) - blk_begin;
    const int n_iters = (nblk + BPS - 1) / BPS;

    // ---- shared memory carve-up (ring first, 1024-byte aligned for the swizzle atoms)
    const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* ring_ptr = smem_raw + (ring - smem_u32(smem_raw));
    uint64_t* bars = reinterpret_cast<uint64_t*>(ring_ptr + STAGES * C::STAGE_BYTES);     // full[STAGES], empty[STAGES] (8-byte aligned)
    float* scales_s = reinterpret_cast<float*>(bars + 2 * STAGES);                         // [STAGES][2][BPS][HB]
    uint32_t* flags_s = reinterpret_cast<uint32_t*>(scales_s + STAGES * C::SCALE_FLOATS);  // [STAGES][BPS]
    int32_t* table_s = reinterpret_cast<int32_t*>(flags_s + STAGES * BPS);                 // [kMaxChunkBlocks]
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 33);              // producer lane 0 + 32 cp.async arrivals
            mbar_init(empty0 + 8 * s, C::CONSUMERS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    const int32_t* table = a.tables + decode_table_row(a, req, status) * a.table_stride + (a.prefix_tokens >> 4) + blk_begin;
    for (int i = threadIdx.x; i < nblk; i += C::THREADS) table_s[i] = table[i];
    __syncthreads();

    State<C::MTILES> st;
#pragma unroll
    for (int i = 0; i < C::MTILES; ++i) st.o[i][0] = st.o[i][1] = st.o[i][2] = st.o[i][3] = 0.f;
    st.m[0] = st.m[1] = -INFINITY;
    st.l[0] = st.l[1] = 0.f;
    const int h = warp % HB, slot = warp / HB;  // consumer role (unused by the producer warp)
    const int g = lane >> 2, t = lane & 3;
    const int kvh = hg * HB + h;
    const int rowk = perm8(g);  // K rows rowk, rowk+8 <-> MMA rows g, g+8; also this thread's V / output chunk
    bool timed_out = false;

    if (warp == C::CONSUMERS) {
        // =========================== producer warp ===========================
        for (int it = 0; it < n_iters; ++it) {
            const int s = it % STAGES, round = it / STAGES;
            if (!mbar_wait(empty0 + 8 * s, (round & 1) ^ 1)) { timed_out = true; break; }
            const uint32_t fb = full0 + 8 * s;
            if (lane == 0) {
                uint32_t bytes = 0;
                int64_t phys[BPS];
#pragma unroll
                for (int j = 0; j < BPS; ++j) {
                    const int bi = it * BPS + j;
                    phys[j] = bi < nblk ? (int64_t)table_s[bi] : -1;
                    bool ok = bi < nblk && phys[j] >= 0 && phys[j] < a.n_pool_blocks;
                    if (bi < nblk && !ok && status) atomicOr(status, SFB_STATUS_BAD_BLOCK_ID);
                    if (!ok) phys[j] = -1;
                    flags_s[s * BPS + j] = ok ? 1u : 0u;
                    if (ok) bytes += 2 * HB * C::TILE;
                }
                mbar_expect_tx(fb, bytes);
#pragma unroll
                for (int j = 0; j < BPS; ++j)
                    if (phys[j] >= 0) {
                        const uint32_t kd = ring + s * C::STAGE_BYTES + j * HB * C::TILE;
                        tma_load_5d(kd, &kmap, fb, hg * HB, (int)phys[j]);
                        tma_load_5d(kd + C::KV_STAGE_BYTES, &vmap, fb, hg * HB, (int)phys[j]);
                    }
            }
            if (FP8 && lane < 2 * C::CONSUMERS) {
                const int which = lane / C::CONSUMERS, r = lane % C::CONSUMERS;
                const int j = r / HB, hh = r % HB, bi = it * BPS + j;
                if (bi < nblk) {
                    const int64_t p = table_s[bi];
                    if (p >= 0 && p < a.n_pool_blocks) {
                        const float* src = which ? a.v_scale + p * a.vs_stride[0] + (hg * HB + hh) * a.vs_stride[1]
                                                 : a.k_scale + p * a.ks_stride[0] + (hg * HB + hh) * a.ks_stride[1];
                        cp_async_4(smem_u32(scales_s + s * C::SCALE_FLOATS + lane), src);
                    }
                }
            }
            cp_async_arrive_noinc(fb);
        }
    } else {
        // =========================== consumer warps ===========================
        // Query fragments (B operand of S^T = K.Q^T): column g = query head g of the group.
        uint32_t qf[C::KSTEPS][2];
        float colq0, colq1;  // softmax scale in log2 units for the score columns 2t, 2t+1 this thread holds
        {
            const QT* qrow = reinterpret_cast<const QT*>(a.q) + req * a.q_stride[0] + (int64_t)(kvh * group + g) * a.q_stride[1];
            uint2 raw[C::KSTEPS];
#pragma unroll
            for (int ks = 0; ks < C::KSTEPS; ++ks) {
                constexpr int per_chunk = C::EPC / 4;
                const int cc = ks / per_chunk, jj = ks % per_chunk;  // cc = sub*2 + ci
                const int d0 = (cc >> 1) * C::EPR + (t + 4 * (cc & 1)) * C::EPC + 4 * jj;
                raw[ks] = make_uint2(0u, 0u);
                if (g < group) raw[ks] = *reinterpret_cast<const uint2*>(qrow + d0);
            }
            float colexp = 1.f;
            if constexpr (QBF16 && !BF) {
                // A bf16 query feeding the fp16 MMA of an e4m3 pool.  bf16 reaches 3e38, fp16 65504: the row is first
                // scaled by a power of two that puts its largest magnitude into [2^13, 2^14) (exact in fp32; the 8-bit
                // bf16 significand then fits fp16's 11 bits, and what falls below fp16's range is 2^-37 of the row's
                // maximum), and the power goes back into the column's softmax scale.
                float amax = 0.f;
#pragma unroll
                for (int ks = 0; ks < C::KSTEPS; ++ks) {
                    amax = fmaxf(amax, fmaxf(fabsf(__uint_as_float(raw[ks].x << 16)), fabsf(__uint_as_float(raw[ks].x & 0xffff0000u))));
                    amax = fmaxf(amax, fmaxf(fabsf(__uint_as_float(raw[ks].y << 16)), fabsf(__uint_as_float(raw[ks].y & 0xffff0000u))));
                }
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));  // the four threads of a quad hold one query row
                int e = 0;
                if (amax > 0.f && amax < INFINITY) e = min(max((int)((__float_as_uint(amax) >> 23) & 0xffu) - 127 - 13, -100), 114);
                const float down = __uint_as_float((uint32_t)(127 - e) << 23);  // 2^-e
                colexp = __uint_as_float((uint32_t)(127 + e) << 23);            // 2^e
#pragma unroll
                for (int ks = 0; ks < C::KSTEPS; ++ks) {
                    const float f0 = __uint_as_float(raw[ks].x << 16) * down, f1 = __uint_as_float(raw[ks].x & 0xffff0000u) * down;
                    const float f2 = __uint_as_float(raw[ks].y << 16) * down, f3 = __uint_as_float(raw[ks].y & 0xffff0000u) * down;
                    qf[ks][0] = pack2<false>(f0, f1);
                    qf[ks][1] = pack2<false>(f2, f3);
                }
            } else {
#pragma unroll
                for (int ks = 0; ks < C::KSTEPS; ++ks) {
                    qf[ks][0] = raw[ks].x;
                    qf[ks][1] = raw[ks].y;
                }
            }
            const float qscale = a.scale * kLog2e;
            colq0 = qscale * __shfl_sync(0xffffffffu, colexp, (2 * t) * 4);      // lanes 4c .. 4c+3 hold query row c
            colq1 = qscale * __shfl_sync(0xffffffffu, colexp, (2 * t + 1) * 4);
        }
        for (int it = 0; it < n_iters; ++it) {
            const int s = it % STAGES, round = it / STAGES;
            if (!mbar_wait(full0 + 8 * s, round & 1)) { timed_out = true; break; }
            if (flags_s[s * BPS + slot]) {
                const int bi = it * BPS + slot;
                const int n_valid = min(16, tok_end - ((blk_begin + bi) << 4));
                const uint32_t kt = ring + s * C::STAGE_BYTES + (slot * HB + h) * C::TILE;
                const uint32_t vt = kt + C::KV_STAGE_BYTES;
                float ksc = 1.f, vsc = 1.f;
                if constexpr (FP8) {
                    ksc = scales_s[s * C::SCALE_FLOATS + slot * HB + h];
                    vsc = scales_s[s * C::SCALE_FLOATS + C::CONSUMERS + slot * HB + h];
                }
                // ---- S^T = K . Q^T, two accumulators to shorten the dependency chain
                float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int cc = 0; cc < 2 * NSUB; ++cc) {
                    const int c = t + 4 * (cc & 1);
                    const uint32_t addr = kt + (cc >> 1) * kTileBytes + rowk * 128 + ((c ^ rowk) << 4);
                    const uint4 r0 = lds128(addr), r1 = lds128(addr + 8 * 128);
                    if constexpr (FP8) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const uint32_t w0 = word(r0, j), w1 = word(r1, j);
                            const uint32_t af[4] = {e4m3x2_to_f16x2((uint16_t)w0), e4m3x2_to_f16x2((uint16_t)w1),
                                                    e4m3x2_to_f16x2((uint16_t)(w0 >> 16)), e4m3x2_to_f16x2((uint16_t)(w1 >> 16))};
                            const int ks = cc * 4 + j;
                            if (j & 1) mma16816<BF>(sb, af, qf[ks][0], qf[ks][1]);
                            else mma16816<BF>(sa, af, qf[ks][0], qf[ks][1]);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            const uint32_t af[4] = {word(r0, 2 * j), word(r1, 2 * j), word(r0, 2 * j + 1), word(r1, 2 * j + 1)};
                            const int ks = cc * 2 + j;
                            if (j & 1) mma16816<BF>(sb, af, qf[ks][0], qf[ks][1]);
                            else mma16816<BF>(sa, af, qf[ks][0], qf[ks][1]);
                        }
                    }
                }
                // ---- online softmax in log2 units; the V scale rides in the exponent
                const float qk0 = colq0 * ksc, qk1 = colq1 * ksc;
                const float lv = FP8 ? __log2f(vsc) : 0.f;
                const float ivsc = FP8 ? (vsc > 0.f ? __frcp_rn(vsc) : 0.f) : 1.f;
                float x0 = fmaf(sa[0] + sb[0], qk0, lv), x1 = fmaf(sa[1] + sb[1], qk1, lv);
                float x2 = fmaf(sa[2] + sb[2], qk0, lv), x3 = fmaf(sa[3] + sb[3], qk1, lv);
                if (n_valid < 16) {
                    if (rowk >= n_valid) x0 = x1 = -INFINITY;
                    if (rowk + 8 >= n_valid) x2 = x3 = -INFINITY;
                }
                float mx0 = fmaxf(x0, x2), mx1 = fmaxf(x1, x3);
#pragma unroll
                for (int o = 4; o <= 16; o <<= 1) {
                    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
                    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
                }
                const float mn0 = fmaxf(st.m[0], mx0), mn1 = fmaxf(st.m[1], mx1);
                if (__any_sync(0xffffffffu, mn0 > st.m[0] || mn1 > st.m[1])) {
                    const float c0 = fast_exp2(st.m[0] - mn0), c1 = fast_exp2(st.m[1] - mn1);  // -inf - finite -> 0
                    st.l[0] *= (mn0 > st.m[0]) ? c0 : 1.f;
                    st.l[1] *= (mn1 > st.m[1]) ? c1 : 1.f;
                    const float f0 = (mn0 > st.m[0]) ? c0 : 1.f, f1 = (mn1 > st.m[1]) ? c1 : 1.f;
#pragma unroll
                    for (int i = 0; i < C::MTILES; ++i) {
                        st.o[i][0] *= f0; st.o[i][1] *= f1; st.o[i][2] *= f0; st.o[i][3] *= f1;
                    }
                    st.m[0] = mn0;
                    st.m[1] = mn1;
                }
                const float mb0 = st.m[0] == -INFINITY ? 0.f : st.m[0], mb1 = st.m[1] == -INFINITY ? 0.f : st.m[1];
                const float w0 = fast_exp2(x0 - mb0), w1 = fast_exp2(x1 - mb1);
                const float w2 = fast_exp2(x2 - mb0), w3 = fast_exp2(x3 - mb1);
                st.l[0] = fmaf(w0 + w2, ivsc, st.l[0]);
                st.l[1] = fmaf(w1 + w3, ivsc, st.l[1]);
                const uint32_t pb0 = movmatrix_trans(pack2<BF>(w0, w1));
                const uint32_t pb1 = movmatrix_trans(pack2<BF>(w2, w3));
                // ---- O^T += V^T . P^T: this thread feeds tokens t, t+4, t+8, t+12 at its 16-byte column chunk
#pragma unroll
                for (int sub = 0; sub < NSUB; ++sub) {
                    uint4 v[4];
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        const int row = t + 4 * r;
                        v[r] = lds128(vt + sub * kTileBytes + row * 128 + ((rowk ^ (row & 7)) << 4));
                        if (n_valid < 16 && row >= n_valid) v[r] = make_uint4(0u, 0u, 0u, 0u);  // stale slots may hold NaN codes
                    }
#pragma unroll
                    for (int wi = 0; wi < 4; ++wi) {
                        const uint32_t A = word(v[0], wi), B = word(v[1], wi), Cw = word(v[2], wi), Dw = word(v[3], wi);
                        if constexpr (FP8) {
                            const uint32_t p01 = __byte_perm(A, B, 0x5140), p23 = __byte_perm(A, B, 0x7362);
                            const uint32_t q01 = __byte_perm(Cw, Dw, 0x5140), q23 = __byte_perm(Cw, Dw, 0x7362);
                            const uint32_t a0[4] = {e4m3x2_to_f16x2((uint16_t)p01), e4m3x2_to_f16x2((uint16_t)(p01 >> 16)),
                                                    e4m3x2_to_f16x2((uint16_t)q01), e4m3x2_to_f16x2((uint16_t)(q01 >> 16))};
                            const uint32_t a1[4] = {e4m3x2_to_f16x2((uint16_t)p23), e4m3x2_to_f16x2((uint16_t)(p23 >> 16)),
                                                    e4m3x2_to_f16x2((uint16_t)q23), e4m3x2_to_f16x2((uint16_t)(q23 >> 16))};
                            mma16816<BF>(st.o[sub * 8 + wi * 2], a0, pb0, pb1);
                            mma16816<BF>(st.o[sub * 8 + wi * 2 + 1], a1, pb0, pb1);
                        } else {
                            const uint32_t af[4] = {__byte_perm(A, B, 0x5410), __byte_perm(A, B, 0x7632),
                                                    __byte_perm(Cw, Dw, 0x5410), __byte_perm(Cw, Dw, 0x7632)};
                            mma16816<BF>(st.o[sub * 4 + wi], af, pb0, pb1);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * s);
        }
    }
    if (timed_out && status && lane == 0) atomicOr(status, SFB_STATUS_WAIT_TIMEOUT);
    const bool consumer = warp < C::CONSUMERS;

    // ---- merge the block slots of one head (BPS > 1) through the drained ring
    if constexpr (BPS > 1) {
        float* merge = reinterpret_cast<float*>(ring_ptr);  // [slot-1][h][field][lane]
        __syncthreads();
        if (consumer && slot > 0) {
            float* dst = merge + ((slot - 1) * HB + h) * C::MERGE_FLOATS * 32 + lane;
#pragma unroll
            for (int i = 0; i < C::MTILES; ++i)
#pragma unroll
                for (int k = 0; k < 4; ++k) dst[(i * 4 + k) * 32] = st.o[i][k];
            dst[(C::MTILES * 4 + 0) * 32] = st.m[0];
            dst[(C::MTILES * 4 + 1) * 32] = st.m[1];
            dst[(C::MTILES * 4 + 2) * 32] = st.l[0];
            dst[(C::MTILES * 4 + 3) * 32] = st.l[1];
        }
        __syncthreads();
        if (consumer && slot == 0) {
            for (int sl = 1; sl < BPS; ++sl) {
                const float* src = merge + ((sl - 1) * HB + h) * C::MERGE_FLOATS * 32 + lane;
                const float om0 = src[(C::MTILES * 4 + 0) * 32], om1 = src[(C::MTILES * 4 + 1) * 32];
                const float mn0 = fmaxf(st.m[0], om0), mn1 = fmaxf(st.m[1], om1);
                const float b0 = mn0 == -INFINITY ? 0.f : mn0, b1 = mn1 == -INFINITY ? 0.f : mn1;
                const float fs0 = fast_exp2(st.m[0] - b0), fs1 = fast_exp2(st.m[1] - b1);
                const float fo0 = fast_exp2(om0 - b0), fo1 = fast_exp2(om1 - b1);
                st.l[0] = st.l[0] * fs0 + src[(C::MTILES * 4 + 2) * 32] * fo0;
                st.l[1] = st.l[1] * fs1 + src[(C::MTILES * 4 + 3) * 32] * fo1;
#pragma unroll
                for (int i = 0; i < C::MTILES; ++i) {
                    st.o[i][0] = st.o[i][0] * fs0 + src[(i * 4 + 0) * 32] * fo0;
                    st.o[i][1] = st.o[i][1] * fs1 + src[(i * 4 + 1) * 32] * fo1;
                    st.o[i][2] = st.o[i][2] * fs0 + src[(i * 4 + 2) * 32] * fo0;
                    st.o[i][3] = st.o[i][3] * fs1 + src[(i * 4 + 3) * 32] * fo1;
                }
                st.m[0] = mn0;
                st.m[1] = mn1;
            }
        }
    }
    // ---- write the final rows (single-chunk request), or this chunk's partials
    const int used_chunks = (len + (int)a.split.chunk_tokens - 1) / (int)a.split.chunk_tokens;
    const int merge_chunks = used_chunks + (a.prefix_tokens > 0 ? 1 : 0);  // + the shared-prefix partial
    float* part_ml = reinterpret_cast<float*>(a.workspace + a.split.ml_offset);
    float* part_o = reinterpret_cast<float*>(a.workspace + a.split.o_offset);
    if (consumer && slot == 0) {
#pragma unroll
        for (int o = 4; o <= 16; o <<= 1) {
            st.l[0] += __shfl_xor_sync(0xffffffffu, st.l[0], o);
            st.l[1] += __shfl_xor_sync(0xffffffffu, st.l[1], o);
        }
#pragma unroll
        for (int col = 0; col < 2; ++col) {
            const int qh_in_group = 2 * t + col;
            if (qh_in_group >= group) continue;
            const int head = kvh * group + qh_in_group;
            const float l = st.l[col];
            if (merge_chunks == 1) {
                const float inv = l > 0.f ? 1.f / l : 0.f;
                const int64_t dst = req * a.out_stride[0] + (int64_t)head * a.out_stride[1];
#pragma unroll
                for (int sub = 0; sub < NSUB; ++sub) {
                    const int d0 = sub * C::EPR + rowk * C::EPC;
#pragma unroll
                    for (int q4 = 0; q4 < C::EPC / 8; ++q4) {  // 8 outputs = 16 bytes per store
                        uint32_t w[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const int mt = sub * (C::EPC / 2) + q4 * 4 + k;
                            w[k] = pack2<QBF16>(st.o[mt][col] * inv, st.o[mt][2 + col] * inv);
                        }
                        store_out(a, out, dst + d0 + q4 * 8, make_uint4(w[0], w[1], w[2], w[3]));
                    }
                }
            } else {
                const int64_t pslot = ((int64_t)req * n_chunks + chunk) * a.n_heads + head;
                if (g == 0) { part_ml[pslot * 2] = st.m[col]; part_ml[pslot * 2 + 1] = l; }
                float* dst = part_o + pslot * C::D;
#pragma unroll
                for (int sub = 0; sub < NSUB; ++sub) {
                    const int d0 = sub * C::EPR + rowk * C::EPC;
#pragma unroll
                    for (int q4 = 0; q4 < C::EPC / 4; ++q4) {  // 4 floats per store
                        const int mt = sub * (C::EPC / 2) + q4 * 2;
                        *reinterpret_cast<float4*>(dst + d0 + q4 * 4) =
                            make_float4(st.o[mt][col], st.o[mt][2 + col], st.o[mt + 1][col], st.o[mt + 1][2 + col]);
                    }
                }
            }
        }
    }
    if (merge_chunks == 1) return;

    // ---- the thread block that finishes a request's last chunk merges all of its partials
    // (no second launch; the partials it reads are still in L2)
    __shared__ int is_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int* done = reinterpret_cast<int*>(a.workspace + a.split.cnt_offset) + (int64_t)req * gridDim.y + hg;
        is_last = atomicAdd(done, 1) == used_chunks - 1;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    const int heads_here = HB * group;
    const int64_t slot_base = ((int64_t)req * n_chunks) * a.n_heads + hg * heads_here;
    // (a) per (head, chunk) weights exp2(m_c - m) / sum_c l_c exp2(m_c - m) into the drained ring
    float* w_s = reinterpret_cast<float*>(ring_ptr);  // [heads_here][merge_chunks]
    const bool fits = (int64_t)heads_here * merge_chunks * 4 <= (int64_t)STAGES * C::STAGE_BYTES;
    if (fits) {
        for (int hl = threadIdx.x; hl < heads_here; hl += C::THREADS) {
            float m = -INFINITY;
            for (int c = 0; c < merge_chunks; ++c) m = fmaxf(m, __ldcg(part_ml + (slot_base + hl + (int64_t)c * a.n_heads) * 2));
            float l = 0.f;
            for (int c = 0; c < merge_chunks; ++c) {
                const float2 ml = __ldcg(reinterpret_cast<const float2*>(part_ml + (slot_base + hl + (int64_t)c * a.n_heads) * 2));
                const float f = ml.x == -INFINITY ? 0.f : fast_exp2(ml.x - m);
                w_s[hl * merge_chunks + c] = f;
                l = fmaf(ml.y, f, l);
            }
            const float inv = l > 0.f ? 1.f / l : 0.f;
            for (int c = 0; c < merge_chunks; ++c) w_s[hl * merge_chunks + c] *= inv;
        }
        __syncthreads();
        // (b) out[h][d] = sum_c w[h][c] * part_o[c][h][d]; several independent 16-byte loads in flight per thread
        constexpr int VPR = C::D / 4;  // float4 per row
        constexpr int ITEMS = (HB * 8 * VPR + C::THREADS - 1) / C::THREADS;
        const int n_items = heads_here * VPR;
        float4 acc[ITEMS];
#pragma unroll
        for (int k = 0; k < ITEMS; ++k) acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int c = 0; c < merge_chunks; ++c) {
#pragma unroll
            for (int k = 0; k < ITEMS; ++k) {
                const int i = threadIdx.x + k * C::THREADS;
                if (i < n_items) {
                    const int hl = i / VPR, v4 = i - hl * VPR;
                    const float w = w_s[hl * merge_chunks + c];
                    const float4 x = __ldcg(reinterpret_cast<const float4*>(part_o + (slot_base + hl + (int64_t)c * a.n_heads) * C::D) + v4);
                    acc[k].x = fmaf(x.x, w, acc[k].x); acc[k].y = fmaf(x.y, w, acc[k].y);
                    acc[k].z = fmaf(x.z, w, acc[k].z); acc[k].w = fmaf(x.w, w, acc[k].w);
                }
            }
        }
#pragma unroll
        for (int k = 0; k < ITEMS; ++k) {
            const int i = threadIdx.x + k * C::THREADS;
            if (i < n_items) {
                const int hl = i / VPR, v4 = i - hl * VPR;
                store_out(a, out, req * a.out_stride[0] + (int64_t)(hg * heads_here + hl) * a.out_stride[1] + v4 * 4,
                          make_uint2(pack2<QBF16>(acc[k].x, acc[k].y), pack2<QBF16>(acc[k].z, acc[k].w)));
            }
        }
        return;
    }
    // very long splits: plain loop (one output element per thread at a time)
    for (int i = threadIdx.x; i < heads_here * C::D; i += C::THREADS) {
        const int hl = i / C::D, d = i - hl * C::D;
        float m = -INFINITY;
        for (int c = 0; c < merge_chunks; ++c) m = fmaxf(m, __ldcg(part_ml + (slot_base + hl + (int64_t)c * a.n_heads) * 2));
        float l = 0.f, o = 0.f;
        for (int c = 0; c < merge_chunks; ++c) {
            const int64_t ps = slot_base + hl + (int64_t)c * a.n_heads;
            const float mc = __ldcg(part_ml + ps * 2);
            if (mc == -INFINITY) continue;
            const float f = fast_exp2(mc - m);
            l = fmaf(__ldcg(part_ml + ps * 2 + 1), f, l);
            o = fmaf(__ldcg(part_o + ps * C::D + d), f, o);
        }
        store_out(a, out, req * a.out_stride[0] + (int64_t)(hg * heads_here + hl) * a.out_stride[1] + d, from_float<QT>(l > 0.f ? o / l : 0.f));
    }
}

// ---------------------------------------------------------------------------
// Host side: tensor maps and dispatch
// ---------------------------------------------------------------------------
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

// Byte view of a pool [NB, 16, Hkv, D]: dims (128 B, token, 128-B sub-row, head, block), so that one box
// [128, 16, NSUB, HB, 1] lands in shared memory as [head][sub][token][128 B].
bool make_pool_map(CUtensorMap* map, const void* base, const int64_t* stride_elems, int elem, int nsub, int hb, int n_kv_heads,
                   int64_t n_blocks) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[5] = {128, 16, (cuuint64_t)nsub, (cuuint64_t)n_kv_heads, (cuuint64_t)n_blocks};
    cuuint64_t strides[4] = {(cuuint64_t)(stride_elems[1] * elem), 128, (cuuint64_t)(stride_elems[2] * elem),
                             (cuuint64_t)(stride_elems[0] * elem)};
    cuuint32_t box[5] = {128, 16, (cuuint32_t)nsub, (cuuint32_t)hb, 1};
    cuuint32_t es[5] = {1, 1, 1, 1, 1};
    for (int i = 0; i < 4; ++i)
        if (strides[i] % 16 || strides[i] >= (1ull << 40)) return false;
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 5, const_cast<void*>(base), dims, strides, box, es,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// Work list of a split decode: one item per (request, chunk) that has tokens, ordered by size - full chunks first, then
// the partial last chunks from long to short (33 size classes, counting sort in one thread block).  Thread blocks are
// dispatched in list order, so the wave that finishes the launch consists of the smallest items instead of whatever
// request happens to come last; an item is (request << 16 | chunk).
constexpr int kWorkClasses = 33;
constexpr int64_t kWorkListMinItems = 600;  // fewer (request, chunk) slots than about two waves: plain grid order
constexpr int64_t kWorkListMinBytes = 1ll << 30;  // ... or a pool too small for the extra launch (a few microseconds) to pay

__global__ void __launch_bounds__(1024) decode_worklist_kernel(const int32_t* __restrict__ seq_lens, int batch, int max_tokens, int prefix_tokens,
                                                               int chunk_tokens, uint32_t* __restrict__ work, int* __restrict__ n_work) {
    __shared__ int count[kWorkClasses], cursor[kWorkClasses];
    if (threadIdx.x < kWorkClasses) count[threadIdx.x] = 0;
    __syncthreads();
    auto size_class = [&](int tokens) { return tokens >= chunk_tokens ? 0 : 32 - (int)(((int64_t)tokens * 32 - 1) / chunk_tokens); };
    auto request_len = [&](int r) {
        int len = seq_lens[r];
        if (len > max_tokens) len = max_tokens;
        return len - prefix_tokens;
    };
    for (int r = threadIdx.x; r < batch; r += blockDim.x) {
        const int len = request_len(r);
        if (len <= 0) { atomicAdd(&count[32], 1); continue; }  // the kernel's chunk-0 block zero-fills and flags it
        for (int c = 0; c * chunk_tokens < len; ++c) atomicAdd(&count[size_class(min(chunk_tokens, len - c * chunk_tokens))], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int i = 0; i < kWorkClasses; ++i) { cursor[i] = at; at += count[i]; }
        *n_work = at;
    }
    __syncthreads();
    for (int r = threadIdx.x; r < batch; r += blockDim.x) {
        const int len = request_len(r);
        if (len <= 0) { work[atomicAdd(&cursor[32], 1)] = (uint32_t)r << 16; continue; }
        for (int c = 0; c * chunk_tokens < len; ++c)
            work[atomicAdd(&cursor[size_class(min(chunk_tokens, len - c * chunk_tokens))], 1)] = ((uint32_t)r << 16) | (uint32_t)c;
    }
}

template <int KV, int NSUB, int HB, int BPS, bool QBF16>
int launch_cfg(const DecodeArgs& a, cudaStream_t stream) {
    constexpr int STAGES = (HB * BPS * NSUB >= 8) ? 3 : 4;
    using C = Cfg<KV, NSUB, HB, BPS, STAGES>;
    const int elem = KV == KV_E4M3 ? 1 : 2;
    CUtensorMap kmap, vmap;
    if (!make_pool_map(&kmap, a.k, a.k_stride, elem, NSUB, HB, a.n_kv_heads, a.n_pool_blocks) ||
        !make_pool_map(&vmap, a.v, a.v_stride, elem, NSUB, HB, a.n_kv_heads, a.n_pool_blocks))
        return SFB_ERR_UNSUPPORTED;
    auto kern = decode_tma_kernel<KV, NSUB, HB, BPS, STAGES, QBF16>;
    if (const int rc = allow_shared_memory_once(reinterpret_cast<const void*>(kern), C::SMEM_BYTES)) return rc;
    dim3 grid((unsigned)a.split.n_chunks, (unsigned)(a.n_kv_heads / HB), (unsigned)a.batch);
    DecodeArgs args = a;
    const int64_t slots = (int64_t)a.batch * a.split.n_chunks;
    const int64_t bytes_bound = (int64_t)a.batch * a.max_blocks * 16 * a.n_kv_heads * a.head_dim * elem * 2;  // every table full
    if (a.split.n_chunks > 1 && a.split.n_chunks <= 65536 && slots >= kWorkListMinItems && slots <= 0x7fffffffLL && bytes_bound >= kWorkListMinBytes &&
        a.workspace) {
        int* n_work = reinterpret_cast<int*>(a.workspace + a.split.work_offset);
        uint32_t* work = reinterpret_cast<uint32_t*>(a.workspace + a.split.work_offset + 256);
        decode_worklist_kernel<<<1, 1024, 0, stream>>>(a.seq_lens, a.batch, a.max_blocks * 16, a.prefix_tokens, (int)a.split.chunk_tokens, work, n_work);
        SFB_CUDA_CHECK(cudaGetLastError());
        args.work = work;
        args.n_work = n_work;
        grid = dim3((unsigned)slots, (unsigned)(a.n_kv_heads / HB), 1);
    }
    kern<<<grid, C::THREADS, C::SMEM_BYTES, stream>>>(kmap, vmap, args);
    SFB_CUDA_CHECK(cudaGetLastError());
    return SFB_OK;
}

template <int KV, int NSUB, bool QBF16>
int launch_heads(const DecodeArgs& a, cudaStream_t stream) {
    const int hkv = a.n_kv_heads;
    if (hkv % 8 == 0) return launch_cfg<KV, NSUB, 8, 1, QBF16>(a, stream);
    if (hkv % 4 == 0) return launch_cfg<KV, NSUB, 4, 2, QBF16>(a, stream);
    if (hkv % 2 == 0) return launch_cfg<KV, NSUB, 2, 4, QBF16>(a, stream);
    return launch_cfg<KV, NSUB, 1, 4, QBF16>(a, stream);
}

template <int KV, bool QBF16>
int launch_rows(const DecodeArgs& a, cudaStream_t stream) {
    const int row_bytes = a.head_dim * (KV == KV_E4M3 ? 1 : 2);
    if (row_bytes == 128) return launch_heads<KV, 1, QBF16>(a, stream);
    if (row_bytes == 256) return launch_heads<KV, 2, QBF16>(a, stream);
    return SFB_ERR_UNSUPPORTED;
}

}  // namespace

int launch_decode_tma(const DecodeArgs& a, cudaStream_t stream) {
    const int group = a.n_heads / a.n_kv_heads;
    if (a.block_size != 16 || group > 8 || a.q_dtype == SFB_F32) return SFB_ERR_UNSUPPORTED;
    if (a.split.chunk_tokens / 16 > kMaxChunkBlocks) return SFB_ERR_UNSUPPORTED;
    if (a.batch > 65535 || a.n_pool_blocks > 0x7fffffffLL) return SFB_ERR_UNSUPPORTED;
    // vector accesses on q / out rows
    if (reinterpret_cast<uintptr_t>(a.q) % 16 || reinterpret_cast<uintptr_t>(a.out) % 16) return SFB_ERR_UNSUPPORTED;
    for (int i = 0; i < 2; ++i)
        if (a.q_stride[i] % 8 || a.out_stride[i] % 8) return SFB_ERR_UNSUPPORTED;
    const bool qbf16 = a.q_dtype == SFB_BF16;
    switch (a.kv_dtype) {
        case SFB_F8E4M3: return qbf16 ? launch_rows<KV_E4M3, true>(a, stream) : launch_rows<KV_E4M3, false>(a, stream);
        case SFB_BF16: return launch_rows<KV_BF16, true>(a, stream);
        case SFB_F16: return launch_rows<KV_F16, false>(a, stream);
    }
    return SFB_ERR_UNSUPPORTED;
}

}  // namespace sfb
