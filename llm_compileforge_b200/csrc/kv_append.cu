// KV cache write and FP8 quantise-on-append.
//
// Slot rule restated from python_runtime/engine/cache_manager.py:154-159 of the
// reference: token at position p of a request goes to (table[p / bs], p % bs).
// Quantiser restated from compiler/quantize/fp8_kv_cache.py:81-89, applied to
// every touched (block, kv_head) slice: amax over the slice (unwritten slots
// count as zero), scale = amax/448 (1.0 when amax == 0, at least 1e-12),
// codes = e4m3(x / scale) with an IEEE division.
//
// One warp owns one (block, kv_head) slice: it pulls the slice's rows with
// 128-bit loads (rows that precede this call's tokens come from the request's
// unquantised tail copy, rows after them are zero), keeps them in registers,
// reduces |x| with shuffles (packed 16-bit max), divides through a correctly
// rounded reciprocal + one FMA correction, then writes codes, scale and - while
// the block is still open - the refreshed tail copy.  Single pass over the source; bound:
// HBM bandwidth.

#include <type_traits>

#include "sfb_common.cuh"

namespace sfb {
namespace {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;

template <typename T>
struct Src;  // 16-byte chunk of the source dtype
template <>
struct Src<float> {
    static constexpr int N = 4;
    __device__ static void unpack(const uint4& r, float* o) {
        o[0] = __uint_as_float(r.x); o[1] = __uint_as_float(r.y);
        o[2] = __uint_as_float(r.z); o[3] = __uint_as_float(r.w);
    }
};
template <>
struct Src<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ static void unpack(const uint4& r, float* o) {
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            o[2 * i] = __uint_as_float(w[i] << 16);
            o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};
template <>
struct Src<__half> {
    static constexpr int N = 8;
    __device__ static void unpack(const uint4& r, float* o) {
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            o[2 * i] = f.x; o[2 * i + 1] = f.y;
        }
    }
};

// Running |x| maximum over 16-byte chunks, NaN-propagating like torch's abs().max().
// 16-bit sources stay packed (one AND and one packed max per two values).
template <typename ST>
struct AbsMax;
template <>
struct AbsMax<float> {
    float m = 0.f;
    __device__ void add(const uint4& r) {
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) asm("max.NaN.f32 %0, %0, %1;" : "+f"(m) : "f"(fabsf(__uint_as_float(w[i]))));
    }
    __device__ float value() const { return m; }
};
template <>
struct AbsMax<__nv_bfloat16> {
    uint32_t m = 0u;
    __device__ void add(const uint4& r) {
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) asm("max.NaN.bf16x2 %0, %0, %1;" : "+r"(m) : "r"(w[i] & 0x7fff7fffu));
    }
    __device__ float value() const {
        float r = __uint_as_float(m << 16);
        asm("max.NaN.f32 %0, %0, %1;" : "+f"(r) : "f"(__uint_as_float(m & 0xffff0000u)));
        return r;
    }
};
template <>
struct AbsMax<__half> {
    uint32_t m = 0u;
    __device__ void add(const uint4& r) {
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) asm("max.NaN.f16x2 %0, %0, %1;" : "+r"(m) : "r"(w[i] & 0x7fff7fffu));
    }
    __device__ float value() const {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&m));
        float r = f.x;
        asm("max.NaN.f32 %0, %0, %1;" : "+f"(r) : "f"(f.y));
        return r;
    }
};

__device__ __forceinline__ float warp_max_nan(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, v, o);
        asm("max.NaN.f32 %0, %0, %1;" : "+f"(v) : "f"(other));
    }
    return v;
}

// scale rule of fp8_kv_cache.py:81-86 (a NaN in the slice makes amax, hence the scale, NaN)
__device__ __forceinline__ float scale_from_amax(float amax) {
    if (amax != amax) return amax;
    if (amax == 0.f) return 1.0f;
    return fmaxf(__fdiv_rn(amax, 448.0f), 1e-12f);
}

// x / scale for every element of a slice.  The reference divides (fp8_kv_cache.py:89), so the
// quotient must be the correctly rounded one.  With r = RN(1/scale): q = RN(x r),
// q' = RN(q + RN(x - q scale) r) is that quotient (the residual is exact in an FMA; this is the
// fast path of IEEE float division) as long as no intermediate leaves the normal range, which
// holds for scales in [2^-60, 2^60]: there |q| <= 448 (1 + 2^-23), and an x small enough for the
// residual to underflow gives a quotient far below the smallest e4m3 step.  Other scales, NaN
// included, take the division instruction.
struct Divider {
    float scale, rcp;
    bool fast;
    __device__ static Divider make(float s) {
        Divider d;
        d.scale = s;
        d.rcp = __frcp_rn(s);
        d.fast = s >= 0x1p-60f && s <= 0x1p60f;
        return d;
    }
    // the quotient without its sign repaired: +0 where the true quotient is -0 (x = -0.0, or a negative x that underflows)
    __device__ __forceinline__ float quick_unsigned_zero(float x) const {
        const float q = __fmul_rn(x, rcp);
        return __fmaf_rn(__fmaf_rn(-q, scale, x), rcp, q);
    }
    // two quotients at once on the packed fp32 pipe (fmul2 / ffma2: each half rounds like the scalar instruction, so the
    // result is bit-identical; half the instructions)
    __device__ __forceinline__ float2 quick2_unsigned_zero(float2 x) const {
        const float2 r2 = make_float2(rcp, rcp), ns2 = make_float2(-scale, -scale);
        const float2 q = __fmul2_rn(x, r2);
        return __ffma2_rn(__ffma2_rn(q, ns2, x), r2, q);
    }
    __device__ __forceinline__ float quick(float x) const {
        return copysignf(quick_unsigned_zero(x), x);  // scale > 0: the quotient has x's sign, also when it is zero (-0.0 encodes as 0x80)
    }
};

// N source values -> N codes packed little-endian into 32-bit words.  For 16-bit sources the sign of a zero quotient is
// put back on the packed codes - the four source sign bytes gathered with one byte permute and OR-ed in (a no-op for
// non-zero quotients, whose codes already carry it) - instead of one copysign per value.
template <int N>
__device__ __forceinline__ void encode_quick(const float* x, const uint4& raw, const Divider& div, uint32_t* words) {
    if constexpr (N == 8) {
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float2 qa = div.quick2_unsigned_zero(make_float2(x[4 * i], x[4 * i + 1]));
            const float2 qb = div.quick2_unsigned_zero(make_float2(x[4 * i + 2], x[4 * i + 3]));
            uint16_t lo = float2_to_e4m3x2(qa.x, qa.y);
            uint16_t hi = float2_to_e4m3x2(qb.x, qb.y);
            words[i] = ((uint32_t)lo | ((uint32_t)hi << 16)) | (__byte_perm(w[2 * i], w[2 * i + 1], 0x7531) & 0x80808080u);
        }
    } else {
#pragma unroll
        for (int i = 0; i < N / 4; ++i) {
            uint16_t lo = float2_to_e4m3x2(div.quick(x[4 * i]), div.quick(x[4 * i + 1]));
            uint16_t hi = float2_to_e4m3x2(div.quick(x[4 * i + 2]), div.quick(x[4 * i + 3]));
            words[i] = (uint32_t)lo | ((uint32_t)hi << 16);
        }
    }
}
// the rare out-of-range scale: IEEE division instruction, kept out of line and register-to-register
template <typename ST>
__device__ __noinline__ uint2 encode_exact_chunk(uint4 raw, float scale) {
    constexpr int N = Src<ST>::N;
    float x[N];
    Src<ST>::unpack(raw, x);
    uint32_t words[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < N / 4; ++i) {
        uint16_t lo = float2_to_e4m3x2(__fdiv_rn(x[4 * i], scale), __fdiv_rn(x[4 * i + 1], scale));
        uint16_t hi = float2_to_e4m3x2(__fdiv_rn(x[4 * i + 2], scale), __fdiv_rn(x[4 * i + 3], scale));
        words[i] = (uint32_t)lo | ((uint32_t)hi << 16);
    }
    return make_uint2(words[0], words[1]);
}

// CPL = 16-byte source chunks each lane keeps; a slice has bs * D / N chunks.
// Grid: x strides over the blocks a request touches, y = request, z = K / V.
template <typename ST, int CPL, bool FP8, bool EVEN, bool FIRST>
// The quantising kernel for 16-bit sources is held to 96 registers (five thread blocks per SM instead of four): measured 1.4 %
// faster on 638 k appended tokens than the 128 the compiler takes by itself; six (80 registers) and eight (64) are slower.
__global__ void __launch_bounds__(kThreads, (FP8 && sizeof(ST) == 2 && CPL <= 8 && EVEN) ? 5 : 1) cache_write_kernel(AppendArgs a) {
    constexpr bool first_pass = FIRST;
    constexpr int N = Src<ST>::N;
    const int req = blockIdx.y, which = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bs = a.block_size, dim = a.head_dim;
    const int n_new = a.cu_tokens[req + 1] - a.cu_tokens[req];
    if (n_new <= 0) return;
    const int start = a.start_pos[req], end = start + n_new;
    const int first_blk = start / bs;
    const int last_blk = min((end - 1) / bs, a.max_blocks - 1);
    // pass 0 handles each request's first touched block (the one that reads the tail copy),
    // pass 1 all later ones (the last of which rewrites the tail copy)
    int blk = first_pass ? first_blk : first_blk + 1 + (int)blockIdx.x;
    const int blk_step = first_pass ? (1 << 30) : (int)gridDim.x;

    const ST* src = reinterpret_cast<const ST*>(which ? a.v_new : a.k_new) + (int64_t)a.cu_tokens[req] * (which ? a.vnew_stride[0] : a.new_stride[0]);
    const int64_t src_tok = which ? a.vnew_stride[0] : a.new_stride[0];
    const int64_t src_head = which ? a.vnew_stride[1] : a.new_stride[1];
    const int64_t* ps = which ? a.v_stride : a.k_stride;
    // rows of the table / tail arrays this request uses; a row outside either array skips the request
    const int64_t trow = a.table_rows ? a.table_rows[req] : req;
    if (trow < 0 || trow >= a.n_table_rows) return;
    const int32_t* table = a.tables + trow * a.table_stride;
    const int64_t tail_row = a.tail_rows ? a.tail_rows[req] : req;
    if (FP8 && (tail_row < 0 || tail_row >= a.n_tail_rows)) return;
    const int cpr = dim / N;            // chunks per row
    const int n_chunks = bs * cpr;

    // This lane's chunk j of a slice sits at row (token slot) row_of(j), column col_of(j).  When the chunks
    // of a row divide a warp evenly (every usual head_dim) the column is the same for all j.
    constexpr bool even = EVEN;  // (32 % cpr) == 0, checked by the launcher
    const int r0 = even ? lane / cpr : 0, rpp = even ? 32 / cpr : 0, c0 = even ? (lane % cpr) * N : 0;
    auto row_of = [&](int j) -> int {
        const int i = lane + 32 * j;
        if (i >= n_chunks) return 1 << 20;
        return even ? r0 + j * rpp : i / cpr;
    };
    auto col_of = [&](int j) -> int { return even ? c0 : ((lane + 32 * j) % cpr) * N; };

    if constexpr (!FP8) {
        for (; blk <= last_blk; blk += blk_step) {
            const int64_t phys = table[blk];
            if (phys < 0 || phys >= a.n_pool_blocks) continue;
            const int lo = blk * bs;
            ST* pool = reinterpret_cast<ST*>(which ? a.v_cache : a.k_cache) + phys * ps[0];
            for (int h = warp; h < a.n_kv_heads; h += kWarps)
                for (int i = lane; i < n_chunks; i += 32) {
                    int t = i / cpr, c = i - t * cpr, p = lo + t;
                    if (p >= start && p < end) {
                        uint4 v = ldg_stream(src + (int64_t)(p - start) * src_tok + h * src_head + c * N);
                        *reinterpret_cast<uint4*>(pool + t * ps[1] + h * ps[2] + c * N) = v;
                    }
                }
        }
    } else {
        uint8_t* pool_base = reinterpret_cast<uint8_t*>(which ? a.v_cache : a.k_cache);
        float* scales = which ? a.v_scale : a.k_scale;
        const int64_t* ss = which ? a.vs_stride : a.ks_stride;
        const int64_t* ts = which ? a.vt_stride : a.kt_stride;
        ST* tail = reinterpret_cast<ST*>(which ? a.v_tail : a.k_tail) + tail_row * ts[0];
        if (warp >= a.n_kv_heads) return;

        // The warp walks its (block, head) slices with the next slice's rows already in flight
        // while the current one is reduced and encoded.
        const bool full_lanes = n_chunks == 32 * CPL;  // every lane owns CPL chunks of a slice: no row check needed
        auto fetch = [&](int fb, int fh, uint4 (&raw)[CPL]) {
            const int lo = fb * bs;
            if (full_lanes && lo >= start && lo + bs <= end) {  // a block that lies wholly inside the appended range: plain loads
                const ST* base = src + (int64_t)(lo - start) * src_tok + fh * src_head;
#pragma unroll
                for (int j = 0; j < CPL; ++j) raw[j] = ldg_stream(base + (int64_t)row_of(j) * src_tok + col_of(j));
                return;
            }
#pragma unroll
            for (int j = 0; j < CPL; ++j) {
                raw[j] = make_uint4(0, 0, 0, 0);
                const int p = lo + row_of(j);  // lanes past the slice get a row beyond `end`
                if (FIRST && p < start) raw[j] = *reinterpret_cast<const uint4*>(tail + row_of(j) * ts[1] + fh * ts[2] + col_of(j));
                else if (p < end) raw[j] = ldg_stream(src + (int64_t)(p - start) * src_tok + fh * src_head + col_of(j));
            }
        };
        int h = warp;
        uint4 raw[CPL], nxt[CPL];
        if (blk <= last_blk) fetch(blk, h, raw);
        while (blk <= last_blk) {
            int nb = blk, nh = h + kWarps;
            if (nh >= a.n_kv_heads) { nh = warp; nb = blk + blk_step; }
            const bool more = nb <= last_blk;
            if (more) fetch(nb, nh, nxt);

            const int64_t phys = table[blk];
            if (phys >= 0 && phys < a.n_pool_blocks) {
                const int lo = blk * bs;
                const bool still_open = end < lo + bs;  // this block keeps free slots after the call
                uint8_t* pool = pool_base + phys * ps[0];
                AbsMax<ST> am;
#pragma unroll
                for (int j = 0; j < CPL; ++j) am.add(raw[j]);
                const float scale = scale_from_amax(warp_max_nan(am.value()));
                if (lane == 0) scales[phys * ss[0] + h * ss[1]] = scale;
                const Divider div = Divider::make(scale);
                // lane-constant parts of the destination addresses (row_of(j) = r0 + j*rpp when EVEN)
                uint8_t* const dst_h = pool + h * ps[2];
                ST* const tail_h = tail + h * ts[2];
                auto emit = [&](int j, uint2 words) {
                    uint8_t* dst = dst_h + row_of(j) * ps[1] + col_of(j);
                    if constexpr (N == 8) *reinterpret_cast<uint2*>(dst) = words;
                    else *reinterpret_cast<uint32_t*>(dst) = words.x;
                    if (still_open) *reinterpret_cast<uint4*>(tail_h + row_of(j) * ts[1] + col_of(j)) = raw[j];
                };
                if (div.fast) {  // one branch per slice, not per chunk
                    auto fast_loop = [&](auto full_c) {
#pragma unroll
                        for (int j = 0; j < CPL; ++j) {
                            if (decltype(full_c)::value || row_of(j) < bs) {
                                float x[N];
                                Src<ST>::unpack(raw[j], x);
                                uint32_t w[N / 4];
                                encode_quick<N>(x, raw[j], div, w);
                                emit(j, make_uint2(w[0], N == 8 ? w[N / 4 - 1] : 0u));
                            }
                        }
                    };
                    if (full_lanes) fast_loop(std::true_type{});
                    else fast_loop(std::false_type{});
                } else {
#pragma unroll
                    for (int j = 0; j < CPL; ++j)  // unrolled: a run-time index would put the chunk registers on the stack
                        if (row_of(j) < bs) emit(j, encode_exact_chunk<ST>(raw[j], scale));
                }
            }
            if (!more) break;
#pragma unroll
            for (int j = 0; j < CPL; ++j) raw[j] = nxt[j];
            blk = nb;
            h = nh;
        }
    }
}

template <typename ST, bool FP8>
int launch_t(const AppendArgs& a, cudaStream_t stream) {
    constexpr int N = Src<ST>::N;
    const int n_chunks = a.block_size * a.head_dim / N;
    const int cpl = (n_chunks + 31) / 32;
    // a request that appends n tokens starting mid-block touches at most this many blocks
    const int touched = (a.max_new_tokens + a.block_size - 2) / a.block_size + 1;
    if (a.batch > 65535) return fail(SFB_ERR_UNSUPPORTED, "cache_write: batch %d exceeds the grid limit 65535", a.batch);
    if (cpl > 32) return fail(SFB_ERR_UNSUPPORTED, "cache_write: a (block, head) slice of %d x %d elements is too large", a.block_size, a.head_dim);
    // Two launches: the first touched block of every request reads the tail copy,
    // the last one rewrites it; stream order keeps the read before the write when
    // an append spans several blocks.
    for (int pass = 0; pass < 2; ++pass) {
        // pass 0: one thread block per request for its first touched block; pass 1: up to 32 thread
        // blocks per request stride over its remaining blocks (few idle blocks for short requests)
        const int count = pass == 0 ? 1 : (touched - 1 < 32 ? touched - 1 : 32);
        if (count <= 0) continue;
        dim3 grid((unsigned)count, (unsigned)a.batch, 2);
        const bool even = 32 % (a.head_dim / N) == 0;
        auto go = [&](auto cpl_c, auto even_c, auto first_c) {
            cache_write_kernel<ST, decltype(cpl_c)::value, FP8, decltype(even_c)::value, decltype(first_c)::value>
                <<<grid, kThreads, 0, stream>>>(a);
        };
        auto by_pass = [&](auto cpl_c, auto even_c) {
            if (pass == 0) go(cpl_c, even_c, std::true_type{});
            else go(cpl_c, even_c, std::false_type{});
        };
        auto by_even = [&](auto cpl_c) {
            if (even) by_pass(cpl_c, std::true_type{});
            else by_pass(cpl_c, std::false_type{});
        };
        if (!FP8 || cpl <= 4) by_even(std::integral_constant<int, 4>{});
        else if (cpl <= 8) by_even(std::integral_constant<int, 8>{});
        else if (cpl <= 16) by_even(std::integral_constant<int, 16>{});
        else by_even(std::integral_constant<int, 32>{});
        SFB_CUDA_CHECK(cudaGetLastError());
    }
    return SFB_OK;
}

}  // namespace

int launch_cache_write(const AppendArgs& a, cudaStream_t stream) {
    const bool fp8 = a.kv_dtype == SFB_F8E4M3;
    switch (a.src_dtype) {
        case SFB_F32: return fp8 ? launch_t<float, true>(a, stream) : launch_t<float, false>(a, stream);
        case SFB_BF16: return fp8 ? launch_t<__nv_bfloat16, true>(a, stream) : launch_t<__nv_bfloat16, false>(a, stream);
        case SFB_F16: return fp8 ? launch_t<__half, true>(a, stream) : launch_t<__half, false>(a, stream);
    }
    return fail(SFB_ERR_INVALID_ARG, "cache_write: source dtype %d", a.src_dtype);
}

}  // namespace sfb
