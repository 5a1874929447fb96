/*
 * sfb.h — C ABI of the B200 (sm_100a) attention hot-path library, libsfb.so.
 *
 * One thin C surface for the operators LLM-CompileForge routes through its HAL
 * `OpExecutor.execute(op_name, inputs, **kwargs)` seam
 * (python_runtime/hal/interface.py:51-61) and that its Rust runtime reaches
 * through `Executable::execute(op_name, stream, &[SfaMemRef], &mut [SfaMemRef])`
 * (runtime/src/hal/traits.rs:115-137).  Tensors travel as the reference's own
 * descriptors (include/sfa.h:41-99): MLIR memref layout, element strides.
 *
 * Conventions
 *   - Every pointer inside a descriptor is a DEVICE pointer (`device` must be
 *     SFB_DEVICE_CUDA); `aligned + offset*elem_size` is element 0.
 *   - Strides are in elements.  The innermost dimension must be contiguous;
 *     all other strides are honoured, so a layer view of the engine's
 *     `[NB, layers, bs, heads, dim]` slab
 *     (python_runtime/engine/cache_manager.py:106-113) is consumed in place.
 *   - Element types are passed out of band as SFBDType (elem_size alone cannot
 *     tell fp16 from bf16, or e4m3 codes from bytes).
 *   - The caller owns every buffer, including the workspace.  The library
 *     allocates no device memory (the `_mlir_ciface_*` shims excepted, which
 *     follow the reference's callee-allocates convention).
 *   - Calls enqueue work on `stream` (a cudaStream_t, NULL = default stream)
 *     and return without synchronising.  Return value: SFB_OK or a negative
 *     SFBStatus; `sfb_last_error()` gives the text for the calling thread.
 *   - Functions are re-entrant for distinct workspaces.
 */
#ifndef SFB_H
#define SFB_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SFB_ABI_VERSION 1

#if defined(__GNUC__)
#define SFB_API __attribute__((visibility("default")))
#else
#define SFB_API
#endif

/* ── Tensor descriptors: binary-identical to include/sfa.h:41-99 ─────────── */
#ifdef SFA_H
typedef SFATensorRaw1 SFBMemRef1;
typedef SFATensorRaw2 SFBMemRef2;
typedef SFATensorRaw3 SFBMemRef3;
typedef SFATensorRaw4 SFBMemRef4;
typedef SFATensor SFBTensor;
#define SFB_DEVICE_CPU SFA_CPU
#define SFB_DEVICE_CUDA SFA_CUDA
#else
#define SFB_MEMREF(R)                                                                  \
    struct {                                                                           \
        void* allocated;                                                               \
        void* aligned;                                                                 \
        int64_t offset;                                                                \
        int64_t sizes[R];                                                              \
        int64_t strides[R];                                                            \
    }
typedef SFB_MEMREF(1) SFBMemRef1; /* 40 bytes */
typedef SFB_MEMREF(2) SFBMemRef2; /* 56 bytes */
typedef SFB_MEMREF(3) SFBMemRef3; /* 72 bytes */
typedef SFB_MEMREF(4) SFBMemRef4; /* 88 bytes */
enum { SFB_DEVICE_CPU = 1, SFB_DEVICE_CUDA = 2 };
typedef struct {
    int32_t device;    /* SFB_DEVICE_CUDA */
    int32_t rank;      /* 1..4 */
    int32_t elem_size; /* bytes per element */
    union {
        SFBMemRef1 r1;
        SFBMemRef2 r2;
        SFBMemRef3 r3;
        SFBMemRef4 r4;
    };
} SFBTensor; /* 104 bytes, union at offset 16 */
#endif

typedef enum {
    SFB_OK = 0,
    SFB_ERR_INVALID_ARG = -1,  /* bad descriptor, shape, stride or dtype combination */
    SFB_ERR_UNSUPPORTED = -2,  /* valid request this build has no kernel for */
    SFB_ERR_WORKSPACE = -3,    /* workspace missing or too small */
    SFB_ERR_CUDA = -4,         /* a CUDA runtime/driver call failed */
    SFB_ERR_DEVICE_STATUS = -5, /* a kernel flagged bad data (sfb_read_status) */
    SFB_ERR_OUT_OF_BLOCKS = -6  /* block manager: pool or device table rows exhausted */
} SFBStatus;

typedef enum {
    SFB_F32 = 0,
    SFB_BF16 = 1,
    SFB_F16 = 2,
    SFB_F8E4M3 = 3 /* torch.float8_e4m3fn codes, one byte each */
} SFBDType;

/* Bits a kernel may set in the workspace status word. */
enum {
    SFB_STATUS_BAD_BLOCK_ID = 1, /* block-table entry outside [0, NB): block skipped */
    SFB_STATUS_EMPTY_REQUEST = 2, /* seq_len <= 0: output row zero-filled */
    SFB_STATUS_WAIT_TIMEOUT = 4, /* a bounded device-side wait gave up */
    SFB_STATUS_UNSORTED_POSITIONS = 8 /* sfb_attention_dense: a positional mask whose positions decrease somewhere */
};

SFB_API int sfb_abi_version(void);
SFB_API const char* sfb_last_error(void);
SFB_API const char* sfb_status_string(int status);

/* ── Paged-attention decode ─────────────────────────────────────────────────
 * Replaces kernels/paged_attention.py:200-227 `paged_attention` (CPU path
 * :21-73) and is the kernel behind the HAL op name `paged_attention` that
 * sf-dialect/include/Sf/HALOps.td:184-189 reserves.
 *
 *   q            [B, H, D]            q_dtype (F32 | BF16 | F16)
 *   k_cache      [NB, bs, Hkv, D]     kv_dtype; F32/BF16/F16 must equal q_dtype,
 *   v_cache      [NB, bs, Hkv, D]       F8E4M3 pairs with a BF16/F16 q
 *   k_scale      [NB, Hkv] float32    F8E4M3 only (else NULL): dequantised value
 *   v_scale      [NB, Hkv] float32      = code * scale (fp8_kv_cache.py:95-105)
 *   block_tables [B, max_blocks] int32  row r lists request r's physical blocks
 *   seq_lens     [B] int32            attended tokens; clamped to max_blocks*bs
 *                                       like paged_attention.py:37-48
 *   table_rows   [B] int32 or NULL    batch position r reads table row
 *                                       table_rows[r] (block_tables may then have any
 *                                       number of rows, e.g. the block manager's
 *                                       device-resident tables); NULL = row r
 *   out          [B, H, D]            q_dtype
 *
 * Query head h reads kv head h / (H / Hkv) (paged_attention.py:57-60); no mask;
 * one query token per request.  Entries of a table row past ceil(L/bs) are
 * never dereferenced.  `scale` <= 0 selects 1/sqrt(D) (:31-32).
 *
 * The KV length of a request is cut into chunks of `chunk_tokens` tokens
 * (multiple of bs; 0 = library default) processed by different thread blocks;
 * when max_blocks*bs > chunk_tokens the partial results go through `workspace`
 * (size from sfb_paged_attention_workspace_bytes) and a combine kernel.  The
 * first 4 bytes of a non-NULL workspace are the status word (zeroed by each
 * call before its kernels run). */
SFB_API int64_t sfb_paged_attention_workspace_bytes(int64_t batch, int64_t n_heads, int64_t head_dim,
                                            int64_t max_blocks, int64_t block_size, int64_t chunk_tokens);

SFB_API int sfb_paged_attention_decode(const SFBTensor* q, const SFBTensor* k_cache, const SFBTensor* v_cache,
                               const SFBTensor* k_scale, const SFBTensor* v_scale,
                               const SFBTensor* block_tables, const SFBTensor* seq_lens,
                               const SFBTensor* table_rows, SFBTensor* out, int q_dtype, int kv_dtype,
                               float scale, int64_t chunk_tokens, void* workspace, int64_t workspace_bytes,
                               void* stream);

/* Copies the workspace status word to the host (synchronises `stream`).
 * Returns SFB_OK when it is zero, SFB_ERR_DEVICE_STATUS otherwise; *bits (may
 * be NULL) receives the SFB_STATUS_* mask. */
SFB_API int sfb_read_status(const void* workspace, int32_t* bits, void* stream);

/* ── Decode without a caller workspace ───────────────────────────────────────
 * No counterpart in the reference: this entry point exists only for hosts that
 * cannot allocate device memory at the point of the call - a runtime whose KV
 * block pool already owns all free HBM, or a dlopen-style host with no
 * allocator binding.  Same arguments and results as sfb_paged_attention_decode,
 * but the split-K partials and the status word live in a fixed device array
 * inside the library (SFB_STATIC_SCRATCH_BYTES per GPU, resident from the
 * moment the library's image is loaded on that GPU until the process exits).
 *
 *   - Allocates nothing: no cudaMalloc / cudaFree, no allocating library call.
 *   - A call whose split needs more than SFB_STATIC_SCRATCH_BYTES
 *     (sfb_paged_attention_workspace_bytes tells) fails with SFB_ERR_WORKSPACE;
 *     raise chunk_tokens or use the workspace form.
 *   - The first call on each device looks up the array's device address (with
 *     that device current); make that first call outside any stream capture.
 *   - All calls on a GPU share the one array and it keeps the previous call's
 *     contents.  The status word is cleared by every call; everything else is
 *     overwritten before it is read.  Two calls that can overlap on the GPU
 *     (different streams without ordering) race on it: serialise them.
 * sfb_read_status_static reads that array's status word like sfb_read_status. */
#define SFB_STATIC_SCRATCH_BYTES (16 * 1024 * 1024)

SFB_API int sfb_paged_attention_decode_static(const SFBTensor* q, const SFBTensor* k_cache, const SFBTensor* v_cache,
                                              const SFBTensor* k_scale, const SFBTensor* v_scale,
                                              const SFBTensor* block_tables, const SFBTensor* seq_lens,
                                              const SFBTensor* table_rows, SFBTensor* out, int q_dtype,
                                              int kv_dtype, float scale, int64_t chunk_tokens, void* stream);
SFB_API int sfb_read_status_static(int32_t* bits, void* stream);

/* ── KV cache write / FP8 quantise-on-append ───────────────────────────────
 * Replaces CacheManager.write_paged (python_runtime/engine/cache_manager.py:139-171;
 * Rust twin BlockManager::write_kv, runtime/src/cache/block.rs:348-403) for the
 * HAL op name `cache_write` (HALOps.td:195-199), fused with
 * FP8KVCacheQuantizer.quantize_block (compiler/quantize/fp8_kv_cache.py:66-93)
 * when the pool holds e4m3 codes.
 *
 *   k_new, v_new [T, Hkv, D]  src_dtype; tokens packed request after request
 *   cu_tokens    [B+1] int32  request r owns rows cu_tokens[r] .. cu_tokens[r+1]-1
 *   start_pos    [B] int32    position of request r's first new token
 *   block_tables [B, max_blocks] int32
 *   k_cache, v_cache [NB, bs, Hkv, D]  kv_dtype (== src_dtype, or F8E4M3)
 *   k_scale, v_scale [NB, Hkv] float32 (F8E4M3 only)
 *   k_tail, v_tail   [B, bs, Hkv, D] src_dtype (F8E4M3 only): unquantised copy of
 *                    each request's open (partially filled) block, owned by the
 *                    caller, read and updated by this call
 *   tail_rows        [B] int32 or NULL: request r's tail copy is row tail_rows[r]
 *                    (a stable slot while batch order changes); NULL = row r
 *   table_rows       [B] int32 or NULL: request r's table is row table_rows[r] of
 *                    block_tables (which may then have any number of rows); NULL = row r.
 *                    A request whose table or tail row lies outside its array is skipped.
 *
 * Token at position p goes to slot (table[p / bs], p % bs) (cache_manager.py:154-159).
 * FP8: after the call every touched (block, kv_head) slice holds exactly
 * quantize_block(slice contents, unwritten slots = 0): scale = amax/448
 * (1.0 when amax == 0, at least 1e-12), codes = e4m3(x / scale), bit-exact.
 * `max_new_tokens` >= max_r (cu_tokens[r+1]-cu_tokens[r]) sizes the launch. */
SFB_API int sfb_cache_write(const SFBTensor* k_new, const SFBTensor* v_new, const SFBTensor* cu_tokens,
                    const SFBTensor* start_pos, const SFBTensor* block_tables, SFBTensor* k_cache,
                    SFBTensor* v_cache, SFBTensor* k_scale, SFBTensor* v_scale, SFBTensor* k_tail,
                    SFBTensor* v_tail, const SFBTensor* tail_rows, const SFBTensor* table_rows,
                    int src_dtype, int kv_dtype, int64_t max_new_tokens, void* stream);

/* ── Chunked prefill over the paged pool ────────────────────────────────────
 * Replaces kernels/flash_attention.py:179-202 `flash_attention_fwd` (CPU path
 * :28-46, dense causal SDPA) for the serving case the reference only sketches:
 * a chunk of new tokens attending causally to prefix + chunk, with K/V read
 * through the block table (kernels/paged_attention.py:36-48) so that a radix
 * prefix shared by several requests is the same physical blocks in every table
 * (runtime/src/cache/block.rs:214-232).  The chunk's own K/V must already be in
 * the pool (sfb_cache_write first).
 *
 *   q, out       [T, H, D]   dtype; chunks packed request after request
 *   cu_q         [R+1] int32 request r owns rows cu_q[r] .. cu_q[r+1]-1
 *   ctx_lens     [R] int32   cached tokens of request r including this chunk;
 *                            query i of the chunk sits at ctx_len - n_q + i and
 *                            sees positions 0 .. its own (causal != 0); with
 *                            causal == 0 every query sees all ctx_len tokens
 *   block_tables [R, max_blocks] int32
 *   k_cache, v_cache [NB, bs, Hkv, D] dtype (same as q)
 *
 * BF16 / F16 with D = 128 and bs = 16 run on the tcgen05 kernel; every other
 * shape takes the decode kernels with one row per query token.  `workspace`
 * (sfb_prefill_workspace_bytes) holds the status word, the counter the
 * tcgen05 kernel's resident thread blocks draw their work items from (one
 * workspace per call in flight) and, for that second route, 8 bytes per
 * query token.  max_q_tokens >= the longest chunk. */
SFB_API int64_t sfb_prefill_workspace_bytes(int64_t total_q_tokens);
SFB_API int sfb_prefill_paged(const SFBTensor* q, const SFBTensor* k_cache, const SFBTensor* v_cache,
                              const SFBTensor* block_tables, const SFBTensor* cu_q, const SFBTensor* ctx_lens,
                              SFBTensor* out, int dtype, float scale, int causal, int64_t max_q_tokens,
                              void* workspace, int64_t workspace_bytes, void* stream);

/* Same, with the visible length of every query row given explicitly instead of the
 * causal rule: row t of the packed batch attends to positions 0 .. row_limits[t]-1 of
 * its request (clamped to ctx_len; a row whose limit is <= 0 gets a zero output).
 * This is how the reference backend's positional attention mask is served
 * (python_runtime/hal/pytorch_backend/_ops_attention.py:33-43: key j is visible to
 * query i iff pos[i] >= pos[j], which for non-decreasing positions is a prefix of
 * keys) and the top-left aligned causal mask of the Rust runtime's dense attention
 * (runtime/src/engine/kernels.rs:246-252: row i sees keys 0..i).
 *   row_limits  [T] int32, contiguous */
SFB_API int sfb_prefill_paged_rows(const SFBTensor* q, const SFBTensor* k_cache, const SFBTensor* v_cache,
                                   const SFBTensor* block_tables, const SFBTensor* cu_q, const SFBTensor* ctx_lens,
                                   const SFBTensor* row_limits, SFBTensor* out, int dtype, float scale,
                                   int64_t max_q_tokens, void* workspace, int64_t workspace_bytes, void* stream);

/* ── Dense attention ──────────────────────────────────────────────────────────
 * softmax(q k^T scale + mask) v over dense [B, H, S, D] operands (k, v: [B, Hkv, Skv, D],
 * H a multiple of Hkv); any batch / head / token strides that are multiples of 16 bytes,
 * D contiguous, so a position-major [B, S, H, D] buffer is passed as a permuted view.
 * Replaces the reference backend's scaled_dot_product_attention
 * (python_runtime/hal/pytorch_backend/_ops_attention.py:13-53) and the Rust runtime's
 * dense attention (runtime/src/engine/kernels.rs:97-302: fp32, head-major operands,
 * q pre-scaled -> pass scale = 1; decode = SFB_MASK_NONE, prefill = SFB_MASK_CAUSAL_TOP_LEFT).
 * Masks are prefixes of keys per query row:
 *   SFB_MASK_NONE                 every key
 *   SFB_MASK_CAUSAL_TOP_LEFT      row i sees keys 0..i (torch's is_causal, kernels.rs:246-252)
 *   SFB_MASK_CAUSAL_BOTTOM_RIGHT  row i sees keys 0..Skv-Sq+i (a chunk at the end of its context)
 *   SFB_MASK_POSITIONS            `positions` [B or 1, S] f32, Sq = Skv = S: key j is visible to
 *                                 query i iff positions[i] >= positions[j], the reference's
 *                                 positional mask (_ops_attention.py:33-43).  The positions must
 *                                 not decrease along S; otherwise SFB_STATUS_UNSORTED_POSITIONS is
 *                                 set in the status word and the output is unspecified.
 * scale <= 0 means 1/sqrt(D).  `workspace` (sfb_attention_dense_workspace_bytes) holds the
 * status word (first 4 bytes, sfb_read_status) and the repacked operands: the attention
 * itself runs on the chunked-prefill kernels over a private pool of 16-token blocks. */
enum { SFB_MASK_NONE = 0, SFB_MASK_CAUSAL_TOP_LEFT = 1, SFB_MASK_CAUSAL_BOTTOM_RIGHT = 2, SFB_MASK_POSITIONS = 3 };
SFB_API int64_t sfb_attention_dense_workspace_bytes(int64_t batch, int64_t n_heads, int64_t n_kv_heads, int64_t q_len, int64_t kv_len,
                                                    int64_t head_dim, int dtype);
SFB_API int sfb_attention_dense(const SFBTensor* q, const SFBTensor* k, const SFBTensor* v, const SFBTensor* positions, SFBTensor* out,
                                int dtype, float scale, int mask_mode, void* workspace, int64_t workspace_bytes, void* stream);

/* ── Dense read of the paged pool ─────────────────────────────────────────────
 * The `cache_read` operator the dialect reserves beside paged_attention / cache_write
 * (sf-dialect/include/Sf/HALOps.td:190-194) and CacheManager.read_paged
 * (python_runtime/engine/cache_manager.py:173-197): out[r, t] = the pool row of token t of
 * request r through its block table, zero for t >= seq_lens[r] (with seq_lens[r] = the table's
 * capacity this is read_paged exactly).  Call once for K and once for V.
 *   cache        [NB, bs, Hkv, D] cache_dtype;  scale [NB, Hkv] f32 with an e4m3 pool, else NULL
 *   block_tables [R, max_blocks] int32;  seq_lens [R] int32
 *   out          [R, max_seq_len, Hkv, D] out_dtype, contiguous (f32 / bf16 / f16; for an e4m3
 *                pool value = code * scale, the reference's dequantize_block,
 *                compiler/quantize/fp8_kv_cache.py:95-105)
 * `status` (may be NULL): device int32 that receives SFB_STATUS_BAD_BLOCK_ID. */
SFB_API int sfb_cache_read(const SFBTensor* cache, const SFBTensor* scale, const SFBTensor* block_tables, const SFBTensor* seq_lens,
                           SFBTensor* out, int cache_dtype, int out_dtype, void* status, void* stream);

/* ── Decode with a shared (radix) prefix ────────────────────────────────────
 * Same result as sfb_paged_attention_decode for requests whose first
 * `shared_prefix_blocks` table entries are the same physical blocks in EVERY
 * row - what RadixCache.match_prefix + BlockManager::assign_cached_blocks /
 * share_prefix produce for a common system prompt
 * (python_runtime/engine/cache/radix_cache.py:68-103,
 * runtime/src/cache/block.rs:214-232,273-306) - but the prefix is read once
 * for the whole batch instead of once per request: the batch's queries attend
 * to it as one dense [B*H/Hkv x prefix] contraction per kv head on the tcgen05
 * kernel, each request's remaining tokens go through the split decode kernel,
 * and the thread block finishing a request merges both partial results.
 * The caller guarantees the rows really share those blocks (only row 0's are
 * read) and that every seq_len exceeds the prefix.  BF16 / F16, head_dim 128,
 * block_size 16.  Workspace from sfb_shared_prefix_workspace_bytes. */
SFB_API int64_t sfb_shared_prefix_workspace_bytes(int64_t batch, int64_t n_heads, int64_t head_dim, int64_t max_blocks,
                                                  int64_t block_size, int64_t chunk_tokens, int64_t shared_prefix_blocks);
SFB_API int sfb_paged_attention_decode_shared_prefix(const SFBTensor* q, const SFBTensor* k_cache, const SFBTensor* v_cache,
                                                     const SFBTensor* block_tables, const SFBTensor* seq_lens,
                                                     SFBTensor* out, int dtype, float scale, int64_t shared_prefix_blocks,
                                                     int64_t chunk_tokens, void* workspace, int64_t workspace_bytes,
                                                     void* stream);

/* ── FP8 quantise / dequantise ──────────────────────────────────────────────
 * Replaces FP8KVCacheQuantizer.quantize_block / dequantize_block
 * (compiler/quantize/fp8_kv_cache.py:66-105); HAL op names `quantize` /
 * `dequantize` (HALOps.td:202-211).
 *
 *   x      [N0, N1, N2, N3]  x_dtype (F32 | BF16 | F16)
 *   codes  [N0, N1, N2, N3]  uint8 e4m3
 *   scales float32: SFB_QUANT_PER_TENSOR -> [1] (the reference's single scale for
 *          the tensor passed in); SFB_QUANT_PER_BLOCK_HEAD -> [N0, N2], one per
 *          x[b, :, h, :] slice (the KV pool layout [NB, bs, Hkv, D]). */
enum { SFB_QUANT_PER_TENSOR = 0, SFB_QUANT_PER_BLOCK_HEAD = 1 };

SFB_API int sfb_quantize_fp8(const SFBTensor* x, SFBTensor* codes, SFBTensor* scales, int x_dtype, int granularity,
                     void* stream);
SFB_API int sfb_dequantize_fp8(const SFBTensor* codes, const SFBTensor* scales, SFBTensor* out, int out_dtype,
                       int granularity, void* stream);

/* ── RMSNorm (optionally fused with a residual add) ─────────────────────────
 * Replaces the HAL op `rms_norm` (python_runtime/hal/pytorch_backend/_ops_norm.py:30-45)
 * and kernels/rms_norm.py:85-106 `fused_rms_norm_add`.
 *
 *   x, out   [rows, hidden] dtype;  residual [rows, hidden] dtype or NULL
 *   weight   [hidden] dtype or NULL
 *   out = s * rsqrt(mean(s^2) + eps) * weight,  s = x (+ residual)
 * Arithmetic is float32 with one final rounding to `dtype` (the HAL op's rule,
 * _ops_norm.py:35-45). */
SFB_API int sfb_rms_norm(const SFBTensor* x, const SFBTensor* residual, const SFBTensor* weight, SFBTensor* out,
                 int dtype, float eps, void* stream);

/* ── Head-partitioned decode with the output gathered in-kernel ─────────────────
 * The reference's tensor-parallel attention ends in an all-gather of the per-rank
 * heads through its Communicator (python_runtime/hal/communicator.py:17-72,
 * runtime/src/comm/).  Here GPU `rank` of `world` (<= 8, one node) holds kv heads
 * [rank*Hkv, (rank+1)*Hkv) of the pool and the matching H query heads, and the
 * decode kernel stores its [B, H, D] result directly into heads [rank*H, (rank+1)*H)
 * of EVERY GPU's [B, H*world, D] output (plain peer stores over NVLink; no TMA, no
 * multicast).  `out_all` describes this GPU's copy; peer_out[p] is the base address
 * of GPU p's copy (peer_out[rank] the local one; all copies have out_all's layout).
 * The buffers must be mapped for peer access by the caller (CUDA IPC / symmetric
 * memory).  Follow it on the same stream with sfb_peer_signal_wait: after that the
 * local copy is complete.  The signal says "arrived", nothing says "consumed": a
 * GPU that has passed its wait may start the next step's stores while a slower peer
 * still reads this one.  Alternate between TWO output sets by step parity and queue
 * the reader of a step on the same stream before the next decode; the stores of step
 * n + 2 then cannot start before every peer has signalled step n + 1, i.e. after
 * its reader of step n.  Only the shapes of the TMA decode kernel are supported. */
SFB_API int sfb_paged_attention_decode_gather(const SFBTensor* q, const SFBTensor* k_cache, const SFBTensor* v_cache,
                                              const SFBTensor* k_scale, const SFBTensor* v_scale,
                                              const SFBTensor* block_tables, const SFBTensor* seq_lens,
                                              const SFBTensor* table_rows, SFBTensor* out_all, void* const* peer_out,
                                              int world, int rank, int q_dtype, int kv_dtype, float scale,
                                              int64_t chunk_tokens, void* workspace, int64_t workspace_bytes, void* stream);

/* Tells every peer that this GPU's stores of step `step` have landed and waits (bounded:
 * about a second, then SFB_STATUS_WAIT_TIMEOUT is OR-ed into *status, a device int32 or
 * NULL) until every peer has said the same.  peer_flags[p] = GPU p's device array of
 * `world` uint32 slots, zero before the first step; `step` must grow by one per call.
 * `phases`: SFB_PEER_SIGNAL | SFB_PEER_WAIT in one launch (the multi-GPU use), or one of
 * them alone (ranks emulated on ONE device must queue all signals before any wait). */
enum { SFB_PEER_SIGNAL = 1, SFB_PEER_WAIT = 2 };
SFB_API int sfb_peer_signal_wait(void* const* peer_flags, int world, int rank, uint32_t step, int phases, void* status,
                                 void* stream);

/* ── Block manager with device-resident tables ───────────────────────────────
 * Replaces BlockManager (runtime/src/cache/block.rs:84-346; Python twin in the
 * engine): reference-counted physical blocks, LIFO free list, per-request ordered
 * tables, prefix hits prepended (assign_cached_blocks), share_prefix,
 * ensure_blocks, free / free_block.  Block ids and their order are identical to
 * the reference's for the same call sequence.
 *
 * sfb_bm_attach_device_tables gives the manager a device array
 * int32 [rows, max_blocks]; every request then owns a stable row (sfb_bm_row)
 * and sfb_bm_sync sends only entries changed since the last sync (one scatter kernel
 * on the given stream, reading pinned host memory; asynchronous).  Pass that
 * array as `block_tables` and the requests' rows as `table_rows` to the decode
 * entry points.  Negative returns are SFBStatus values (SFB_ERR_OUT_OF_BLOCKS for
 * the reference's OutOfMemoryError). */
typedef struct SFBBlockManager SFBBlockManager;
SFB_API SFBBlockManager* sfb_bm_create(int64_t num_blocks, int64_t block_size);
SFB_API void sfb_bm_destroy(SFBBlockManager* bm);
SFB_API int sfb_bm_attach_device_tables(SFBBlockManager* bm, void* d_tables, int64_t rows, int64_t max_blocks);
SFB_API int64_t sfb_bm_allocate(SFBBlockManager* bm, const char* request_id, int64_t num_tokens, int32_t* out, int64_t cap);
SFB_API void sfb_bm_free(SFBBlockManager* bm, const char* request_id);
SFB_API void sfb_bm_free_block(SFBBlockManager* bm, int64_t block_id);
SFB_API int sfb_bm_assign_cached_blocks(SFBBlockManager* bm, const char* request_id, const int32_t* block_ids, int64_t n);
SFB_API int sfb_bm_ensure_blocks(SFBBlockManager* bm, const char* request_id, int64_t target_tokens);
SFB_API int sfb_bm_ensure_blocks_batch(SFBBlockManager* bm, const char* const* request_ids, const int64_t* target_tokens,
                                       int64_t n);
SFB_API int64_t sfb_bm_share_prefix(SFBBlockManager* bm, const char* src_request_id, const char* dst_request_id,
                                    int64_t prefix_len);
SFB_API void sfb_bm_increment_ref_count(SFBBlockManager* bm, int64_t block_id);
SFB_API int64_t sfb_bm_ref_count(const SFBBlockManager* bm, int64_t block_id);
SFB_API int64_t sfb_bm_num_free_blocks(const SFBBlockManager* bm);
SFB_API int64_t sfb_bm_get_blocks(const SFBBlockManager* bm, const char* request_id, int32_t* out, int64_t cap);
SFB_API int64_t sfb_bm_row(const SFBBlockManager* bm, const char* request_id);
SFB_API int64_t sfb_bm_sync(SFBBlockManager* bm, void* stream);

/* ── Chunked prefill over an e4m3 pool ────────────────────────────────────────
 * sfb_prefill_paged for a pool of FP8 codes with per-(block, kv head) scales (the layout
 * sfb_cache_write produces).  The blocks the batch attends to are expanded once into a
 * 16-bit scratch pool inside `workspace` (value = code * scale in q's type) and the
 * ordinary prefill runs over it; workspace size from sfb_prefill_fp8_workspace_bytes
 * (max_blocks = columns of block_tables).  Status word as for sfb_prefill_paged. */
SFB_API int64_t sfb_prefill_fp8_workspace_bytes(int64_t total_q_tokens, int64_t n_requests, int64_t max_blocks, int64_t n_kv_heads,
                                                int64_t head_dim);
SFB_API int sfb_prefill_paged_fp8(const SFBTensor* q, const SFBTensor* k_cache, const SFBTensor* v_cache, const SFBTensor* k_scale,
                                  const SFBTensor* v_scale, const SFBTensor* block_tables, const SFBTensor* cu_q,
                                  const SFBTensor* ctx_lens, SFBTensor* out, int q_dtype, float scale, int causal,
                                  int64_t max_q_tokens, void* workspace, int64_t workspace_bytes, void* stream);

/* ── RMSNorm fused into the following matmul ───────────────────────────────────
 * Replaces fused_rms_norm_matmul (python_runtime/hal/pytorch_backend/_ops_norm.py:47-65):
 *   y = (x * rsqrt(mean(x^2, -1) + eps) * rms_weight) @ mat_weight,  x [M, K], mat_weight [K, N].
 * The row factor commutes with the contraction, so the weight is folded once
 * (sfb_fold_norm_weight: folded = diag(rms_weight) mat_weight; weights are static while
 * serving) and sfb_fused_rms_norm_matmul runs y = rstd(x) * (x @ folded) on the tensor
 * cores from the raw activations, taking each row's sum of squares from the tiles it
 * multiplies.  bf16 / fp16, fp32 accumulation, one rounding of y; K and N multiples of 8,
 * rows contiguous and 16-byte aligned.  `workspace` (device, may be NULL) of
 * sfb_fused_rms_norm_matmul_workspace_bytes(M) bytes: its first word is the status word
 * (sfb_read_status; SFB_STATUS_WAIT_TIMEOUT if a bounded wait inside the kernel ran out),
 * the rest holds per-row statistics when the shape is large enough for a statistics pre-pass
 * to pay (2048 rows up, or wherever a cluster of two thread blocks per 256 x 256 tile is the
 * cheaper shape: that kernel needs the pre-pass); without it the statistics are always taken
 * inside the single-block GEMM kernel. */
SFB_API int64_t sfb_fused_rms_norm_matmul_workspace_bytes(int64_t rows);
/* Host arithmetic only (no device call): the tile shape sfb_fused_rms_norm_matmul runs for an [rows, K] x [K, cols]
 * problem on a device with `sms` SMs that can hold `clusters` clusters of two thread blocks, with or without a full
 * workspace.  plan6 = {clusters of two (0/1), tile width, pipeline stages, K steps per stage, statistics pre-pass (0/1),
 * rows of x per TMA box}. */
SFB_API int sfb_fused_rms_norm_matmul_plan(int64_t rows, int64_t cols, int sms, int clusters, int has_workspace, int32_t* plan6);
SFB_API int sfb_fold_norm_weight(const SFBTensor* rms_weight, const SFBTensor* mat_weight, SFBTensor* folded, int dtype, void* stream);
SFB_API int sfb_fused_rms_norm_matmul(const SFBTensor* x, const SFBTensor* folded_weight, SFBTensor* out, int dtype, float eps,
                                      void* workspace, int64_t workspace_bytes, void* stream);

/* ── `_mlir_ciface_*` convention ─────────────────────────────────────────────
 * The reference's runtime calls compiled kernels as
 *   void _mlir_ciface_<name>(void* sret, const memref* in0, ...)
 * (runtime/src/hal/cpu/executable.rs:23-29,159-200): the callee allocates each
 * output, writes its memref descriptor into `sret`, and the caller frees
 * `allocated` with the library's `serveforge_free`
 * (runtime/src/hal/cpu/device.rs:94-109).  This shim has the signature and
 * epsilon (1e-5) of the reference's golden kernel tests/data/golden/rms_norm.c:35-75,
 * with device pointers; it synchronises before returning.  On failure
 * `allocated` is NULL (the convention has no error channel). */
SFB_API void _mlir_ciface_sfb_rms_norm_f32(void* sret, const SFBMemRef2* x, const SFBMemRef1* w);
SFB_API void serveforge_free(void* ptr);

/* The attention operators in the same convention, under the operator names the dialect
 * reserves (sf-dialect/include/Sf/HALOps.td:184-211: paged_attention, cache_read,
 * cache_write, quantize, dequantize) plus the dense attention of
 * python_runtime/hal/pytorch_backend/_ops_attention.py:13-53 and
 * runtime/src/engine/kernels.rs:97-302; one symbol per element type (_f32, _bf16).
 * Operands beyond the dialect's own lists (sequence lengths, the pools, the per-request
 * token ranges) are what the engine holds as state around those operators.  Outputs are
 * contiguous, consecutive descriptors in `sret`; int32 index operands.
 *   paged_attention(q [B,H,D], key_cache, value_cache [NB,bs,Hkv,D], block_table [B,max_blocks],
 *                   seq_lens [B]) -> [B,H,D]
 *   cache_write(key, value [T,Hkv,D], cu_tokens [B+1], start_pos [B], block_table, key_cache,
 *               value_cache): writes the pools, no result (`sret` untouched)
 *   cache_read(block_table [R,max_blocks], seq_lens [R], key_cache, value_cache)
 *                   -> key, value [R, max_blocks*bs, Hkv, D]
 *   quantize(x [NB,bs,Hkv,D]) -> codes [NB,bs,Hkv,D] u8 (e4m3), scales [NB,Hkv] f32
 *   dequantize(codes, scales) -> [NB,bs,Hkv,D]
 *   scaled_dot_product_attention / causal_attention(q [B,H,Sq,D], k, v [B,Hkv,Skv,D]) -> [B,H,Sq,D]
 *                   (scale 1/sqrt(D); causal = row i sees keys 0..i) */
#define SFB_DECLARE_CIFACE(sfx)                                                                                                    \
    SFB_API void _mlir_ciface_sfb_paged_attention_##sfx(void* sret, const SFBMemRef3* q, const SFBMemRef4* key_cache,              \
                                                        const SFBMemRef4* value_cache, const SFBMemRef2* block_table,             \
                                                        const SFBMemRef1* seq_lens);                                              \
    SFB_API void _mlir_ciface_sfb_cache_write_##sfx(void* sret, const SFBMemRef3* key, const SFBMemRef3* value,                    \
                                                    const SFBMemRef1* cu_tokens, const SFBMemRef1* start_pos,                     \
                                                    const SFBMemRef2* block_table, const SFBMemRef4* key_cache,                   \
                                                    const SFBMemRef4* value_cache);                                               \
    SFB_API void _mlir_ciface_sfb_cache_read_##sfx(void* sret, const SFBMemRef2* block_table, const SFBMemRef1* seq_lens,          \
                                                   const SFBMemRef4* key_cache, const SFBMemRef4* value_cache);                   \
    SFB_API void _mlir_ciface_sfb_quantize_##sfx(void* sret, const SFBMemRef4* x);                                                 \
    SFB_API void _mlir_ciface_sfb_dequantize_##sfx(void* sret, const SFBMemRef4* codes, const SFBMemRef2* scales);                 \
    SFB_API void _mlir_ciface_sfb_scaled_dot_product_attention_##sfx(void* sret, const SFBMemRef4* q, const SFBMemRef4* k,         \
                                                                     const SFBMemRef4* v);                                        \
    SFB_API void _mlir_ciface_sfb_causal_attention_##sfx(void* sret, const SFBMemRef4* q, const SFBMemRef4* k, const SFBMemRef4* v);
SFB_DECLARE_CIFACE(f32)
SFB_DECLARE_CIFACE(bf16)
#undef SFB_DECLARE_CIFACE

#ifdef __cplusplus
}
#endif

#endif /* SFB_H */
