"""Tensor-level operators: torch CUDA tensors in, one libsfb call each.

These are the device-resident forms (block tables and lengths already dense
int32 tensors on the GPU) that a serving loop calls every step; the
dict-based signatures of the reference's ``kernels`` package are in
``kernels_api.py`` and the HAL ``OpExecutor`` in ``hal.py``.
"""

from __future__ import annotations

import torch

from . import _lib
from ._lib import check, current_stream, desc, dtype_code

BLOCK_SIZE = 16


def _as_codes(t: torch.Tensor) -> torch.Tensor:
    """uint8 and float8_e4m3fn tensors are both accepted for code pools."""
    return t.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t


def decode_workspace_bytes(batch: int, n_heads: int, head_dim: int, max_blocks: int, block_size: int = BLOCK_SIZE,
                           chunk_tokens: int = 0) -> int:
    n = _lib.load().sfb_paged_attention_workspace_bytes(batch, n_heads, head_dim, max_blocks, block_size, chunk_tokens)
    if n < 0:
        raise ValueError("invalid decode workspace query")
    return int(n)


def paged_attention_decode(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_tables: torch.Tensor,
    seq_lens: torch.Tensor,
    *,
    k_scale: torch.Tensor | None = None,
    v_scale: torch.Tensor | None = None,
    scale: float | None = None,
    chunk_tokens: int = 0,
    workspace: torch.Tensor | None = None,
    out: torch.Tensor | None = None,
    table_rows: torch.Tensor | None = None,
) -> torch.Tensor:
    """Decode attention of ``q [B,H,D]`` over a paged pool ``[NB,bs,Hkv,D]``.

    ``block_tables`` int32 ``[B,max_blocks]``, ``seq_lens`` int32 ``[B]``, both on
    the device.  An e4m3 pool (uint8 or float8_e4m3fn) needs ``k_scale`` /
    ``v_scale`` float32 ``[NB,Hkv]``.  ``workspace`` (uint8) is allocated when
    the split needs one and none is given; pass a persistent one in a serving
    loop (size from :func:`decode_workspace_bytes`).  With ``table_rows`` (int32 ``[B]``) batch
    position r reads row ``table_rows[r]`` of ``block_tables`` (device-resident tables of
    :class:`llm_compileforge_b200.block_manager.BlockManager`)."""
    lib = _lib.load()
    fp8 = k_scale is not None
    kc, vc = (_as_codes(k_cache), _as_codes(v_cache)) if fp8 else (k_cache, v_cache)
    kv_code = _lib.SFB_F8E4M3 if fp8 else dtype_code(k_cache.dtype)
    if out is None:
        out = torch.empty_like(q)
    b, h, d = q.shape
    need = decode_workspace_bytes(b, h, d, block_tables.shape[1], k_cache.shape[1], chunk_tokens)
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=q.device)
    elif workspace.numel() * workspace.element_size() < need:
        raise ValueError(f"decode workspace holds {workspace.numel() * workspace.element_size()} B, {need} needed")
    check(lib.sfb_paged_attention_decode(
        desc(q, "q"), desc(kc, "k_cache"), desc(vc, "v_cache"), desc(k_scale, "k_scale"), desc(v_scale, "v_scale"),
        desc(block_tables, "block_tables"), desc(seq_lens, "seq_lens"), desc(table_rows, "table_rows"), desc(out, "out"),
        dtype_code(q.dtype), kv_code, float(scale) if scale is not None else 0.0, int(chunk_tokens),
        workspace.data_ptr(), workspace.numel() * workspace.element_size(), current_stream(q.device),
    ))
    return out


def paged_attention_decode_gather(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_tables: torch.Tensor,
    seq_lens: torch.Tensor,
    out_all: torch.Tensor,
    peer_out_ptrs: "list[int]",
    rank: int,
    *,
    k_scale: torch.Tensor | None = None,
    v_scale: torch.Tensor | None = None,
    scale: float | None = None,
    chunk_tokens: int = 0,
    workspace: torch.Tensor | None = None,
    table_rows: torch.Tensor | None = None,
) -> torch.Tensor:
    """Decode of this GPU's heads (``q [B,H,D]`` against its kv-head shard of the pool) whose result is stored
    into heads ``[rank*H, (rank+1)*H)`` of every GPU's ``[B, H*world, D]`` output: ``out_all`` is the local copy,
    ``peer_out_ptrs[p]`` the device address of GPU p's copy (peer-mapped by the caller, same layout).  Follow it
    with :func:`peer_signal_wait` on the same stream; then ``out_all`` is complete."""
    import ctypes

    lib = _lib.load()
    world = len(peer_out_ptrs)
    fp8 = k_scale is not None
    kc, vc = (_as_codes(k_cache), _as_codes(v_cache)) if fp8 else (k_cache, v_cache)
    b, h, d = q.shape
    need = decode_workspace_bytes(b, h, d, block_tables.shape[1], k_cache.shape[1], chunk_tokens)
    if workspace is None:
        workspace = torch.zeros(need, dtype=torch.uint8, device=q.device)
    ptrs = (ctypes.c_void_p * world)(*[int(x) for x in peer_out_ptrs])
    check(lib.sfb_paged_attention_decode_gather(
        desc(q, "q"), desc(kc, "k_cache"), desc(vc, "v_cache"), desc(k_scale, "k_scale"), desc(v_scale, "v_scale"),
        desc(block_tables, "block_tables"), desc(seq_lens, "seq_lens"), desc(table_rows, "table_rows"), desc(out_all, "out_all"),
        ptrs, world, int(rank), dtype_code(q.dtype), _lib.SFB_F8E4M3 if fp8 else dtype_code(k_cache.dtype),
        float(scale) if scale is not None else 0.0, int(chunk_tokens), workspace.data_ptr(), workspace.numel(),
        current_stream(q.device),
    ))
    return out_all


def peer_signal_wait(peer_flag_ptrs: "list[int]", rank: int, step: int, status: torch.Tensor | None, device: torch.device,
                     phases: int = 3) -> None:
    """Signal step ``step`` to every peer and wait (bounded) for theirs; ``peer_flag_ptrs[p]`` is the device address of
    GPU p's ``uint32 [world]`` flag array, ``status`` an int32 device tensor that collects ``SFB_STATUS_WAIT_TIMEOUT``;
    ``phases`` 1 = signal only, 2 = wait only, 3 = both (ranks emulated on one device queue all signals before any wait)."""
    import ctypes

    world = len(peer_flag_ptrs)
    ptrs = (ctypes.c_void_p * world)(*[int(x) for x in peer_flag_ptrs])
    check(_lib.load().sfb_peer_signal_wait(ptrs, world, int(rank), ctypes.c_uint32(step & 0xFFFFFFFF), int(phases),
                                           status.data_ptr() if status is not None else None, current_stream(device)))


def read_status(workspace: torch.Tensor) -> int:
    """Status bits left by the last decode call that used ``workspace``
    (synchronises the current stream)."""
    import ctypes

    bits = ctypes.c_int32(0)
    rc = _lib.load().sfb_read_status(workspace.data_ptr(), ctypes.byref(bits), current_stream(workspace.device))
    if rc not in (_lib.SFB_OK, _lib.SFB_ERR_DEVICE_STATUS):
        check(rc)
    return int(bits.value)


def cache_write(
    k_new: torch.Tensor,
    v_new: torch.Tensor,
    cu_tokens: torch.Tensor,
    start_pos: torch.Tensor,
    block_tables: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    *,
    max_new_tokens: int,
    k_scale: torch.Tensor | None = None,
    v_scale: torch.Tensor | None = None,
    k_tail: torch.Tensor | None = None,
    v_tail: torch.Tensor | None = None,
    tail_rows: torch.Tensor | None = None,
    table_rows: torch.Tensor | None = None,
) -> None:
    """Scatter new K/V tokens ``[T,Hkv,D]`` into their paged slots; with scales
    and tails given the pool holds e4m3 codes and the write quantises on append.
    ``table_rows`` / ``tail_rows`` (int32 ``[B]``) name each request's row of
    ``block_tables`` / of the tails when those are stable per-request arrays."""
    lib = _lib.load()
    fp8 = k_scale is not None
    kc, vc = (_as_codes(k_cache), _as_codes(v_cache)) if fp8 else (k_cache, v_cache)
    check(lib.sfb_cache_write(
        desc(k_new, "k_new"), desc(v_new, "v_new"), desc(cu_tokens, "cu_tokens"), desc(start_pos, "start_pos"),
        desc(block_tables, "block_tables"), desc(kc, "k_cache"), desc(vc, "v_cache"), desc(k_scale, "k_scale"),
        desc(v_scale, "v_scale"), desc(k_tail, "k_tail"), desc(v_tail, "v_tail"), desc(tail_rows, "tail_rows"),
        desc(table_rows, "table_rows"), dtype_code(k_new.dtype),
        _lib.SFB_F8E4M3 if fp8 else dtype_code(k_cache.dtype), int(max_new_tokens), current_stream(k_new.device),
    ))


def quantize_fp8(x: torch.Tensor, per_block_head: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """e4m3 codes (``float8_e4m3fn``, same shape) and float32 scale(s).

    ``per_block_head=False``: one scale for the whole tensor (0-dim), the
    reference's ``quantize_block``.  ``True``: ``x`` is ``[NB,bs,Hkv,D]`` and
    scales are ``[NB,Hkv]``."""
    lib = _lib.load()
    if x.dim() > 4:
        raise ValueError("quantize_fp8 takes tensors of rank <= 4")
    xv = x if x.dim() >= 1 else x.reshape(1)
    codes = torch.empty(xv.shape, dtype=torch.uint8, device=x.device)
    if per_block_head:
        scales = torch.empty((x.shape[0], x.shape[2]), dtype=torch.float32, device=x.device)
    else:
        scales = torch.empty((1,), dtype=torch.float32, device=x.device)
    if xv.stride(-1) != 1:
        xv = xv.contiguous()
    check(lib.sfb_quantize_fp8(
        desc(xv, "x"), desc(codes, "codes"), desc(scales, "scales"), dtype_code(x.dtype),
        _lib.SFB_QUANT_PER_BLOCK_HEAD if per_block_head else _lib.SFB_QUANT_PER_TENSOR, current_stream(x.device),
    ))
    codes = codes.view(torch.float8_e4m3fn).reshape(x.shape)
    return codes, (scales if per_block_head else scales.reshape(()))


def dequantize_fp8(codes: torch.Tensor, scales: torch.Tensor, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """``codes.float() * scale``; scales 0-dim / 1 element (whole tensor) or
    ``[NB,Hkv]`` for a ``[NB,bs,Hkv,D]`` pool."""
    lib = _lib.load()
    cv = _as_codes(codes)
    if cv.dim() == 0:
        cv = cv.reshape(1)
    if cv.stride(-1) != 1:
        cv = cv.contiguous()
    per_block_head = scales.dim() == 2
    sv = scales if per_block_head else scales.reshape(1)
    out = torch.empty(cv.shape, dtype=out_dtype, device=codes.device)
    check(lib.sfb_dequantize_fp8(
        desc(cv, "codes"), desc(sv, "scales"), desc(out, "out"), dtype_code(out_dtype),
        _lib.SFB_QUANT_PER_BLOCK_HEAD if per_block_head else _lib.SFB_QUANT_PER_TENSOR, current_stream(codes.device),
    ))
    return out.reshape(codes.shape)


def rms_norm(
    x: torch.Tensor,
    weight: torch.Tensor | None,
    eps: float = 1e-5,
    residual: torch.Tensor | None = None,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """``s * rsqrt(mean(s^2) + eps) * weight`` with ``s = x (+ residual)``;
    float32 arithmetic, one rounding to ``x.dtype``."""
    lib = _lib.load()
    hidden = x.shape[-1]
    x2 = x.reshape(-1, hidden)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    r2 = None
    if residual is not None:
        if residual.shape != x.shape or residual.dtype != x.dtype:
            raise ValueError("residual must match x in shape and dtype")
        r2 = residual.reshape(-1, hidden)
        if r2.stride(-1) != 1:
            r2 = r2.contiguous()
    w = weight
    if w is not None and w.dtype != x.dtype:
        w = w.to(x.dtype)
    if w is not None and not w.is_contiguous():
        w = w.contiguous()
    o2 = torch.empty_like(x2) if out is None else out.reshape(-1, hidden)
    check(lib.sfb_rms_norm(desc(x2, "x"), desc(r2, "residual"), desc(w, "weight"), desc(o2, "out"),
                           dtype_code(x.dtype), float(eps), current_stream(x.device)))
    return o2.reshape(x.shape) if out is None else out


def prefill_workspace_bytes(total_q_tokens: int) -> int:
    return int(_lib.load().sfb_prefill_workspace_bytes(int(total_q_tokens)))


def prefill_paged(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_tables: torch.Tensor,
    cu_q: torch.Tensor,
    ctx_lens: torch.Tensor,
    *,
    max_q_tokens: int,
    scale: float | None = None,
    causal: bool = True,
    workspace: torch.Tensor | None = None,
    out: torch.Tensor | None = None,
    k_scale: torch.Tensor | None = None,
    v_scale: torch.Tensor | None = None,
    row_limits: torch.Tensor | None = None,
) -> torch.Tensor:
    """Attention of packed query chunks ``q [T,H,D]`` over prefix + chunk read from
    the paged pool.  Request ``r`` owns rows ``cu_q[r]:cu_q[r+1]``; its chunk ends
    at cached position ``ctx_lens[r] - 1`` (the chunk's K/V are already in the pool).
    With ``k_scale`` / ``v_scale`` (float32 ``[NB,Hkv]``) the pool holds e4m3 codes; the attended blocks are expanded
    into a 16-bit scratch inside the workspace first (:func:`prefill_fp8_workspace_bytes`).
    ``row_limits`` (int32 ``[T]``) replaces the causal rule: row ``t`` attends to positions ``0 .. row_limits[t]-1``."""
    lib = _lib.load()
    if out is None:
        out = torch.empty_like(q)
    if row_limits is not None:
        if k_scale is not None:
            raise ValueError("prefill_paged: row_limits are not implemented over an e4m3 pool")
        if workspace is None:
            workspace = torch.empty(prefill_workspace_bytes(q.shape[0]), dtype=torch.uint8, device=q.device)
        check(lib.sfb_prefill_paged_rows(
            desc(q, "q"), desc(k_cache, "k_cache"), desc(v_cache, "v_cache"), desc(block_tables, "block_tables"),
            desc(cu_q, "cu_q"), desc(ctx_lens, "ctx_lens"), desc(row_limits, "row_limits"), desc(out, "out"), dtype_code(q.dtype),
            float(scale) if scale is not None else 0.0, int(max_q_tokens), workspace.data_ptr(),
            workspace.numel() * workspace.element_size(), current_stream(q.device),
        ))
        return out
    if k_scale is not None:
        kc, vc = _as_codes(k_cache), _as_codes(v_cache)
        need = prefill_fp8_workspace_bytes(q.shape[0], block_tables.shape[0], block_tables.shape[1], kc.shape[2], kc.shape[3])
        if workspace is None:
            workspace = torch.empty(need, dtype=torch.uint8, device=q.device)
        check(lib.sfb_prefill_paged_fp8(
            desc(q, "q"), desc(kc, "k_cache"), desc(vc, "v_cache"), desc(k_scale, "k_scale"), desc(v_scale, "v_scale"),
            desc(block_tables, "block_tables"), desc(cu_q, "cu_q"), desc(ctx_lens, "ctx_lens"), desc(out, "out"), dtype_code(q.dtype),
            float(scale) if scale is not None else 0.0, 1 if causal else 0, int(max_q_tokens), workspace.data_ptr(),
            workspace.numel() * workspace.element_size(), current_stream(q.device),
        ))
        return out
    need = prefill_workspace_bytes(q.shape[0])
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=q.device)
    check(lib.sfb_prefill_paged(
        desc(q, "q"), desc(k_cache, "k_cache"), desc(v_cache, "v_cache"), desc(block_tables, "block_tables"),
        desc(cu_q, "cu_q"), desc(ctx_lens, "ctx_lens"), desc(out, "out"), dtype_code(q.dtype),
        float(scale) if scale is not None else 0.0, 1 if causal else 0, int(max_q_tokens), workspace.data_ptr(),
        workspace.numel() * workspace.element_size(), current_stream(q.device),
    ))
    return out


MASK_MODES = {"none": _lib.SFB_MASK_NONE, "causal": _lib.SFB_MASK_CAUSAL_TOP_LEFT, "causal_bottom_right": _lib.SFB_MASK_CAUSAL_BOTTOM_RIGHT,
              "positions": _lib.SFB_MASK_POSITIONS}


def attention_dense(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, mask: str = "none", positions: torch.Tensor | None = None,
                    scale: float | None = None, out: torch.Tensor | None = None, workspace: torch.Tensor | None = None,
                    return_workspace: bool = False):
    """``softmax(q k^T scale + mask) v`` for dense ``q [B,H,Sq,D]``, ``k, v [B,Hkv,Skv,D]`` (any batch / head / token strides).
    ``mask``: ``"none"``, ``"causal"`` (row i sees keys 0..i), ``"causal_bottom_right"`` (row i sees keys 0..Skv-Sq+i) or
    ``"positions"`` with ``positions [B or 1, S]`` float32: key j visible to query i iff ``positions[i] >= positions[j]``
    (the reference backend's positional mask; positions must not decrease - the status word says so otherwise, read it
    with :func:`read_status` on the returned workspace)."""
    lib = _lib.load()
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("attention_dense: q, k, v must be [B, H, S, D]")
    if mask not in MASK_MODES:
        raise ValueError(f"attention_dense: mask {mask!r} not in {sorted(MASK_MODES)}")
    if out is None:
        out = torch.empty_like(q, memory_format=torch.contiguous_format)
    b, h, sq, d = q.shape
    need = int(lib.sfb_attention_dense_workspace_bytes(b, h, k.shape[1], sq, k.shape[2], d, dtype_code(q.dtype)))
    if need < 0:
        raise ValueError("attention_dense: bad shape")
    if workspace is None:
        workspace = torch.empty(max(need, 256), dtype=torch.uint8, device=q.device)
    if positions is not None:
        positions = positions.to(torch.float32).contiguous()
    check(lib.sfb_attention_dense(
        desc(q, "q"), desc(k, "k"), desc(v, "v"), desc(positions, "positions"), desc(out, "out"), dtype_code(q.dtype),
        float(scale) if scale is not None else 0.0, MASK_MODES[mask], workspace.data_ptr(),
        workspace.numel() * workspace.element_size(), current_stream(q.device),
    ))
    return (out, workspace) if return_workspace else out


def cache_read(cache: torch.Tensor, block_tables: torch.Tensor, seq_lens: torch.Tensor, max_seq_len: int, *,
               scale: torch.Tensor | None = None, out_dtype: torch.dtype | None = None, status: torch.Tensor | None = None) -> torch.Tensor:
    """Dense ``[R, max_seq_len, Hkv, D]`` copy of the pool rows the block tables point at (zero past ``seq_lens[r]``), the
    reference's ``CacheManager.read_paged`` (python_runtime/engine/cache_manager.py:173-197).  With ``scale [NB,Hkv]`` the
    pool holds e4m3 codes and the result is ``code * scale`` in ``out_dtype`` (default float32)."""
    lib = _lib.load()
    fp8 = scale is not None
    pool = _as_codes(cache) if fp8 else cache
    odt = out_dtype or (torch.float32 if fp8 else cache.dtype)
    out = torch.empty((block_tables.shape[0], int(max_seq_len), pool.shape[2], pool.shape[3]), dtype=odt, device=cache.device)
    check(lib.sfb_cache_read(
        desc(pool, "cache"), desc(scale, "scale"), desc(block_tables, "block_tables"), desc(seq_lens, "seq_lens"), desc(out, "out"),
        _lib.SFB_F8E4M3 if fp8 else dtype_code(cache.dtype), dtype_code(odt), status.data_ptr() if status is not None else None,
        current_stream(cache.device),
    ))
    return out


def prefill_fp8_workspace_bytes(total_q_tokens: int, n_requests: int, max_blocks: int, n_kv_heads: int, head_dim: int) -> int:
    return int(_lib.load().sfb_prefill_fp8_workspace_bytes(int(total_q_tokens), int(n_requests), int(max_blocks), int(n_kv_heads), int(head_dim)))


def paged_attention_decode_shared_prefix(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_tables: torch.Tensor,
    seq_lens: torch.Tensor,
    shared_prefix_blocks: int,
    *,
    scale: float | None = None,
    chunk_tokens: int = 0,
    workspace: torch.Tensor | None = None,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """Decode for a batch whose first ``shared_prefix_blocks`` table entries are the same
    physical blocks in every row (a radix-shared prefix): the prefix is read once for
    the whole batch.  Same result as :func:`paged_attention_decode`."""
    lib = _lib.load()
    if out is None:
        out = torch.empty_like(q)
    b, h, d = q.shape
    need = int(lib.sfb_shared_prefix_workspace_bytes(b, h, d, block_tables.shape[1], k_cache.shape[1], chunk_tokens,
                                                     shared_prefix_blocks))
    if need < 0:
        raise ValueError("invalid shared-prefix workspace query")
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=q.device)
    check(lib.sfb_paged_attention_decode_shared_prefix(
        desc(q, "q"), desc(k_cache, "k_cache"), desc(v_cache, "v_cache"), desc(block_tables, "block_tables"),
        desc(seq_lens, "seq_lens"), desc(out, "out"), dtype_code(q.dtype), float(scale) if scale is not None else 0.0,
        int(shared_prefix_blocks), int(chunk_tokens), workspace.data_ptr(), workspace.numel() * workspace.element_size(),
        current_stream(q.device),
    ))
    return out


def fold_norm_weight(rms_weight: torch.Tensor, mat_weight: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``diag(rms_weight) @ mat_weight`` (``[K] , [K,N] -> [K,N]``): the weight :func:`fused_rms_norm_matmul` multiplies by.
    Done once per weight pair; weights do not change while serving."""
    if out is None:
        out = torch.empty_like(mat_weight)
    check(_lib.load().sfb_fold_norm_weight(desc(rms_weight, "rms_weight"), desc(mat_weight, "mat_weight"), desc(out, "folded"),
                                           dtype_code(mat_weight.dtype), current_stream(mat_weight.device)))
    return out


def fused_rms_norm_matmul(x: torch.Tensor, folded_weight: torch.Tensor, eps: float = 1e-5, out: torch.Tensor | None = None,
                          workspace: torch.Tensor | None = None) -> torch.Tensor:
    """``rms_norm(x) @ W`` with the norm's weight already folded into ``folded_weight`` (:func:`fold_norm_weight`):
    ``x [..., K]`` bf16 / fp16, result ``[..., N]``; one tcgen05 GEMM on the raw activations, the row factor applied to the
    accumulators.  ``workspace`` (uint8, :func:`norm_matmul_workspace_bytes`; allocated when missing) carries the status word
    (:func:`read_status`) and the per-row statistics of a pre-pass, which large shapes use (from 2048 rows up, or whenever the
    two-thread-block kernel is the cheaper shape)."""
    k = x.shape[-1]
    x2 = x.reshape(-1, k)
    n = folded_weight.shape[1]
    if out is None:
        out = torch.empty((x2.shape[0], n), dtype=x.dtype, device=x.device)
    out2 = out.reshape(-1, n)
    if workspace is None:
        workspace = torch.empty(norm_matmul_workspace_bytes(x2.shape[0]), dtype=torch.uint8, device=x.device)
    check(_lib.load().sfb_fused_rms_norm_matmul(desc(x2, "x"), desc(folded_weight, "folded_weight"), desc(out2, "out"), dtype_code(x.dtype),
                                                float(eps), workspace.data_ptr(), workspace.numel(), current_stream(x.device)))
    return out2.reshape(*x.shape[:-1], n)


def norm_matmul_workspace_bytes(rows: int) -> int:
    return int(_lib.load().sfb_fused_rms_norm_matmul_workspace_bytes(int(rows)))


def norm_matmul_plan(rows: int, cols: int, *, sms: int = 148, clusters: int = 74, has_workspace: bool = True) -> dict:
    """The tile shape :func:`fused_rms_norm_matmul` runs for ``[rows, K] x [K, cols]`` (host arithmetic, no device needed)."""
    import ctypes

    out = (ctypes.c_int32 * 6)()
    check(_lib.load().sfb_fused_rms_norm_matmul_plan(int(rows), int(cols), int(sms), int(clusters), int(bool(has_workspace)), out))
    keys = ("pair", "tile_n", "stages", "k_steps_per_stage", "prepass", "x_box_rows")
    return dict(zip(keys, (int(v) for v in out)))
