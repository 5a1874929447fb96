"""Drop-ins for the reference's ``kernels`` package and FP8 KV quantiser.

Same names, argument meaning and error behaviour as the reference functions
they replace; every call runs on the GPU through libsfb (no Triton, no CPU
fallback: a CPU tensor raises ``ValueError``).

    kernels/paged_attention.py:200-227   paged_attention
    kernels/flash_attention.py:179-202   flash_attention_fwd
    kernels/rms_norm.py:85-106           fused_rms_norm_add
    compiler/quantize/fp8_kv_cache.py    FP8KVCacheQuantizer
"""

from __future__ import annotations

import math
from collections.abc import Mapping, Sequence

import torch

from . import ops
from .tables import dense_block_tables, pick_chunk_tokens, shared_prefix_blocks


def paged_attention(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_tables: Mapping[str, Sequence[int]],
    seq_lens: Mapping[str, int],
    block_size: int = 16,
    scale: float | None = None,
    *,
    k_scale: torch.Tensor | None = None,
    v_scale: torch.Tensor | None = None,
    chunk_tokens: int = 0,
    share_prefix: bool = True,
) -> dict[str, torch.Tensor]:
    """PagedAttention with block-table indirection (paged_attention.py:200-227).

    ``q [B,H,D]``; ``k_cache``/``v_cache`` ``[NB,block_size,Hkv,D]``; returns
    ``{request_id: [H,D]}``.  ``k_scale``/``v_scale`` (keyword-only, float32
    ``[NB,Hkv]``) switch to an e4m3 code pool dequantised inside the kernel.
    When every table starts with the same physical blocks (a radix-shared prefix of at
    least 16 blocks, 64 or more requests) and the pool is bf16/fp16 with head_dim 128, that prefix is read once
    for the whole batch (``share_prefix=False`` turns this off); results are the same."""
    if k_cache.shape[1] != block_size:
        raise ValueError(f"k_cache block dimension {k_cache.shape[1]} != block_size {block_size}")
    if not block_tables:
        return {}
    dense, lens, rids = dense_block_tables(block_tables, seq_lens, block_size, n_pool_blocks=k_cache.shape[0])
    if len(rids) > q.shape[0]:
        raise IndexError(f"{len(rids)} block tables for {q.shape[0]} query rows")
    dev = q.device
    if chunk_tokens <= 0:
        chunk_tokens = pick_chunk_tokens(lens.tolist())
    if (share_prefix and k_scale is None and q.dtype in (torch.bfloat16, torch.float16) and q.shape[-1] == 128
            and block_size == 16 and q.shape[1] // k_cache.shape[2] <= 8):
        n_shared = shared_prefix_blocks(block_tables, seq_lens, block_size)
        # below ~64 requests the prefix stays in L2 and the plain kernel is as fast (measured crossover)
        if n_shared >= 16 and n_shared < dense.shape[1] and len(rids) >= 64:
            out = ops.paged_attention_decode_shared_prefix(
                q[: len(rids)], k_cache, v_cache, dense.to(dev, non_blocking=True), lens.to(dev, non_blocking=True),
                n_shared, scale=scale, chunk_tokens=chunk_tokens)
            return {rid: out[i] for i, rid in enumerate(rids)}
    out = ops.paged_attention_decode(
        q[: len(rids)], k_cache, v_cache, dense.to(dev, non_blocking=True), lens.to(dev, non_blocking=True),
        k_scale=k_scale, v_scale=v_scale, scale=scale, chunk_tokens=chunk_tokens,
    )
    return {rid: out[i] for i, rid in enumerate(rids)}


def flash_attention_fwd(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float | None = None, causal: bool = True
) -> torch.Tensor:
    """FlashAttention forward (kernels/flash_attention.py:179-202): ``q, k, v``
    ``[batch, heads, seq, head_dim]`` -> same shape; ``causal`` defaults to True,
    ``scale`` to ``1/sqrt(head_dim)``.

    Runs through the library's dense-attention entry point, which repacks K/V as a
    private paged pool (16-token blocks, identity tables) and uses the chunked-prefill
    kernels; K/V may have fewer heads than Q (GQA).  As in the reference's CPU path,
    ``causal=True`` needs equal query and key lengths."""
    if q.dim() != 4 or k.shape != v.shape or k.shape[0] != q.shape[0] or k.shape[-1] != q.shape[-1]:
        raise ValueError("flash_attention_fwd expects q [B,H,S,D] and k, v [B,Hkv,Skv,D]")
    if causal and q.shape[2] != k.shape[2]:
        raise ValueError("causal flash_attention_fwd needs equal query and key lengths")
    return ops.attention_dense(q, k, v, mask="causal" if causal else "none", scale=scale)


def chunked_prefill(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_tables: Mapping[str, Sequence[int]],
    ctx_lens: Mapping[str, int],
    n_tokens: Mapping[str, int],
    block_size: int = 16,
    scale: float | None = None,
    k_scale: torch.Tensor | None = None,
    v_scale: torch.Tensor | None = None,
) -> dict[str, torch.Tensor]:
    """Causal attention of each request's newest ``n_tokens[rid]`` tokens over all
    of its ``ctx_lens[rid]`` cached tokens (prefix + chunk), K/V through the block
    tables.  ``q [T,H,D]`` packs the chunks in dict order (the scheduler's
    ``ScheduledRequest.n_tokens`` / ``block_table``, runtime/src/engine/types.rs:85-94).
    ``k_scale`` / ``v_scale`` ``[NB,Hkv]``: the pool holds e4m3 codes.  Returns ``{rid: [n_tokens, H, D]}``."""
    if k_cache.shape[1] != block_size:
        raise ValueError(f"k_cache block dimension {k_cache.shape[1]} != block_size {block_size}")
    rids = list(block_tables)
    lens = {r: ctx_lens[r] for r in rids}
    dense, ll, _ = dense_block_tables(block_tables, lens, block_size, n_pool_blocks=k_cache.shape[0])
    counts = [int(n_tokens[r]) for r in rids]
    for r, n in zip(rids, counts):
        if n <= 0 or n > min(int(ctx_lens[r]), len(block_tables[r]) * block_size):
            raise ValueError(f"request {r!r}: chunk of {n} tokens does not fit its context")
    cu = torch.zeros(len(rids) + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(counts, dtype=torch.int32).cumsum(0)
    if int(cu[-1]) != q.shape[0]:
        raise ValueError(f"q has {q.shape[0]} rows, the chunks add up to {int(cu[-1])}")
    dev = q.device
    out = ops.prefill_paged(q, k_cache, v_cache, dense.to(dev, non_blocking=True), cu.to(dev), ll.to(dev, non_blocking=True),
                            max_q_tokens=max(counts), scale=scale, causal=True, k_scale=k_scale, v_scale=v_scale)
    return {r: out[int(cu[i]) : int(cu[i + 1])] for i, r in enumerate(rids)}


def fused_rms_norm_add(
    input_tensor: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6
) -> torch.Tensor:
    """RMSNorm + residual connection, fused (kernels/rms_norm.py:85-106; note the
    1e-6 default).  Intermediates are float32 with one final rounding."""
    return ops.rms_norm(input_tensor, weight, eps=eps, residual=residual)


class FP8KVCacheQuantizer:
    """GPU twin of compiler/quantize/fp8_kv_cache.py:19-140."""

    SUPPORTED_HARDWARE: list[str] = ["H100", "H200", "B100", "B200", "MI300", "Ascend 910B", "Ascend 910C"]

    def __init__(self, block_size: int = 16, fp8_max: float = 448.0) -> None:
        if block_size <= 0:
            raise ValueError(f"block_size must be positive, got {block_size}")
        if fp8_max != 448.0:
            raise ValueError("only the e4m3 range (fp8_max = 448) is implemented")
        self.block_size = block_size
        self.fp8_max = fp8_max

    def check_hardware_support(self, device_name: str) -> bool:
        return any(hw in device_name for hw in self.SUPPORTED_HARDWARE)

    def quantize_block(self, kv_block: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """One scale for the whole tensor passed in (fp8_kv_cache.py:66-93)."""
        return ops.quantize_fp8(kv_block, per_block_head=False)

    def dequantize_block(self, quant_block: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
        """``quant_block.float() * scale`` (fp8_kv_cache.py:95-105)."""
        return ops.dequantize_fp8(quant_block, scale, torch.float32)

    def quantize_kv(self, k: torch.Tensor, v: torch.Tensor):
        k_quant, k_scale = self.quantize_block(k)
        v_quant, v_scale = self.quantize_block(v)
        return k_quant, k_scale, v_quant, v_scale

    def dequantize_kv(self, k_quant, k_scale, v_quant, v_scale):
        return self.dequantize_block(k_quant, k_scale), self.dequantize_block(v_quant, v_scale)

    # per-(block, kv_head) layout used by the paged pool
    def quantize_pool(self, pool: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """``quantize_block`` applied to every ``pool[b, :, h, :]`` slice of a
        ``[NB,bs,Hkv,D]`` pool: codes ``[NB,bs,Hkv,D]`` and scales ``[NB,Hkv]``."""
        return ops.quantize_fp8(pool, per_block_head=True)

    def dequantize_pool(self, codes: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
        return ops.dequantize_fp8(codes, scales, torch.float32)


def default_scale(head_dim: int) -> float:
    return 1.0 / math.sqrt(head_dim)
