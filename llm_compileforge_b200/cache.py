"""Paged KV cache for a serving loop: the GPU twin of the reference's CacheManager.

The reference's engine keeps one slab ``[num_blocks, layers, block_size, heads, dim]``
per K and V (python_runtime/engine/cache_manager.py:103-121), writes new tokens with
``write_paged`` (:139-171: slot = ``(table[pos // bs], pos % bs)``), and for decode gathers
the whole cache into a dense tensor with ``read_paged`` (:173-197) before calling dense
SDPA (python_runtime/engine/mlir_executor.py:400-419).  ``PagedKVCache`` keeps the same
slab layout and the same per-step protocol (``begin_step(block_tables)`` then per-layer
calls), but ``write`` is the fused cache-write / FP8 quantise-on-append kernel and
``attend`` / ``prefill`` run attention straight off the paged pool: nothing is densified.

With ``fp8=True`` the slabs hold e4m3 codes, with per-(block, layer, kv_head) float32
scales and a per-request copy of the open block (``tails``) that quantise-on-append needs.
"""

from __future__ import annotations

from collections.abc import Mapping, Sequence

import torch

from . import ops
from .tables import dense_block_tables, pick_chunk_tokens


class PagedKVCache:
    def __init__(self, num_blocks: int, num_layers: int, num_kv_heads: int, head_dim: int, block_size: int = 16,
                 dtype: torch.dtype = torch.bfloat16, fp8: bool = False, max_requests: int = 256,
                 device: str | torch.device = "cuda") -> None:
        self.num_blocks, self.num_layers, self.block_size = num_blocks, num_layers, block_size
        self.num_kv_heads, self.head_dim, self.dtype, self.fp8 = num_kv_heads, head_dim, dtype, fp8
        self.device = torch.device(device)
        shape = (num_blocks, num_layers, block_size, num_kv_heads, head_dim)  # cache_manager.py:106-113
        store = torch.uint8 if fp8 else dtype
        self.k_slab = torch.zeros(shape, dtype=store, device=self.device)
        self.v_slab = torch.zeros(shape, dtype=store, device=self.device)
        if fp8:
            self.k_scale = torch.ones((num_blocks, num_layers, num_kv_heads), dtype=torch.float32, device=self.device)
            self.v_scale = torch.ones_like(self.k_scale)
            tail_shape = (max_requests, num_layers, block_size, num_kv_heads, head_dim)
            self.k_tail = torch.zeros(tail_shape, dtype=dtype, device=self.device)
            self.v_tail = torch.zeros_like(self.k_tail)
        self._free_slots = list(range(max_requests - 1, -1, -1))
        self._slot_of: dict[str, int] = {}
        self._rids: list[str] = []
        self._tables: dict[str, list[int]] = {}
        self._dense = None
        self._slots_dev = None

    # ── per-step state (CacheManager.begin_step, cache_manager.py:125-128) ─────────
    def begin_step(self, block_tables: Mapping[str, Sequence[int]]) -> None:
        """Tables of the requests scheduled this step, in the order their tokens are packed."""
        self._tables = {r: list(t) for r, t in block_tables.items()}
        self._rids = list(self._tables)
        for r in self._rids:
            if r not in self._slot_of:
                if not self._free_slots:
                    raise RuntimeError("PagedKVCache: more live requests than max_requests")
                self._slot_of[r] = self._free_slots.pop()
        dense, _, _ = dense_block_tables(self._tables, {}, self.block_size, n_pool_blocks=self.num_blocks)
        self._dense = dense.to(self.device, non_blocking=True)
        self._slots_dev = torch.tensor([self._slot_of[r] for r in self._rids], dtype=torch.int32).to(self.device)

    def release(self, rid: str) -> None:
        """Forget a finished request (its tail slot becomes reusable; blocks belong to the block manager)."""
        slot = self._slot_of.pop(rid, None)
        if slot is not None:
            self._free_slots.append(slot)

    def _layer(self, layer: int):
        return self.k_slab[:, layer], self.v_slab[:, layer]  # strided views, consumed in place

    # ── write_paged (cache_manager.py:139-171) ─────────────────────────────────────
    def write(self, layer: int, k_new: torch.Tensor, v_new: torch.Tensor, n_tokens: Sequence[int], start_pos: Sequence[int]) -> None:
        """``k_new, v_new [T, Hkv, D]`` pack ``n_tokens[i]`` new tokens of request i (table order)
        whose first token sits at position ``start_pos[i]``."""
        cu = torch.zeros(len(n_tokens) + 1, dtype=torch.int32)
        cu[1:] = torch.tensor(list(n_tokens), dtype=torch.int32).cumsum(0)
        start = torch.tensor(list(start_pos), dtype=torch.int32)
        k_cache, v_cache = self._layer(layer)
        kw = {}
        if self.fp8:
            kw = dict(k_scale=self.k_scale[:, layer], v_scale=self.v_scale[:, layer], k_tail=self.k_tail[:, layer],
                      v_tail=self.v_tail[:, layer], tail_rows=self._slots_dev)
        ops.cache_write(k_new, v_new, cu.to(self.device, non_blocking=True), start.to(self.device, non_blocking=True), self._dense,
                        k_cache, v_cache, max_new_tokens=max(n_tokens), **kw)

    # ── decode attention straight off the pool (replaces read_paged + dense SDPA) ──
    def attend(self, layer: int, q: torch.Tensor, seq_lens: Sequence[int], scale: float | None = None) -> torch.Tensor:
        """``q [B, H, D]`` (one token per request, table order) -> ``[B, H, D]``."""
        lens = torch.tensor(list(seq_lens), dtype=torch.int32).to(self.device, non_blocking=True)
        k_cache, v_cache = self._layer(layer)
        kw = dict(k_scale=self.k_scale[:, layer], v_scale=self.v_scale[:, layer]) if self.fp8 else {}
        return ops.paged_attention_decode(q, k_cache, v_cache, self._dense, lens, scale=scale,
                                          chunk_tokens=pick_chunk_tokens(list(seq_lens)), **kw)

    def prefill(self, layer: int, q: torch.Tensor, n_tokens: Sequence[int], ctx_lens: Sequence[int], scale: float | None = None) -> torch.Tensor:
        """Causal attention of each request's newest ``n_tokens[i]`` tokens (``q [T, H, D]`` packed) over its
        ``ctx_lens[i]`` cached tokens.  An e4m3 pool is expanded to 16 bits for the attended blocks first."""
        cu = torch.zeros(len(n_tokens) + 1, dtype=torch.int32)
        cu[1:] = torch.tensor(list(n_tokens), dtype=torch.int32).cumsum(0)
        ctx = torch.tensor(list(ctx_lens), dtype=torch.int32)
        k_cache, v_cache = self._layer(layer)
        fp8kw = dict(k_scale=self.k_scale[:, layer], v_scale=self.v_scale[:, layer]) if self.fp8 else {}
        return ops.prefill_paged(q, k_cache, v_cache, self._dense, cu.to(self.device), ctx.to(self.device),
                                 max_q_tokens=max(n_tokens), scale=scale, **fp8kw)

    # ── read_paged (cache_manager.py:173-197), for debugging and parity checks only ─
    def read_dense(self, layer: int, rid: str, length: int) -> tuple[torch.Tensor, torch.Tensor]:
        """Dense ``[length, Hkv, D]`` float32 K and V of one request (dequantised for an FP8 pool)."""
        ids = torch.as_tensor(self._tables[rid][: -(-length // self.block_size)], device=self.device)
        k, v = self.k_slab[ids, layer], self.v_slab[ids, layer]
        if self.fp8:
            k = k.view(torch.float8_e4m3fn).float() * self.k_scale[ids, layer][:, None, :, None]
            v = v.view(torch.float8_e4m3fn).float() * self.v_scale[ids, layer][:, None, :, None]
        return k.flatten(0, 1)[:length].float(), v.flatten(0, 1)[:length].float()
