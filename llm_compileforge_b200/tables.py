"""Block-table wire formats: the reference's dicts <-> the dense int32 arrays of the C ABI.

The reference passes ``block_tables: dict[str, list[int]]`` and
``seq_lens: dict[str, int]`` (kernels/paged_attention.py:25-26); row ``i`` of
``q`` belongs to the i-th key in insertion order (:36,:54).  The C ABI takes
``int32 [B, max_blocks]`` and ``int32 [B]``.
"""

from __future__ import annotations

from collections.abc import Mapping, Sequence

import torch


def dense_block_tables(
    block_tables: Mapping[str, Sequence[int]],
    seq_lens: Mapping[str, int],
    block_size: int,
    n_pool_blocks: int | None = None,
    min_width: int = 1,
) -> tuple[torch.Tensor, torch.Tensor, list[str]]:
    """Dense CPU (pinned when CUDA is available) tables in dict insertion order.

    Follows kernels/paged_attention.py:37-48: a missing length means the whole
    table (``len(table)*block_size``), a length beyond the table's capacity is
    truncated to it, blocks past ``ceil(L/bs)`` are dropped.  Raises
    ``ValueError`` for a request that would attend to zero tokens (the reference
    fails in ``torch.cat`` there) or a block id outside the pool."""
    rids = list(block_tables.keys())
    lens: list[int] = []
    used: list[Sequence[int]] = []
    for rid in rids:
        table = block_tables[rid]
        length = seq_lens.get(rid, len(table) * block_size)
        length = min(int(length), len(table) * block_size)
        if length <= 0:
            raise ValueError(f"request {rid!r} attends to zero tokens")
        n = -(-length // block_size)
        used.append(table[:n])
        lens.append(length)
    width = max([min_width] + [len(t) for t in used])
    pin = torch.cuda.is_available()
    dense = torch.zeros((len(rids), width), dtype=torch.int32, pin_memory=pin)
    for i, t in enumerate(used):
        row = torch.as_tensor(list(t), dtype=torch.int64)
        if n_pool_blocks is not None and row.numel() and (int(row.min()) < 0 or int(row.max()) >= n_pool_blocks):
            raise ValueError(f"request {rids[i]!r}: block id outside the pool of {n_pool_blocks} blocks")
        dense[i, : len(t)] = row.to(torch.int32)
    lens_t = torch.tensor(lens, dtype=torch.int32)
    if pin:
        lens_t = lens_t.pin_memory()
    return dense, lens_t, rids


def partition_by_request(lengths: Sequence[int], world_size: int) -> list[list[int]]:
    """Contiguous request ranges balanced by attended tokens: rank ``g`` gets the
    requests whose running token sum falls in the g-th equal share.  Contiguity
    keeps the all-gathered output in request order."""
    total = sum(lengths)
    parts: list[list[int]] = [[] for _ in range(world_size)]
    acc = 0
    for i, n in enumerate(lengths):
        mid = acc + n / 2
        g = min(world_size - 1, int(mid * world_size / total)) if total else i % world_size
        parts[g].append(i)
        acc += n
    return parts


def pick_chunk_tokens(lengths: Sequence[int], n_sm: int = 148, head_groups: int = 1) -> int:
    """KV split size for the decode kernel.  A work item is (request, chunk, group of kv heads one thread block takes);
    two thread blocks are resident per SM.  The largest of 2048/1024/512 that still makes about one and a half waves of
    items (the size-ordered work list puts the small items into the last wave, and fewer, larger items pay the per-item
    cost less often: 256 requests of 0.2-8 k tokens take 219 us at 2048 against 231 us at 1024 and 238 us at 512);
    for a small batch the smallest multiple of 64 tokens, up to 1024, whose items fit ONE wave - a second, ragged wave
    leaves most slots idle for as long as a whole item takes (64 requests of 1-4 k tokens: 49 us at 640 against 56 us at
    256, which makes 2.2 waves); else 256."""
    import numpy as np

    slots = 2 * n_sm
    lens = np.asarray([int(n) for n in lengths if int(n) > 0], dtype=np.int64)
    if lens.size == 0:
        return 256
    groups = max(1, int(head_groups))
    items = lambda cand: int(np.sum(-(-lens // cand))) * groups
    for cand in (2048, 1024, 512):
        if items(cand) * 10 >= 14 * slots:
            return cand
    for cand in range(256, 1025, 64):
        if items(cand) <= slots:
            return cand
    return 256


def shared_prefix_blocks(block_tables: Mapping[str, Sequence[int]], seq_lens: Mapping[str, int], block_size: int) -> int:
    """Number of leading table entries that are the same physical blocks in EVERY request and lie
    wholly inside every request's attended length minus one token (each request keeps at least one
    token of its own after the prefix).  This is what a radix-cache hit on a common prompt yields
    (python_runtime/engine/cache/radix_cache.py:68-103: matched blocks are prepended to the table)."""
    tables = list(block_tables.values())
    if len(tables) < 2:
        return 0
    limit = min(len(t) for t in tables)
    for rid, t in block_tables.items():
        length = min(int(seq_lens.get(rid, len(t) * block_size)), len(t) * block_size)
        limit = min(limit, (length - 1) // block_size)
    first = tables[0]
    n = 0
    while n < limit and all(t[n] == first[n] for t in tables[1:]):
        n += 1
    return n
