"""Block manager of the paged KV pool, host side of ``sfb_bm_*``.

Same surface as the reference's ``BlockManager``
(runtime/src/cache/block.rs:84-346, exported to Python by
runtime/src/ffi.rs and driven by python_runtime/engine/llm_engine.py):
``allocate / free / free_block / assign_cached_blocks / ensure_blocks /
share_prefix / get_blocks / num_free_blocks / num_allocated_blocks /
increment_ref_count / utilization`` with the same block ids in the same
order for the same call sequence, ``OutOfMemoryError`` when the pool is
exhausted and ``ValueError`` / ``KeyError`` where the reference returns
``Err(String)``.

New here: :meth:`attach_device_tables` gives every request a stable row of
a device-resident ``int32 [rows, max_blocks]`` array; :meth:`sync` uploads
only the entries that changed, and :meth:`rows` yields the ``table_rows``
tensor the decode entry points take.  The library is required - there is
no Python fallback.
"""

from __future__ import annotations

import ctypes
from typing import Iterable, Sequence

import torch

from . import _lib


class OutOfMemoryError(RuntimeError):
    """The block pool (or the device table) cannot satisfy the request (block.rs:62-78)."""


def _raise(rc: int) -> None:
    msg = _lib.load().sfb_last_error().decode()
    if rc == _lib.SFB_ERR_OUT_OF_BLOCKS:
        raise OutOfMemoryError(msg)
    raise ValueError(msg)


class BlockManager:
    def __init__(self, num_blocks: int, block_size: int = 16):
        if num_blocks <= 0:
            raise ValueError("num_blocks must be positive")
        if block_size <= 0:
            raise ValueError("block_size must be positive")
        self._lib = _lib.load()
        self._h = self._lib.sfb_bm_create(int(num_blocks), int(block_size))
        if not self._h:
            raise ValueError(self._lib.sfb_last_error().decode())
        self.num_blocks = int(num_blocks)
        self.block_size = int(block_size)
        self.device_tables: torch.Tensor | None = None
        # counts the calls that can give a request a device-table row or take one away; callers that cache
        # request -> row lookups (the step pipeline) compare it instead of asking for every row on every step
        self.row_generation = 0

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.sfb_bm_destroy(h)

    # ── allocation (block.rs:146-268) ────────────────────────────────────────
    def allocate(self, request_id: str, num_tokens: int) -> list[int]:
        self.row_generation += 1
        cap = -(-int(num_tokens) // self.block_size)
        buf = (ctypes.c_int32 * max(cap, 1))()
        n = self._lib.sfb_bm_allocate(self._h, request_id.encode(), int(num_tokens), buf, cap)
        if n < 0:
            _raise(n)
        return list(buf[:n])

    def free(self, request_id: str) -> None:
        self.row_generation += 1
        self._lib.sfb_bm_free(self._h, request_id.encode())

    def free_block(self, block_id: int) -> None:
        self._lib.sfb_bm_free_block(self._h, int(block_id))

    def assign_cached_blocks(self, request_id: str, block_ids: Sequence[int]) -> None:
        self.row_generation += 1
        ids = (ctypes.c_int32 * max(len(block_ids), 1))(*[int(b) for b in block_ids])
        rc = self._lib.sfb_bm_assign_cached_blocks(self._h, request_id.encode(), ids, len(block_ids))
        if rc < 0:
            _raise(rc)

    def ensure_blocks(self, request_id: str, target_tokens: int) -> None:
        self.row_generation += 1  # an unknown request is created here (block.rs:236-268)
        rc = self._lib.sfb_bm_ensure_blocks(self._h, request_id.encode(), int(target_tokens))
        if rc < 0:
            _raise(rc)

    def ensure_blocks_batch(self, request_ids: Sequence[str], target_tokens: "Sequence[int] | torch.Tensor") -> None:
        """``ensure_blocks`` for every request of a step in one call (the scheduler's
        pre-step growth, runtime/src/engine/scheduler.rs:239-246)."""
        n = len(request_ids)
        key = tuple(request_ids)
        if getattr(self, "_batch_key", None) != key:  # the id array is rebuilt only when the batch changes
            self._batch_key = key
            self._batch_ids = (ctypes.c_char_p * max(n, 1))(*[r.encode() for r in request_ids])
        if isinstance(target_tokens, torch.Tensor):
            t64 = target_tokens.to(dtype=torch.int64, device="cpu").contiguous()
            targets = ctypes.cast(ctypes.c_void_p(t64.data_ptr()), ctypes.POINTER(ctypes.c_int64))
        else:
            targets = (ctypes.c_int64 * max(n, 1))(*[int(t) for t in target_tokens])
        rc = self._lib.sfb_bm_ensure_blocks_batch(self._h, self._batch_ids, targets, n)
        if rc < 0:
            _raise(rc)

    def share_prefix(self, src_request_id: str, dst_request_id: str, prefix_len: int) -> list[int]:
        self.row_generation += 1
        n = self._lib.sfb_bm_share_prefix(self._h, src_request_id.encode(), dst_request_id.encode(), int(prefix_len))
        if n < 0:
            _raise(n)
        return self.get_blocks(dst_request_id)

    # ── queries (block.rs:310-346) ───────────────────────────────────────────
    def get_blocks(self, request_id: str) -> list[int]:
        rid = request_id.encode()
        n = self._lib.sfb_bm_get_blocks(self._h, rid, None, 0)
        if n < 0:
            raise KeyError(f"Unknown request_id: {request_id}")
        buf = (ctypes.c_int32 * max(n, 1))()
        self._lib.sfb_bm_get_blocks(self._h, rid, buf, n)
        return list(buf[:n])

    def num_free_blocks(self) -> int:
        return int(self._lib.sfb_bm_num_free_blocks(self._h))

    def num_allocated_blocks(self) -> int:
        return self.num_blocks - self.num_free_blocks()

    def increment_ref_count(self, block_id: int) -> None:
        self._lib.sfb_bm_increment_ref_count(self._h, int(block_id))

    def ref_count(self, block_id: int) -> int:
        return int(self._lib.sfb_bm_ref_count(self._h, int(block_id)))

    def utilization(self) -> float:
        return self.num_allocated_blocks() / self.num_blocks if self.num_blocks else 0.0

    # ── device-resident tables ───────────────────────────────────────────────
    def attach_device_tables(self, rows: int, max_blocks: int, device: torch.device | str = "cuda") -> torch.Tensor:
        """Create the ``int32 [rows, max_blocks]`` device array the kernels read; call before the first allocation."""
        tables = torch.zeros((int(rows), int(max_blocks)), dtype=torch.int32, device=device)
        rc = self._lib.sfb_bm_attach_device_tables(self._h, ctypes.c_void_p(tables.data_ptr()), int(rows), int(max_blocks))
        if rc < 0:
            _raise(rc)
        self.device_tables = tables
        return tables

    def row(self, request_id: str) -> int:
        r = int(self._lib.sfb_bm_row(self._h, request_id.encode()))
        if r < 0:
            raise KeyError(f"Unknown request_id: {request_id}")
        return r

    def rows(self, request_ids: Iterable[str]) -> torch.Tensor:
        """``table_rows`` for a batch: the table row of each request, in batch order (int32, on the tables' device)."""
        assert self.device_tables is not None, "attach_device_tables() first"
        return torch.tensor([self.row(r) for r in request_ids], dtype=torch.int32, device=self.device_tables.device)

    def sync(self, stream: torch.cuda.Stream | None = None) -> int:
        """Upload table entries changed since the last sync; returns how many int32 entries went over."""
        assert self.device_tables is not None, "attach_device_tables() first"
        st = stream if stream is not None else torch.cuda.current_stream(self.device_tables.device)
        with torch.cuda.device(self.device_tables.device):
            n = self._lib.sfb_bm_sync(self._h, ctypes.c_void_p(st.cuda_stream))
        if n < 0:
            _raise(n)
        return int(n)
