"""Attention half of a decode step, driven from HOST buffers, several steps in flight.

What the reference's engine does per decode step for the attention layer
(python_runtime/engine/_inference_loop.py:187-289: schedule, grow the block
tables, write the step's K/V - ``_write_kv_outputs`` :141-171 - attend, hand
the result back to the host) with everything that does not depend on the
previous step's result overlapped:

* copy-in stream:   q / new K / new V / positions, pinned host -> device staging slot
* compute stream:   table delta scatter, ``cache_write``, ``paged_attention`` (decode)
* copy-out stream:  result -> pinned host slot

``depth`` slots rotate, so the copies of step s+1 run while step s computes;
the pool, the tables and the open-tail copies are touched on the compute
stream only, in submission order.  Block tables live on the device
(:class:`~llm_compileforge_b200.block_manager.BlockManager`): a step uploads
the ids of blocks that were added, nothing else.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import torch

from . import ops
from .block_manager import BlockManager


@dataclass
class _Slot:
    q: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor
    meta: torch.Tensor       # [3, B] int32 on the device: positions, attended lengths, table rows
    meta_host: torch.Tensor  # pinned twin
    out: torch.Tensor
    out_host: torch.Tensor
    copied_in: torch.cuda.Event
    computed: torch.cuda.Event
    copied_out: torch.cuda.Event
    arena: torch.Tensor | None = None     # q | k | v staging as one byte range (a single copy fills it when the host side is laid out alike)
    in_begin: torch.cuda.Event | None = None   # with time_copies: the copies' own device time
    out_begin: torch.cuda.Event | None = None
    busy: bool = False
    n: int = 0


class AttentionStepPipeline:
    """``submit()`` one step's host inputs, ``result()`` its host output; up to ``depth`` steps in flight."""

    def __init__(self, block_manager: BlockManager, k_cache: torch.Tensor, v_cache: torch.Tensor, *, max_batch: int,
                 n_heads: int, dtype: torch.dtype, k_scale: torch.Tensor | None = None, v_scale: torch.Tensor | None = None,
                 k_tail: torch.Tensor | None = None, v_tail: torch.Tensor | None = None, scale: float | None = None,
                 chunk_tokens: int = 0, depth: int = 2, time_copies: bool = False):
        assert block_manager.device_tables is not None, "attach_device_tables() first"
        self.bm = block_manager
        self.tables = block_manager.device_tables
        self.dev = self.tables.device
        self.k_cache, self.v_cache = k_cache, v_cache
        self.fp8 = k_scale is not None
        self.kw = dict(k_scale=k_scale, v_scale=v_scale) if self.fp8 else {}
        self.tails = dict(k_tail=k_tail, v_tail=v_tail) if self.fp8 else {}
        if self.fp8:
            assert k_tail is not None and k_tail.shape[0] >= self.tables.shape[0], "one tail row per table row"
        self.scale, self.chunk = scale, int(chunk_tokens)
        nb, bs, hkv, d = k_cache.shape
        self.block_size = bs
        self.compute = torch.cuda.Stream(self.dev)
        self.copy_in = torch.cuda.Stream(self.dev)
        self.copy_out = torch.cuda.Stream(self.dev)
        self.workspace = torch.zeros(ops.decode_workspace_bytes(max_batch, n_heads, d, self.tables.shape[1], bs, self.chunk),
                                     dtype=torch.uint8, device=self.dev)
        self.cu_one = torch.arange(max_batch + 1, dtype=torch.int32, device=self.dev)

        self.time_copies = bool(time_copies)
        self.h2d_ms = self.d2h_ms = 0.0   # device time of the copies of the steps whose result() was taken (time_copies)
        self.h2d_timed = self.d2h_timed = 0  # bytes those times cover
        esz = torch.empty((), dtype=dtype).element_size()
        nq, nk = max_batch * n_heads * d * esz, max_batch * hkv * d * esz

        def slot() -> _Slot:
            ev = lambda: torch.cuda.Event(enable_timing=self.time_copies)
            arena = torch.empty(nq + 2 * nk, dtype=torch.uint8, device=self.dev)
            return _Slot(
                q=arena[:nq].view(dtype).view(max_batch, n_heads, d),
                k=arena[nq : nq + nk].view(dtype).view(max_batch, hkv, d),
                v=arena[nq + nk :].view(dtype).view(max_batch, hkv, d),
                meta=torch.empty((3, max_batch), dtype=torch.int32, device=self.dev),
                meta_host=torch.empty((3, max_batch), dtype=torch.int32).pin_memory(),
                out=torch.empty((max_batch, n_heads, d), dtype=dtype, device=self.dev),
                out_host=torch.empty((max_batch, n_heads, d), dtype=dtype).pin_memory(),
                copied_in=ev(), computed=ev(), copied_out=ev(), arena=arena,
                in_begin=ev() if self.time_copies else None, out_begin=ev() if self.time_copies else None)

        self.slots = [slot() for _ in range(depth)]
        self.submitted = 0
        self.table_entries_sent = 0
        self._rows_key: tuple | None = None
        self._rows: torch.Tensor | None = None
        self.h2d_bytes = 0  # of the last submit
        self.d2h_bytes = 0

    def submit(self, request_ids: Sequence[str], q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor,
               positions: torch.Tensor, packed: torch.Tensor | None = None) -> int:
        """Queue one decode step.  ``q [B,H,D]``, ``k_new / v_new [B,Hkv,D]`` and ``positions [B]`` (int32: where each
        request's new token goes; it then attends to ``positions + 1`` tokens) are host tensors, pinned for the
        copies to be asynchronous.  ``packed``: the same q, k_new, v_new as ONE pinned uint8 buffer (q's bytes, then k's,
        then v's - see :meth:`host_arena`); a full batch then goes over in a single copy.  Returns a ticket for :meth:`result`."""
        n = len(request_ids)
        ticket = self.submitted
        s = self.slots[ticket % len(self.slots)]
        if s.busy:
            s.copied_out.synchronize()  # its result buffer is about to be reused
        # table row of every request: looked up again whenever the batch or the manager's set of requests has changed (an
        # id that was freed and admitted again may sit in another row)
        key = (self.bm.row_generation, tuple(request_ids))
        if key != self._rows_key:
            self._rows_key = key
            self._rows = torch.tensor([self.bm.row(r) for r in request_ids], dtype=torch.int32)
        s.meta_host[0, :n] = positions
        torch.add(positions, 1, out=s.meta_host[1, :n])
        s.meta_host[2, :n] = self._rows
        # copy-in first (the slot's staging buffers are free once the step that last used them has computed), so that the
        # host's table work below runs while the copies are already moving
        self.copy_in.wait_event(s.computed)
        with torch.cuda.stream(self.copy_in):
            if s.in_begin is not None:
                s.in_begin.record()
            if packed is not None and n == s.q.shape[0]:  # q | k | v back to back in one pinned buffer: one copy instead of three
                s.arena.copy_(packed, non_blocking=True)
            else:
                s.q[:n].copy_(q, non_blocking=True)
                s.k[:n].copy_(k_new, non_blocking=True)
                s.v[:n].copy_(v_new, non_blocking=True)
            s.meta.copy_(s.meta_host, non_blocking=True)
            s.copied_in.record()
        # host: grow the tables to cover the new token (runtime/src/engine/scheduler.rs:239-246), queue the delta
        self.bm.ensure_blocks_batch(request_ids, s.meta_host[1, :n])
        self.table_entries_sent = self.bm.sync(self.compute)
        self.compute.wait_event(s.copied_in)
        self.compute.wait_event(s.copied_out)  # the previous result has left s.out
        with torch.cuda.stream(self.compute):
            pos, lens, rows = s.meta[0, :n], s.meta[1, :n], s.meta[2, :n]
            ops.cache_write(s.k[:n], s.v[:n], self.cu_one[: n + 1], pos, self.tables, self.k_cache, self.v_cache,
                            max_new_tokens=1, tail_rows=rows if self.fp8 else None, table_rows=rows, **self.kw, **self.tails)
            ops.paged_attention_decode(s.q[:n], self.k_cache, self.v_cache, self.tables, lens, scale=self.scale,
                                       chunk_tokens=self.chunk, workspace=self.workspace, out=s.out[:n], table_rows=rows,
                                       **self.kw)
            s.computed.record()
        self.copy_out.wait_event(s.computed)
        with torch.cuda.stream(self.copy_out):
            if s.out_begin is not None:
                s.out_begin.record()
            s.out_host[:n].copy_(s.out[:n], non_blocking=True)
            s.copied_out.record()
        s.busy, s.n = True, n
        self.submitted += 1
        e = q.element_size()
        self.h2d_bytes = (q.numel() + k_new.numel() + v_new.numel()) * e + s.meta_host.numel() * 4 + self.table_entries_sent * 8
        self.d2h_bytes = q.numel() * e
        return ticket

    def host_arena(self) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
        """A pinned buffer laid out like a staging slot: ``(packed uint8, q [B,H,D], k [B,Hkv,D], v [B,Hkv,D])`` views of it, for
        callers that fill their step inputs in place and pass ``packed`` to :meth:`submit`."""
        s = self.slots[0]
        packed = torch.empty(s.arena.numel(), dtype=torch.uint8).pin_memory()
        nq, nk = s.q.numel() * s.q.element_size(), s.k.numel() * s.k.element_size()
        return (packed, packed[:nq].view(s.q.dtype).view(s.q.shape), packed[nq : nq + nk].view(s.k.dtype).view(s.k.shape),
                packed[nq + nk :].view(s.v.dtype).view(s.v.shape))

    def result(self, ticket: int) -> torch.Tensor:
        """Host tensor ``[B,H,D]`` of a submitted step (valid until ``depth`` more steps were submitted)."""
        assert self.submitted - len(self.slots) <= ticket < self.submitted, "ticket no longer in flight"
        s = self.slots[ticket % len(self.slots)]
        s.copied_out.synchronize()
        if self.time_copies and s.busy:
            self.h2d_ms += s.in_begin.elapsed_time(s.copied_in)
            self.d2h_ms += s.out_begin.elapsed_time(s.copied_out)
            e = s.q.element_size()
            self.h2d_timed += (s.n * (s.q.shape[1] + 2 * s.k.shape[1]) * s.q.shape[2]) * e + s.meta_host.numel() * 4
            self.d2h_timed += s.n * s.q.shape[1] * s.q.shape[2] * e
        s.busy = False
        return s.out_host[: s.n]

    def drain(self) -> None:
        for s in self.slots:
            if s.busy:
                s.copied_out.synchronize()
        self.compute.synchronize()

    def status(self) -> int:
        """Status bits of the decode kernel's last run (synchronises the compute stream)."""
        with torch.cuda.stream(self.compute):
            return ops.read_status(self.workspace)
