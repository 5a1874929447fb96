"""Collective plumbing for the multi-GPU partitions of the decode path.

Attention needs no exchange step: requests are independent, and within a
request the kv-head groups are independent.  The only collective is the
all-gather that brings per-GPU outputs to every device when the caller wants
them in one place.  ``TorchDistCommunicator`` implements the reference's
5-member ``Communicator`` interface (python_runtime/hal/communicator.py:17-72:
``all_reduce``, ``all_gather`` along the last dimension, ``broadcast``, ``rank``,
``world_size``) over ``torch.distributed`` - NCCL on NVLink/NVSwitch for GPU
tensors, Gloo for CPU tensors (the multi-rank tests).
"""

from __future__ import annotations

from collections.abc import Sequence

import torch
import torch.distributed as dist

try:
    from python_runtime.hal.communicator import Communicator  # type: ignore
except Exception:  # noqa: BLE001
    from abc import ABC, abstractmethod

    class Communicator(ABC):  # type: ignore[no-redef]
        """Same contract as python_runtime/hal/communicator.py:17-72."""

        @abstractmethod
        def all_reduce(self, tensor: torch.Tensor, op: str = "sum") -> torch.Tensor: ...

        @abstractmethod
        def all_gather(self, tensor: torch.Tensor) -> torch.Tensor: ...

        @abstractmethod
        def broadcast(self, tensor: torch.Tensor, src: int) -> torch.Tensor: ...

        @property
        @abstractmethod
        def rank(self) -> int: ...

        @property
        @abstractmethod
        def world_size(self) -> int: ...


_OPS = {"sum": dist.ReduceOp.SUM, "min": dist.ReduceOp.MIN, "max": dist.ReduceOp.MAX, "avg": dist.ReduceOp.SUM}


class TorchDistCommunicator(Communicator):
    """``Communicator`` over an initialised ``torch.distributed`` process group."""

    def __init__(self, group: dist.ProcessGroup | None = None) -> None:
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        self._group = group

    @property
    def rank(self) -> int:
        return dist.get_rank(self._group)

    @property
    def world_size(self) -> int:
        return dist.get_world_size(self._group)

    def all_reduce(self, tensor: torch.Tensor, op: str = "sum") -> torch.Tensor:
        if op not in _OPS:
            raise ValueError(f"unknown reduction {op!r}")
        out = tensor.clone()
        dist.all_reduce(out, op=_OPS[op], group=self._group)
        if op == "avg":
            out = out / self.world_size
        return out

    def all_gather(self, tensor: torch.Tensor) -> torch.Tensor:
        """Concatenation of every rank's tensor along the last dimension."""
        return torch.cat(self._gather_parts(tensor.contiguous()), dim=-1)

    def _gather_parts(self, t: torch.Tensor) -> list[torch.Tensor]:
        parts = [torch.empty_like(t) for _ in range(self.world_size)]
        dist.all_gather(parts, t, group=self._group)
        return parts

    def broadcast(self, tensor: torch.Tensor, src: int) -> torch.Tensor:
        out = tensor.clone()
        dist.broadcast(out, src=src, group=self._group)
        return out

    # ── decode-path helpers ──────────────────────────────────────────────────
    def gather_requests(self, out_local: torch.Tensor, counts: Sequence[int]) -> torch.Tensor:
        """Partition by request: rank ``g`` holds ``out_local [counts[g], H, D]`` for a
        contiguous request range; returns ``[sum(counts), H, D]`` in request order on
        every rank (rows are padded to the largest count for the collective)."""
        width = max(counts)
        padded = out_local.new_zeros((width,) + tuple(out_local.shape[1:]))
        padded[: out_local.shape[0]] = out_local
        parts = self._gather_parts(padded)
        return torch.cat([parts[g][: counts[g]] for g in range(self.world_size)], dim=0)

    def gather_heads(self, out_local: torch.Tensor) -> torch.Tensor:
        """Partition by kv head: rank ``g`` holds ``out_local [B, H/G, D]`` for its
        query-head slice; returns ``[B, H, D]`` (heads of rank 0 first)."""
        b, hg, d = out_local.shape
        flat = self.all_gather(out_local.reshape(b, hg * d))
        return flat.view(b, self.world_size * hg, d)


def kv_head_shard(t: torch.Tensor, rank: int, world_size: int, dim: int) -> torch.Tensor:
    """View of rank ``rank``'s slice of a head axis (``k_cache[:, :, g]`` style
    partition for the 8-GPU configuration: one kv head, or H/Hkv query heads, per GPU)."""
    n = t.shape[dim]
    if n % world_size:
        raise ValueError(f"axis of {n} heads does not divide over {world_size} ranks")
    per = n // world_size
    return t.narrow(dim, rank * per, per)


class PeerGather:
    """Output buffers for head-partitioned decode whose all-gather happens inside the decode kernel.

    Every rank allocates TWO copies of the whole ``[batch, heads_per_rank * world, head_dim]`` output plus a
    ``uint32 [world]`` flag array in peer-mapped (symmetric) memory; rank g's decode stores its heads into every rank's
    copy (:func:`ops.paged_attention_decode_gather`) and :meth:`signal_wait` closes the step.  One node, at most 8 ranks.
    The NCCL path (:meth:`TorchDistCommunicator.gather_heads`) stays the portable fallback for callers that cannot map peers.

    Why two copies: there is a "data has arrived" flag per step and no "data has been consumed" flag.  Once rank g has
    passed its wait for step n, its decode of step n + 1 starts storing into the peers' buffers while a slower peer p may
    still be reading step n.  Steps therefore alternate between the two copies (step parity): g's stores of step n + 2
    reuse step n's copy, and g only gets there after p's flag for step n + 1, which p's stream sets after everything it
    queued for step n.  The rule this leaves to the caller: whatever reads the tensor :meth:`decode` returns must be
    queued on the same stream before the next :meth:`decode`, and the tensor is only valid until the decode after next.
    """

    def __init__(self, batch: int, heads_per_rank: int, head_dim: int, dtype: torch.dtype, device: torch.device,
                 group: "dist.ProcessGroup | None" = None) -> None:
        import torch.distributed._symmetric_memory as symm_mem

        grp = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(grp), dist.get_world_size(grp)
        if self.world > 8:
            raise ValueError("PeerGather covers one node: at most 8 ranks")
        self.device = device
        self.outs, self._out_hdls, self.out_ptrs_by_parity = [], [], []
        for _ in range(2):
            buf = symm_mem.empty((batch, heads_per_rank * self.world, head_dim), dtype=dtype, device=device)
            hdl = symm_mem.rendezvous(buf, grp)
            self.outs.append(buf)
            self._out_hdls.append(hdl)
            self.out_ptrs_by_parity.append([int(p) for p in hdl.buffer_ptrs])
        self.flags = symm_mem.empty((self.world,), dtype=torch.int32, device=device)
        self.flags.zero_()
        self._flag_hdl = symm_mem.rendezvous(self.flags, grp)
        self.flag_ptrs = [int(p) for p in self._flag_hdl.buffer_ptrs]
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.step = 0
        torch.cuda.synchronize(device)
        dist.barrier(grp)  # every rank's flags are zero before anybody signals

    @property
    def out(self) -> torch.Tensor:
        """The copy the last completed :meth:`decode` filled."""
        return self.outs[step_buffer(self.step)]

    def decode(self, q, k_cache, v_cache, block_tables, seq_lens, **kw) -> torch.Tensor:
        from . import ops

        which = step_buffer(self.step + 1)
        ops.paged_attention_decode_gather(q, k_cache, v_cache, block_tables, seq_lens, self.outs[which],
                                          self.out_ptrs_by_parity[which], self.rank, **kw)
        self.signal_wait()
        return self.outs[which]

    def signal_wait(self) -> None:
        from . import ops

        self.step += 1
        ops.peer_signal_wait(self.flag_ptrs, self.rank, self.step, self.status, self.device)

    def timed_out(self) -> bool:
        """True when a wait gave up (synchronises)."""
        return bool(int(self.status.item()) != 0)


def step_buffer(step: int) -> int:
    """Which of the two output copies step ``step`` (1, 2, ...) of a :class:`PeerGather` uses."""
    return step & 1
