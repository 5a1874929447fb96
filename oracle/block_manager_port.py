"""CPU restatement of the reference's KV block manager.  TEST INFRASTRUCTURE ONLY:
imported by tests/ as the checker, never by the product.

Follows runtime/src/cache/block.rs of the reference (Rust; no Rust toolchain on
the build machines, so this is a restatement, pinned by the Rust file's own unit
tests restated in tests/test_block_manager.py):

  new                    block.rs:92-111   free list = [0 .. num_blocks)
  allocate               block.rs:146-172  ceil(tokens / block_size) blocks, popped from
                                           the END of the free list; an existing request
                                           is refused with needed = 0
  free                   block.rs:176-195  saturating decrement; a block whose count
                                           reaches 0 is pushed to the END of the free list
  free_block             block.rs:198-210
  assign_cached_blocks   block.rs:214-232  counts += 1 (unknown ids skipped), ids PREPENDED
  ensure_blocks          block.rs:236-268
  share_prefix           block.rs:273-306
  get_blocks ...         block.rs:310-346
"""

from __future__ import annotations


class OutOfMemory(Exception):
    def __init__(self, needed: int, free: int, total: int):
        super().__init__(f"OutOfMemory: need {needed} blocks but only {free} free (total pool: {total})")
        self.needed, self.free, self.total = needed, free, total


class BlockManagerPort:
    def __init__(self, num_blocks: int, block_size: int):
        if num_blocks <= 0:
            raise ValueError("num_blocks must be positive")
        if block_size <= 0:
            raise ValueError("block_size must be positive")
        self.num_blocks, self.block_size = num_blocks, block_size
        self.ref = [0] * num_blocks
        self.free_blocks = list(range(num_blocks))
        self.block_tables: dict[str, list[int]] = {}

    def _pop(self) -> int:
        bid = self.free_blocks.pop()
        self.ref[bid] += 1
        return bid

    def _drop(self, bid: int) -> None:
        self.ref[bid] = max(self.ref[bid] - 1, 0)
        if self.ref[bid] == 0:
            self.free_blocks.append(bid)

    def allocate(self, request_id: str, num_tokens: int) -> list[int]:
        if request_id in self.block_tables:
            raise OutOfMemory(0, len(self.free_blocks), self.num_blocks)
        needed = -(-num_tokens // self.block_size)
        if needed > len(self.free_blocks):
            raise OutOfMemory(needed, len(self.free_blocks), self.num_blocks)
        table = [self._pop() for _ in range(needed)]
        self.block_tables[request_id] = table
        return list(table)

    def free(self, request_id: str) -> None:
        for bid in self.block_tables.pop(request_id, []):
            if 0 <= bid < self.num_blocks:
                self._drop(bid)

    def free_block(self, block_id: int) -> None:
        if 0 <= block_id < self.num_blocks:
            self._drop(block_id)

    def assign_cached_blocks(self, request_id: str, block_ids) -> None:
        for bid in block_ids:
            if 0 <= bid < self.num_blocks:
                self.ref[bid] += 1
        self.block_tables[request_id] = list(block_ids) + self.block_tables.get(request_id, [])

    def ensure_blocks(self, request_id: str, target_tokens: int) -> None:
        existing = len(self.block_tables.get(request_id, [])) * self.block_size
        if existing >= target_tokens:
            return
        n_extra = -(-(target_tokens - existing) // self.block_size)
        if n_extra > len(self.free_blocks):
            raise OutOfMemory(n_extra, len(self.free_blocks), self.num_blocks)
        table = self.block_tables.setdefault(request_id, [])
        for _ in range(n_extra):
            table.append(self._pop())

    def share_prefix(self, src: str, dst: str, prefix_len: int) -> list[int]:
        if src not in self.block_tables:
            raise ValueError(f"Source request '{src}' not found")
        if dst in self.block_tables:
            raise ValueError(f"Destination request '{dst}' already has blocks")
        n = -(-prefix_len // self.block_size)
        table = self.block_tables[src]
        if n > len(table):
            raise ValueError(f"Source has {len(table)} blocks, cannot share {n}")
        shared = table[:n]
        for bid in shared:
            if not 0 <= bid < self.num_blocks:  # block.rs:292-294: counts raised so far stay, no table for dst
                raise ValueError(f"block {bid} not found in share_prefix")
            self.ref[bid] += 1
        self.block_tables[dst] = list(shared)
        return list(shared)

    def get_blocks(self, request_id: str) -> list[int]:
        if request_id not in self.block_tables:
            raise KeyError(f"Unknown request_id: {request_id}")
        return list(self.block_tables[request_id])

    def num_free_blocks(self) -> int:
        return len(self.free_blocks)

    def num_allocated_blocks(self) -> int:
        return self.num_blocks - len(self.free_blocks)

    def ref_count(self, block_id: int) -> int:
        return self.ref[block_id] if 0 <= block_id < self.num_blocks else -1

    def increment_ref_count(self, block_id: int) -> None:
        if 0 <= block_id < self.num_blocks:
            self.ref[block_id] += 1

    def utilization(self) -> float:
        return self.num_allocated_blocks() / self.num_blocks if self.num_blocks else 0.0
