"""Block manager: the reference's own unit tests restated as known-answer tests
(runtime/src/cache/block.rs:478-611), then a randomised differential run of the
C++ manager against the oracle port - block ids, order, counts and errors must
match call for call."""

import random

import pytest

from llm_compileforge_b200.block_manager import BlockManager, OutOfMemoryError
from oracle.block_manager_port import BlockManagerPort, OutOfMemory

IMPLS = [BlockManager, BlockManagerPort]
OOM = (OutOfMemoryError, OutOfMemory)


@pytest.mark.parametrize("cls", IMPLS)
class TestReferenceCases:
    def test_creation(self, cls):
        bm = cls(1000, 16)
        assert (bm.num_blocks, bm.block_size, bm.num_free_blocks()) == (1000, 16, 1000)

    def test_invalid_params(self, cls):
        with pytest.raises(ValueError):
            cls(0, 16)
        with pytest.raises(ValueError):
            cls(100, 0)

    def test_allocate_basic(self, cls):
        bm = cls(1000, 16)
        assert len(bm.allocate("req_1", 32)) == 2
        assert bm.num_free_blocks() == 998

    def test_allocate_exact_block_boundary(self, cls):
        assert len(cls(1000, 16).allocate("req_1", 16)) == 1

    def test_allocate_one_token_needs_one_block(self, cls):
        assert len(cls(1000, 16).allocate("req_1", 1)) == 1

    def test_free_returns_blocks(self, cls):
        bm = cls(1000, 16)
        bm.allocate("req_1", 32)
        assert bm.num_free_blocks() == 998
        bm.free("req_1")
        assert bm.num_free_blocks() == 1000

    def test_free_unknown_is_noop(self, cls):
        bm = cls(1000, 16)
        bm.free("nonexistent")
        assert bm.num_free_blocks() == 1000

    def test_out_of_memory(self, cls):
        bm = cls(10, 16)
        with pytest.raises(OOM) as e:
            bm.allocate("req_1", 200)  # 13 blocks, 10 in the pool
        assert "need 13 blocks but only 10 free (total pool: 10)" in str(e.value)
        assert bm.num_free_blocks() == 10

    def test_share_prefix(self, cls):
        bm = cls(1000, 16)
        src = bm.allocate("src", 64)
        assert len(src) == 4
        shared = bm.share_prefix("src", "dst", 32)
        assert shared == src[:2] and bm.get_blocks("dst") == shared

    def test_share_prefix_ref_count(self, cls):
        bm = cls(1000, 16)
        bm.allocate("src", 32)
        bm.share_prefix("src", "dst", 16)
        bm.free("src")
        assert bm.num_free_blocks() == 999
        bm.free("dst")
        assert bm.num_free_blocks() == 1000

    def test_free_block_single(self, cls):
        bm = cls(1000, 16)
        blocks = bm.allocate("req_1", 32)
        bm.free_block(blocks[0])
        assert bm.num_free_blocks() == 999

    def test_assign_cached_blocks(self, cls):
        bm = cls(1000, 16)
        bm.assign_cached_blocks("req_1", [0, 1])
        assert bm.get_blocks("req_1") == [0, 1]
        bm.ensure_blocks("req_1", 48)
        bm.assign_cached_blocks("req_1", [7])
        assert bm.get_blocks("req_1") == [7, 0, 1, 999]  # prepended; the new block is the pool's last id

    def test_utilization(self, cls):
        bm = cls(100, 16)
        assert abs(bm.utilization()) < 1e-3
        bm.allocate("req_1", 160)
        assert abs(bm.utilization() - 0.1) < 1e-3

    def test_get_blocks_unknown(self, cls):
        with pytest.raises(KeyError):
            cls(10, 16).get_blocks("unknown")

    def test_lifo_order(self, cls):
        # free list is popped from its end (block.rs:165) and freed ids go back on the end (:190)
        bm = cls(8, 4)
        assert bm.allocate("a", 8) == [7, 6]
        assert bm.allocate("b", 4) == [5]
        bm.free("a")
        assert bm.allocate("c", 12) == [6, 7, 4]

    def test_allocate_twice_is_refused(self, cls):
        bm = cls(8, 4)
        bm.allocate("a", 4)
        with pytest.raises(OOM) as e:
            bm.allocate("a", 4)
        assert "need 0 blocks" in str(e.value)

    def test_ids_from_outside_the_pool(self, cls):
        # block.rs:214-232 takes any id into the table and counts only the ones it knows; free skips the others
        # (:184) and share_prefix refuses them (:292-294)
        bm = cls(8, 16)
        bm.assign_cached_blocks("a", [0, 999, -5])
        assert bm.get_blocks("a") == [0, 999, -5]
        assert bm.ref_count(0) == 1
        with pytest.raises(ValueError, match="block 999 not found in share_prefix"):
            bm.share_prefix("a", "b", 48)
        assert bm.ref_count(0) == 2  # raised before the unknown id was met, as in the reference
        with pytest.raises(KeyError):
            bm.get_blocks("b")
        assert bm.share_prefix("a", "c", 16) == [0]
        bm.free("a")
        bm.free("c")
        assert bm.ref_count(0) == 1 and bm.num_free_blocks() == 8

    def test_share_prefix_errors(self, cls):
        bm = cls(8, 4)
        bm.allocate("a", 8)
        with pytest.raises(ValueError):
            bm.share_prefix("nope", "b", 4)
        with pytest.raises(ValueError):
            bm.share_prefix("a", "a", 4)
        with pytest.raises(ValueError):
            bm.share_prefix("a", "b", 100)


def _same(call, *impls):
    """Run `call` on every implementation; all raise the same kind of error or return equal values."""
    results = []
    for bm in impls:
        try:
            results.append(("ok", call(bm)))
        except OOM as e:
            results.append(("oom", str(e)))
        except KeyError:
            results.append(("key", None))
        except ValueError:
            results.append(("value", None))
    assert all(r == results[0] for r in results), results
    return results[0]


@pytest.mark.parametrize("seed", range(6))
def test_differential_random_trace(seed):
    rng = random.Random(seed)
    nb, bs = rng.choice([(12, 4), (64, 16), (257, 16)])
    a, b = BlockManager(nb, bs), BlockManagerPort(nb, bs)
    live: list[str] = []
    counter = 0
    for _ in range(1500):
        op = rng.random()
        if op < 0.30:
            counter += 1
            rid = f"r{counter}"
            tokens = rng.randint(0, 6 * bs)
            if _same(lambda m: m.allocate(rid, tokens), a, b)[0] == "ok":
                live.append(rid)
        elif op < 0.50 and live:
            rid = live.pop(rng.randrange(len(live)))
            _same(lambda m: m.free(rid), a, b)
        elif op < 0.65 and live:
            rid = rng.choice(live)
            tokens = rng.randint(0, 10 * bs)
            _same(lambda m: m.ensure_blocks(rid, tokens), a, b)
        elif op < 0.75 and live:
            counter += 1
            src, dst, plen = rng.choice(live), f"s{counter}", rng.randint(0, 5 * bs)
            if _same(lambda m: m.share_prefix(src, dst, plen), a, b)[0] == "ok":
                live.append(dst)
        elif op < 0.85 and live:
            # prefix hit: blocks held by some live request are prepended to a (possibly new) request
            src = rng.choice(live)
            ids = b.get_blocks(src)[: rng.randint(0, 3)]
            counter += 1
            dst = rng.choice(live + [f"c{counter}"])
            _same(lambda m: m.assign_cached_blocks(dst, ids), a, b)
            if dst not in live:
                live.append(dst)
        elif op < 0.90:
            bid = rng.randrange(nb)
            if b.ref[bid] > 1:  # radix eviction releases one holder of a block that stays referenced
                _same(lambda m: m.free_block(bid), a, b)
        elif op < 0.93:
            bid = rng.randrange(nb)
            if b.ref[bid] > 0:
                _same(lambda m: m.increment_ref_count(bid), a, b)
        else:
            rid = rng.choice(live) if live and rng.random() < 0.8 else "unknown"
            _same(lambda m: m.get_blocks(rid), a, b)
        assert a.num_free_blocks() == b.num_free_blocks()
    for rid in live:
        assert a.get_blocks(rid) == b.get_blocks(rid)
    assert [a.ref_count(i) for i in range(nb)] == b.ref


@pytest.mark.gpu
def test_device_tables_follow_the_host_tables_and_feed_decode():
    """Requests come, grow and go; after every sync the device rows equal the host tables, and a decode that
    reads them through table_rows equals a decode over freshly built dense tables."""
    import torch

    from llm_compileforge_b200 import ops
    from llm_compileforge_b200.tables import dense_block_tables

    dev = torch.device("cuda:0")
    rng = random.Random(3)
    nb, bs, hkv, h, d = 96, 16, 2, 8, 128
    bm = BlockManager(nb, bs)
    tables = bm.attach_device_tables(rows=8, max_blocks=12, device=dev)
    g = torch.Generator().manual_seed(0)
    k = torch.randn((nb, bs, hkv, d), generator=g).to(torch.bfloat16).to(dev)
    v = torch.randn((nb, bs, hkv, d), generator=g).to(torch.bfloat16).to(dev)
    lengths: dict[str, int] = {}
    n_new = 0
    for step in range(40):
        churn = True
        if len(lengths) < 8 and rng.random() < 0.5:
            n_new += 1
            rid = f"r{n_new}"
            lengths[rid] = rng.randint(1, 60)
            if lengths and rng.random() < 0.3 and len(lengths) > 1:
                src = rng.choice([r for r in lengths if r != rid])
                share = min(lengths[src], lengths[rid]) // bs * bs
                bm.share_prefix(src, rid, share)
                bm.ensure_blocks(rid, lengths[rid])
            else:
                bm.allocate(rid, lengths[rid])
        elif lengths and rng.random() < 0.25:
            rid = rng.choice(list(lengths))
            bm.free(rid)
            del lengths[rid]
        else:
            churn = False
        grew = 0
        for rid in lengths:  # every live request decodes one more token
            if lengths[rid] < 12 * bs - 1:
                lengths[rid] += 1
                before = len(bm.get_blocks(rid))
                bm.ensure_blocks(rid, lengths[rid])
                grew += len(bm.get_blocks(rid)) - before
        sent = bm.sync()
        host = tables.cpu()
        for rid in lengths:
            blocks = bm.get_blocks(rid)
            assert host[bm.row(rid), : len(blocks)].tolist() == blocks
        if not churn:
            assert sent == grew  # a steady decode step uploads the new tail blocks and nothing else
        if not lengths:
            continue
        order = list(lengths)
        rng.shuffle(order)  # batch order is free: rows stay put
        q = torch.randn((len(order), h, d), generator=g).to(torch.bfloat16).to(dev)
        lens = torch.tensor([lengths[r] for r in order], dtype=torch.int32, device=dev)
        got = ops.paged_attention_decode(q, k, v, tables, lens, table_rows=bm.rows(order))
        dense, dl, rids = dense_block_tables({r: bm.get_blocks(r) for r in order}, {r: lengths[r] for r in order}, bs)
        assert rids == order
        want = ops.paged_attention_decode(q, k, v, dense.to(dev), dl.to(dev))
        assert torch.equal(got, want)


@pytest.mark.gpu
def test_table_row_out_of_range_is_flagged():
    import torch

    from llm_compileforge_b200 import _lib, ops

    dev = torch.device("cuda:0")
    k = torch.randn((8, 16, 2, 128), device=dev).to(torch.bfloat16)
    q = torch.randn((2, 8, 128), device=dev).to(torch.bfloat16)
    tables = torch.zeros((4, 4), dtype=torch.int32, device=dev)
    lens = torch.tensor([20, 20], dtype=torch.int32, device=dev)
    ws = torch.zeros(ops.decode_workspace_bytes(2, 8, 128, 4), dtype=torch.uint8, device=dev)
    ops.paged_attention_decode(q, k, k, tables, lens, table_rows=torch.tensor([1, 9], dtype=torch.int32, device=dev), workspace=ws)
    assert ops.read_status(ws) & _lib.SFB_STATUS_BAD_BLOCK_ID


@pytest.mark.parametrize("cls", IMPLS)
def test_replay_of_the_reference_radix_cache_trace(cls):
    """tests/golden/block_manager_trace.json: every call the reference's RadixCache and a small serving loop made on a block
    manager (recorded by tests/golden/make_block_trace.py), with results; the C++ manager must answer each one the same."""
    import json
    import os

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "block_manager_trace.json")
    errors = {"OutOfMemory": OOM, "KeyError": (KeyError,), "ValueError": (ValueError,)}
    for trace in json.load(open(path)):
        bm = cls(trace["num_blocks"], trace["block_size"])
        for i, call in enumerate(trace["calls"]):
            fn = getattr(bm, call["op"])
            if "raises" in call:
                with pytest.raises(errors[call["raises"]]):
                    fn(*call["args"])
            else:
                got = fn(*call["args"])
                want = call["ok"]
                assert (got == want) or (isinstance(want, float) and abs(got - want) < 1e-9), (i, call, got)
            assert bm.num_free_blocks() == call["free"], (i, call)
