"""AttentionStepPipeline: host-driven decode steps, two in flight, over block-manager tables.
Every step's result must equal the plain one-step-at-a-time path (dense tables rebuilt per
step, everything on one stream) bit for bit, FP8 codes and scales included."""

import pytest
import torch

from llm_compileforge_b200 import ops
from llm_compileforge_b200.block_manager import BlockManager
from llm_compileforge_b200.step_pipeline import AttentionStepPipeline
from llm_compileforge_b200.tables import dense_block_tables

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fp8", [True, False])
def test_pipelined_steps_equal_serial_steps(fp8):
    dev = torch.device("cuda:0")
    nb, bs, hkv, h, d, rows, width = 200, 16, 2, 8, 128, 6, 16
    g = torch.Generator().manual_seed(5)
    lengths = {f"r{i}": int(n) for i, n in enumerate(torch.randint(1, 150, (rows,), generator=g))}

    def fresh():
        bm = BlockManager(nb, bs)
        tables = bm.attach_device_tables(rows, width, dev)
        kc = torch.zeros((nb, bs, hkv, d), dtype=torch.uint8 if fp8 else torch.bfloat16, device=dev)
        st = dict(bm=bm, tables=tables, kc=kc, vc=torch.zeros_like(kc))
        if fp8:
            st.update(ks=torch.ones((nb, hkv), device=dev), vs=torch.ones((nb, hkv), device=dev),
                      kt=torch.zeros((rows, bs, hkv, d), dtype=torch.bfloat16, device=dev),
                      vt=torch.zeros((rows, bs, hkv, d), dtype=torch.bfloat16, device=dev))
        return st

    def prompt(st):  # prefill every request's context through cache_write
        gp = torch.Generator().manual_seed(6)
        for rid, n in lengths.items():
            st["bm"].allocate(rid, n)
        st["bm"].sync()
        for i, (rid, n) in enumerate(lengths.items()):
            k = (torch.randn((n, hkv, d), generator=gp) * 2).to(torch.bfloat16).to(dev)
            v = (torch.randn((n, hkv, d), generator=gp) * 2).to(torch.bfloat16).to(dev)
            row = torch.tensor([st["bm"].row(rid)], dtype=torch.int32, device=dev)
            extra = dict(k_scale=st["ks"], v_scale=st["vs"], k_tail=st["kt"], v_tail=st["vt"], tail_rows=row) if fp8 else {}
            ops.cache_write(k, v, torch.tensor([0, n], dtype=torch.int32, device=dev), torch.zeros(1, dtype=torch.int32, device=dev),
                            st["tables"], st["kc"], st["vc"], max_new_tokens=n, table_rows=row, **extra)
        torch.cuda.synchronize()

    a, b = fresh(), fresh()
    prompt(a)
    prompt(b)
    fp8kw = lambda st: dict(k_scale=st["ks"], v_scale=st["vs"]) if fp8 else {}
    pipe = AttentionStepPipeline(a["bm"], a["kc"], a["vc"], max_batch=rows, n_heads=h, dtype=torch.bfloat16, depth=2,
                                 **(dict(k_scale=a["ks"], v_scale=a["vs"], k_tail=a["kt"], v_tail=a["vt"]) if fp8 else {}))
    gs = torch.Generator().manual_seed(7)
    live = list(lengths)
    pos = dict(lengths)
    tickets, wants = [], []
    for step in range(24):
        if step == 9:
            live = live[1:]  # a request finishes; the batch shrinks and its order changes
            live.reverse()
        n = len(live)
        q = torch.randn((n, h, d), generator=gs).to(torch.bfloat16).pin_memory()
        k = (torch.randn((n, hkv, d), generator=gs) * 2).to(torch.bfloat16).pin_memory()
        v = (torch.randn((n, hkv, d), generator=gs) * 2).to(torch.bfloat16).pin_memory()
        p = torch.tensor([pos[r] for r in live], dtype=torch.int32).pin_memory()
        tickets.append(pipe.submit(live, q, k, v, p))
        # the same step the plain way on the second state
        b["bm"].ensure_blocks_batch(live, (p + 1).tolist())
        dense, lens, rids = dense_block_tables({r: b["bm"].get_blocks(r) for r in live}, {r: pos[r] + 1 for r in live}, bs)
        rows_t = torch.tensor([b["bm"].row(r) for r in live], dtype=torch.int32, device=dev)
        extra = dict(k_tail=b["kt"], v_tail=b["vt"], tail_rows=rows_t, **fp8kw(b)) if fp8 else {}
        ops.cache_write(k.to(dev), v.to(dev), torch.arange(n + 1, dtype=torch.int32, device=dev), p.to(dev), dense.to(dev),
                        b["kc"], b["vc"], max_new_tokens=1, **extra)
        wants.append(ops.paged_attention_decode(q.to(dev), b["kc"], b["vc"], dense.to(dev), lens.to(dev), **fp8kw(b)).cpu())
        if len(tickets) >= 2:
            t = tickets.pop(0)
            assert torch.equal(pipe.result(t), wants[t]), f"step {t}"
        for r in live:
            pos[r] += 1
    while tickets:
        t = tickets.pop(0)
        assert torch.equal(pipe.result(t), wants[t]), f"step {t}"
    pipe.drain()
    assert pipe.status() == 0
    torch.cuda.synchronize()
    # the two pools hold the same bytes wherever a live request's table points
    for r in live:
        ids = a["bm"].get_blocks(r)
        assert ids == b["bm"].get_blocks(r)
        assert torch.equal(a["kc"][ids], b["kc"][ids]) and torch.equal(a["vc"][ids], b["vc"][ids])
        if fp8:
            assert torch.equal(a["ks"][ids], b["ks"][ids]) and torch.equal(a["vs"][ids], b["vs"][ids])


def test_readmitted_request_id_gets_its_new_table_row():
    """A request id that is freed and admitted again (preemption) may sit in another row of the device tables while the
    tuple of ids of the batch stays the same: the pipeline must look its row up again."""
    dev = torch.device("cuda:0")
    nb, bs, hkv, h, d = 64, 16, 2, 8, 128
    g = torch.Generator().manual_seed(8)
    bm = BlockManager(nb, bs)
    tables = bm.attach_device_tables(4, 8, dev)
    kc = torch.zeros((nb, bs, hkv, d), dtype=torch.bfloat16, device=dev)
    vc = torch.zeros_like(kc)
    pipe = AttentionStepPipeline(bm, kc, vc, max_batch=2, n_heads=h, dtype=torch.bfloat16, depth=2)

    def admit(rid, n):  # allocate and write a prompt of n tokens
        bm.allocate(rid, n)
        bm.sync()
        row = torch.tensor([bm.row(rid)], dtype=torch.int32, device=dev)
        k = torch.randn((n, hkv, d), generator=g).to(torch.bfloat16).to(dev)
        v = torch.randn((n, hkv, d), generator=g).to(torch.bfloat16).to(dev)
        ops.cache_write(k, v, torch.tensor([0, n], dtype=torch.int32, device=dev), torch.zeros(1, dtype=torch.int32, device=dev), tables, kc, vc,
                        max_new_tokens=n, table_rows=row)
        torch.cuda.synchronize()

    def step(pos):
        q = torch.randn((2, h, d), generator=g).to(torch.bfloat16).pin_memory()
        k = torch.randn((2, hkv, d), generator=g).to(torch.bfloat16).pin_memory()
        v = torch.randn((2, hkv, d), generator=g).to(torch.bfloat16).pin_memory()
        got = pipe.result(pipe.submit(["a", "b"], q, k, v, torch.tensor(pos, dtype=torch.int32).pin_memory())).clone()
        dense, lens, _ = dense_block_tables({r: bm.get_blocks(r) for r in ("a", "b")}, {"a": pos[0] + 1, "b": pos[1] + 1}, bs)
        want = ops.paged_attention_decode(q.to(dev), kc, vc, dense.to(dev), lens.to(dev))  # the pools already hold the new token
        assert torch.equal(got, want.cpu())

    admit("a", 20)
    admit("b", 33)
    admit("c", 5)
    step([20, 33])
    row_before = bm.row("a")
    bm.free("a")
    bm.free("c")  # rows come back last-freed-first: "a" now takes the row "c" had
    admit("a", 27)
    assert bm.row("a") != row_before
    step([27, 34])
    assert pipe.status() == 0
