"""Head-partitioned decode with the gather done by the kernel's own stores.  On one GPU the "peers" are buffers of the
same device and the launch order is: every rank's decode, every rank's signal, then every rank's wait (kernels that
wait for one another must never be queued the other way round on a single device)."""

import pytest
import torch

from llm_compileforge_b200 import _lib, ops
from llm_compileforge_b200.comm import kv_head_shard

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fp8,world", [(False, 2), (True, 4), (True, 1)])
def test_decode_gather_equals_unpartitioned_decode(fp8, world):
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(21 + world)
    b, hkv, group, d, nb, bs = 5, world * 1, 4, 128, 64, 16
    h = hkv * group
    lens = torch.tensor([17, 100, 333, 1, 250], dtype=torch.int32)
    width = 24
    tables = torch.stack([torch.randperm(nb, generator=g)[:width] for _ in range(b)]).to(torch.int32)
    q = torch.randn((b, h, d), generator=g).to(torch.bfloat16).to(dev)
    if fp8:
        k = torch.randint(0, 256, (nb, bs, hkv, d), generator=g, dtype=torch.uint8)
        v = torch.randint(0, 256, (nb, bs, hkv, d), generator=g, dtype=torch.uint8)
        k[(k & 0x7F) == 0x7F] = 0x3C  # no NaN codes
        v[(v & 0x7F) == 0x7F] = 0x3C
        ks = (torch.rand((nb, hkv), generator=g) * 0.02 + 0.001).to(dev)
        vs = (torch.rand((nb, hkv), generator=g) * 0.02 + 0.001).to(dev)
    else:
        k = torch.randn((nb, bs, hkv, d), generator=g).to(torch.bfloat16)
        v = torch.randn((nb, bs, hkv, d), generator=g).to(torch.bfloat16)
        ks = vs = None
    k, v, tables_d, lens_d = k.to(dev), v.to(dev), tables.to(dev), lens.to(dev)
    kw = dict(k_scale=ks, v_scale=vs) if fp8 else {}
    want = ops.paged_attention_decode(q, k, v, tables_d, lens_d, chunk_tokens=64, **kw)

    copies = [torch.full((b, h, d), float("nan"), dtype=torch.bfloat16, device=dev) for _ in range(world)]
    flags = [torch.zeros(world, dtype=torch.int32, device=dev) for _ in range(world)]
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    out_ptrs = [c.data_ptr() for c in copies]
    flag_ptrs = [f.data_ptr() for f in flags]
    for step in (1, 2):  # two steps in a row: the flags count up
        for c in copies:
            c.fill_(float("nan"))
        for r in range(world):
            kw_r = dict(k_scale=kv_head_shard(ks, r, world, 1), v_scale=kv_head_shard(vs, r, world, 1)) if fp8 else {}
            ops.paged_attention_decode_gather(kv_head_shard(q, r, world, 1), kv_head_shard(k, r, world, 2), kv_head_shard(v, r, world, 2),
                                              tables_d, lens_d, copies[r], out_ptrs, r, chunk_tokens=64, **kw_r)
        for phase in (_lib.SFB_PEER_SIGNAL, _lib.SFB_PEER_WAIT):
            for r in range(world):
                ops.peer_signal_wait(flag_ptrs, r, step, status, dev, phases=phase)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        # every copy holds the same bytes; against the unpartitioned launch only the summation order differs
        # (one kv head per launch picks another tiling than `hkv` heads per launch)
        tol = 2e-2 + 2.0 ** -7 * want.float().abs().max().item()
        for r in range(world):
            assert torch.equal(copies[r], copies[0]), f"copy of rank {r}, step {step}"
            assert flags[r].tolist() == [step] * world
        assert not torch.isnan(copies[0].float()).any()
        assert (copies[0].float() - want.float()).abs().max().item() <= tol


def test_signal_wait_gives_up_with_a_status_bit():
    """A peer that never signals: the wait ends by itself and reports it; nothing hangs."""
    dev = torch.device("cuda:0")
    flags = [torch.zeros(2, dtype=torch.int32, device=dev) for _ in range(2)]
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    ops.peer_signal_wait([f.data_ptr() for f in flags], 0, 1, status, dev)  # rank 1 never runs
    torch.cuda.synchronize()
    assert int(status.item()) & _lib.SFB_STATUS_WAIT_TIMEOUT
    assert flags[1].tolist() == [1, 0] and flags[0].tolist() == [1, 0]


def test_two_output_sets_keep_a_slow_readers_step_intact():
    """The race the two output sets close: rank 0 has passed its wait for step 1 and stores step 2 while rank 1 has not
    read step 1 yet.  With the copies alternating by step parity (comm.step_buffer) step 1's bytes stay whole until the
    reader has run; the same sequence over ONE copy would have mixed rows of step 2 into it."""
    from llm_compileforge_b200.comm import step_buffer

    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(77)
    world, b, group, d, nb, bs = 2, 6, 4, 128, 48, 16
    hkv, h = world, world * group
    tables = torch.stack([torch.randperm(nb, generator=g)[:8] for _ in range(b)]).to(torch.int32).to(dev)
    lens = torch.tensor([5, 64, 128, 33, 90, 17], dtype=torch.int32, device=dev)
    k = torch.randn((nb, bs, hkv, d), generator=g).to(torch.bfloat16).to(dev)
    v = torch.randn((nb, bs, hkv, d), generator=g).to(torch.bfloat16).to(dev)
    qs = [torch.randn((b, h, d), generator=g).to(torch.bfloat16).to(dev) for _ in range(2)]  # the queries of steps 1 and 2
    want = [ops.paged_attention_decode(q, k, v, tables, lens, chunk_tokens=64) for q in qs]
    sets = [[torch.zeros((b, h, d), dtype=torch.bfloat16, device=dev) for _ in range(world)] for _ in range(2)]
    flags = [torch.zeros(world, dtype=torch.int32, device=dev) for _ in range(world)]
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    flag_ptrs = [f.data_ptr() for f in flags]

    def decode(step, r):
        copies = sets[step_buffer(step)]
        ops.paged_attention_decode_gather(kv_head_shard(qs[step - 1], r, world, 1), kv_head_shard(k, r, world, 2), kv_head_shard(v, r, world, 2),
                                          tables, lens, copies[r], [c.data_ptr() for c in copies], r, chunk_tokens=64)

    assert step_buffer(1) != step_buffer(2) and step_buffer(1) == step_buffer(3)
    for r in range(world):
        decode(1, r)
    for phase in (_lib.SFB_PEER_SIGNAL, _lib.SFB_PEER_WAIT):
        for r in range(world):
            ops.peer_signal_wait(flag_ptrs, r, 1, status, dev, phases=phase)
    decode(2, 0)  # the fast rank is already in step 2 ...
    seen_by_slow_rank = sets[step_buffer(1)][1].clone()  # ... when the slow rank's reader of step 1 runs
    decode(2, 1)
    for phase in (_lib.SFB_PEER_SIGNAL, _lib.SFB_PEER_WAIT):
        for r in range(world):
            ops.peer_signal_wait(flag_ptrs, r, 2, status, dev, phases=phase)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    tol = 2e-2 + 2.0 ** -7 * want[0].float().abs().max().item()
    assert (seen_by_slow_rank.float() - want[0].float()).abs().max().item() <= tol
    assert torch.equal(seen_by_slow_rank, sets[step_buffer(1)][0])
    assert (sets[step_buffer(2)][1].float() - want[1].float()).abs().max().item() <= tol
