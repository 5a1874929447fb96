"""World-size-2 checks of the multi-GPU host logic with Gloo ranks on the CPU:
request partition + output gather, kv-head partition + output gather, and the
Communicator interface.  Per-rank attention is computed by the CPU oracle (these
tests have no GPU); the gathered result must equal the unpartitioned oracle."""

import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, mode: str, result_dir: str) -> None:
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    from llm_compileforge_b200 import workloads as wl
    from llm_compileforge_b200.comm import TorchDistCommunicator, kv_head_shard
    from llm_compileforge_b200.tables import partition_by_request
    from oracle import reference_port as ref

    comm = TorchDistCommunicator()
    assert comm.rank == rank and comm.world_size == world
    w = wl.make_decode_workload(wl.C2, batch=7, max_len=200)
    rids = list(w.block_tables)
    full = ref.paged_attention(w.q, w.k_cache, w.v_cache, w.block_tables, w.seq_lens, scale=w.scale)
    full = torch.stack([full[r] for r in rids])
    if mode == "interface":
        t = torch.full((2, 3), float(rank + 1))
        assert torch.equal(comm.all_reduce(t), torch.full((2, 3), 3.0))
        assert torch.equal(comm.all_reduce(t, "max"), torch.full((2, 3), 2.0))
        assert torch.equal(comm.all_reduce(t, "avg"), torch.full((2, 3), 1.5))
        g = comm.all_gather(t)
        assert g.shape == (2, 6) and torch.equal(g[:, :3], torch.full((2, 3), 1.0)) and torch.equal(g[:, 3:], torch.full((2, 3), 2.0))
        assert torch.equal(comm.broadcast(t, src=1), torch.full((2, 3), 2.0))
        with pytest.raises(ValueError):
            comm.all_reduce(t, "prod")
        got = full
    elif mode == "requests":
        parts = partition_by_request(w.lengths, world)
        mine = parts[rank]
        sub_t = {rids[i]: w.block_tables[rids[i]] for i in mine}
        sub_l = {rids[i]: w.seq_lens[rids[i]] for i in mine}
        local = ref.paged_attention(w.q[mine], w.k_cache, w.v_cache, sub_t, sub_l, scale=w.scale)
        local = torch.stack([local[rids[i]] for i in mine]) if mine else w.q.new_zeros((0,) + tuple(w.q.shape[1:]))
        got = comm.gather_requests(local, [len(p) for p in parts])
    else:  # kv heads: rank g owns kv heads [g*Hkv/G, ...) and the matching query heads
        k = kv_head_shard(w.k_cache, rank, world, dim=2)
        v = kv_head_shard(w.v_cache, rank, world, dim=2)
        q = kv_head_shard(w.q, rank, world, dim=1)
        local = ref.paged_attention(q, k, v, w.block_tables, w.seq_lens, scale=w.scale)
        got = comm.gather_heads(torch.stack([local[r] for r in rids]))
    assert got.shape == full.shape
    assert torch.equal(got, full), f"{mode}: gathered result differs from the unpartitioned oracle"
    with open(os.path.join(result_dir, f"ok_{mode}_{rank}"), "w") as f:
        f.write("ok")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["interface", "requests", "heads"])
def test_two_ranks_gloo(mode, tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, mode, str(tmp_path)), nprocs=2, join=True)
    assert sorted(os.listdir(tmp_path)) == [f"ok_{mode}_0", f"ok_{mode}_1"]
