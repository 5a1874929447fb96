"""Chunked prefill / dense attention on the GPU against the oracle and the
reference-made fixtures.  bf16/fp16 with head_dim 128 run on the tcgen05 kernel,
everything else on the decode kernels (one row per query token)."""

import math

import numpy as np
import pytest
import torch

import llm_compileforge_b200 as pkg
from helpers import assert_f32_close, assert_half_close, from_bits, golden
from llm_compileforge_b200 import ops
from llm_compileforge_b200 import workloads as wl
from llm_compileforge_b200.tables import dense_block_tables
from oracle import c_oracle
from oracle import reference_port as ref

pytestmark = pytest.mark.gpu


def test_flash_attention_reference_kat_fp32(cuda):
    """python_runtime/hal/tests/test_triton_kernels.py:83-105 (seed 42, causal) and :107-127."""
    g = golden("prefill.npz")
    q, k, v = (torch.from_numpy(g[f"flash_kat.{n}"]).to(cuda) for n in "qkv")
    got = pkg.flash_attention_fwd(q, k, v, causal=True).cpu()
    assert_f32_close(got, torch.from_numpy(g["flash_kat.out"]), what="flash causal")
    got = pkg.flash_attention_fwd(q, k, v, causal=False).cpu()
    assert_f32_close(got, torch.from_numpy(g["flash_kat.out_noncausal"]), what="flash non-causal")
    got = pkg.flash_attention_fwd(q, k, v, scale=0.5).cpu()
    want = ref.flash_attention_fwd(q.cpu(), k.cpu(), v.cpu(), scale=0.5)
    assert_f32_close(got, want, what="flash custom scale")
    one = pkg.flash_attention_fwd(torch.randn(1, 1, 16, 32, device=cuda), torch.randn(1, 1, 16, 32, device=cuda),
                                  torch.randn(1, 1, 16, 32, device=cuda))
    assert one.shape == (1, 1, 16, 32)


def test_chunked_prefill_small_fixture(cuda):
    """Config-4 shape, reduced: 3 requests share a 64-token prefix, 48-token chunks, GQA 8/2, D 128, bf16."""
    g = golden("prefill.npz")
    pw = wl.make_prefill_workload(n_requests=3, prefix_len=64, chunk_len=48, n_heads=8, n_kv_heads=2, head_dim=128)
    want = from_bits(g["prefill_small.out"], torch.bfloat16)
    out = pkg.chunked_prefill(pw.q.to(cuda), pw.k_cache.to(cuda), pw.v_cache.to(cuda), pw.block_tables, pw.ctx_lens,
                              {r: 48 for r in pw.block_tables}, scale=pw.scale)
    for i, rid in enumerate(pw.block_tables):
        assert_half_close(out[rid].cpu(), want[i], what=f"chunked prefill {rid}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("n_q,ctx", [(1, 1), (5, 5), (128, 128), (129, 300), (200, 200), (77, 1000), (512, 2560), (300, 301)])
def test_tcgen05_prefill_ragged(cuda, dtype, n_q, ctx):
    """Ragged chunk / context sizes against the plain-C oracle (double accumulation)."""
    g = torch.Generator().manual_seed(n_q * 7 + ctx)
    h, hkv, d = 4, 2, 128
    nblk = -(-ctx // 16)
    nb = nblk + 5
    table = torch.randperm(nb, generator=g)[:nblk].tolist()
    k = torch.randn((nb, 16, hkv, d), generator=g).to(dtype)
    v = torch.randn((nb, 16, hkv, d), generator=g).to(dtype)
    q = torch.randn((n_q, h, d), generator=g).to(dtype)
    want = torch.from_numpy(c_oracle.chunk_prefill(q.float().numpy(), k.float().numpy(), v.float().numpy(),
                                                   np.array(table, dtype=np.int32), ctx, 1 / math.sqrt(d)))
    out = pkg.chunked_prefill(q.to(cuda), k.to(cuda), v.to(cuda), {"r": table}, {"r": ctx}, {"r": n_q})
    assert_half_close(out["r"].cpu(), want, what=f"{dtype} n_q {n_q} ctx {ctx}")


def test_prefill_multi_request_shared_prefix_and_generic_route(cuda):
    """Several requests with different chunk lengths sharing prefix blocks; the same
    inputs in float32 / head_dim 64 go through the decode-kernel route."""
    g = torch.Generator().manual_seed(3)
    for dtype, d, tol in ((torch.bfloat16, 128, None), (torch.float32, 64, 1e-5), (torch.bfloat16, 64, None)):
        h, hkv = 8, 4
        shared = [3, 9, 1, 12]  # 64-token shared prefix
        tables = {"a": shared + [5, 6, 7], "b": shared + [2], "c": shared + [8, 10, 11, 13, 14]}
        ctx = {"a": 64 + 40, "b": 64 + 16, "c": 64 + 70}
        nq = {"a": 40, "b": 16, "c": 70}
        k = torch.randn((16, 16, hkv, d), generator=g).to(dtype)
        v = torch.randn((16, 16, hkv, d), generator=g).to(dtype)
        q = torch.randn((sum(nq.values()), h, d), generator=g).to(dtype)
        out = pkg.chunked_prefill(q.to(cuda), k.to(cuda), v.to(cuda), tables, ctx, nq)
        at = 0
        for r in tables:
            want = torch.from_numpy(c_oracle.chunk_prefill(q[at : at + nq[r]].float().numpy(), k.float().numpy(), v.float().numpy(),
                                                           np.array(tables[r], dtype=np.int32), ctx[r], 1 / math.sqrt(d)))
            if tol:
                assert_f32_close(out[r].cpu(), want, rel=tol, what=f"generic route {r}")
            else:
                assert_half_close(out[r].cpu(), want, what=f"{dtype} D{d} {r}")
            at += nq[r]


@pytest.mark.parametrize("h,hkv", [(6, 2), (8, 8), (2, 1), (12, 3)])
def test_tcgen05_prefill_single_tile_chunks_head_groups(cuda, h, hkv):
    """Chunks of at most 128 rows: with an even number of query heads per kv head two heads share a work item (one per
    tensor-memory tile slot); with an odd number (3 per kv head, or 1) every head runs alone with the second slot empty."""
    g = torch.Generator().manual_seed(100 + h)
    d = 128
    nq = {"a": 77, "b": 128, "c": 3}
    ctx = {"a": 500, "b": 128, "c": 1027}
    blocks = {r: -(-c // 16) for r, c in ctx.items()}
    nb = sum(blocks.values()) + 3
    perm = torch.randperm(nb, generator=g).tolist()
    tables, at = {}, 0
    for r, n in blocks.items():
        tables[r] = perm[at : at + n]
        at += n
    k = torch.randn((nb, 16, hkv, d), generator=g).to(torch.bfloat16)
    v = torch.randn((nb, 16, hkv, d), generator=g).to(torch.bfloat16)
    q = torch.randn((sum(nq.values()), h, d), generator=g).to(torch.bfloat16)
    out = pkg.chunked_prefill(q.to(cuda), k.to(cuda), v.to(cuda), tables, ctx, nq)
    at = 0
    for r in tables:
        want = torch.from_numpy(c_oracle.chunk_prefill(q[at : at + nq[r]].float().numpy(), k.float().numpy(), v.float().numpy(),
                                                       np.array(tables[r], dtype=np.int32), ctx[r], 1 / math.sqrt(d)))
        assert_half_close(out[r].cpu(), want, what=f"H {h}/{hkv} {r}")
        at += nq[r]


def test_prefill_many_ragged_items_per_thread_block(cuda):
    """More work items than SMs, of very different sizes: every resident thread block runs several items back to back (K / V
    stream, Q tiles and first score tile of the next item issued during the current one's last step), including requests whose
    second query tile is empty, one-token chunks and contexts that end inside a 16-token block.  Every request against the
    plain-C oracle."""
    g = torch.Generator().manual_seed(29)
    h, hkv, d = 8, 2, 128
    n_req = 28
    nq = {f"r{i}": int(torch.randint(1, 300, (1,), generator=g)) for i in range(n_req)}
    nq["r3"], nq["r7"], nq["r11"] = 1, 128, 257
    ctx = {r: n + int(torch.randint(0, 400, (1,), generator=g)) for r, n in nq.items()}
    ctx["r5"] = nq["r5"]  # no prefix at all
    blocks = {r: -(-c // 16) for r, c in ctx.items()}
    nb = sum(blocks.values()) + 7
    perm = torch.randperm(nb, generator=g).tolist()
    tables, at = {}, 0
    for r, n in blocks.items():
        tables[r] = perm[at : at + n]
        at += n
    k = torch.randn((nb, 16, hkv, d), generator=g).to(torch.bfloat16)
    v = torch.randn((nb, 16, hkv, d), generator=g).to(torch.bfloat16)
    q = torch.randn((sum(nq.values()), h, d), generator=g).to(torch.bfloat16)
    assert 2 * h * n_req > 148  # two query blocks for the longest chunk: more items than a B200 has SMs
    out = pkg.chunked_prefill(q.to(cuda), k.to(cuda), v.to(cuda), tables, ctx, nq)
    kf, vf = k.float().numpy(), v.float().numpy()
    at = 0
    for r in tables:
        want = torch.from_numpy(c_oracle.chunk_prefill(q[at : at + nq[r]].float().numpy(), kf, vf, np.array(tables[r], dtype=np.int32), ctx[r],
                                                       1 / math.sqrt(d)))
        assert_half_close(out[r].cpu(), want, what=f"ragged batch {r} n_q {nq[r]} ctx {ctx[r]}")
        at += nq[r]


def test_prefill_matches_decode_for_last_token(cuda):
    """The last query row of a chunk is exactly a decode step over the same cache."""
    pw = wl.make_prefill_workload(n_requests=2, prefix_len=128, chunk_len=100, n_heads=8, n_kv_heads=2, head_dim=128)
    dk, dv = pw.k_cache.to(cuda), pw.v_cache.to(cuda)
    out = pkg.chunked_prefill(pw.q.to(cuda), dk, dv, pw.block_tables, pw.ctx_lens, {r: 100 for r in pw.block_tables}, scale=pw.scale)
    last_q = torch.stack([pw.q[99], pw.q[199]]).to(cuda)
    dec = pkg.paged_attention(last_q, dk, dv, pw.block_tables, pw.ctx_lens, scale=pw.scale)
    for i, r in enumerate(pw.block_tables):
        assert (out[r][-1].float() - dec[r].float()).abs().max() <= 2e-2


def test_hal_scaled_dot_product_attention(cuda):
    """HAL op of pytorch_backend/_ops_attention.py:13-53: no mask, is_causal, GQA, and the positional float mask that
    the reference drops when is_causal=True; an explicit mask without a fallback executor is refused."""
    g = torch.Generator().manual_seed(11)
    be = pkg.B200Backend(device=cuda)
    q = torch.randn((2, 8, 96, 128), generator=g).to(torch.bfloat16)
    k = torch.randn((2, 2, 96, 128), generator=g).to(torch.bfloat16)
    v = torch.randn((2, 2, 96, 128), generator=g).to(torch.bfloat16)
    kx, vx = k.repeat_interleave(4, dim=1), v.repeat_interleave(4, dim=1)
    for causal in (False, True):
        got = be.execute("scaled_dot_product_attention", [q.to(cuda), k.to(cuda), v.to(cuda)], is_causal=causal, scale=0.11)
        want = torch.nn.functional.scaled_dot_product_attention(q.float(), kx.float(), vx.float(), is_causal=causal, scale=0.11)
        assert_half_close(got.cpu(), want.to(torch.bfloat16), what=f"sdpa causal={causal}")
    pos = torch.arange(96, dtype=torch.float32).view(1, 1, 96, 1).expand(2, 1, 96, 1).to(cuda)
    got = be.execute("scaled_dot_product_attention", [q.to(cuda), k.to(cuda), v.to(cuda), pos], is_causal=True)
    want = torch.nn.functional.scaled_dot_product_attention(q.float(), kx.float(), vx.float(), is_causal=True)
    assert_half_close(got.cpu(), want.to(torch.bfloat16), what="sdpa positional mask + is_causal")
    with pytest.raises(ValueError):
        be.execute("scaled_dot_product_attention", [q.to(cuda), k.to(cuda), v.to(cuda)],
                   attn_mask=torch.ones((96, 96), dtype=torch.bool, device=cuda))


def test_config4_full_sampled(cuda):
    """Config 4 at full size (32 requests, 2048-token shared prefix + 512-token chunk, H 32/8, D 128, bf16) on the tcgen05
    kernel; the oracle checks a seeded sample of requests, and every request's rows that attend to the shared prefix
    only through identical blocks must agree with request 0's on the one property the layout guarantees: the last row
    of two requests differs (private chunks differ) while status stays clean."""
    pw = wl.make_prefill_workload()
    rids = list(pw.block_tables)
    out = pkg.chunked_prefill(pw.q.to(cuda), pw.k_cache.to(cuda), pw.v_cache.to(cuda), pw.block_tables, pw.ctx_lens,
                              {r: pw.chunk_len for r in rids}, scale=pw.scale)
    pick = torch.randperm(len(rids), generator=torch.Generator().manual_seed(4))[:3].tolist()
    for i in pick:
        rid = rids[i]
        q = pw.q[i * pw.chunk_len : (i + 1) * pw.chunk_len]
        want = ref.chunked_prefill(q, pw.k_cache, pw.v_cache, pw.block_tables[rid], pw.ctx_lens[rid], scale=pw.scale)
        assert_half_close(out[rid].cpu(), want, what=f"config 4 {rid}")
    assert not torch.equal(out[rids[0]][-1], out[rids[1]][-1])
    assert all(torch.isfinite(out[r]).all() for r in rids)
