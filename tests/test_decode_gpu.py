"""Paged-attention decode on the GPU against the CPU oracle and the reference's
golden vectors.  Calls go through the C ABI (kernels_api / ops -> libsfb)."""

import math

import numpy as np
import pytest
import torch

import llm_compileforge_b200 as pkg
from helpers import (assert_f32_close, assert_half_close, from_bits, golden, stack_outputs, tables_to_dict)
from llm_compileforge_b200 import ops
from llm_compileforge_b200 import workloads as wl
from llm_compileforge_b200.tables import dense_block_tables
from oracle import reference_port as ref

pytestmark = pytest.mark.gpu

KAT_NAMES = {"kat_mha": ["req_1"], "kat_gqa": ["req_1"], "kat_multi": ["req_1", "req_2"],
             "edges": ["nolen", "toolong", "surplus", "shared", "one"]}


@pytest.mark.parametrize("case", list(KAT_NAMES))
def test_reference_kats_fp32(cuda, case):
    g = golden("paged_decode_kats.npz")
    q, k, v = (torch.from_numpy(g[f"{case}.{n}"]) for n in "qkv")
    names = KAT_NAMES[case]
    tables, lens = tables_to_dict(g[f"{case}.tables"], g[f"{case}.table_lens"], g[f"{case}.seq_lens"], names)
    want = torch.from_numpy(g[f"{case}.out"])
    out = pkg.paged_attention(q.to(cuda), k.to(cuda), v.to(cuda), tables, lens, block_size=16)
    assert list(out) == names
    got = stack_outputs(out, names).cpu()
    assert got.dtype == torch.float32 and got.shape == want.shape
    assert_f32_close(got, want, what=case)
    # the reference's own acceptance line (python_runtime/hal/tests/test_triton_kernels.py:250, cos >= 0.999)
    assert torch.nn.functional.cosine_similarity(got.flatten(), want.flatten(), dim=0) >= 0.999


@pytest.mark.parametrize("chunk", [0, 16, 64, 128])
def test_config1_full_fp32(cuda, chunk):
    g = golden("paged_decode_c1.npz")
    w = wl.make_decode_workload(wl.C1)
    want = torch.from_numpy(g["out"])
    out = pkg.paged_attention(w.q.to(cuda), w.k_cache.to(cuda), w.v_cache.to(cuda), w.block_tables, w.seq_lens,
                              block_size=16, scale=w.scale, chunk_tokens=chunk)
    got = stack_outputs(out, list(w.block_tables)).cpu()
    assert got.shape == (8, 12, 64)
    assert_f32_close(got, want, what=f"config 1 chunk {chunk}")
    truth = ref.paged_attention_f64(w.q, w.k_cache, w.v_cache, w.block_tables, w.seq_lens, scale=w.scale)
    assert_f32_close(got, stack_outputs(truth, list(w.block_tables)).float(), what="config 1 vs float64")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("chunk", [0, 64])
def test_config2_small_half(cuda, dtype, chunk):
    w = wl.make_decode_workload(wl.C2, batch=6, max_len=400)
    q, k, v = w.q.to(dtype), w.k_cache.to(dtype), w.v_cache.to(dtype)
    if dtype == torch.bfloat16:
        want = from_bits(golden("paged_decode_c2_small.npz")["out"], torch.bfloat16)
    else:
        want = stack_outputs(ref.paged_attention(q, k, v, w.block_tables, w.seq_lens, scale=w.scale), list(w.block_tables))
    out = pkg.paged_attention(q.to(cuda), k.to(cuda), v.to(cuda), w.block_tables, w.seq_lens, scale=w.scale, chunk_tokens=chunk)
    got = stack_outputs(out, list(w.block_tables)).cpu()
    assert got.dtype == dtype
    assert_half_close(got, want, what=f"config 2 small {dtype}")
    truth = stack_outputs(ref.paged_attention_f64(q, k, v, w.block_tables, w.seq_lens, scale=w.scale), list(w.block_tables))
    assert_half_close(got, truth, what="config 2 small vs float64")


def test_config2_full_sampled(cuda):
    """Full config 2 on the GPU; the oracle checks a seeded sample of requests."""
    w = wl.make_decode_workload(wl.C2)
    out = pkg.paged_attention(w.q.to(cuda), w.k_cache.to(cuda), w.v_cache.to(cuda), w.block_tables, w.seq_lens, scale=w.scale)
    rids = list(w.block_tables)
    pick = [rids[i] for i in torch.randperm(len(rids), generator=torch.Generator().manual_seed(3))[:6].tolist()]
    rows = [rids.index(r) for r in pick]
    sub_t = {r: w.block_tables[r] for r in pick}
    sub_l = {r: w.seq_lens[r] for r in pick}
    want = ref.paged_attention(w.q[rows], w.k_cache, w.v_cache, sub_t, sub_l, scale=w.scale)
    assert_half_close(stack_outputs(out, pick).cpu(), stack_outputs(want, pick), what="config 2 full")


def test_strided_layer_view_and_shared_blocks(cuda):
    """The engine's slab [NB, layers, bs, heads, dim] is consumed through a layer
    view without a copy (python_runtime/engine/cache_manager.py:106-113), and a
    physical block may sit in several tables (prefix sharing)."""
    g = torch.Generator().manual_seed(11)
    nb, layers, hkv, d, h = 24, 3, 2, 64, 8
    slab_k = torch.randn((nb, layers, 16, hkv, d), generator=g)
    slab_v = torch.randn((nb, layers, 16, hkv, d), generator=g)
    q = torch.randn((3, h, d), generator=g)
    shared = [5, 9]
    tables = {"a": shared + [1, 2], "b": shared + [7], "c": shared}
    lens = {"a": 60, "b": 40, "c": 32}
    dk, dv = slab_k.to(cuda), slab_v.to(cuda)
    for layer in range(layers):
        want = ref.paged_attention(q, slab_k[:, layer], slab_v[:, layer], tables, lens)
        view_k, view_v = dk[:, layer], dv[:, layer]
        assert not view_k.is_contiguous()
        out = pkg.paged_attention(q.to(cuda), view_k, view_v, tables, lens)
        assert_f32_close(stack_outputs(out, list(tables)).cpu(), stack_outputs(want, list(tables)), what=f"layer {layer}")


def test_device_status_flags_bad_block_and_empty_request(cuda):
    g = torch.Generator().manual_seed(2)
    k = torch.randn((6, 16, 2, 32), generator=g).to(cuda)
    q = torch.randn((2, 4, 32), generator=g).to(cuda)
    tables = torch.tensor([[0, 99, 2], [1, 3, 4]], dtype=torch.int32, device=cuda)  # 99 is outside the pool
    lens = torch.tensor([40, 0], dtype=torch.int32, device=cuda)
    ws = torch.zeros(ops.decode_workspace_bytes(2, 4, 32, 3, 16, 16), dtype=torch.uint8, device=cuda)
    out = ops.paged_attention_decode(q, k, k, tables, lens, chunk_tokens=16, workspace=ws)
    bits = ops.read_status(ws)
    assert bits == 1 | 2
    assert torch.count_nonzero(out[1]) == 0  # empty request: zero row
    # the bad block is skipped: result equals attention over blocks 0 and 2's tokens only
    kk = k.cpu()
    keep = torch.cat([kk[0], kk[2][:8]], 0)  # tokens 0..15 and 32..39
    lg = torch.einsum("hd,thd->ht", q[0].cpu(), keep.repeat_interleave(2, dim=1)) / math.sqrt(32)
    want = torch.einsum("ht,thd->hd", torch.softmax(lg, -1), keep.repeat_interleave(2, dim=1))
    assert_f32_close(out[0].cpu(), want, rel=1e-5)
    # a clean call resets the word
    lens2 = torch.tensor([33, 20], dtype=torch.int32, device=cuda)
    tables2 = torch.tensor([[0, 5, 2], [1, 3, 4]], dtype=torch.int32, device=cuda)
    ops.paged_attention_decode(q, k, k, tables2, lens2, chunk_tokens=16, workspace=ws)
    assert ops.read_status(ws) == 0


def test_hal_backend_dense_and_dict_forms(cuda):
    w = wl.make_decode_workload(wl.C1)
    be = pkg.B200Backend()
    q, k, v = w.q.to(cuda), w.k_cache.to(cuda), w.v_cache.to(cuda)
    as_dict = be.execute("paged_attention", [q, k, v, w.block_tables], seq_lens=w.seq_lens, scale=w.scale, chunk_tokens=128)
    dense, lens, rids = dense_block_tables(w.block_tables, w.seq_lens, 16)
    as_dense = be.execute("paged_attention", [q, k, v, dense.to(cuda)], seq_lens=lens.to(cuda), scale=w.scale, chunk_tokens=128)
    assert torch.equal(stack_outputs(as_dict, rids), as_dense)
    want = torch.from_numpy(golden("paged_decode_c1.npz")["out"])
    assert_f32_close(as_dense.cpu(), want)


def _random_case(seed, batch, heads, kv_heads, dim, max_len, dtype, layers=None):
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(1, max_len + 1, (batch,), generator=g).tolist()
    lens[0] = max_len  # at least one request of full length
    if batch > 1:
        lens[1] = 1
    nb = sum(-(-n // 16) for n in lens) + 3
    tables = wl.random_tables(lens, nb, seed=seed + 1)
    q = torch.randn((batch, heads, dim), generator=g).to(dtype)
    shape = (nb, 16, kv_heads, dim) if layers is None else (nb, layers, 16, kv_heads, dim)
    k = torch.randn(shape, generator=g).to(dtype)
    v = torch.randn(shape, generator=g).to(dtype)
    return q, k, v, tables, {r: n for r, n in zip(tables, lens)}


@pytest.mark.parametrize("dtype,dim", [(torch.bfloat16, 64), (torch.bfloat16, 128), (torch.float16, 64), (torch.float16, 128)])
@pytest.mark.parametrize("heads,kv_heads", [(8, 8), (32, 4), (16, 2), (8, 1), (32, 16), (6, 2), (5, 1)])
def test_tensor_core_path_shapes(cuda, dtype, dim, heads, kv_heads):
    """Shapes the TMA + tensor-core kernel covers (128- and 256-byte rows, 1..8 query
    heads per kv head, every head-group layout), single pass and split."""
    q, k, v, tables, lens = _random_case(100 + heads + dim, 5, heads, kv_heads, dim, 200, dtype)
    want = ref.paged_attention_f64(q, k, v, tables, lens)
    rids = list(tables)
    for chunk in (0, 48):
        out = pkg.paged_attention(q.to(cuda), k.to(cuda), v.to(cuda), tables, lens, chunk_tokens=chunk)
        assert_half_close(stack_outputs(out, rids).cpu(), stack_outputs(want, rids), what=f"{dtype} D{dim} H{heads}/{kv_heads} chunk {chunk}")


@pytest.mark.parametrize("heads,kv_heads,dim", [(32, 8, 128), (64, 8, 128), (8, 1, 128), (16, 4, 256), (12, 2, 128)])
@pytest.mark.parametrize("qdtype", [torch.bfloat16, torch.float16])
def test_tensor_core_path_fp8(cuda, heads, kv_heads, dim, qdtype):
    q, k, v, tables, lens = _random_case(300 + heads + dim, 6, heads, kv_heads, dim, 300, torch.bfloat16)
    k, v = k * 2, v * 2
    k[3] *= 50.0  # blocks with very different scales exercise the scale-in-exponent path
    v[5] *= 0.001
    v[7] *= 300.0
    kc, ks = ref.fp8_quantize_pool_fast(k)
    vc, vs = ref.fp8_quantize_pool_fast(v)
    kd, vd = ref.fp8_dequantize_pool(kc, ks), ref.fp8_dequantize_pool(vc, vs)
    q = q.to(qdtype)
    want = ref.paged_attention_f64(q, kd, vd, tables, lens)
    want32 = ref.paged_attention(q.float(), kd, vd, tables, lens)  # the reference's own arithmetic
    rids = list(tables)
    for chunk in (0, 64):
        out = pkg.paged_attention(q.to(cuda), kc.to(cuda), vc.to(cuda), tables, lens, k_scale=ks.to(cuda), v_scale=vs.to(cuda),
                                  chunk_tokens=chunk)
        got = stack_outputs(out, rids).cpu()
        # 2e-2 absolute for O(1) rows; a row dominated by the 300x block is O(1000), where the
        # 16-bit output grid and the 16-bit probability operand are coarser in absolute terms:
        # allow 2^-8 of the row's largest magnitude on top
        w64 = stack_outputs(want, rids)
        tol = 2e-2 + 2.0 ** -8 * w64.abs().amax(dim=-1, keepdim=True)
        assert ((got.double() - w64).abs() <= tol).all()
        assert ((got.double() - stack_outputs(want32, rids).double()).abs() <= tol).all()
        from helpers import cos_deficit
        assert cos_deficit(got, stack_outputs(want, rids)) <= 1e-4


def test_fp8_mixed_scales_with_rows_of_order_one(cuda):
    """Blocks whose K and V scales differ by orders of magnitude while every output row stays O(1): the contract's own
    tolerance (2e-2 absolute, cosine deficit 1e-4) with nothing added."""
    q, k, v, tables, lens = _random_case(41, 6, 32, 8, 128, 280, torch.bfloat16)
    g = torch.Generator().manual_seed(42)
    nb = k.shape[0]
    # K: per-block gains 1/16 .. 16 change the logits' spread block by block; V: gains 1/32 .. 1, so no block dominates the row
    k = (k.float() * (2.0 ** torch.randint(-4, 5, (nb, 1, 1, 1), generator=g)) * 0.25).to(torch.bfloat16)
    v = (v.float() * (2.0 ** torch.randint(-5, 1, (nb, 1, 1, 1), generator=g).float())).to(torch.bfloat16)
    kc, ks = ref.fp8_quantize_pool_fast(k)
    vc, vs = ref.fp8_quantize_pool_fast(v)
    assert ks.max() / ks[ks > 0].min() > 100 and vs.max() / vs[vs > 0].min() > 10
    kd, vd = ref.fp8_dequantize_pool(kc, ks), ref.fp8_dequantize_pool(vc, vs)
    want = ref.paged_attention_f64(q, kd, vd, tables, lens)
    rids = list(tables)
    assert stack_outputs(want, rids).abs().max() < 4.0
    for chunk in (0, 64):
        out = pkg.paged_attention(q.to(cuda), kc.to(cuda), vc.to(cuda), tables, lens, k_scale=ks.to(cuda), v_scale=vs.to(cuda), chunk_tokens=chunk)
        assert_half_close(stack_outputs(out, rids).cpu(), stack_outputs(want, rids), what=f"mixed scales, chunk {chunk}")


@pytest.mark.parametrize("gain", [1e5, 3e4, 1e-6, 1e-30])
def test_fp8_decode_bf16_query_outside_fp16_range(cuda, gain):
    """A bf16 query is fed to the fp16 tensor-core path of an e4m3 pool.  Magnitudes beyond fp16's 65504, or far below its
    smallest normal, must neither overflow to infinity nor lose the row: heads of very different magnitude share a batch."""
    q, k, v, tables, lens = _random_case(77, 4, 16, 4, 128, 120, torch.bfloat16)
    q = q.float()
    q[:, ::2] *= gain          # every other head scaled, the rest left at N(0,1)
    q[0, 1] = 0.0              # an all-zero query row
    q = q.to(torch.bfloat16)
    kc, ks = ref.fp8_quantize_pool_fast(k)
    vc, vs = ref.fp8_quantize_pool_fast(v)
    kd, vd = ref.fp8_dequantize_pool(kc, ks), ref.fp8_dequantize_pool(vc, vs)
    want = ref.paged_attention_f64(q, kd, vd, tables, lens)
    rids = list(tables)
    out = pkg.paged_attention(q.to(cuda), kc.to(cuda), vc.to(cuda), tables, lens, k_scale=ks.to(cuda), v_scale=vs.to(cuda))
    got = stack_outputs(out, rids).cpu()
    assert torch.isfinite(got.float()).all()
    assert_half_close(got, stack_outputs(want, rids), what=f"query gain {gain:g}")


def test_tensor_core_path_strided_slab_and_bad_block(cuda):
    q, k, v, tables, lens = _random_case(7, 4, 16, 4, 64, 150, torch.bfloat16, layers=2)
    dk, dv = k.to(cuda), v.to(cuda)
    rids = list(tables)
    for layer in range(2):
        want = ref.paged_attention_f64(q, k[:, layer], v[:, layer], tables, lens)
        out = pkg.paged_attention(q.to(cuda), dk[:, layer], dv[:, layer], tables, lens)
        assert_half_close(stack_outputs(out, rids).cpu(), stack_outputs(want, rids), what=f"slab layer {layer}")
    # out-of-pool block id: skipped and flagged, the kernel keeps running
    dense, ll, _ = dense_block_tables(tables, lens, 16)
    dense = dense.clone()
    dense[0, 1] = 10_000
    ws = torch.zeros(ops.decode_workspace_bytes(4, 16, 64, dense.shape[1], 16, 32), dtype=torch.uint8, device=cuda)
    out = ops.paged_attention_decode(q.to(cuda), dk[:, 0], dv[:, 0], dense.to(cuda), ll.to(cuda), chunk_tokens=32, workspace=ws)
    assert ops.read_status(ws) == 1
    assert torch.isfinite(out.float()).all()
    want = ref.paged_attention_f64(q, k[:, 0], v[:, 0], tables, lens)
    assert_half_close(out[1:].cpu(), stack_outputs(want, rids)[1:], what="rows without the bad block")


def test_stale_slots_past_length_are_ignored(cuda):
    """Slots after a request's last token may hold anything (NaN bit patterns
    included); they must not leak into the result."""
    q, k, v, tables, lens = _random_case(9, 3, 8, 2, 64, 90, torch.bfloat16)
    want = ref.paged_attention_f64(q, k, v, tables, lens)
    k2, v2 = k.clone(), v.clone()
    for r, n in lens.items():
        last = tables[r][(n - 1) // 16]
        if n % 16:
            k2[last, n % 16 :] = float("nan")
            v2[last, n % 16 :] = float("nan")
    out = pkg.paged_attention(q.to(cuda), k2.to(cuda), v2.to(cuda), tables, lens)
    rids = list(tables)
    assert_half_close(stack_outputs(out, rids).cpu(), stack_outputs(want, rids), what="stale slots")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("n_req,prefix_blocks,heads,kv_heads", [(32, 128, 32, 8), (5, 16, 8, 2), (150, 20, 8, 8), (1, 16, 8, 1)])
def test_shared_prefix_decode_matches_plain_decode(cuda, dtype, n_req, prefix_blocks, heads, kv_heads):
    """Radix-shared prefix (identical leading block ids in every table): the cascade route
    (prefix once on the tcgen05 kernel + per-request remainder, merged in-kernel) equals the
    oracle and the plain decode kernel."""
    g = torch.Generator().manual_seed(n_req + prefix_blocks)
    d = 128
    own = torch.randint(1, 200, (n_req,), generator=g).tolist()
    own[0] = 1
    own_blocks = [-(-n // 16) for n in own]
    nb = prefix_blocks + sum(own_blocks) + 4
    perm = torch.randperm(nb, generator=g).tolist()
    shared = perm[:prefix_blocks]
    tables, lens, at = {}, {}, prefix_blocks
    for i in range(n_req):
        tables[f"r{i}"] = shared + perm[at : at + own_blocks[i]]
        lens[f"r{i}"] = prefix_blocks * 16 + own[i]
        at += own_blocks[i]
    q = torch.randn((n_req, heads, d), generator=g).to(dtype)
    k = torch.randn((nb, 16, kv_heads, d), generator=g).to(dtype)
    v = torch.randn((nb, 16, kv_heads, d), generator=g).to(dtype)
    rids = list(tables)
    from llm_compileforge_b200.tables import shared_prefix_blocks

    assert shared_prefix_blocks(tables, lens, 16) == (prefix_blocks if n_req > 1 else 0)
    dense, ll, _ = dense_block_tables(tables, lens, 16)
    dq, dk, dv = q.to(cuda), k.to(cuda), v.to(cuda)
    plain = ops.paged_attention_decode(dq, dk, dv, dense.to(cuda), ll.to(cuda), chunk_tokens=64)
    want = stack_outputs(ref.paged_attention_f64(q, k, v, tables, lens), rids)
    for chunk in (0, 64):
        ws_bytes = _lib_ws(n_req, heads, d, dense.shape[1], chunk, prefix_blocks)
        ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=cuda)
        got = ops.paged_attention_decode_shared_prefix(dq, dk, dv, dense.to(cuda), ll.to(cuda), prefix_blocks, chunk_tokens=chunk, workspace=ws)
        assert ops.read_status(ws) == 0
        assert_half_close(got.cpu(), want, what=f"shared prefix chunk {chunk}")
        assert (got.float() - plain.float()).abs().max() <= 2e-2
    if n_req > 1:  # the dict API finds the shared prefix by itself
        auto = pkg.paged_attention(dq, dk, dv, tables, lens)
        assert_half_close(stack_outputs(auto, rids).cpu(), want, what="auto shared prefix")


def _lib_ws(b, h, d, max_blocks, chunk, prefix_blocks):
    from llm_compileforge_b200 import _lib

    return int(_lib.load().sfb_shared_prefix_workspace_bytes(b, h, d, max_blocks, 16, chunk, prefix_blocks))


def test_work_list_with_shared_prefix_and_ragged_lengths(cuda):
    """A batch large enough for the size-ordered work list (>= 600 (request, chunk) slots over >= 1 GiB of addressable pool):
    plain decode and the shared-prefix route both take their items from the list; lengths from 1 token to several chunks,
    an empty request in the middle.  The oracle checks a sample; the two routes must agree everywhere."""
    g = torch.Generator().manual_seed(77)
    n_req, heads, kv_heads, d, prefix_blocks = 384, 32, 8, 128, 16
    own = torch.randint(1, 1100, (n_req,), generator=g).tolist()
    own[5], own[6] = 1, 1024
    own_blocks = [-(-n // 16) for n in own]
    nb = prefix_blocks + sum(own_blocks) + 7
    perm = torch.randperm(nb, generator=g).tolist()
    shared = perm[:prefix_blocks]
    tables, lens, at = {}, {}, prefix_blocks
    for i in range(n_req):
        tables[f"r{i}"] = shared + perm[at : at + own_blocks[i]]
        lens[f"r{i}"] = prefix_blocks * 16 + own[i]
        at += own_blocks[i]
    gen = torch.Generator(device=cuda).manual_seed(78)
    q = torch.randn((n_req, heads, d), generator=gen, device=cuda).to(torch.bfloat16)
    k = torch.randn((nb, 16, kv_heads, d), generator=gen, device=cuda).to(torch.bfloat16)
    v = torch.randn((nb, 16, kv_heads, d), generator=gen, device=cuda).to(torch.bfloat16)
    rids = list(tables)
    dense, ll, _ = dense_block_tables(tables, lens, 16)
    assert n_req * -(-dense.shape[1] * 16 // 256) >= 600 and n_req * dense.shape[1] * 16 * kv_heads * d * 2 * 2 >= 1 << 30
    dt, dl = dense.to(cuda), ll.to(cuda)
    ws = torch.zeros(ops.decode_workspace_bytes(n_req, heads, d, dense.shape[1], 16, 256), dtype=torch.uint8, device=cuda)
    plain = ops.paged_attention_decode(q, k, v, dt, dl, chunk_tokens=256, workspace=ws)
    assert ops.read_status(ws) == 0
    ws2 = torch.zeros(_lib_ws(n_req, heads, d, dense.shape[1], 256, prefix_blocks), dtype=torch.uint8, device=cuda)
    casc = ops.paged_attention_decode_shared_prefix(q, k, v, dt, dl, prefix_blocks, chunk_tokens=256, workspace=ws2)
    assert ops.read_status(ws2) == 0
    assert (casc.float() - plain.float()).abs().max().item() <= 2e-2
    pick = [5, 6, 17, 200, 383]
    kc, vc = k.cpu(), v.cpu()
    want = ref.paged_attention_f64(q.cpu()[pick], kc, vc, {rids[i]: tables[rids[i]] for i in pick}, {rids[i]: lens[rids[i]] for i in pick})
    for j, i in enumerate(pick):
        assert_half_close(plain[i].cpu(), want[rids[i]], what=f"work list, request {i}")
    # an empty request among the others: flagged, zero row, every other row unchanged
    dl2 = dl.clone()
    dl2[100] = 0
    again = ops.paged_attention_decode(q, k, v, dt, dl2, chunk_tokens=256, workspace=ws)
    assert ops.read_status(ws) & 2  # SFB_STATUS_EMPTY_REQUEST
    assert float(again[100].float().abs().max()) == 0.0
    keep = [i for i in range(n_req) if i != 100]
    assert torch.equal(again[keep], plain[keep])


@pytest.mark.gpu
def test_second_device_of_one_process(cuda):
    """One process driving two GPUs: per-kernel settings (the shared-memory opt-in, the cluster occupancy query) are made
    per device, so the kernels launch on cuda:1 after they have run on cuda:0."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from llm_compileforge_b200 import ops, workloads as wl
    q, k, v, tables, lens = _random_case(77, 5, 32, 8, 128, 200, torch.bfloat16)
    want = ref.paged_attention_f64(q, k, v, tables, lens)
    rids = list(tables)
    x, rw, w, eps = wl.make_norm_matmul_inputs(2100, 264, 2600, torch.bfloat16, seed=3)
    want_nm = ref.fused_rms_norm_matmul(x, rw, w, eps)
    for dev in (torch.device("cuda:0"), torch.device("cuda:1")):
        with torch.cuda.device(dev):
            out = pkg.paged_attention(q.to(dev), k.to(dev), v.to(dev), tables, lens, chunk_tokens=48)
            assert_half_close(stack_outputs(out, rids).cpu(), stack_outputs(want, rids), what=f"decode on {dev}")
            got = ops.fused_rms_norm_matmul(x.to(dev), ops.fold_norm_weight(rw.to(dev), w.to(dev)), eps=eps)
            from helpers import assert_half_close_ulp
            assert_half_close_ulp(got.cpu(), want_nm, what=f"norm-matmul on {dev}")
