"""FP8-e4m3 KV path on the GPU: quantise / dequantise operators, quantise-on-append
through the cache write, and decode over code pools.  Codes and scales are
compared bit for bit with the oracle and the reference-made fixtures."""

import numpy as np
import pytest
import torch

import llm_compileforge_b200 as pkg
from helpers import assert_half_close_ulp, assert_half_close, from_bits, golden, stack_outputs
from llm_compileforge_b200 import ops
from llm_compileforge_b200 import workloads as wl
from llm_compileforge_b200.tables import dense_block_tables
from oracle import reference_port as ref

pytestmark = pytest.mark.gpu


def test_quantize_block_whole_tensor_kat(cuda):
    g = golden("fp8_quantize.npz")
    quant = pkg.FP8KVCacheQuantizer(block_size=16)
    k = torch.from_numpy(g["whole.k"]).to(cuda)
    v = torch.from_numpy(g["whole.v"]).to(cuda)
    k_q, k_s, v_q, v_s = quant.quantize_kv(k, v)
    assert k_q.dtype == torch.float8_e4m3fn and k_s.dim() == 0 and k_s.dtype == torch.float32
    assert np.array_equal(k_q.view(torch.uint8).cpu().numpy(), g["whole.k_codes"])
    assert np.array_equal(v_q.view(torch.uint8).cpu().numpy(), g["whole.v_codes"])
    assert k_s.item() == g["whole.k_scale"].item() and v_s.item() == g["whole.v_scale"].item()
    k_fp, _ = quant.dequantize_kv(k_q, k_s, v_q, v_s)
    assert np.array_equal(k_fp.cpu().numpy(), g["whole.k_deq"])
    # the reference's acceptance lines (tests/test_quantize.py:299-300,311): cos >= 0.99, zero block exact
    assert torch.nn.functional.cosine_similarity(k.flatten(), k_fp.flatten(), dim=0) >= 0.99
    z_q, z_s = quant.quantize_block(torch.zeros(16, 4, 64, device=cuda))
    assert z_s.item() == 1.0 and torch.count_nonzero(quant.dequantize_block(z_q, z_s)) == 0


def test_quantize_pool_per_block_head(cuda):
    g = golden("fp8_quantize.npz")
    pool = from_bits(g["pool.x"], torch.bfloat16).to(cuda)
    codes, scales = pkg.FP8KVCacheQuantizer().quantize_pool(pool)
    assert np.array_equal(codes.view(torch.uint8).cpu().numpy(), g["pool.codes"])
    assert np.array_equal(scales.cpu().numpy(), g["pool.scales"])
    deq = pkg.FP8KVCacheQuantizer().dequantize_pool(codes, scales)
    assert np.array_equal(deq.cpu().numpy(), g["pool.deq"])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_encoder_matches_torch_cast_on_wide_inputs(cuda, dtype):
    """Every bf16 bit pattern (and random float32 / float16 values) through the
    whole-tensor quantiser with the scale pinned to 1 by a 448 sentinel."""
    if dtype == torch.bfloat16:
        bits = np.arange(65536, dtype=np.uint32).astype(np.uint16)
        x = torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)
        x = x[torch.isfinite(x) & (x.abs() <= 448)]
    else:
        gen = torch.Generator().manual_seed(9)
        x = (torch.randn(1 << 20, generator=gen) * torch.exp(torch.randn(1 << 20, generator=gen) * 3)).clamp(-448, 448).to(dtype)
    x = torch.cat([x, torch.tensor([448.0], dtype=dtype)])
    codes, scale = ops.quantize_fp8(x.to(cuda))
    assert scale.item() == 1.0
    want = x.float().to(torch.float8_e4m3fn).view(torch.uint8)
    assert torch.equal(codes.view(torch.uint8).cpu(), want)


def _append_all(cuda, pool_shape, tables, lengths, data_k, data_v, pieces, src_dtype=torch.bfloat16):
    """Drive ops.cache_write over several calls; returns codes, scales."""
    nb, bs, hkv, d = pool_shape
    b = len(lengths)
    kc = torch.zeros(pool_shape, dtype=torch.uint8, device=cuda)
    vc = torch.zeros_like(kc)
    ks = torch.ones((nb, hkv), dtype=torch.float32, device=cuda)
    vs = torch.ones_like(ks)
    kt = torch.zeros((b, bs, hkv, d), dtype=src_dtype, device=cuda)
    vt = torch.zeros_like(kt)
    dense, _, _ = dense_block_tables(tables, {}, bs)
    dense = dense.to(cuda)
    done = [0] * b
    for step in pieces:  # step[r] = tokens request r appends in this call
        ns = [min(step[r], lengths[r] - done[r]) for r in range(b)]
        cu = torch.tensor([0] + list(np.cumsum(ns)), dtype=torch.int32)
        newk = torch.cat([data_k[r][done[r] : done[r] + ns[r]] for r in range(b)]).to(cuda)
        newv = torch.cat([data_v[r][done[r] : done[r] + ns[r]] for r in range(b)]).to(cuda)
        start = torch.tensor(done, dtype=torch.int32)
        if newk.shape[0]:
            ops.cache_write(newk, newv, cu.to(cuda), start.to(cuda), dense, kc, vc, max_new_tokens=max(ns),
                            k_scale=ks, v_scale=vs, k_tail=kt, v_tail=vt)
        done = [done[r] + ns[r] for r in range(b)]
    assert done == list(lengths)
    return kc, vc, ks, vs


def test_quantise_on_append_bit_exact(cuda):
    """Ragged appends (whole prompt, then single tokens, then chunks) leave exactly
    quantize_block(slice) in every touched (block, kv_head) slice."""
    gen = torch.Generator().manual_seed(21)
    hkv, d, bs = 4, 128, 16
    lengths = [53, 16, 1, 130, 37]
    nb = 40
    tables = wl.random_tables(lengths, nb, seed=3)
    data_k = [(torch.randn((n, hkv, d), generator=gen) * 2).to(torch.bfloat16) for n in lengths]
    data_v = [(torch.randn((n, hkv, d), generator=gen) * 2).to(torch.bfloat16) for n in lengths]
    data_k[1][3:9] = 0  # zero rows inside a block
    data_v[2][:] = 0    # an all-zero slice: scale 1.0
    pieces = [[20, 16, 1, 64, 5]] + [[1, 0, 0, 1, 1]] * 14 + [[19, 0, 0, 52, 18]]
    kc, vc, ks, vs = _append_all(cuda, (nb, bs, hkv, d), tables, lengths, data_k, data_v, pieces)
    pool_k = torch.zeros((nb, bs, hkv, d), dtype=torch.bfloat16)
    pool_v = torch.zeros_like(pool_k)
    for r, n in enumerate(lengths):
        ref.cache_write(pool_k, data_k[r], tables[f"req_{r}"], range(n))
        ref.cache_write(pool_v, data_v[r], tables[f"req_{r}"], range(n))
    want_kc, want_ks = ref.fp8_quantize_pool_fast(pool_k)
    want_vc, want_vs = ref.fp8_quantize_pool_fast(pool_v)
    touched = sorted(b for t in tables.values() for b in t)
    assert torch.equal(kc.cpu()[touched], want_kc[touched])
    assert torch.equal(vc.cpu()[touched], want_vc[touched])
    assert torch.equal(ks.cpu()[touched], want_ks[touched])
    assert torch.equal(vs.cpu()[touched], want_vs[touched])
    # the per-slice loop form of the oracle (the reference function called slice by slice) on a few blocks
    for b in touched[:3]:
        c, s = ref.fp8_quantize_pool(pool_k[b : b + 1])
        assert torch.equal(kc.cpu()[b : b + 1], c) and torch.equal(ks.cpu()[b : b + 1], s)


def test_plain_cache_write_slots(cuda):
    """Non-quantised pools: token p lands in (table[p // bs], p % bs), bit-exact."""
    gen = torch.Generator().manual_seed(4)
    hkv, d, bs, nb = 2, 64, 16, 12
    lengths = [21, 40]
    tables = {"a": [7, 2], "b": [9, 0, 4]}
    for dtype in (torch.float32, torch.bfloat16):
        data = [torch.randn((n, hkv, d), generator=gen).to(dtype) for n in lengths]
        pool_k = torch.zeros((nb, bs, hkv, d), dtype=dtype, device=cuda)
        pool_v = torch.zeros_like(pool_k)
        dense, _, _ = dense_block_tables(tables, {}, bs)
        cu = torch.tensor([0, 21, 61], dtype=torch.int32, device=cuda)
        start = torch.zeros(2, dtype=torch.int32, device=cuda)
        new = torch.cat(data).to(cuda)
        ops.cache_write(new, new * 2, cu, start, dense.to(cuda), pool_k, pool_v, max_new_tokens=40)
        want = torch.zeros((nb, bs, hkv, d), dtype=dtype)
        for r, rid in enumerate(tables):
            ref.cache_write(want, data[r], tables[rid], range(lengths[r]))
        assert torch.equal(pool_k.cpu(), want)
        assert torch.equal(pool_v.cpu(), want * 2)


@pytest.mark.parametrize("chunk", [0, 64])
def test_fp8_decode_small_vs_reference(cuda, chunk):
    g = golden("fp8_decode_c3_small.npz")
    w = wl.make_decode_workload(wl.C3, batch=4, max_len=300)
    kc, ks = ops.quantize_fp8(w.k_cache.to(cuda), per_block_head=True)
    vc, vs = ops.quantize_fp8(w.v_cache.to(cuda), per_block_head=True)
    assert np.array_equal(ks.cpu().numpy(), g["k_scales"]) and np.array_equal(vs.cpu().numpy(), g["v_scales"])
    assert int(kc.view(torch.uint8).long().sum()) == int(g["k_codes_sum"])
    out = pkg.paged_attention(w.q.to(cuda), kc, vc, w.block_tables, w.seq_lens, scale=w.scale,
                              k_scale=ks, v_scale=vs, chunk_tokens=chunk)
    got = stack_outputs(out, list(w.block_tables)).cpu()
    assert got.dtype == torch.bfloat16
    assert_half_close(got, torch.from_numpy(g["out"]), what="fp8 decode small")


def test_fp8_config3_sampled(cuda):
    """Config 3 at full batch on the GPU (append whole sequences, then decode);
    the oracle checks a seeded sample of requests."""
    shape = wl.C3
    lengths = wl.config_lengths(shape)
    nb = wl.pool_blocks_for(shape, lengths)
    tables = wl.random_tables(lengths, nb, 1005 + shape.index)
    hkv, d, bs = shape.n_kv_heads, shape.head_dim, shape.block_size
    b = len(lengths)
    gen = torch.Generator(device=cuda).manual_seed(77)
    total = sum(lengths)
    newk = (torch.randn((total, hkv, d), generator=gen, device=cuda) * 2).to(torch.bfloat16)
    newv = (torch.randn((total, hkv, d), generator=gen, device=cuda) * 2).to(torch.bfloat16)
    q = torch.randn((b, shape.n_heads, d), generator=gen, device=cuda).to(torch.bfloat16)
    kc = torch.zeros((nb, bs, hkv, d), dtype=torch.uint8, device=cuda)
    vc = torch.zeros_like(kc)
    ks = torch.ones((nb, hkv), dtype=torch.float32, device=cuda)
    vs = torch.ones_like(ks)
    kt = torch.zeros((b, bs, hkv, d), dtype=torch.bfloat16, device=cuda)
    vt = torch.zeros_like(kt)
    dense, lens, rids = dense_block_tables(tables, {r: n for r, n in zip(tables, lengths)}, bs)
    cu = torch.tensor([0] + list(np.cumsum(lengths)), dtype=torch.int32, device=cuda)
    ops.cache_write(newk, newv, cu, torch.zeros(b, dtype=torch.int32, device=cuda), dense.to(cuda), kc, vc,
                    max_new_tokens=max(lengths), k_scale=ks, v_scale=vs, k_tail=kt, v_tail=vt)
    out = ops.paged_attention_decode(q, kc, vc, dense.to(cuda), lens.to(cuda), k_scale=ks, v_scale=vs)
    pick = torch.randperm(b, generator=torch.Generator().manual_seed(5))[:5].tolist()
    cu_h = cu.cpu().tolist()
    for r in pick:
        n = lengths[r]
        table = tables[rids[r]]
        pool_k = torch.zeros((len(table), bs, hkv, d), dtype=torch.bfloat16)
        pool_v = torch.zeros_like(pool_k)
        local = list(range(len(table)))
        ref.cache_write(pool_k, newk[cu_h[r] : cu_h[r + 1]].cpu(), local, range(n))
        ref.cache_write(pool_v, newv[cu_h[r] : cu_h[r + 1]].cpu(), local, range(n))
        wkc, wks = ref.fp8_quantize_pool_fast(pool_k)
        wvc, wvs = ref.fp8_quantize_pool_fast(pool_v)
        ids = torch.as_tensor(table)
        assert torch.equal(kc.cpu()[ids], wkc) and torch.equal(ks.cpu()[ids], wks)
        assert torch.equal(vc.cpu()[ids], wvc) and torch.equal(vs.cpu()[ids], wvs)
        want = ref.paged_attention(q[r : r + 1].float().cpu(), ref.fp8_dequantize_pool(wkc, wks),
                                   ref.fp8_dequantize_pool(wvc, wvs), {"x": local}, {"x": n})
        assert_half_close(out[r].cpu(), want["x"], what=f"config 3 request {r}")


def test_fp8_config5_full_sampled(cuda):
    """Config 5 at full size on one GPU (2048 requests, ~11 M tokens, 22.7 GB of codes): whole sequences appended
    group by group through quantise-on-append, one decode over everything; the oracle checks a seeded sample of
    requests (codes and scales bit for bit, attention output within the half-precision tolerance), and two
    size-independent properties hold for ALL requests: the output is finite, and it is a convex combination of
    the request's dequantised V rows, so it lies inside their per-dimension [min, max] envelope (checked on the sample)."""
    shape = wl.C5
    lengths = wl.config_lengths(shape)
    nb = wl.pool_blocks_for(shape, lengths)
    tables = wl.random_tables(lengths, nb, 1005 + shape.index)
    hkv, d, bs = shape.n_kv_heads, shape.head_dim, shape.block_size
    b = len(lengths)
    rids = list(tables)
    dense, lens, _ = dense_block_tables(tables, {r: n for r, n in zip(rids, lengths)}, bs)
    dense_d = dense.to(cuda)
    kc = torch.zeros((nb, bs, hkv, d), dtype=torch.uint8, device=cuda)
    vc = torch.zeros_like(kc)
    ks = torch.ones((nb, hkv), dtype=torch.float32, device=cuda)
    vs = torch.ones_like(ks)
    kt = torch.zeros((b, bs, hkv, d), dtype=torch.bfloat16, device=cuda)
    vt = torch.zeros_like(kt)
    pick = sorted(torch.randperm(b, generator=torch.Generator().manual_seed(5))[:4].tolist())
    kept = {}
    group = 128
    for lo in range(0, b, group):
        ls = lengths[lo : lo + group]
        gen = torch.Generator(device=cuda).manual_seed(500 + lo)
        total = sum(ls)
        newk = (torch.randn((total, hkv, d), generator=gen, device=cuda) * 2).to(torch.bfloat16)
        newv = (torch.randn((total, hkv, d), generator=gen, device=cuda) * 2).to(torch.bfloat16)
        cu = [0] + list(np.cumsum(ls))
        ops.cache_write(newk, newv, torch.tensor(cu, dtype=torch.int32, device=cuda), torch.zeros(len(ls), dtype=torch.int32, device=cuda),
                        dense_d[lo : lo + len(ls)], kc, vc, max_new_tokens=max(ls), k_scale=ks, v_scale=vs,
                        k_tail=kt[lo : lo + len(ls)], v_tail=vt[lo : lo + len(ls)])
        for r in pick:
            if lo <= r < lo + len(ls):
                kept[r] = (newk[cu[r - lo] : cu[r - lo + 1]].cpu(), newv[cu[r - lo] : cu[r - lo + 1]].cpu())
        del newk, newv
    q = torch.randn((b, shape.n_heads, d), generator=torch.Generator(device=cuda).manual_seed(9), device=cuda).to(torch.bfloat16)
    out = ops.paged_attention_decode(q, kc, vc, dense_d, lens.to(cuda), k_scale=ks, v_scale=vs)
    assert torch.isfinite(out).all()
    for r in pick:
        n = lengths[r]
        table = tables[rids[r]]
        local = list(range(len(table)))
        pool_k = torch.zeros((len(table), bs, hkv, d), dtype=torch.bfloat16)
        pool_v = torch.zeros_like(pool_k)
        ref.cache_write(pool_k, kept[r][0], local, range(n))
        ref.cache_write(pool_v, kept[r][1], local, range(n))
        wkc, wks = ref.fp8_quantize_pool_fast(pool_k)
        wvc, wvs = ref.fp8_quantize_pool_fast(pool_v)
        ids = torch.as_tensor(table, device=cuda)
        assert torch.equal(kc[ids].cpu(), wkc) and torch.equal(ks[ids].cpu(), wks)
        assert torch.equal(vc[ids].cpu(), wvc) and torch.equal(vs[ids].cpu(), wvs)
        v_deq = ref.fp8_dequantize_pool(wvc, wvs)
        want = ref.paged_attention(q[r : r + 1].float().cpu(), ref.fp8_dequantize_pool(wkc, wks), v_deq, {"x": local}, {"x": n})
        assert_half_close(out[r].cpu(), want["x"], what=f"config 5 request {r} (length {n})")
        rows = v_deq.flatten(0, 1)[:n]  # [n, Hkv, D]
        lo_env = rows.amin(0).repeat_interleave(shape.n_heads // hkv, 0) - 2e-2
        hi_env = rows.amax(0).repeat_interleave(shape.n_heads // hkv, 0) + 2e-2
        got = out[r].float().cpu()
        assert bool(((got >= lo_env) & (got <= hi_env)).all()), "attention output outside the convex hull of V"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_append_division_is_exact_over_many_scales(cuda, dtype):
    """The append kernel divides through a reciprocal plus one FMA correction; the codes
    must equal torch's true division on a few million values spread over many block
    scales (tiny, huge, powers of two, all-ones mantissas)."""
    gen = torch.Generator().manual_seed(123)
    nb, hkv, d, bs = 1500, 2, 128, 16
    x = torch.randn((nb, bs, hkv, d), generator=gen)
    gain = torch.exp2(torch.randint(-24 if dtype != torch.float16 else -10, 24 if dtype != torch.float16 else 10, (nb, 1, hkv, 1), generator=gen).float())
    gain = gain * (1 + torch.rand((nb, 1, hkv, 1), generator=gen))
    x = (x * gain).to(dtype)
    x[5, :, 0] = 0
    x[6, :, 1, :] = torch.tensor(448.0).to(dtype)                       # scale exactly 1
    x[7, 0, 0, 0] = torch.tensor(float.fromhex("0x1.fffffep+3")).to(dtype)  # all-ones mantissa amax (fp32 source)
    tables = {"r": list(range(nb))}
    dense, _, _ = dense_block_tables(tables, {}, bs)
    kc = torch.zeros((nb, bs, hkv, d), dtype=torch.uint8, device=cuda)
    vc = torch.zeros_like(kc)
    ks = torch.ones((nb, hkv), dtype=torch.float32, device=cuda)
    vs = torch.ones_like(ks)
    kt = torch.zeros((1, bs, hkv, d), dtype=dtype, device=cuda)
    vt = torch.zeros_like(kt)
    new = x.reshape(nb * bs, hkv, d).to(cuda)
    cu = torch.tensor([0, nb * bs], dtype=torch.int32, device=cuda)
    ops.cache_write(new, new.flip(0).contiguous(), cu, torch.zeros(1, dtype=torch.int32, device=cuda), dense.to(cuda), kc, vc,
                    max_new_tokens=nb * bs, k_scale=ks, v_scale=vs, k_tail=kt, v_tail=vt)
    want_c, want_s = ref.fp8_quantize_pool_fast(x)
    assert torch.equal(ks.cpu(), want_s)
    assert torch.equal(kc.cpu(), want_c)
    want_c, want_s = ref.fp8_quantize_pool_fast(x.reshape(nb * bs, hkv, d).flip(0).reshape(nb, bs, hkv, d))
    assert torch.equal(vc.cpu(), want_c) and torch.equal(vs.cpu(), want_s)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_chunked_prefill_over_fp8_pool(cuda, dtype):
    """Chunks that attend to an e4m3 pool (earlier chunks of the prompt are already quantised): against the oracle's
    attention over the dequantised pool; three requests share a prefix, ragged chunk and context sizes, a strided
    (layer-sliced) pool and scale layout; the tcgen05 route (D 128) and the decode route (D 64)."""
    for d, h, hkv in ((128, 8, 2), (64, 4, 4)):
        g = torch.Generator().manual_seed(31 + d)
        nb, bs, layers = 40, 16, 2
        shared = [3, 17, 9]
        tables = {"a": shared + [1, 2, 30], "b": shared + [7, 8], "c": shared + [11]}
        ctx = {"a": 90, "b": 70, "c": 50}
        chunk = {"a": 40, "b": 70 - 48, "c": 1}
        src_k = (torch.randn((nb, bs, hkv, d), generator=g) * 2).to(dtype)
        src_v = (torch.randn((nb, bs, hkv, d), generator=g) * 2).to(dtype)
        kc, ks = ref.fp8_quantize_pool_fast(src_k)
        vc, vs = ref.fp8_quantize_pool_fast(src_v)
        k_deq, v_deq = ref.fp8_dequantize_pool(kc, ks), ref.fp8_dequantize_pool(vc, vs)
        # layer-sliced device layout: [NB, layers, bs, Hkv, D] codes and [NB, layers, Hkv] scales, layer 1 is ours
        slab_k = torch.zeros((nb, layers, bs, hkv, d), dtype=torch.uint8, device=cuda)
        slab_v = torch.zeros_like(slab_k)
        sc_k = torch.ones((nb, layers, hkv), dtype=torch.float32, device=cuda)
        sc_v = torch.ones_like(sc_k)
        slab_k[:, 1], slab_v[:, 1] = kc.to(cuda), vc.to(cuda)
        sc_k[:, 1], sc_v[:, 1] = ks.to(cuda), vs.to(cuda)
        q_of = {rid: torch.randn((chunk[rid], h, d), generator=g).to(dtype) for rid in tables}
        # the blocks a request shares with the FIRST request of the batch are expanded once: a long and a short first request
        # must give every request the same bytes
        first = None
        for order in (("a", "b", "c"), ("c", "b", "a")):
            tb = {r: tables[r] for r in order}
            q = torch.cat([q_of[r] for r in order])
            out = pkg.chunked_prefill(q.to(cuda), slab_k[:, 1], slab_v[:, 1], tb, ctx, chunk, k_scale=sc_k[:, 1], v_scale=sc_v[:, 1])
            if first is None:
                first = {r: out[r].clone() for r in order}
                for rid in order:
                    want = ref.chunked_prefill(q_of[rid].float(), k_deq, v_deq, tables[rid], ctx[rid])
                    assert_half_close_ulp(out[rid].cpu(), want.to(dtype), what=f"fp8 prefill {rid} D {d} {dtype}")
            else:
                for rid in order:
                    assert torch.equal(out[rid], first[rid]), f"request {rid} differs when the batch is reordered (D {d})"
