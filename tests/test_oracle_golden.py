"""The CPU oracle against the fixtures produced by the reference's own modules
(tests/golden/make_golden.py).  No GPU, no reference checkout needed."""

import math

import numpy as np
import pytest
import torch

from helpers import assert_f32_close, assert_same, from_bits, golden, tables_to_dict
from llm_compileforge_b200 import workloads as wl
from oracle import c_oracle
from oracle import reference_port as ref


def _dense(tables, lens, bs=16):
    rids = list(tables)
    width = max(len(t) for t in tables.values())
    d = np.zeros((len(rids), width), dtype=np.int32)
    ll = np.zeros(len(rids), dtype=np.int32)
    for i, r in enumerate(rids):
        t = tables[r]
        d[i, : len(t)] = t
        ll[i] = min(lens.get(r, len(t) * bs), len(t) * bs)
    return d, ll


@pytest.mark.parametrize("case", ["kat_mha", "kat_gqa", "kat_multi", "edges"])
def test_paged_decode_kats(case):
    g = golden("paged_decode_kats.npz")
    q, k, v = (torch.from_numpy(g[f"{case}.{n}"]) for n in "qkv")
    names = {"kat_mha": ["req_1"], "kat_gqa": ["req_1"], "kat_multi": ["req_1", "req_2"],
             "edges": ["nolen", "toolong", "surplus", "shared", "one"]}[case]
    tables, lens = tables_to_dict(g[f"{case}.tables"], g[f"{case}.table_lens"], g[f"{case}.seq_lens"], names)
    want = torch.from_numpy(g[f"{case}.out"])
    got = ref.paged_attention(q, k, v, tables, lens, block_size=16)
    # same torch CPU operator, same order of operations: bit-identical
    assert_same(torch.stack([got[r] for r in names]), want)
    # the independent C restatement (double accumulation) agrees to float32 rounding
    d, ll = _dense(tables, lens)
    c = c_oracle.paged_decode(q.numpy(), k.numpy(), v.numpy(), d, ll, 1.0 / math.sqrt(q.shape[-1]))
    assert_f32_close(torch.from_numpy(c), want, rel=2e-6, what=case)
    f64 = ref.paged_attention_f64(q, k, v, tables, lens)
    assert_f32_close(torch.stack([f64[r] for r in names]).float(), want, rel=2e-6, what=case + " f64")


def test_paged_decode_empty_request_raises():
    q = torch.zeros(1, 2, 8)
    k = torch.zeros(2, 16, 2, 8)
    with pytest.raises(ValueError):
        ref.paged_attention(q, k, k, {"a": [0]}, {"a": 0})


def test_config1_full():
    g = golden("paged_decode_c1.npz")
    w = wl.make_decode_workload(wl.C1)
    # the seeded generator reproduces the inputs the fixture was made from
    assert np.isclose(w.k_cache.double().sum().item(), float(g["k_sum"]), rtol=0, atol=1e-6)
    assert np.isclose(w.v_cache.double().sum().item(), float(g["v_sum"]), rtol=0, atol=1e-6)
    assert np.array_equal(w.q.numpy(), g["q"])
    assert w.lengths == g["seq_lens"].tolist()
    want = torch.from_numpy(g["out"])
    assert want.shape == (8, 12, 64)
    got = ref.paged_attention(w.q, w.k_cache, w.v_cache, w.block_tables, w.seq_lens, scale=w.scale)
    assert_same(torch.stack(list(got.values())), want)
    d, ll = _dense(w.block_tables, w.seq_lens)
    c = c_oracle.paged_decode(w.q.numpy(), w.k_cache.numpy(), w.v_cache.numpy(), d, ll, w.scale)
    assert_f32_close(torch.from_numpy(c), want, rel=3e-6, what="c1")


def test_config2_small_bf16():
    g = golden("paged_decode_c2_small.npz")
    w = wl.make_decode_workload(wl.C2, batch=6, max_len=400)
    assert np.isclose(w.k_cache.double().sum().item(), float(g["k_sum"]), rtol=0, atol=1e-6)
    want = from_bits(g["out"], torch.bfloat16)
    got = ref.paged_attention(w.q, w.k_cache, w.v_cache, w.block_tables, w.seq_lens, scale=w.scale)
    assert_same(torch.stack(list(got.values())), want)
    d, ll = _dense(w.block_tables, w.seq_lens)
    kb = w.k_cache.view(torch.int16).numpy().view(np.uint16)
    vb = w.v_cache.view(torch.int16).numpy().view(np.uint16)
    c = torch.from_numpy(c_oracle.paged_decode(w.q.float().numpy(), kb, vb, d, ll, w.scale))
    assert (c - want.float()).abs().max() <= 2e-2


def test_fp8_whole_tensor_kat():
    g = golden("fp8_quantize.npz")
    k = torch.from_numpy(g["whole.k"])
    codes, scale = ref.fp8_quantize_block(k)
    assert np.array_equal(codes.view(torch.uint8).numpy(), g["whole.k_codes"])
    assert scale.numpy() == g["whole.k_scale"]
    assert np.array_equal(ref.fp8_dequantize_block(codes, scale).numpy(), g["whole.k_deq"])
    # plain-C codec reproduces the codes from the same quotient
    q = (k / scale).numpy()
    assert np.array_equal(c_oracle.e4m3_encode(q), g["whole.k_codes"])
    assert np.array_equal(c_oracle.e4m3_decode(g["whole.k_codes"]) * g["whole.k_scale"], g["whole.k_deq"])


def test_fp8_pool_per_block_head():
    g = golden("fp8_quantize.npz")
    pool = from_bits(g["pool.x"], torch.bfloat16)
    codes, scales = ref.fp8_quantize_pool(pool)
    assert np.array_equal(codes.numpy(), g["pool.codes"])
    assert np.array_equal(scales.numpy(), g["pool.scales"])
    codes2, scales2 = ref.fp8_quantize_pool_fast(pool)
    assert torch.equal(codes2, codes) and torch.equal(scales2, scales)
    assert np.array_equal(ref.fp8_dequantize_pool(codes, scales).numpy(), g["pool.deq"])
    c_codes, c_scales = c_oracle.quantize_pool(pool.float().numpy())
    assert np.array_equal(c_codes, g["pool.codes"])
    assert np.array_equal(c_scales, g["pool.scales"])
    # the reference's edge rules: zero block -> scale 1, codes 0; tiny block -> scale clamp
    assert g["pool.scales"][1].tolist() == [1.0, 1.0] and not g["pool.codes"][1].any()
    assert g["pool.scales"][3, 0] == np.float32(1e-12)


def test_e4m3_codec_exhaustive_bf16_inputs():
    bits = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    x = torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16).float()
    want = x.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(c_oracle.e4m3_encode(x.numpy()), want)
    all_codes = np.arange(256, dtype=np.uint8)
    want_dec = torch.from_numpy(all_codes).view(torch.float8_e4m3fn).float().numpy()
    assert np.array_equal(c_oracle.e4m3_decode(all_codes), want_dec, equal_nan=True)


def test_fp8_decode_small():
    g = golden("fp8_decode_c3_small.npz")
    w = wl.make_decode_workload(wl.C3, batch=4, max_len=300)
    kc, ks = ref.fp8_quantize_pool_fast(w.k_cache)
    vc, vs = ref.fp8_quantize_pool_fast(w.v_cache)
    assert int(kc.long().sum()) == int(g["k_codes_sum"]) and int(vc.long().sum()) == int(g["v_codes_sum"])
    assert np.array_equal(ks.numpy(), g["k_scales"]) and np.array_equal(vs.numpy(), g["v_scales"])
    kd, vd = ref.fp8_dequantize_pool(kc, ks), ref.fp8_dequantize_pool(vc, vs)
    got = ref.paged_attention(w.q.float(), kd, vd, w.block_tables, w.seq_lens, scale=w.scale)
    want = torch.from_numpy(g["out"])
    assert_same(torch.stack(list(got.values())), want)
    d, ll = _dense(w.block_tables, w.seq_lens)
    c = c_oracle.paged_decode(w.q.float().numpy(), kc.numpy(), vc.numpy(), d, ll, w.scale, ks.numpy(), vs.numpy())
    assert_f32_close(torch.from_numpy(c), want, rel=3e-6, what="fp8 decode")


def test_kv_append_matches_bulk_quantisation():
    """Appending a request in ragged pieces leaves the same codes and scales as
    quantising the finished pool in one go."""
    g = torch.Generator().manual_seed(5)
    n, hkv, d = 53, 2, 32
    table = [4, 1, 6, 2]
    data = (torch.randn((n, hkv, d), generator=g) * 2).to(torch.bfloat16)
    pool = torch.zeros((8, 16, hkv, d), dtype=torch.bfloat16)
    ref.cache_write(pool, data, table, range(n))
    want_codes, want_scales = ref.fp8_quantize_pool(pool)
    codes = torch.zeros((8, 16, hkv, d), dtype=torch.uint8)
    scales = torch.ones((8, hkv), dtype=torch.float32)
    tail = torch.zeros((16, hkv, d), dtype=torch.bfloat16)
    at = 0
    for piece in (5, 1, 1, 20, 10, 16):
        ref.kv_append_fp8(codes, scales, tail, data[at : at + piece], table, at)
        at += piece
    assert at == n
    touched = table
    assert torch.equal(codes[touched], want_codes[touched])
    assert torch.equal(scales[touched], want_scales[touched])


def test_rms_norm():
    g = golden("rms_norm.npz")
    x, w, eps = wl.make_rms_norm_inputs(rows=8, hidden=4096)
    assert torch.equal(ref.rms_norm_hal(x, w, eps), from_bits(g["hal_bf16.out"], torch.bfloat16))
    xf, wf = torch.from_numpy(g["hal_f32.x"]), torch.from_numpy(g["hal_f32.w"])
    assert torch.equal(ref.rms_norm_hal(xf, wf, 1e-5), torch.from_numpy(g["hal_f32.out"]))
    assert torch.equal(ref.rms_norm_hal(xf, None, 1e-5), torch.from_numpy(g["hal_f32_noweight.out"]))
    c = c_oracle.rms_norm(xf.numpy(), wf.numpy(), 1e-5)
    assert_f32_close(torch.from_numpy(c), torch.from_numpy(g["hal_f32.out"]), rel=2e-6)
    x, r, wg = (torch.from_numpy(g[f"fused_f32.{n}"]) for n in "xrw")
    assert torch.equal(ref.fused_rms_norm_add(x, r, wg, 1e-6), torch.from_numpy(g["fused_f32.out"]))
    assert torch.equal(ref.fused_rms_norm_add(x.bfloat16(), r.bfloat16(), wg.bfloat16(), 1e-6),
                       from_bits(g["fused_bf16.out"], torch.bfloat16))
    c = c_oracle.rms_norm(x.numpy(), wg.numpy(), 1e-6, residual=r.numpy())
    assert_f32_close(torch.from_numpy(c), torch.from_numpy(g["fused_f32.out"]), rel=2e-6)
    # the reference's cross-language precision case (tests/contract/fixtures/generate.py:49-76):
    # expected values computed without eps, tolerance 1e-4
    xs = torch.from_numpy(g["contract_2x4.x"])
    want = xs / torch.sqrt((xs * xs).mean(-1, keepdim=True))
    assert (torch.from_numpy(g["contract_2x4.out"]) - want).abs().max() < 1e-4
    assert (ref.rms_norm_hal(xs, torch.ones(4), 1e-5) - want).abs().max() < 1e-4


def test_flash_and_chunked_prefill():
    g = golden("prefill.npz")
    q, k, v = (torch.from_numpy(g[f"flash_kat.{n}"]) for n in "qkv")
    assert torch.equal(ref.flash_attention_fwd(q, k, v, causal=True), torch.from_numpy(g["flash_kat.out"]))
    assert torch.equal(ref.flash_attention_fwd(q, k, v, causal=False), torch.from_numpy(g["flash_kat.out_noncausal"]))
    pw = wl.make_prefill_workload(n_requests=3, prefix_len=64, chunk_len=48, n_heads=8, n_kv_heads=2, head_dim=128)
    assert np.isclose(pw.k_cache.double().sum().item(), float(g["prefill_small.k_sum"]), atol=1e-6)
    assert np.isclose(pw.q.double().sum().item(), float(g["prefill_small.q_sum"]), atol=1e-6)
    want = from_bits(g["prefill_small.out"], torch.bfloat16)
    for i, (rid, table) in enumerate(pw.block_tables.items()):
        got = ref.chunked_prefill(pw.q[i * 48 : (i + 1) * 48], pw.k_cache, pw.v_cache, table, pw.ctx_lens[rid], scale=pw.scale)
        assert_same(got, want[i])
        c = c_oracle.chunk_prefill(pw.q[i * 48 : (i + 1) * 48].float().numpy(), pw.k_cache.float().numpy(),
                                   pw.v_cache.float().numpy(), np.array(table, dtype=np.int32), pw.ctx_lens[rid], pw.scale)
        assert (torch.from_numpy(c) - want[i].float()).abs().max() <= 2e-2
    # all requests share the prefix blocks: identical ids at the head of every table
    heads = [t[:4] for t in pw.block_tables.values()]
    assert heads[0] == heads[1] == heads[2]


@pytest.mark.parametrize("case", wl.SDPA_MASK_CASES)
def test_hal_sdpa_mask_conventions(case):
    """The restated backend operator against the reference backend's own outputs (tests/golden/sdpa_masks.npz)."""
    inputs, kw = wl.make_sdpa_mask_case(case)
    got = ref.hal_scaled_dot_product_attention(inputs, **kw)
    want = from_bits(golden("sdpa_masks.npz")[case], got.dtype)
    assert_same(got, want.view(got.shape))


def test_positional_mask_is_a_prefix_per_row():
    """What the GPU path relies on: for positions that do not decrease, ``pos[i] >= pos[j]`` selects the first
    ``#{j: pos[j] <= pos[i]}`` keys of the row."""
    inputs, kw = wl.make_sdpa_mask_case("ties_f32")
    q, k, v, mask = inputs
    pos = mask[0, 0, :, 0]
    limits = torch.searchsorted(pos.contiguous(), pos.contiguous(), right=True)
    rows = []
    for i in range(q.shape[2]):
        n = int(limits[i])
        rows.append(torch.nn.functional.scaled_dot_product_attention(q[:, :, i : i + 1], k[:, :, :n], v[:, :, :n], scale=kw["scale"]))
    assert_f32_close(torch.cat(rows, dim=2), ref.hal_scaled_dot_product_attention(inputs, **kw), rel=2e-6)


def test_rust_attention_forward_known_answers():
    """runtime/src/engine/kernels.rs:345-419: the Rust file's own two unit tests, restated."""
    # attention_decode_is_unmasked_dot_product: one head, dim 2, two keys
    q = torch.tensor([[[1.0, 2.0]]])
    k = torch.tensor([[[3.0, 0.0], [0.0, 4.0]]])
    v = torch.tensor([[[5.0, 0.0], [0.0, 6.0]]])
    ctx, _ = ref.attention_forward(q, k, v, is_decode=True)
    e5 = math.exp(-5.0)
    assert abs(ctx[0, 0].item() - e5 / (e5 + 1.0) * 5.0) < 1e-5 and abs(ctx[0, 1].item() - 1.0 / (e5 + 1.0) * 6.0) < 1e-5
    # attention_prefill_applies_causal_mask: seq 2, kv_len 2, dim 1
    q = torch.tensor([[[1.0], [1.0]]])
    k = torch.tensor([[[1.0], [1.0]]])
    v = torch.tensor([[[10.0], [20.0]]])
    ctx, probs = ref.attention_forward(q, k, v, is_decode=False)
    assert probs[0, 0, 0].item() == 1.0 and probs[0, 0, 1].item() == 0.0
    assert abs(probs[0, 1, 0].item() - probs[0, 1, 1].item()) < 1e-6
    assert ctx[0, 0].item() == 10.0 and abs(ctx[1, 0].item() - 15.0) < 1e-6


def test_read_paged_restates_the_sorted_request_order():
    """cache_manager.py:173-197: rows follow the SORTED request ids, whole blocks are copied up to max_seq_len."""
    g = torch.Generator().manual_seed(3)
    slab = torch.randn((6, 2, 4, 1, 2), generator=g)  # [NB, layers, bs, heads, dim]
    tables = {"b": [5, 0], "a": [2]}
    got = ref.read_paged(slab, tables, 6, layer_idx=1)
    assert got.shape == (2, 6, 1, 2)
    assert torch.equal(got[0, :4], slab[2, 1]) and torch.equal(got[0, 4:], torch.zeros(2, 1, 2))
    assert torch.equal(got[1, :4], slab[5, 1]) and torch.equal(got[1, 4:6], slab[0, 1, :2])
