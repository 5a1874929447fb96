"""Dense attention (HAL scaled_dot_product_attention with the reference backend's mask conventions, the Rust runtime's
attention_forward), per-row visible lengths of the prefill kernels, and cache_read - all through the C ABI."""

import pytest
import torch

from helpers import assert_f32_close, assert_half_close, from_bits, golden
from llm_compileforge_b200 import B200Backend, _lib, ops
from llm_compileforge_b200 import workloads as wl
from oracle import reference_port as ref

pytestmark = pytest.mark.gpu


def _close(got, want, what):
    if want.dtype == torch.float32:
        assert_f32_close(got.float().cpu(), want, what=what)
    else:
        assert_half_close(got.float().cpu(), want.float(), what=what)


@pytest.mark.parametrize("case", wl.SDPA_MASK_CASES)
def test_hal_sdpa_mask_conventions_run_natively(cuda, case):
    """Every mask convention of pytorch_backend/_ops_attention.py:13-53 is served WITHOUT a fallback executor and
    matches the reference backend's own output (tests/golden/sdpa_masks.npz) and the restated operator."""
    inputs, kw = wl.make_sdpa_mask_case(case)
    want = ref.hal_scaled_dot_product_attention(inputs, **kw)
    fixture = from_bits(golden("sdpa_masks.npz")[case], want.dtype).view(want.shape)
    got = B200Backend(fallback=None).execute("scaled_dot_product_attention", [t.to(cuda) for t in inputs], **kw)
    assert got.shape == want.shape and got.dtype == want.dtype
    _close(got, want, case)
    _close(got, fixture, case + " (reference fixture)")


def test_decreasing_positions_are_reported_not_guessed(cuda):
    inputs, kw = wl.make_sdpa_mask_case("ties_f32")
    inputs[3] = inputs[3].flip(2).contiguous()  # positions now fall along the sequence: no prefix per row
    dev = [t.to(cuda) for t in inputs]
    with pytest.raises(ValueError, match="fallback"):
        B200Backend(fallback=None).execute("scaled_dot_product_attention", dev, **kw)
    _, ws = ops.attention_dense(dev[0], dev[1], dev[2], mask="positions", positions=dev[3][:, 0, :, 0], return_workspace=True)
    assert ops.read_status(ws) & _lib.SFB_STATUS_UNSORTED_POSITIONS

    class Fallback:  # stands in for PyTorchBackend("cuda"): the call is handed on unchanged
        def execute(self, name, ins, **k):
            return ref.hal_scaled_dot_product_attention([t.cpu() for t in ins], **k).to(ins[0].device)

    got = B200Backend(fallback=Fallback()).execute("scaled_dot_product_attention", dev, **kw)
    assert_f32_close(got.cpu(), ref.hal_scaled_dot_product_attention(inputs, **kw))


@pytest.mark.parametrize("dtype,h,hkv,sq,skv,d,mask", [
    (torch.bfloat16, 4, 2, 300, 300, 128, "causal"),          # tcgen05 route, GQA, ragged tiles
    (torch.bfloat16, 2, 2, 70, 333, 128, "causal_bottom_right"),
    (torch.float16, 2, 1, 129, 40, 128, "none"),
    (torch.float32, 3, 3, 50, 50, 64, "causal"),              # decode route
    (torch.float32, 2, 1, 9, 100, 32, "causal_bottom_right"),
])
def test_attention_dense_masks(cuda, dtype, h, hkv, sq, skv, d, mask):
    g = torch.Generator().manual_seed(sq * 7 + skv)
    b = 2
    q = torch.randn((b, h, sq, d), generator=g).to(dtype)
    k = torch.randn((b, hkv, skv, d), generator=g).to(dtype)
    v = torch.randn((b, hkv, skv, d), generator=g).to(dtype)
    i, j = torch.arange(sq).view(sq, 1), torch.arange(skv).view(1, skv)
    visible = {"none": torch.ones(sq, skv, dtype=torch.bool), "causal": j <= i, "causal_bottom_right": j <= i + skv - sq}[mask]
    rep = h // hkv
    want = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float().repeat_interleave(rep, 1), v.float().repeat_interleave(rep, 1),
                                                            attn_mask=visible)
    # strided operands: q and the output as position-major [B,S,H,D] buffers seen through permuted views
    q_pm = q.permute(0, 2, 1, 3).contiguous().to(cuda)
    out_pm = torch.empty_like(q_pm)
    ops.attention_dense(q_pm.permute(0, 2, 1, 3), k.to(cuda), v.to(cuda), mask=mask, out=out_pm.permute(0, 2, 1, 3))
    got = out_pm.permute(0, 2, 1, 3)
    if dtype == torch.float32:
        assert_f32_close(got.cpu(), want, what=mask)
    else:
        assert_half_close(got.float().cpu(), want, what=mask)


def test_rust_attention_forward_operator(cuda):
    """runtime/src/engine/kernels.rs:97-302: head-major fp32, q pre-scaled, position-major result; prefill masks keys
    after the query's own index, decode masks nothing."""
    g = torch.Generator().manual_seed(5)
    h, s, d = 4, 37, 64
    q = torch.randn((h, s, d), generator=g) * 0.125
    k = torch.randn((h, s, d), generator=g)
    v = torch.randn((h, s, d), generator=g)
    be = B200Backend()
    want, _ = ref.attention_forward(q, k, v, is_decode=False)
    got = be.execute("attention_forward", [q.to(cuda), k.to(cuda), v.to(cuda)], is_decode=False)
    assert got.shape == (s, h * d)
    assert_f32_close(got.cpu(), want, what="prefill")
    want1, _ = ref.attention_forward(q[:, :1], k, v, is_decode=True)
    got1 = be.execute("attention_forward", [q[:, :1].contiguous().to(cuda), k.to(cuda), v.to(cuda)], is_decode=True)
    assert_f32_close(got1.cpu(), want1, what="decode")


@pytest.mark.parametrize("dtype,d", [(torch.bfloat16, 128), (torch.float32, 64)])
def test_prefill_row_limits(cuda, dtype, d):
    """Arbitrary visible lengths per query row (not even monotone), both kernel routes; a limit of zero gives a zero row."""
    g = torch.Generator().manual_seed(11)
    h, hkv, nb, bs = 4, 2, 40, 16
    n_q, ctx = [150, 260], [200, 300]
    pool_k = torch.randn((nb, bs, hkv, d), generator=g).to(dtype)
    pool_v = torch.randn((nb, bs, hkv, d), generator=g).to(dtype)
    tables = torch.stack([torch.randperm(nb, generator=g)[:19] for _ in range(2)]).to(torch.int32)
    q = torch.randn((sum(n_q), h, d), generator=g).to(dtype)
    limits = torch.cat([torch.randint(1, ctx[r] + 1, (n_q[r],), generator=g) for r in range(2)]).to(torch.int32)
    limits[3] = 0
    limits[200] = 10_000  # beyond the context: clamped
    cu = torch.tensor([0, n_q[0], sum(n_q)], dtype=torch.int32)
    out = ops.prefill_paged(q.to(cuda), pool_k.to(cuda), pool_v.to(cuda), tables.to(cuda), cu.to(cuda),
                            torch.tensor(ctx, dtype=torch.int32, device=cuda), max_q_tokens=max(n_q), row_limits=limits.to(cuda))
    want = torch.zeros(q.shape, dtype=torch.float32)
    for r in range(2):
        kk = pool_k[tables[r].long()].flatten(0, 1)[: ctx[r]].float().repeat_interleave(h // hkv, 1)
        vv = pool_v[tables[r].long()].flatten(0, 1)[: ctx[r]].float().repeat_interleave(h // hkv, 1)
        for i in range(n_q[r]):
            t = int(cu[r]) + i
            n = min(int(limits[t]), ctx[r])
            if n > 0:
                s = torch.einsum("hd,nhd->hn", q[t].float(), kk[:n]) / d ** 0.5
                want[t] = torch.einsum("hn,nhd->hd", torch.softmax(s, -1), vv[:n])
    if dtype == torch.float32:
        assert_f32_close(out.cpu(), want)
    else:
        assert_half_close(out.float().cpu(), want)
    assert not out[3].any()


@pytest.mark.parametrize("fp8", [False, True])
def test_cache_read_matches_read_paged(cuda, fp8):
    g = torch.Generator().manual_seed(9)
    nb, layers, bs, hkv, d = 24, 3, 16, 2, 64
    slab = torch.randn((nb, layers, bs, hkv, d), generator=g).to(torch.bfloat16)
    tables = {"b": [5, 0, 7], "a": [2], "c": [9, 11]}
    order = sorted(tables)
    dense = torch.zeros((3, 3), dtype=torch.int32)
    for i, r in enumerate(order):
        dense[i, : len(tables[r])] = torch.tensor(tables[r], dtype=torch.int32)
    cap = torch.tensor([len(tables[r]) * bs for r in order], dtype=torch.int32)
    layer = slab[:, 1]
    if not fp8:
        want = ref.read_paged(slab, tables, 40, layer_idx=1)
        got = ops.cache_read(layer.to(cuda), dense.to(cuda), cap.to(cuda), 40)  # a strided layer view, read in place
        assert torch.equal(got.cpu(), want)
        short = ops.cache_read(layer.to(cuda), dense.to(cuda), torch.tensor([5, 33, 0], dtype=torch.int32, device=cuda), 40)
        assert torch.equal(short.cpu()[0, :5], want[0, :5]) and not short.cpu()[0, 5:].any() and not short.cpu()[2].any()
    else:
        codes, scales = ref.fp8_quantize_pool_fast(layer.contiguous())
        deq = ref.fp8_dequantize_pool(codes, scales)
        want = ref.read_paged(deq, tables, 40)
        got = ops.cache_read(codes.view(torch.uint8).to(cuda), dense.to(cuda), cap.to(cuda), 40, scale=scales.to(cuda))
        assert got.dtype == torch.float32 and torch.equal(got.cpu(), want)  # code * scale in fp32: bit-exact
        be = B200Backend()
        key, value = be.execute("cache_read", [dense.to(cuda)], k_cache=codes.view(torch.uint8).to(cuda), v_cache=codes.view(torch.uint8).to(cuda),
                                k_scale=scales.to(cuda), v_scale=scales.to(cuda), max_seq_len=40, seq_lens=cap.to(cuda))
        assert torch.equal(key.cpu(), want) and torch.equal(value.cpu(), want)


def test_nan_in_unwritten_slots_does_not_reach_the_output(cuda):
    """A pool that was never zero-filled: slots past a request's length hold NaN.  Decode and prefill must both ignore
    them (the reference slices K/V to the length before attending, kernels/paged_attention.py:47-48)."""
    g = torch.Generator().manual_seed(13)
    nb, bs, hkv, h, d = 12, 16, 2, 4, 128
    ctx = 37  # ends inside a block
    k = torch.randn((nb, bs, hkv, d), generator=g).to(torch.bfloat16)
    v = torch.randn((nb, bs, hkv, d), generator=g).to(torch.bfloat16)
    table = torch.tensor([[4, 9, 1]], dtype=torch.int32)
    clean_k, clean_v = k.clone(), v.clone()
    k[1, ctx - 32:] = float("nan")
    v[1, ctx - 32:] = float("nan")
    n_q = 20
    q = torch.randn((n_q, h, d), generator=g).to(torch.bfloat16)
    cu = torch.tensor([0, n_q], dtype=torch.int32, device=cuda)
    cl = torch.tensor([ctx], dtype=torch.int32, device=cuda)
    got = ops.prefill_paged(q.to(cuda), k.to(cuda), v.to(cuda), table.to(cuda), cu, cl, max_q_tokens=n_q)
    want = ops.prefill_paged(q.to(cuda), clean_k.to(cuda), clean_v.to(cuda), table.to(cuda), cu, cl, max_q_tokens=n_q)
    assert not torch.isnan(got.float()).any() and torch.equal(got, want)
    dq = q[-1:].contiguous()
    got_d = ops.paged_attention_decode(dq.to(cuda), k.to(cuda), v.to(cuda), table.to(cuda), cl)
    want_d = ops.paged_attention_decode(dq.to(cuda), clean_k.to(cuda), clean_v.to(cuda), table.to(cuda), cl)
    assert not torch.isnan(got_d.float()).any() and torch.equal(got_d, want_d)
    assert_half_close(got[-1:].float().cpu(), want_d.float().cpu(), what="last prefill row = decode row")
