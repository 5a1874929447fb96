"""A serving loop over PagedKVCache (prefill chunks, then decode steps with a changing
batch, two layers, bf16 and FP8 pools) against the reference's protocol replayed on the CPU:
write_paged slot rule + dense attention over the gathered cache."""

import math

import pytest
import torch

from helpers import assert_half_close
from llm_compileforge_b200.cache import PagedKVCache
from oracle import reference_port as ref

pytestmark = pytest.mark.gpu


class _CpuEngineCache:
    """Reference protocol on the CPU: slab [NB, layers, bs, heads, dim], write_paged slots
    (cache_manager.py:153-160), FP8 by quantize_block per (block, kv_head) slice."""

    def __init__(self, nb, layers, hkv, d, fp8):
        self.k = torch.zeros((nb, layers, 16, hkv, d), dtype=torch.bfloat16)
        self.v = torch.zeros_like(self.k)
        self.fp8 = fp8

    def write(self, layer, table, k_new, v_new, start):
        ref.cache_write(self.k[:, layer], k_new, table, range(start, start + k_new.shape[0]))
        ref.cache_write(self.v[:, layer], v_new, table, range(start, start + v_new.shape[0]))

    def pools(self, layer):
        k, v = self.k[:, layer].contiguous(), self.v[:, layer].contiguous()
        if self.fp8:
            kc, ks = ref.fp8_quantize_pool_fast(k)
            vc, vs = ref.fp8_quantize_pool_fast(v)
            return ref.fp8_dequantize_pool(kc, ks), ref.fp8_dequantize_pool(vc, vs)
        return k, v


@pytest.mark.parametrize("fp8", [False, True])
def test_serving_loop_matches_reference_protocol(cuda, fp8):
    g = torch.Generator().manual_seed(17 + fp8)
    layers, h, hkv, d, nb = 2, 8, 2, 128, 64
    cache = PagedKVCache(nb, layers, hkv, d, dtype=torch.bfloat16, fp8=fp8, max_requests=8, device=cuda)
    cpu = _CpuEngineCache(nb, layers, hkv, d, fp8)
    perm = torch.randperm(nb, generator=g).tolist()
    tables = {"a": perm[0:6], "b": perm[6:10], "c": perm[10:20]}  # capacity 96 / 64 / 160 tokens
    prompt = {"a": 37, "b": 16, "c": 70}
    length = {r: 0 for r in tables}
    gain = 2.0 if fp8 else 1.0

    def new_kv(n):
        return ((torch.randn((n, hkv, d), generator=g) * gain).to(torch.bfloat16), (torch.randn((n, hkv, d), generator=g) * gain).to(torch.bfloat16))

    # ---- prefill: request "c" in two chunks (chunked prefill), "a" and "b" in one
    for step_reqs in ([("a", 37), ("b", 16), ("c", 48)], [("c", 22)]):
        rids = [r for r, _ in step_reqs]
        cache.begin_step({r: tables[r] for r in rids})
        for layer in range(layers):
            ks, vs = zip(*[new_kv(n) for _, n in step_reqs])
            for (r, n), k_new, v_new in zip(step_reqs, ks, vs):
                cpu.write(layer, tables[r], k_new, v_new, length[r])
            cache.write(layer, torch.cat(ks).to(cuda), torch.cat(vs).to(cuda), [n for _, n in step_reqs], [length[r] for r in rids])
            # chunk attention over prefix + chunk, straight off the pool (an FP8 pool: over the quantised earlier chunk too)
            q = torch.randn((sum(n for _, n in step_reqs), h, d), generator=g).to(torch.bfloat16)
            out = cache.prefill(layer, q.to(cuda), [n for _, n in step_reqs], [length[r] + n for r, n in step_reqs]).cpu()
            kp, vp = cpu.pools(layer)
            at = 0
            for r, n in step_reqs:
                if fp8:
                    want = ref.chunked_prefill(q[at : at + n].float(), kp, vp, tables[r], length[r] + n).to(torch.bfloat16)
                    # V (code * scale) and P are each rounded to bf16 before the tensor-core product and the result once
                    # more: three roundings of 2^-9 on values as large as the context's largest V entry
                    tol = 2e-2 + 3 * 2.0 ** -9 * vp.abs().max().item()
                    err = (out[at : at + n].float() - want.float()).abs().max().item()
                    assert err <= tol, f"prefill {r} layer {layer}: {err:.3e} > {tol:.3e}"
                else:
                    want = ref.chunked_prefill(q[at : at + n], kp, vp, tables[r], length[r] + n)
                    assert_half_close(out[at : at + n], want, what=f"prefill {r} layer {layer}")
                at += n
        for r, n in step_reqs:
            length[r] += n
    assert length == prompt

    # ---- decode: batch composition and order change between steps; "b" finishes early
    schedule = [["a", "b", "c"], ["c", "a", "b"], ["b", "c"], ["c", "a"], ["a", "c"]] + [["a", "c"]] * 12
    for step, rids in enumerate(schedule):
        if step == 3:
            cache.release("b")
        cache.begin_step({r: tables[r] for r in rids})
        for layer in range(layers):
            k_new, v_new = new_kv(len(rids))
            for i, r in enumerate(rids):
                cpu.write(layer, tables[r], k_new[i : i + 1], v_new[i : i + 1], length[r])
            cache.write(layer, k_new.to(cuda), v_new.to(cuda), [1] * len(rids), [length[r] for r in rids])
            q = torch.randn((len(rids), h, d), generator=g).to(torch.bfloat16)
            lens = [length[r] + 1 for r in rids]
            out = cache.attend(layer, q.to(cuda), lens).cpu()
            kp, vp = cpu.pools(layer)
            want = ref.paged_attention(q.float(), kp.float(), vp.float(), {r: tables[r] for r in rids}, dict(zip(rids, lens)))
            assert_half_close(out, torch.stack([want[r] for r in rids]), what=f"decode step {step} layer {layer}")
            # the debugging gather agrees with the reference's read_paged view of the same cache
            kd, _ = cache.read_dense(layer, rids[0], lens[0])
            want_k = kp[torch.as_tensor(tables[rids[0]])].flatten(0, 1)[: lens[0]].float()
            assert torch.equal(kd.cpu(), want_k)
        for r in rids:
            length[r] += 1
