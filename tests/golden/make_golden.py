"""Generate tests/golden/*.npz by running the REFERENCE's own Python modules.

Usage (only where the reference checkout is available):

    python tests/golden/make_golden.py /path/to/LLM-CompileForge [--only-norm-matmul]

The reference's functions are imported from that checkout (never copied) and
run on seeded inputs; inputs and outputs are saved as small ``.npz`` fixtures.
The fixtures travel with the repository; the checkout does not, and no test
reads it at run time.  bfloat16 tensors are stored as uint16 bit patterns and
float8 codes as uint8.
"""

from __future__ import annotations

import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))


def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.float8_e4m3fn:
        return t.contiguous().view(torch.uint8).numpy()
    return t.contiguous().numpy()


def dense_tables(tables: dict[str, list[int]]) -> np.ndarray:
    width = max(len(t) for t in tables.values())
    out = np.zeros((len(tables), width), dtype=np.int32)
    for i, t in enumerate(tables.values()):
        out[i, : len(t)] = t
    return out


def norm_matmul_fixture(ref_root: str) -> None:
    """norm_matmul.npz: the reference backend's fused_rms_norm_matmul (pytorch_backend/_ops_norm.py:47-65) on seeded
    inputs that tests rebuild from the same generator; only the outputs are stored."""
    sys.path.insert(0, ref_root)
    sys.path.insert(0, REPO)
    from python_runtime.hal.pytorch_backend import PyTorchBackend

    from llm_compileforge_b200 import workloads as wl

    torch.set_num_threads(1)
    hal = PyTorchBackend("cpu")
    blob = {}
    for name, (m, k, n, dt) in {"bf16_a": (70, 256, 264, torch.bfloat16), "bf16_b": (130, 1000, 512, torch.bfloat16),
                                "f16_a": (5, 64, 8, torch.float16)}.items():
        x, g, w, eps = wl.make_norm_matmul_inputs(m, k, n, dt)
        out = hal.execute("fused_rms_norm_matmul", [x, g, w], eps=eps)
        blob[name + ".out"] = bits(out) if dt == torch.bfloat16 else out.numpy()
        blob[name + ".shape"] = np.array([m, k, n])
    np.savez_compressed(os.path.join(HERE, "norm_matmul.npz"), **blob)


def sdpa_mask_fixture(ref_root: str) -> None:
    """sdpa_masks.npz: the reference backend's scaled_dot_product_attention (pytorch_backend/_ops_attention.py:13-53) on the
    seeded mask cases of workloads.make_sdpa_mask_case; only the outputs are stored."""
    sys.path.insert(0, ref_root)
    sys.path.insert(0, REPO)
    from python_runtime.hal.pytorch_backend import PyTorchBackend

    from llm_compileforge_b200 import workloads as wl

    torch.set_num_threads(1)
    hal = PyTorchBackend("cpu")
    blob = {}
    for name in wl.SDPA_MASK_CASES:
        inputs, kw = wl.make_sdpa_mask_case(name)
        out = hal.execute("scaled_dot_product_attention", inputs, **kw)
        blob[name] = bits(out) if out.dtype == torch.bfloat16 else out.numpy()
    np.savez_compressed(os.path.join(HERE, "sdpa_masks.npz"), **blob)


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    sys.path.insert(0, REPO)
    from compiler.quantize.fp8_kv_cache import FP8KVCacheQuantizer
    from kernels.flash_attention import flash_attention_fwd
    from kernels.paged_attention import paged_attention
    from kernels.rms_norm import fused_rms_norm_add
    from python_runtime.hal.pytorch_backend import PyTorchBackend

    from llm_compileforge_b200 import workloads as wl

    torch.set_num_threads(1)  # fixtures must not depend on thread-count dependent summation
    hal = PyTorchBackend("cpu")
    quant = FP8KVCacheQuantizer(block_size=16)

    # ---- paged decode: the reference's own known-answer set-ups -------------
    # python_runtime/hal/tests/test_triton_kernels.py:207-250 (seed 42, MHA)
    cases = {}
    torch.manual_seed(42)
    k = torch.randn(4, 16, 4, 32)
    v = torch.randn(4, 16, 4, 32)
    q = torch.randn(1, 4, 32)
    tables, lens = {"req_1": [0, 1]}, {"req_1": 20}
    out = paged_attention(q, k, v, tables, lens, block_size=16)
    cases["kat_mha"] = (q, k, v, tables, lens, out)
    # :188-205 GQA 8/2, three blocks, L 40
    torch.manual_seed(42)
    q = torch.randn(1, 8, 32)
    k = torch.randn(4, 16, 2, 32)
    v = torch.randn(4, 16, 2, 32)
    tables, lens = {"req_1": [0, 1, 2]}, {"req_1": 40}
    cases["kat_gqa"] = (q, k, v, tables, lens, paged_attention(q, k, v, tables, lens, block_size=16))
    # :252-269 two requests
    torch.manual_seed(42)
    q = torch.randn(2, 4, 32)
    k = torch.randn(8, 16, 4, 32)
    v = torch.randn(8, 16, 4, 32)
    tables, lens = {"req_1": [0, 1], "req_2": [2, 3]}, {"req_1": 20, "req_2": 30}
    cases["kat_multi"] = (q, k, v, tables, lens, paged_attention(q, k, v, tables, lens, block_size=16))
    # edge semantics: missing seq_len, over-long seq_len, surplus blocks, shared block, L == 1
    torch.manual_seed(7)
    q = torch.randn(5, 4, 32)
    k = torch.randn(12, 16, 2, 32)
    v = torch.randn(12, 16, 2, 32)
    tables = {"nolen": [3, 4], "toolong": [5, 1], "surplus": [0, 2, 7, 9], "shared": [3, 4, 8], "one": [11]}
    lens = {"toolong": 100, "surplus": 17, "shared": 48, "one": 1}
    cases["edges"] = (q, k, v, tables, lens, paged_attention(q, k, v, tables, lens, block_size=16))
    blob = {}
    for name, (q, k, v, tables, lens, out) in cases.items():
        blob[f"{name}.q"] = bits(q)
        blob[f"{name}.k"] = bits(k)
        blob[f"{name}.v"] = bits(v)
        blob[f"{name}.tables"] = dense_tables(tables)
        blob[f"{name}.table_lens"] = np.array([len(t) for t in tables.values()], dtype=np.int32)
        blob[f"{name}.seq_lens"] = np.array([lens.get(r, -1) for r in tables], dtype=np.int32)
        blob[f"{name}.out"] = np.stack([bits(out[r]) for r in tables])
    np.savez_compressed(os.path.join(HERE, "paged_decode_kats.npz"), **blob)

    # ---- config 1 in full (inputs are regenerated from seeds; a checksum guards them)
    w = wl.make_decode_workload(wl.C1)
    out = paged_attention(w.q, w.k_cache, w.v_cache, w.block_tables, w.seq_lens, block_size=16, scale=w.scale)
    np.savez_compressed(
        os.path.join(HERE, "paged_decode_c1.npz"),
        out=np.stack([bits(out[r]) for r in w.block_tables]),
        q=bits(w.q),
        seq_lens=np.array(w.lengths, dtype=np.int32),
        tables=dense_tables(w.block_tables),
        k_sum=np.float64(w.k_cache.double().sum().item()),
        v_sum=np.float64(w.v_cache.double().sum().item()),
    )

    # ---- config 2 shape, reduced (bf16 GQA 32/4, D 64): 6 requests, lengths clipped to 400
    w = wl.make_decode_workload(wl.C2, batch=6, max_len=400)
    out = paged_attention(w.q, w.k_cache, w.v_cache, w.block_tables, w.seq_lens, block_size=16, scale=w.scale)
    np.savez_compressed(
        os.path.join(HERE, "paged_decode_c2_small.npz"),
        out=np.stack([bits(out[r]) for r in w.block_tables]),
        seq_lens=np.array(w.lengths, dtype=np.int32),
        tables=dense_tables(w.block_tables),
        k_sum=np.float64(w.k_cache.double().sum().item()),
        v_sum=np.float64(w.v_cache.double().sum().item()),
    )

    # ---- FP8 quantiser ---------------------------------------------------------
    # tests/test_quantize.py:290-301 (seed 42, whole-tensor scale) ...
    torch.manual_seed(42)
    kk = torch.randn(16, 8, 128)
    vv = torch.randn(16, 8, 128)
    k_q, k_s, v_q, v_s = quant.quantize_kv(kk, vv)
    k_fp, v_fp = quant.dequantize_kv(k_q, k_s, v_q, v_s)
    blob = {"whole.k": bits(kk), "whole.k_codes": bits(k_q), "whole.k_scale": k_s.numpy(), "whole.k_deq": bits(k_fp),
            "whole.v": bits(vv), "whole.v_codes": bits(v_q), "whole.v_scale": v_s.numpy()}
    # ... and per-(block, kv_head) slices of a pool with awkward blocks
    g = torch.Generator().manual_seed(1234)
    pool = (torch.randn((8, 16, 2, 64), generator=g) * 2).to(torch.bfloat16)
    pool[1] = 0  # all-zero block: scale 1.0, codes 0x00 (:82-83)
    pool[2] *= 1e-3
    pool[3, :, 0] = (torch.randn((16, 64), generator=g) * 1e-12).to(torch.bfloat16)  # amax/448 < 1e-12: clamp (:86)
    pool[4, 5:] = 0  # partially written block
    pool[5] *= 3e4
    pool[6, 0, 1, 0] = -0.0
    codes = torch.empty(pool.shape, dtype=torch.uint8)
    scales = torch.empty((8, 2), dtype=torch.float32)
    deq = torch.empty(pool.shape, dtype=torch.float32)
    for b in range(8):
        for h in range(2):
            c, s = quant.quantize_block(pool[b, :, h, :])
            codes[b, :, h, :] = c.view(torch.uint8)
            scales[b, h] = s
            deq[b, :, h, :] = quant.dequantize_block(c, s)
    blob.update({"pool.x": bits(pool), "pool.codes": codes.numpy(), "pool.scales": scales.numpy(), "pool.deq": deq.numpy()})
    np.savez_compressed(os.path.join(HERE, "fp8_quantize.npz"), **blob)

    # ---- FP8 decode: quantise per slice, dequantise, reference decode on the fp32 pool
    w = wl.make_decode_workload(wl.C3, batch=4, max_len=300)
    nb, bs, hkv, d = w.k_cache.shape
    kc = torch.empty((nb, bs, hkv, d), dtype=torch.uint8)
    vc = torch.empty_like(kc)
    ks = torch.empty((nb, hkv), dtype=torch.float32)
    vs = torch.empty_like(ks)
    kd = torch.empty((nb, bs, hkv, d), dtype=torch.float32)
    vd = torch.empty_like(kd)
    for b in range(nb):
        for h in range(hkv):
            c, s = quant.quantize_block(w.k_cache[b, :, h, :])
            kc[b, :, h, :], ks[b, h], kd[b, :, h, :] = c.view(torch.uint8), s, quant.dequantize_block(c, s)
            c, s = quant.quantize_block(w.v_cache[b, :, h, :])
            vc[b, :, h, :], vs[b, h], vd[b, :, h, :] = c.view(torch.uint8), s, quant.dequantize_block(c, s)
    out = paged_attention(w.q.float(), kd, vd, w.block_tables, w.seq_lens, block_size=16, scale=w.scale)
    np.savez_compressed(
        os.path.join(HERE, "fp8_decode_c3_small.npz"),
        out=np.stack([out[r].numpy() for r in w.block_tables]),
        seq_lens=np.array(w.lengths, dtype=np.int32),
        tables=dense_tables(w.block_tables),
        k_codes_sum=np.int64(kc.long().sum().item()),
        v_codes_sum=np.int64(vc.long().sum().item()),
        k_scales=ks.numpy(),
        v_scales=vs.numpy(),
    )

    # ---- RMSNorm -----------------------------------------------------------------
    blob = {}
    x, wgt, eps = wl.make_rms_norm_inputs(rows=8, hidden=4096)
    blob["hal_bf16.out"] = bits(hal.execute("rms_norm", [x, wgt], eps=eps))
    xf = torch.randn((5, 333), generator=torch.Generator().manual_seed(3))
    wf = torch.randn((333,), generator=torch.Generator().manual_seed(4))
    blob["hal_f32.x"], blob["hal_f32.w"] = xf.numpy(), wf.numpy()
    blob["hal_f32.out"] = hal.execute("rms_norm", [xf, wf], eps=1e-5).numpy()
    blob["hal_f32_noweight.out"] = hal.execute("rms_norm", [xf], eps=1e-5).numpy()
    # python_runtime/hal/tests/test_triton_kernels.py:26-43 (seed 42, eps 1e-6)
    torch.manual_seed(42)
    x = torch.randn(4, 128)
    r = torch.randn(4, 128)
    wg = torch.randn(128)
    blob["fused_f32.x"], blob["fused_f32.r"], blob["fused_f32.w"] = x.numpy(), r.numpy(), wg.numpy()
    blob["fused_f32.out"] = fused_rms_norm_add(x, r, wg, eps=1e-6).numpy()
    xb, rb, wb = x.bfloat16(), r.bfloat16(), wg.bfloat16()
    blob["fused_bf16.out"] = bits(fused_rms_norm_add(xb, rb, wb, eps=1e-6))
    # tests/contract/fixtures/generate.py:49-76 "rms_norm_2x4_f32": no eps in the expected values
    xs = torch.tensor([[1.0, 2.0, 3.0, 4.0], [0.5, 1.5, 2.5, 3.5]])
    blob["contract_2x4.x"] = xs.numpy()
    blob["contract_2x4.out"] = hal.execute("rms_norm", [xs, torch.ones(4)], eps=1e-5).numpy()
    np.savez_compressed(os.path.join(HERE, "rms_norm.npz"), **blob)

    # ---- dense causal attention + chunked prefill --------------------------------
    blob = {}
    # python_runtime/hal/tests/test_triton_kernels.py:83-105
    torch.manual_seed(42)
    q = torch.randn(2, 4, 64, 32) / math.sqrt(32)
    k = torch.randn(2, 4, 64, 32) / math.sqrt(32)
    v = torch.randn(2, 4, 64, 32)
    blob["flash_kat.q"], blob["flash_kat.k"], blob["flash_kat.v"] = q.numpy(), k.numpy(), v.numpy()
    blob["flash_kat.out"] = flash_attention_fwd(q, k, v, causal=True).numpy()
    blob["flash_kat.out_noncausal"] = flash_attention_fwd(q, k, v, causal=False).numpy()
    # config-4 shape, reduced: 3 requests share a 64-token prefix, 48-token chunks, GQA 8/2, D 128, bf16
    pw = wl.make_prefill_workload(n_requests=3, prefix_len=64, chunk_len=48, n_heads=8, n_kv_heads=2, head_dim=128)
    outs = []
    for i, (rid, table) in enumerate(pw.block_tables.items()):
        L = pw.ctx_lens[rid]
        ids = torch.as_tensor(table[: -(-L // 16)])
        ks = pw.k_cache[ids].flatten(0, 1)[:L].repeat_interleave(4, dim=1).transpose(0, 1).unsqueeze(0)
        vs = pw.v_cache[ids].flatten(0, 1)[:L].repeat_interleave(4, dim=1).transpose(0, 1).unsqueeze(0)
        qf = torch.zeros((1, 8, L, 128), dtype=torch.bfloat16)
        qf[0, :, L - 48 :] = pw.q[i * 48 : (i + 1) * 48].transpose(0, 1)
        full = flash_attention_fwd(qf, ks, vs, scale=pw.scale, causal=True)
        # cross-check with the HAL op and an explicit additive mask (_ops_attention.py:13-53)
        mask = torch.full((L, L), float("-inf")).triu(1).to(torch.bfloat16)
        full2 = hal.execute("scaled_dot_product_attention", [qf, ks, vs], attn_mask=mask, scale=pw.scale)
        assert (full[0, :, L - 48 :].float() - full2[0, :, L - 48 :].float()).abs().max() < 2e-2
        outs.append(full[0, :, L - 48 :].transpose(0, 1).contiguous())
    blob["prefill_small.out"] = np.stack([bits(o) for o in outs])
    blob["prefill_small.k_sum"] = np.float64(pw.k_cache.double().sum().item())
    blob["prefill_small.q_sum"] = np.float64(pw.q.double().sum().item())
    np.savez_compressed(os.path.join(HERE, "prefill.npz"), **blob)

    norm_matmul_fixture(ref_root)
    sdpa_mask_fixture(ref_root)
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    sys.path.insert(0, REPO)
    from oracle.build_ref import reference_root  # argument, $SFB_REFERENCE_ROOT, or ../reference beside this repository

    root = reference_root(sys.argv[1] if len(sys.argv) > 1 and not sys.argv[1].startswith("--") else None)
    if "--only-norm-matmul" in sys.argv:  # adds that one fixture without rewriting the others
        norm_matmul_fixture(root)
    elif "--only-sdpa-masks" in sys.argv:
        sdpa_mask_fixture(root)
    else:
        main(root)
