"""Per-kernel measurements for the hot path's other kernels (one JSON line each).

    python -m llm_compileforge_b200.kernel_bench [--iters 20] [--chunk-tokens 0] \
        [--only prefill,prefill_fp8,norm_matmul,append,norm,decode_c2,decode_c3,shared_prefix]

``bench.py`` at the repository root reports the headline decode metric; this
module times the remaining kernels on their configurations with CUDA events
(at least 3 warm-ups; inputs larger than L2 or an L2 flush between iterations)
and prints achieved bandwidth / FLOP rate against the measured peaks (tensor kernels against the burst GEMM rate, the
figure for a kernel timed alone; ``frac_of_sustained`` gives the fraction of the seconds-long rate beside it).
"""

from __future__ import annotations

import argparse
import json
import os

import torch

from . import ops
from . import workloads as wl

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d["bf16_tflops_sustained"],
                "kind": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "kind": "fallback"}


class L2Flush:
    def __init__(self, dev, enabled=True):
        self.buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if enabled else None

    def __call__(self):
        if self.buf is not None:
            self.buf.zero_()


def time_ms(fn, iters: int, warmup: int = 3, flush=None) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush:
            flush()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return total / iters


def time_ms_graph(fn, iters: int, warmup: int = 3, flush=None) -> float:
    """Device time of one call replayed from a CUDA graph (no host launch latency
    between the call's memset and kernels)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            fn()
    torch.cuda.synchronize()
    return time_ms(graph.replay, iters, warmup=2, flush=flush)


def bench_prefill(dev, iters, fp8: bool = False):
    """Config 4; with ``fp8`` the pool holds e4m3 codes + per-(block, kv head) scales and the call includes their expansion."""
    pw = wl.make_prefill_workload()  # config 4: 32 requests, 2048 shared prefix + 512 chunk, H 32/8, D 128, bf16
    q, k, v = pw.q.to(dev), pw.k_cache.to(dev), pw.v_cache.to(dev)
    scales = {}
    if fp8:
        (k, ks), (v, vs) = ops.quantize_fp8(k, per_block_head=True), ops.quantize_fp8(v, per_block_head=True)
        scales = dict(k_scale=ks, v_scale=vs)
    rids = list(pw.block_tables)
    width = max(len(t) for t in pw.block_tables.values())
    tables = torch.zeros((len(rids), width), dtype=torch.int32)
    for i, r in enumerate(rids):
        tables[i, : len(pw.block_tables[r])] = torch.tensor(pw.block_tables[r], dtype=torch.int32)
    tables = tables.to(dev)
    cu = (torch.arange(len(rids) + 1, dtype=torch.int32) * pw.chunk_len).to(dev)
    ctx = torch.full((len(rids),), pw.prefix_len + pw.chunk_len, dtype=torch.int32, device=dev)
    ws_bytes = (ops.prefill_fp8_workspace_bytes(q.shape[0], len(rids), width, k.shape[2], k.shape[3]) if fp8
                else ops.prefill_workspace_bytes(q.shape[0]))
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=dev)
    out = torch.empty_like(q)
    fn = lambda: ops.prefill_paged(q, k, v, tables, cu, ctx, max_q_tokens=pw.chunk_len, scale=pw.scale, workspace=ws, out=out, **scales)
    # replayed from a CUDA graph: between the two events the host does nothing, so a busy host (tensor-map encoding and the
    # launch take tens of microseconds) cannot leave a gap in front of the kernel
    ms_eager = time_ms(fn, max(3, iters // 4), flush=L2Flush(dev))
    ms = time_ms_graph(fn, iters, flush=L2Flush(dev))
    flops = wl.prefill_flops(len(rids), pw.n_heads, pw.head_dim, pw.chunk_len, pw.prefix_len)
    p = _peaks()
    tf = flops / (ms / 1e3) / 1e12
    return {"kernel": "prefill_tcgen05" + (" after expand_fp8_blocks" if fp8 else ""),
            "workload": "config 4: 32 requests, 2048-token shared prefix + 512-token chunk, H 32/8, D 128, " + ("bf16 queries over an e4m3 pool" if fp8 else "bf16"),
            "ms": ms, "flops": flops, "achieved_tflops": tf, "peak_tflops": p["bf16_tflops"],
            "frac": tf / p["bf16_tflops"], "frac_of_sustained": tf / p["bf16_tflops_sustained"], "peak_kind": p["kind"],
            "timing": "CUDA graph replay", "ms_eager_launch": ms_eager, "status": ops.read_status(ws)}


def bench_norm_matmul(dev, iters, m=16384, k=4096, n=6144):
    """Llama-3-8B's input norm + fused QKV projection over 16384 tokens (prefill-sized), and the same weight at 256 rows."""
    x, rw, w, eps = wl.make_norm_matmul_inputs(m, k, n)
    x, rw, w = x.to(dev), rw.to(dev), w.to(dev)
    folded = ops.fold_norm_weight(rw, w)
    out = torch.empty((m, n), dtype=x.dtype, device=dev)
    ws = torch.empty(ops.norm_matmul_workspace_bytes(m), dtype=torch.uint8, device=dev)
    fn = lambda: ops.fused_rms_norm_matmul(x, folded, eps=eps, out=out, workspace=ws)
    flush = L2Flush(dev, enabled=m * k * 2 + k * n * 2 < (256 << 20))  # small cases would otherwise sit in L2
    timer = time_ms_graph if m < 2048 else time_ms  # a few-microsecond call is timed from a graph, without host launch gaps
    ms = timer(fn, iters, flush=flush)
    xn = torch.empty_like(x)
    lib = lambda: torch.matmul(ops.rms_norm(x, rw, eps=eps, out=xn), w, out=out)  # unfused: norm kernel, then the library GEMM
    ms_lib = timer(lib, iters, flush=flush)
    flops = 2.0 * m * n * k
    pk = _peaks()
    return {"kernel": "norm_matmul_tcgen05", "workload": f"rms_norm + matmul, x [{m}, {k}] bf16, W [{k}, {n}]", "ms": ms,
            "flops": flops, "achieved_tflops": flops / ms / 1e9, "peak_tflops": pk["bf16_tflops"],
            "frac": flops / ms / 1e9 / pk["bf16_tflops"], "frac_of_sustained": flops / ms / 1e9 / pk["bf16_tflops_sustained"],
            "ms_unfused_norm_then_library_gemm": ms_lib, "weight_gbs": k * n * 2 / ms / 1e6,
            "timing": "CUDA graph replay, L2 flushed" if m < 2048 else "stream launches", "peak_kind": pk["kind"], "status": ops.read_status(ws)}


def bench_append(dev, iters):
    shape = wl.C3
    lengths = wl.config_lengths(shape)
    nb = wl.pool_blocks_for(shape, lengths)
    tables = wl.random_tables(lengths, nb, 1005 + shape.index)
    hkv, d, bs = shape.n_kv_heads, shape.head_dim, shape.block_size
    b, total = len(lengths), sum(lengths)
    width = max(len(t) for t in tables.values())
    dense = torch.zeros((b, width), dtype=torch.int32)
    for i, t in enumerate(tables.values()):
        dense[i, : len(t)] = torch.tensor(t, dtype=torch.int32)
    dense = dense.to(dev)
    gen = torch.Generator(device=dev).manual_seed(5)
    k_new = (torch.randn((total, hkv, d), generator=gen, device=dev) * 2).to(torch.bfloat16)
    v_new = (torch.randn((total, hkv, d), generator=gen, device=dev) * 2).to(torch.bfloat16)
    kc = torch.zeros((nb, bs, hkv, d), dtype=torch.uint8, device=dev)
    vc = torch.zeros_like(kc)
    ks = torch.ones((nb, hkv), dtype=torch.float32, device=dev)
    vs = torch.ones_like(ks)
    kt = torch.zeros((b, bs, hkv, d), dtype=torch.bfloat16, device=dev)
    vt = torch.zeros_like(kt)
    cu = torch.zeros(b + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(lengths).cumsum(0)
    cu = cu.to(dev)
    start = torch.zeros(b, dtype=torch.int32, device=dev)
    fn = lambda: ops.cache_write(k_new, v_new, cu, start, dense, kc, vc, max_new_tokens=max(lengths), k_scale=ks, v_scale=vs,
                                 k_tail=kt, v_tail=vt)
    ms = time_ms(fn, iters)  # 2.1 GB of source + 1 GB of codes per pass: far larger than L2
    byts = wl.append_algorithmic_bytes(total, hkv, d)
    p = _peaks()
    gbs = byts / (ms / 1e3) / 1e9
    return {"kernel": "cache_write_kernel (FP8 quantise-on-append)", "workload": f"config 3: {b} requests, {total} tokens appended, Hkv 8, D 128, bf16 -> e4m3",
            "ms": ms, "bytes": byts, "achieved_gbs": gbs, "peak_gbs": p["hbm_gbs"], "frac": gbs / p["hbm_gbs"],
            "frac_of_nominal_8TBs": gbs / 8000.0, "peak_kind": p["kind"]}


def bench_norm(dev, iters, rows):
    x, w, eps = wl.make_rms_norm_inputs(rows=rows)
    x, w = x.to(dev), w.to(dev)
    out = torch.empty_like(x)
    fn = lambda: ops.rms_norm(x, w, eps, out=out)
    ms = time_ms(fn, iters, flush=L2Flush(dev))
    ms_copy = time_ms(lambda: out.copy_(x), iters, flush=L2Flush(dev))  # a plain copy of the same bytes, for scale
    byts = wl.rms_norm_algorithmic_bytes(rows, x.shape[1], 2)
    p = _peaks()
    gbs = byts / (ms / 1e3) / 1e9
    return {"kernel": "rms_norm_vec_kernel", "workload": f"[{rows}, 4096] bf16, eps 1e-5, L2 flushed between iterations", "ms": ms,
            "bytes": byts, "achieved_gbs": gbs, "peak_gbs": p["hbm_gbs"], "frac": gbs / p["hbm_gbs"],
            "frac_of_nominal_8TBs": gbs / 8000.0, "peak_kind": p["kind"], "ms_copy_same_bytes": ms_copy}


def bench_decode(dev, iters, shape, chunk_tokens=0):
    import bench as root_bench  # the repository-level benchmark owns the serving-state builder

    st = root_bench.DecodeState(shape, shape.batch, 4, dev, seed_offset=0)
    chunk = root_bench.pick_chunk_tokens(st.lengths, chunk_tokens)
    ws = torch.zeros(ops.decode_workspace_bytes(st.batch, shape.n_heads, shape.head_dim, st.tables.shape[1], 16, chunk),
                     dtype=torch.uint8, device=dev)
    out = torch.empty_like(st.q)
    kw = dict(k_scale=st.k_scale, v_scale=st.v_scale) if st.fp8 else {}
    fn = lambda: ops.paged_attention_decode(st.q, st.k_cache, st.v_cache, st.tables, st.len_steps[0], chunk_tokens=chunk,
                                            workspace=ws, out=out, **kw)
    pool_bytes = 2 * st.k_cache.numel() * st.k_cache.element_size()
    flush = L2Flush(dev, enabled=pool_bytes < (1 << 30))
    ms_eager = time_ms(fn, iters, flush=flush)
    ms = time_ms_graph(fn, iters, flush=flush)
    byts = st.algorithmic_bytes(0)
    p = _peaks()
    gbs = byts / (ms / 1e3) / 1e9
    return {"kernel": "decode_tma_kernel (split-K, in-kernel merge)", "workload": f"{shape.name}, {st.batch} requests, chunk {chunk}", "ms": ms, "bytes": byts,
            "achieved_gbs": gbs, "peak_gbs": p["hbm_gbs"], "frac": gbs / p["hbm_gbs"], "frac_of_nominal_8TBs": gbs / 8000.0,
            "tokens_per_s": st.batch / (ms / 1e3), "peak_kind": p["kind"], "timing": "CUDA graph replay", "ms_eager_launch": ms_eager}


def bench_shared_prefix(dev, iters, n_requests=32):
    """Decode step right after config 4's prefill: requests that share a 2048-token prefix and own 512 tokens."""
    pw = wl.make_prefill_workload(n_requests=n_requests)
    k, v = pw.k_cache.to(dev), pw.v_cache.to(dev)
    rids = list(pw.block_tables)
    b = len(rids)
    width = max(len(t) for t in pw.block_tables.values())
    tables = torch.zeros((b, width), dtype=torch.int32)
    for i, r in enumerate(rids):
        tables[i, : len(pw.block_tables[r])] = torch.tensor(pw.block_tables[r], dtype=torch.int32)
    tables = tables.to(dev)
    lens = torch.full((b,), pw.prefix_len + pw.chunk_len, dtype=torch.int32, device=dev)
    q = pw.q[:b].contiguous().to(dev)
    out = torch.empty_like(q)
    pb = pw.prefix_len // 16
    ws1 = torch.zeros(ops.decode_workspace_bytes(b, pw.n_heads, pw.head_dim, width, 16, 256), dtype=torch.uint8, device=dev)
    plain = lambda: ops.paged_attention_decode(q, k, v, tables, lens, chunk_tokens=256, workspace=ws1, out=out)
    from . import _lib
    ws2 = torch.zeros(int(_lib.load().sfb_shared_prefix_workspace_bytes(b, pw.n_heads, pw.head_dim, width, 16, 256, pb)),
                      dtype=torch.uint8, device=dev)
    shared = lambda: ops.paged_attention_decode_shared_prefix(q, k, v, tables, lens, pb, chunk_tokens=256, workspace=ws2, out=out)
    flush = L2Flush(dev)
    ms_plain = time_ms_graph(plain, iters, flush=flush)
    ms_shared = time_ms_graph(shared, iters, flush=flush)
    e = 2
    plain_bytes = wl.decode_algorithmic_bytes([pw.prefix_len + pw.chunk_len] * b, pw.n_heads, pw.n_kv_heads, pw.head_dim, e, e, e, False)
    return {"kernel": "shared-prefix decode (tcgen05 prefix + TMA remainder)", "workload": f"{b} requests, 2048-token shared prefix + 512 own tokens, H 32/8, D 128, bf16",
            "ms_plain_decode": ms_plain, "ms_shared_prefix": ms_shared, "speedup": ms_plain / ms_shared,
            "plain_algorithmic_bytes": plain_bytes, "plain_achieved_gbs": plain_bytes / (ms_plain / 1e3) / 1e9,
            "equivalent_gbs": plain_bytes / (ms_shared / 1e3) / 1e9, "timing": "CUDA graph replay, L2 flushed"}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="prefill,norm_matmul,append,norm,decode_c2,decode_c3,shared_prefix")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--chunk-tokens", type=int, default=0)
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("kernel_bench needs a CUDA device")
    dev = torch.device("cuda:0")
    which = args.only.split(",")
    import sys
    sys.path.insert(0, ROOT)
    if "prefill" in which:
        print(json.dumps(bench_prefill(dev, args.iters)), flush=True)
    if "prefill_fp8" in which:
        print(json.dumps(bench_prefill(dev, args.iters, fp8=True)), flush=True)
    if "norm_matmul" in which:
        print(json.dumps(bench_norm_matmul(dev, args.iters)), flush=True)
        print(json.dumps(bench_norm_matmul(dev, args.iters, m=256)), flush=True)
    if "append" in which:
        print(json.dumps(bench_append(dev, args.iters)), flush=True)
    if "norm" in which:
        print(json.dumps(bench_norm(dev, args.iters, 256)), flush=True)
        print(json.dumps(bench_norm(dev, args.iters, 16384)), flush=True)
    if "shared_prefix" in which:
        for n in (32, 128, 512):
            print(json.dumps(bench_shared_prefix(dev, args.iters, n)), flush=True)
    if "decode_c2" in which:
        print(json.dumps(bench_decode(dev, args.iters, wl.C2, args.chunk_tokens)), flush=True)
    if "decode_c3" in which:
        print(json.dumps(bench_decode(dev, args.iters, wl.C3, args.chunk_tokens)), flush=True)


if __name__ == "__main__":
    main()
