"""Benchmark of the paged FP8-KV decode hot path (one JSON line on stdout).

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...        # the reference's CPU algorithm on the host cores

Workload: the Llama-3-70B-shaped FP8-KV decode configuration (64 query heads,
8 kv heads, head_dim 128, block_size 16, 2048 requests, lognormal context
lengths with median 4096 clipped to [256, 32768], e4m3 KV with per-(block,
kv_head) float32 scales) - the whole configuration resident on EACH GPU, requests
partitioned across GPUs (weak scaling, no data-path collective).

One step = one decode iteration of the hot path: quantise-on-append of one new
token per request into the paged FP8 pool, then paged attention of one query
token per request over the pool (split-K kernel, partial results merged in-kernel).  ``value`` is decode
tokens/s with every input already in HBM; ``e2e`` is the same step driven
through ``AttentionStepPipeline`` with host (pinned) inputs: every step q, new
K/V and positions are copied to the device, the block tables are grown on the
host and their delta sent, and the attention output is copied back to the host,
all inside the timed region, three steps in flight (one-step-at-a-time figure
beside it).  The KV pool and the block tables are device state, as in serving.

Inputs are synthetic (seeded); the 22.7 GB code pool is far larger than L2, so
no flush is needed between steps.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from llm_compileforge_b200 import workloads as wl  # noqa: E402

METRIC = "paged_fp8_decode_tokens_per_s"
UNIT = "tokens/s"
NOMINAL_HBM_GBS = 8000.0
# dram__bytes_read.sum + dram__bytes_write.sum over algorithmic bytes of the decode kernel, from the ncu capture of a
# 128-request case of the same shape (1.259 GB read + 0.077 GB written for 1.253 GB algorithmic);
# the full launch is beyond the capture size rule, and its traffic grows with the KV tokens read.
TRAFFIC_PER_ALGORITHMIC_BYTE = 1.066


# steps the end-to-end pass keeps in flight: with three, a step's host->device copy has two compute steps to hide behind, which
# still holds when eight ranks share the host's PCIe uplinks and cores
IN_FLIGHT = 3


def parse_args() -> argparse.Namespace:
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", choices=["b200", "reference"], default="b200")
    p.add_argument("--workload", choices=["c5", "c3", "c2"], default="c5")
    p.add_argument("--batch", type=int, default=0, help="requests per GPU (0 = the configuration's batch)")
    p.add_argument("--chunk-tokens", type=int, default=0, help="KV split size (0 = heuristic)")
    p.add_argument("--gather", nargs="?", const="nccl", default=None, choices=["nccl", "peer"],
                   help="gather the outputs inside the step: nccl = all-gather after the decode; peer (head partition only) = "
                        "the decode kernel stores its heads into every GPU's output over NVLink, then one signal kernel")
    p.add_argument("--partition", choices=["request", "head"], default="request",
                   help="request: every GPU serves its own requests (weak scaling, default); head: the configuration's "
                        "requests on every GPU with 1/N of the kv heads each (strong scaling, the 8-GPU layout of config 5)")
    p.add_argument("--kernel", choices=["decode", "append", "norm", "prefill", "norm_matmul"], default="decode",
                   help="decode (default): the headline step.  The others print one line for that kernel of the path alone "
                        "(device time against its roofline, the oracle port timed on the host cores beside it); 1 GPU")
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--headline-only", action="store_true",
                   help="skip the extra objects of the default run: `kernels` (every other kernel of the path, 1 GPU) and "
                        "`head_partition` (the configuration split by kv head with the output gathered, N GPUs)")
    p.add_argument("--cpu-sample", type=int, default=48, help="requests in the CPU-baseline sample")
    return p.parse_args()


def shape_of(name: str) -> wl.DecodeShape:
    return {"c5": wl.C5, "c3": wl.C3, "c2": wl.C2}[name]


def peaks() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def bind_to_gpu_cpus(index: int) -> str:
    """Restrict this process to the CPUs that sit next to its GPU (read-only NVML query of the device's CPU affinity, then
    this process's own scheduler affinity) before any pinned host buffer is allocated: first-touch then places the buffers
    in that socket's memory and the host<->device copies stay off the socket interconnect.  Changes nothing on the GPU."""
    try:
        import pynvml

        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(ClockSampler._physical_index(index))
        n_cpu = os.cpu_count() or 1
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (n_cpu + 63) // 64)
        cpus = {64 * w + b for w, word in enumerate(words) for b in range(64) if (int(word) >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return f"{len(cpus)} CPUs next to GPU {index}"
    except Exception as e:  # noqa: BLE001
        return f"unbound ({type(e).__name__})"
    return "unbound"


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs
    (read-only NVML queries every few milliseconds; nvidia-smi as a fallback)."""

    def __init__(self, index: int):
        self.index = index
        self.sm: list[int] = []
        self.sm_max = None
        self.reasons: set[str] = set()
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._nvml = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index(index))
            self.sm_max = int(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
        except Exception:  # noqa: BLE001
            self._nvml = None

    @staticmethod
    def _physical_index(index: int) -> int:
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            parts = [p for p in vis.split(",") if p.strip()]
            if index < len(parts) and parts[index].strip().isdigit():
                return int(parts[index])
        return index

    def _sample_nvml(self) -> None:
        n = self._nvml
        self.sm.append(int(n.nvmlDeviceGetClockInfo(self._handle, n.NVML_CLOCK_SM)))
        bits = int(n.nvmlDeviceGetCurrentClocksEventReasons(self._handle)) if hasattr(n, "nvmlDeviceGetCurrentClocksEventReasons") \
            else int(n.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle))
        names = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}
        for bit, name in names.items():
            if bits & bit:
                self.reasons.add(name)

    def _sample_smi(self) -> None:
        fields = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
                  "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        out = subprocess.run(["nvidia-smi", "-i", str(self.index), f"--query-gpu={fields}", "--format=csv,noheader,nounits"],
                             capture_output=True, text=True, timeout=5).stdout
        for line in out.strip().splitlines():
            r = [c.strip() for c in line.split(",")]
            if r and r[0].isdigit():
                self.sm.append(int(r[0]))
                self.sm_max = int(r[1]) if r[1].isdigit() else self.sm_max
                for i, name in enumerate(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]):
                    if len(r) > 2 + i and r[2 + i].lower() == "active":
                        self.reasons.add(name)

    def _run(self) -> None:
        while not self._stop.is_set():
            try:
                if self._nvml:
                    self._sample_nvml()
                else:
                    self._sample_smi()
            except Exception:  # noqa: BLE001
                pass
            self._stop.wait(0.005 if self._nvml else 0.1)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self) -> dict:
        sm = sorted(self.sm)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.sm_max, "reasons": sorted(self.reasons),
                "samples": len(sm)}


def pick_chunk_tokens(lengths: list[int], requested: int) -> int:
    from llm_compileforge_b200.tables import pick_chunk_tokens as heuristic

    return requested if requested > 0 else heuristic(lengths)


class DecodeState:
    """Device-resident serving state for one GPU: the FP8 pool, tables, tails."""

    def __init__(self, shape: wl.DecodeShape, batch: int, steps_total: int, dev: torch.device, seed_offset: int):
        from llm_compileforge_b200 import ops

        self.shape, self.dev = shape, dev
        bs, hkv, d = shape.block_size, shape.n_kv_heads, shape.head_dim
        self.fp8 = shape.kv_fp8
        self.lengths = wl.config_lengths(shape, batch) if seed_offset == 0 else _rank_lengths(shape, batch, seed_offset)
        self.batch = len(self.lengths)
        extra = -(-(steps_total + 1) // bs) + 1  # room for the tokens appended while benchmarking
        self.n_blocks = wl.pool_blocks_for(shape, self.lengths, extra)
        # Block placement: the block manager hands out ids from a free list left in a seeded random order (a pool that
        # has served and released other requests), request i owns row i of the device-resident tables.  Tables cover
        # the device-timed pass up front; the end-to-end pass grows them step by step like a live engine.
        self.bm = _shuffled_block_manager(self.n_blocks, bs, 1005 + shape.index + seed_offset)
        width = max(wl.blocks_for(n, bs) for n in self.lengths) + extra
        self.tables = self.bm.attach_device_tables(self.batch, width, dev)
        self.rids = [f"req_{i}" for i in range(self.batch)]
        for rid, n in zip(self.rids, self.lengths):
            self.bm.allocate(rid, n + steps_total // 3 + 2)
        assert [self.bm.row(r) for r in self.rids] == list(range(self.batch))
        self.bm.sync(torch.cuda.current_stream(dev))
        kv_dtype = torch.uint8 if self.fp8 else shape.dtype
        self.k_cache = torch.zeros((self.n_blocks, bs, hkv, d), dtype=kv_dtype, device=dev)
        self.v_cache = torch.zeros_like(self.k_cache)
        if self.fp8:
            self.k_scale = torch.ones((self.n_blocks, hkv), dtype=torch.float32, device=dev)
            self.v_scale = torch.ones_like(self.k_scale)
            self.k_tail = torch.zeros((self.batch, bs, hkv, d), dtype=shape.dtype, device=dev)
            self.v_tail = torch.zeros_like(self.k_tail)
        else:
            self.k_scale = self.v_scale = self.k_tail = self.v_tail = None
        # fill the pool through the product's own cache write, a group of requests at a time
        gen = torch.Generator(device=dev).manual_seed(1002 + shape.index + seed_offset)
        gain = 2.0 if self.fp8 else 1.0
        group = 64
        for lo in range(0, self.batch, group):
            ls = self.lengths[lo : lo + group]
            total = sum(ls)
            k_new = (torch.randn((total, hkv, d), generator=gen, device=dev) * gain).to(shape.dtype)
            v_new = (torch.randn((total, hkv, d), generator=gen, device=dev) * gain).to(shape.dtype)
            cu = torch.zeros(len(ls) + 1, dtype=torch.int32)
            cu[1:] = torch.tensor(ls).cumsum(0)
            ops.cache_write(k_new, v_new, cu.to(dev), torch.zeros(len(ls), dtype=torch.int32, device=dev),
                            self.tables[lo : lo + len(ls)], self.k_cache, self.v_cache, max_new_tokens=max(ls),
                            k_scale=self.k_scale, v_scale=self.v_scale,
                            k_tail=None if not self.fp8 else self.k_tail[lo : lo + len(ls)],
                            v_tail=None if not self.fp8 else self.v_tail[lo : lo + len(ls)])
            del k_new, v_new
        torch.cuda.synchronize(dev)
        self.q = torch.randn((self.batch, shape.n_heads, d), generator=gen, device=dev).to(shape.dtype)
        self.new_k = (torch.randn((self.batch, hkv, d), generator=gen, device=dev) * gain).to(shape.dtype)
        self.new_v = (torch.randn((self.batch, hkv, d), generator=gen, device=dev) * gain).to(shape.dtype)
        self.cu_one = torch.arange(self.batch + 1, dtype=torch.int32, device=dev)
        base = torch.tensor(self.lengths, dtype=torch.int32)
        self.pos_steps_host = (base[None, :] + torch.arange(steps_total, dtype=torch.int32)[:, None]).contiguous().pin_memory()
        self.pos_steps = self.pos_steps_host.to(dev)          # position of the token appended in step s
        self.len_steps_host = (self.pos_steps_host + 1).pin_memory()
        self.len_steps = self.len_steps_host.to(dev)          # attended length in step s

    def algorithmic_bytes(self, step: int) -> int:
        s = self.shape
        lens = [n + step + 1 for n in self.lengths]
        e = 2 if s.dtype in (torch.bfloat16, torch.float16) else 4
        return wl.decode_algorithmic_bytes(lens, s.n_heads, s.n_kv_heads, s.head_dim, 1 if self.fp8 else e, e, e, self.fp8,
                                           s.block_size)


def _shuffled_block_manager(n_blocks: int, block_size: int, seed: int):
    """A block manager whose free list is a seeded permutation of the pool: take every block, give each a second
    holder, drop the request, then release the blocks one by one in permuted order."""
    from llm_compileforge_b200.block_manager import BlockManager

    bm = BlockManager(n_blocks, block_size)
    bm.allocate("_all", n_blocks * block_size)
    for b in range(n_blocks):
        bm.increment_ref_count(b)
    bm.free("_all")
    for b in torch.randperm(n_blocks, generator=torch.Generator().manual_seed(seed)).tolist():
        bm.free_block(b)
    assert bm.num_free_blocks() == n_blocks
    return bm


def _rank_lengths(shape: wl.DecodeShape, batch: int | None, offset: int) -> list[int]:
    b = shape.batch if batch is None else batch
    if shape.index == 5:
        return wl.lognormal_lengths(b, 4096, 256, 32768, 1004 + shape.index + offset)
    if shape.index == 3:
        return wl.lognormal_lengths(b, 2048, 128, 8192, 1004 + shape.index + offset)
    return wl.uniform_lengths(b, 1024, 4096, 1004 + shape.index + offset)


def cpu_baseline(shape: wl.DecodeShape, lengths: list[int], n_sample: int, repeats: int = 1) -> dict:
    """The reference's CPU algorithm (oracle port: dequantise the request's
    blocks, gather, GQA-expand, SDPA per request) on the host cores, on a seeded
    sample of the workload's requests."""
    from oracle import reference_port as ref

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    pick = torch.randperm(len(lengths), generator=torch.Generator().manual_seed(99))[:n_sample].tolist()
    ls = [lengths[i] for i in pick]
    bs, hkv, d = shape.block_size, shape.n_kv_heads, shape.head_dim
    nb = sum(wl.blocks_for(n, bs) for n in ls)
    tables, at = {}, 0
    for i, n in enumerate(ls):
        tables[f"r{i}"] = list(range(at, at + wl.blocks_for(n, bs)))
        at += wl.blocks_for(n, bs)
    g = torch.Generator().manual_seed(7)
    q = torch.randn((len(ls), shape.n_heads, d), generator=g).to(shape.dtype)
    seq = {f"r{i}": n for i, n in enumerate(ls)}
    if shape.kv_fp8:
        kc = torch.randint(0, 0x7E, (nb, bs, hkv, d), generator=g, dtype=torch.uint8)
        vc = torch.randint(0, 0x7E, (nb, bs, hkv, d), generator=g, dtype=torch.uint8)
        ks = torch.rand((nb, hkv), generator=g) * 0.02 + 0.01
        vs = torch.rand((nb, hkv), generator=g) * 0.02 + 0.01

        def run():
            kd, vd = ref.fp8_dequantize_pool(kc, ks), ref.fp8_dequantize_pool(vc, vs)
            return ref.paged_attention(q.float(), kd, vd, tables, seq)
    else:
        k = torch.randn((nb, bs, hkv, d), generator=g).to(shape.dtype)
        v = torch.randn((nb, bs, hkv, d), generator=g).to(shape.dtype)

        def run():
            return ref.paged_attention(q, k, v, tables, seq)

    run()  # warm-up
    best = math.inf
    for _ in range(max(1, repeats)):
        t0 = time.perf_counter()
        run()
        best = min(best, time.perf_counter() - t0)
    return {"value": len(ls) / best, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{len(ls)} seeded requests of the workload ({sum(ls)} KV tokens), best of {max(1, repeats)}, "
                      f"{best:.3f} s per pass, torch CPU threads = {cores}"}


def run_reference(args: argparse.Namespace, rank: int) -> None:
    if rank != 0:
        return
    shape = shape_of(args.workload)
    lengths = wl.config_lengths(shape, args.batch or None)
    n_sample = min(args.cpu_sample, len(lengths))
    from oracle import reference_port as ref  # noqa: F401  (the reference arm runs the oracle port)

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    # each step is one pass over the bounded sample
    times = []
    base = None
    for i in range(args.warmup + args.steps):
        r = cpu_baseline(shape, lengths, n_sample, repeats=1)
        if i >= args.warmup:
            times.append(n_sample / r["value"])
        base = r
    ms = 1e3 * sum(times) / len(times)
    value = n_sample / (ms / 1e3)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": workload_config(shape, len(lengths), args, 0),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": base["sample"]},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def _best_of(fn, repeats: int = 3) -> float:
    """Seconds of the fastest of `repeats` calls after one warm-up call."""
    fn()
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        fn()
        best = min(best, time.perf_counter() - t0)
    return best


KERNEL_KINDS = ("append", "norm_256", "norm_16384", "prefill", "prefill_fp8", "decode_c2", "decode_c3", "norm_matmul")


def kernel_entry(kind: str, iters: int, dev: torch.device, cpu: bool = True) -> dict:
    """One kernel of the path, timed alone on its configuration (``llm_compileforge_b200.kernel_bench``: CUDA events,
    >= 3 warm-ups, inputs larger than L2 or an L2 flush between iterations) with the SM clocks sampled while it runs, its
    roofline fraction, and the reference's CPU algorithm (oracle port) on a bounded sample of the same workload."""
    from llm_compileforge_b200 import kernel_bench as kb
    from oracle import reference_port as ref

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    with ClockSampler(dev.index or 0) as clocks:
        if kind == "append":
            r = kb.bench_append(dev, iters)
        elif kind in ("norm_256", "norm_16384"):
            r = kb.bench_norm(dev, iters, int(kind.split("_")[1]))
        elif kind in ("prefill", "prefill_fp8"):
            r = kb.bench_prefill(dev, iters, fp8=kind == "prefill_fp8")
        elif kind in ("decode_c2", "decode_c3"):
            r = kb.bench_decode(dev, iters, wl.C2 if kind == "decode_c2" else wl.C3)
        elif kind == "norm_matmul":
            r = kb.bench_norm_matmul(dev, iters)
        else:
            raise KeyError(kind)
        torch.cuda.synchronize(dev)
    tensor = "achieved_tflops" in r
    unit = "TFLOP/s" if tensor else "GB/s"
    entry = {"kernel": r["kernel"], "workload": r["workload"], "ms": r["ms"], "bound": "tensor" if tensor else "hbm",
             "achieved": r["achieved_tflops"] if tensor else r["achieved_gbs"], "peak": r["peak_tflops"] if tensor else r["peak_gbs"],
             "unit": unit, "frac": r["frac"],
             "peak_kind": f"of {r['peak_kind']}" + (" (burst GEMM rate: the kernel is timed alone)" if tensor else ""),
             "clocks": clocks.summary(), "device_status": r.get("status", 0)}
    for k in ("frac_of_sustained", "frac_of_nominal_8TBs", "tokens_per_s", "timing", "ms_copy_same_bytes", "ms_eager_launch"):
        if k in r:
            entry[k] = r[k]
    if not cpu:
        return entry
    if kind == "append":
        n_tok, hkv, d = 262144, 8, 128
        g = torch.Generator().manual_seed(5)
        pool = (torch.randn((n_tok // 16, 16, hkv, d), generator=g) * 2).to(torch.bfloat16)
        sec = _best_of(lambda: ref.fp8_quantize_pool_fast(pool))
        value = wl.append_algorithmic_bytes(n_tok, hkv, d, 2) / 2 / sec / 1e9  # one of K / V
        sample = f"{n_tok} tokens of one of K/V (Hkv 8, D 128) through the per-(block, head) quantiser, best of 3, {sec:.3f} s"
    elif kind in ("norm_256", "norm_16384"):
        rows = int(kind.split("_")[1])
        x, w, eps = wl.make_rms_norm_inputs(rows=rows, hidden=4096)
        sec = _best_of(lambda: ref.rms_norm_hal(x, w, eps))
        value = wl.rms_norm_algorithmic_bytes(rows, 4096, 2) / sec / 1e9
        sample = f"the same [{rows}, 4096] bf16 rows, best of 3, {sec:.4f} s"
    elif kind in ("prefill", "prefill_fp8"):
        pw = wl.make_prefill_workload(n_requests=1)
        rid = next(iter(pw.block_tables))
        sec = _best_of(lambda: ref.chunked_prefill(pw.q, pw.k_cache, pw.v_cache, pw.block_tables[rid], pw.ctx_lens[rid], scale=pw.scale))
        value = wl.prefill_flops(1, pw.n_heads, pw.head_dim, pw.chunk_len, pw.prefix_len) / sec / 1e12
        sample = f"one of the 32 requests (2048-token prefix + 512-token chunk), best of 3, {sec:.3f} s"
    elif kind in ("decode_c2", "decode_c3"):
        shape = wl.C2 if kind == "decode_c2" else wl.C3
        lengths = wl.config_lengths(shape)
        base = cpu_baseline(shape, lengths, 16, repeats=2)
        st_bytes = wl.decode_algorithmic_bytes(lengths, shape.n_heads, shape.n_kv_heads, shape.head_dim, 1 if shape.kv_fp8 else 2, 2, 2,
                                               shape.kv_fp8, shape.block_size)
        value = base["value"] * st_bytes / len(lengths) / 1e9  # requests/s of the sample x mean bytes per request
        sample = base["sample"] + "; GB/s = requests/s x the workload's mean algorithmic bytes per request"
    else:
        x, g, w, eps = wl.make_norm_matmul_inputs(2048, 4096, 6144)
        sec = _best_of(lambda: ref.fused_rms_norm_matmul(x, g, w, eps))
        value = 2.0 * 2048 * 4096 * 6144 / sec / 1e12
        sample = f"2048 of the 16384 rows against the same [4096, 6144] weight, best of 3, {sec:.3f} s"
    entry["cpu_baseline"] = {"value": value, "unit": unit, "cores": cores, "kind": "port", "sample": sample}
    return entry


def run_kernel_line(args: argparse.Namespace) -> None:
    """One JSON line for a single kernel of the path (not the headline step)."""
    dev = torch.device("cuda", 0)
    iters = max(args.steps, 3)
    kind = {"append": "append", "norm": "norm_16384", "prefill": "prefill", "norm_matmul": "norm_matmul"}[args.kernel]
    e = kernel_entry(kind, iters, dev)
    metric = {"append": "fp8_quantize_on_append_GBps", "norm": "rms_norm_GBps", "prefill": "chunked_prefill_TFLOPs",
              "norm_matmul": "fused_rms_norm_matmul_TFLOPs"}[args.kernel]
    roof = {"bound": e["bound"], "achieved": e["achieved"], "peak": e["peak"], "unit": e["unit"], "frac": e["frac"], "traffic": None,
            "peak_kind": e["peak_kind"]}
    line = {"metric": metric, "value": e["achieved"], "unit": e["unit"], "n_gpus": 1, "steps": iters, "warmup": 3, "ms_per_step": e["ms"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "data": "synthetic",
            "config": {"workload": e["workload"], "kernel": e["kernel"]}, "roofline": roof, "cpu_baseline": e["cpu_baseline"],
            "clocks": e["clocks"], "device_status": e["device_status"]}
    print(json.dumps(line), flush=True)


def head_partition_report(args: argparse.Namespace, world: int, rank: int, dev: torch.device, one_gpu_ms: float) -> dict | None:
    """The configuration split by kv head over the GPUs of the run (one kv head = eight query heads per GPU at eight
    GPUs): every GPU decodes ALL requests for its heads and ends the step holding the whole [B, H, D] output - gathered
    by NCCL after the decode, and by the decode kernel's own peer stores plus one signal kernel.  Strong scaling:
    `one_gpu_ms` is this run's own per-step time of one GPU serving the whole configuration."""
    import dataclasses

    import torch.distributed as dist

    from llm_compileforge_b200 import ops
    from llm_compileforge_b200.comm import PeerGather

    full = shape_of(args.workload)
    if full.n_kv_heads % world:
        return None
    shape = dataclasses.replace(full, n_heads=full.n_heads // world, n_kv_heads=full.n_kv_heads // world)
    total = args.warmup + args.steps
    st = DecodeState(shape, args.batch or shape.batch, 2 * total + 2, dev, seed_offset=0)
    chunk = pick_chunk_tokens(st.lengths, args.chunk_tokens)
    workspace = torch.zeros(ops.decode_workspace_bytes(st.batch, shape.n_heads, shape.head_dim, st.tables.shape[1], shape.block_size, chunk),
                            dtype=torch.uint8, device=dev)
    out = torch.empty_like(st.q)
    gathered = torch.empty((world,) + tuple(out.shape), dtype=out.dtype, device=dev)
    peer = PeerGather(st.batch, shape.n_heads, shape.head_dim, shape.dtype, dev)
    fp8kw = dict(k_scale=st.k_scale, v_scale=st.v_scale) if st.fp8 else {}
    tailkw = dict(k_tail=st.k_tail, v_tail=st.v_tail) if st.fp8 else {}

    def step(s: int, mode: str, ev=None) -> None:
        ops.cache_write(st.new_k, st.new_v, st.cu_one, st.pos_steps[s], st.tables, st.k_cache, st.v_cache, max_new_tokens=1, **fp8kw, **tailkw)
        if ev:
            ev[0].record()
        if mode == "peer":
            peer.decode(st.q, st.k_cache, st.v_cache, st.tables, st.len_steps[s], chunk_tokens=chunk, workspace=workspace, **fp8kw)
        else:
            ops.paged_attention_decode(st.q, st.k_cache, st.v_cache, st.tables, st.len_steps[s], scale=None, chunk_tokens=chunk,
                                       workspace=workspace, out=out, **fp8kw)
        if ev:
            ev[1].record()
        if mode == "nccl":
            dist.all_gather_into_tensor(gathered, out)

    def sync_all() -> None:
        torch.cuda.synchronize(dev)
        dist.barrier()
        torch.cuda.synchronize(dev)

    report = {"workload": f"{full.name}: {st.batch} requests on every GPU, {shape.n_kv_heads} of {full.n_kv_heads} kv heads "
                          f"({shape.n_heads} query heads) per GPU, output gathered on every GPU"}
    off = 0
    for mode in ("nccl", "peer"):
        for s in range(args.warmup):
            step(off + s, mode)
        sync_all()
        check = None
        if mode == "peer":  # the peer-stored output of the last warm-up step against decode + NCCL all-gather of the same step
            ops.paged_attention_decode(st.q, st.k_cache, st.v_cache, st.tables, st.len_steps[off + args.warmup - 1], scale=None,
                                       chunk_tokens=chunk, workspace=workspace, out=out, **fp8kw)
            dist.all_gather_into_tensor(gathered, out)
            same = torch.equal(gathered.permute(1, 0, 2, 3).reshape(peer.out.shape), peer.out) and not peer.timed_out()
            flag = torch.tensor([int(same)], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            check = "equal" if int(flag.item()) else "MISMATCH"
            sync_all()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for i in range(args.steps):
            step(off + args.warmup + i, mode, evs[i])
        t1.record()
        sync_all()
        t = torch.tensor([t0.elapsed_time(t1), sum(a.elapsed_time(b) for a, b in evs) / args.steps], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t[0].item() / args.steps
        entry = {"tokens_per_s": st.batch / (ms / 1e3), "ms_per_step": ms, "decode_call_ms": t[1].item(),
                 "decode_gbs_per_gpu": st.algorithmic_bytes(off + args.warmup + args.steps // 2) / (t[1].item() / 1e3) / 1e9,
                 "strong_scaling_vs_one_gpu": one_gpu_ms / ms}
        if check:
            entry["gather_check"] = check
        report["gather_" + mode] = entry
        off += total
    st_bits = ops.read_status(workspace) | (4 if peer.timed_out() else 0)
    flag = torch.tensor([st_bits], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    report["device_status"] = int(flag.item())
    report["one_gpu_ms_per_step"] = one_gpu_ms
    return report if rank == 0 else {}


def workload_config(shape: wl.DecodeShape, batch: int, args: argparse.Namespace, chunk: int) -> dict:
    return {
        "workload": f"{shape.name} paged decode, {batch} requests per GPU, H {shape.n_heads}/{shape.n_kv_heads}, "
                    f"D {shape.head_dim}, block 16, {'e4m3 KV + fp32 scales' if shape.kv_fp8 else 'bf16 KV'}",
        "requests_per_gpu": batch, "partition": "by kv head" if getattr(args, "partition", "request") == "head" and args.gpus > 1 else "by request",
        "chunk_tokens": chunk,
        "l2": "pool (GBs) >> L2, no flush needed", "step": "kv append (1 token/request) + split-K decode (in-kernel merge)",
    }


def main() -> None:
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.kernel != "decode":
        if not torch.cuda.is_available():
            raise SystemExit("bench.py --kernel needs a CUDA device")
        if rank == 0:
            run_kernel_line(args)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path); use --impl reference for the CPU arm")

    import torch.distributed as dist

    from llm_compileforge_b200 import B200Backend, ops

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    host_binding = bind_to_gpu_cpus(local_rank) if world > 1 else "single rank: not bound"
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    shape = shape_of(args.workload)
    by_head = args.partition == "head" and world > 1
    if by_head:
        if shape.n_kv_heads % world:
            raise SystemExit(f"{shape.n_kv_heads} kv heads do not divide over {world} GPUs")
        import dataclasses

        shape = dataclasses.replace(shape, n_heads=shape.n_heads // world, n_kv_heads=shape.n_kv_heads // world)
    total_steps = args.warmup + args.steps
    # three passes (device-resident, end-to-end one step at a time, end-to-end pipelined) each append `total_steps` tokens
    st = DecodeState(shape, args.batch or shape.batch, 3 * total_steps + 2, dev, seed_offset=0 if by_head else rank * 100)
    chunk = pick_chunk_tokens(st.lengths, args.chunk_tokens)
    ws_bytes = ops.decode_workspace_bytes(st.batch, shape.n_heads, shape.head_dim, st.tables.shape[1], shape.block_size, chunk)
    workspace = torch.zeros(ws_bytes, dtype=torch.uint8, device=dev)
    n_chunks = -(-st.tables.shape[1] * shape.block_size // chunk)
    pool_bound = st.batch * st.tables.shape[1] * shape.block_size * shape.n_kv_heads * shape.head_dim * (1 if st.fp8 else 2) * 2
    worklist = n_chunks > 1 and st.batch * n_chunks >= 600 and pool_bound >= (1 << 30)
    out = torch.empty_like(st.q)
    gathered = torch.empty((world,) + tuple(out.shape), dtype=out.dtype, device=dev) if (args.gather == "nccl" and world > 1) else None
    peer = None
    if args.gather == "peer" and world > 1:
        if not by_head:
            raise SystemExit("--gather peer goes with --partition head")
        from llm_compileforge_b200.comm import PeerGather

        peer = PeerGather(st.batch, shape.n_heads, shape.head_dim, shape.dtype, dev)
    # (head partition: rank g's slab is heads [g*H/N, (g+1)*H/N) of every request; `gathered[g]` is that slab)
    be = B200Backend(device=dev)
    fp8kw = dict(k_scale=st.k_scale, v_scale=st.v_scale) if st.fp8 else {}
    tailkw = dict(k_tail=st.k_tail, v_tail=st.v_tail) if st.fp8 else {}

    def step_device(s: int, ev=None) -> None:
        ops.cache_write(st.new_k, st.new_v, st.cu_one, st.pos_steps[s], st.tables, st.k_cache, st.v_cache,
                        max_new_tokens=1, **fp8kw, **tailkw)
        if ev:
            ev[0].record()
        if peer is not None:
            peer.decode(st.q, st.k_cache, st.v_cache, st.tables, st.len_steps[s], chunk_tokens=chunk, workspace=workspace, **fp8kw)
        else:
            ops.paged_attention_decode(st.q, st.k_cache, st.v_cache, st.tables, st.len_steps[s], scale=None,
                                       chunk_tokens=chunk, workspace=workspace, out=out, **fp8kw)
        if ev:
            ev[1].record()
        if gathered is not None:
            dist.all_gather_into_tensor(gathered, out)

    def sync_all() -> None:
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(dev)

    # ---- device-resident timing -------------------------------------------------
    for s in range(args.warmup):
        step_device(s)
    sync_all()
    gather_check = None
    if peer is not None:
        # the peer-stored output of the last warm-up step against decode + NCCL all-gather of the same step
        ops.paged_attention_decode(st.q, st.k_cache, st.v_cache, st.tables, st.len_steps[args.warmup - 1], scale=None,
                                   chunk_tokens=chunk, workspace=workspace, out=out, **fp8kw)
        parts = torch.empty((world,) + tuple(out.shape), dtype=out.dtype, device=dev)
        dist.all_gather_into_tensor(parts, out)
        same = torch.equal(parts.permute(1, 0, 2, 3).reshape(peer.out.shape), peer.out) and not peer.timed_out()
        flag = torch.tensor([int(same)], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        gather_check = "peer-stored output == decode + NCCL all-gather on every rank" if int(flag.item()) else "MISMATCH"
        sync_all()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        t_start.record()
        for i in range(args.steps):
            step_device(args.warmup + i, evs[i])
        t_end.record()
        sync_all()
    elapsed_ms = t_start.elapsed_time(t_end)
    decode_ms = sum(a.elapsed_time(b) for a, b in evs) / args.steps  # the decode call: status memset + decode kernel
    status = ops.read_status(workspace)

    # ---- end to end: host buffers in, host result out, through the step pipeline -----------
    # Every step copies q, new K, new V and positions from pinned host memory, grows the block tables on the host,
    # sends the table delta, appends, attends, and copies the result back to pinned host memory.  Two passes:
    # one step at a time (submit, then wait for its result), then with IN_FLIGHT steps in flight.
    from llm_compileforge_b200.step_pipeline import AttentionStepPipeline

    in_flight_max = IN_FLIGHT + (1 if world >= 4 else 0)  # one more step in flight when several ranks share the host's links
    pipe = AttentionStepPipeline(st.bm, st.k_cache, st.v_cache, max_batch=st.batch, n_heads=shape.n_heads, dtype=shape.dtype,
                                 chunk_tokens=chunk, depth=in_flight_max, time_copies=True, **fp8kw, **tailkw)
    # one pinned arena per rank, laid out like the pipeline's staging slot: q | new K | new V go over in a single copy
    host_packed, host_q, host_k, host_v = pipe.host_arena()
    host_q.copy_(st.q)
    host_k.copy_(st.new_k)
    host_v.copy_(st.new_v)
    sync_all()

    def run_e2e(first: int, n: int, in_flight: int) -> tuple[float, int, int]:
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        h2d = d2h = 0
        t0.record()
        pending: list[int] = []
        for i in range(n):
            pending.append(pipe.submit(st.rids, host_q, host_k, host_v, st.pos_steps_host[first + i], packed=host_packed))
            h2d += pipe.h2d_bytes
            d2h += pipe.d2h_bytes
            if len(pending) >= in_flight:
                pipe.result(pending.pop(0))  # the caller reads every step's result on the host
        while pending:
            pipe.result(pending.pop(0))
        t1.record()
        torch.cuda.synchronize(dev)
        return t0.elapsed_time(t1), h2d // max(n, 1), d2h // max(n, 1)

    off = total_steps
    run_e2e(off, args.warmup, 1)
    sync_all()
    serial_ms, _, _ = run_e2e(off + args.warmup, args.steps, 1)
    sync_all()
    off += total_steps
    run_e2e(off, args.warmup, in_flight_max)
    sync_all()
    pipe.h2d_ms = pipe.d2h_ms = 0.0
    pipe.h2d_timed = pipe.d2h_timed = 0
    e2e_ms, h2d, d2h = run_e2e(off + args.warmup, args.steps, in_flight_max)
    sync_all()
    status |= pipe.status()
    # device time of the copies themselves in the pipelined pass (CUDA events on the copy streams)
    h2d_gbs = pipe.h2d_timed / max(pipe.h2d_ms, 1e-9) / 1e6
    d2h_gbs = pipe.d2h_timed / max(pipe.d2h_ms, 1e-9) / 1e6

    if world > 1:
        t = torch.tensor([elapsed_ms, e2e_ms, decode_ms, serial_ms, -h2d_gbs, -d2h_gbs], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms, e2e_ms, decode_ms, serial_ms = t.tolist()[:4]
        h2d_gbs, d2h_gbs = -t[4].item(), -t[5].item()  # the slowest rank's copy rates
        tot = torch.tensor([st.batch], dtype=torch.int64, device=dev)
        dist.all_reduce(tot)
        total_requests = st.batch if by_head else int(tot.item())
    else:
        total_requests = st.batch

    extras: dict = {}
    cpu_line = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_line = cpu_baseline(shape, st.lengths, min(args.cpu_sample, st.batch), repeats=3)
    algorithmic = st.algorithmic_bytes(args.warmup + args.steps // 2)
    state_batch = st.batch
    peer_used, peer_gave_up = peer is not None, bool(peer is not None and peer.timed_out())
    if not args.headline_only and not by_head and (world > 1 or (args.workload == "c5" and not args.batch)):
        # the other kernels of the path (1 GPU) / the configuration's own kv-head layout (N GPUs): free the headline state first
        del pipe, st, workspace, out, gathered, peer
        torch.cuda.empty_cache()
        try:
            if world == 1:
                extras["kernels"] = {k: kernel_entry(k, 20, dev, cpu=not args.no_cpu_baseline) for k in KERNEL_KINDS if k != "norm_matmul"}
            elif args.workload == "c5" and shape.n_kv_heads % world == 0:
                rep = head_partition_report(args, world, rank, dev, elapsed_ms / args.steps)
                if rep:
                    extras["head_partition"] = rep
        except Exception as e:  # noqa: BLE001  (the headline line is still printed)
            extras["extras_error"] = f"{type(e).__name__}: {e}"

    if rank == 0:
        ms_per_step = elapsed_ms / args.steps
        value = total_requests / (ms_per_step / 1e3)
        peak, peak_kind = peaks()
        alg = algorithmic
        achieved = alg / (decode_ms / 1e3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong" if by_head else "weak", "vs_baseline": None,
            "dtype": "e4m3 KV, bf16 q/out, f32 accumulate" if shape.kv_fp8 else "bf16",
            "data": "synthetic", "config": workload_config(shape, state_batch, args, chunk),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": alg * TRAFFIC_PER_ALGORITHMIC_BYTE, "peak_kind": f"of {peak_kind}", "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS,
                         "kernel": "decode_tma_kernel (split-K, in-kernel merge)", "algorithmic_bytes_per_launch": alg,
                         "avg_launch_ms": decode_ms},
            "e2e": {"value": total_requests / (e2e_ms / args.steps / 1e3), "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "steps_in_flight": in_flight_max,
                    "h2d_gbs_per_rank": h2d_gbs, "d2h_gbs_per_rank": d2h_gbs,
                    "one_step_at_a_time": total_requests / (serial_ms / args.steps / 1e3),
                    "table_upload": "device-resident tables; only ids of added blocks are sent", "host_binding": host_binding},
            # per step: cache_write_kernel + decode_tma_kernel (split merge is in-kernel), + decode_worklist_kernel when the
            # split has >= 600 (request, chunk) slots over a pool bound of >= 1 GiB (the launcher's rule), + the peer signal kernel
            "gpu_launches": args.steps * (2 + int(worklist) + int(peer_used)),
            "clocks": clocks.summary(),
            "device_status": status | (4 if peer_gave_up else 0),
        }
        if args.gather:
            line["config"]["gather"] = args.gather
        if gather_check:
            line["gather_check"] = gather_check
        if cpu_line:
            line["cpu_baseline"] = cpu_line
        line.update(extras)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
