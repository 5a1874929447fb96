"""Host-side logic: table adapters, request partitioning, workload generators,
HAL dispatch and fallback chaining.  CPU only."""

import pytest
import torch

from llm_compileforge_b200 import workloads as wl
from llm_compileforge_b200.hal import B200Backend, OpExecutor
from llm_compileforge_b200.tables import dense_block_tables, partition_by_request, pick_chunk_tokens


def test_dense_tables_follow_reference_rules():
    tables = {"nolen": [3, 4], "toolong": [5, 1], "surplus": [0, 2, 7, 9], "one": [11]}
    lens = {"toolong": 100, "surplus": 17, "one": 1}
    dense, ll, rids = dense_block_tables(tables, lens, 16, n_pool_blocks=12)
    assert rids == ["nolen", "toolong", "surplus", "one"]  # insertion order, not sorted
    assert ll.tolist() == [32, 32, 17, 1]  # missing -> capacity; over-long -> capacity
    assert dense.dtype == torch.int32 and dense.shape == (4, 2)
    assert dense[2].tolist() == [0, 2]  # blocks past ceil(17/16) dropped
    assert dense[3].tolist() == [11, 0]


def test_partition_is_contiguous_and_balanced():
    lengths = wl.config_lengths(wl.C5, batch=512)
    parts = partition_by_request(lengths, 8)
    flat = [i for p in parts for i in p]
    assert flat == list(range(512))
    loads = [sum(lengths[i] for i in p) for p in parts]
    assert max(loads) <= 1.15 * (sum(lengths) / 8)


def test_split_size_fills_whole_waves():
    """KV split of the decode kernel: large batches take the largest split that still makes about 1.4 waves of
    (request, chunk) items on the 2 x 148 SM slots; a small batch the smallest split whose items fit one wave."""
    slots = 2 * 148
    items = lambda lens, c: sum(-(-n // c) for n in lens)
    for shape, want in ((wl.C5, 2048), (wl.C3, 2048), (wl.C2, 640)):
        lens = wl.config_lengths(shape)
        c = pick_chunk_tokens(lens)
        assert c == want and c % 16 == 0
        assert items(lens, c) * 10 >= 14 * slots or items(lens, c) <= slots
    assert pick_chunk_tokens([]) == 256 and pick_chunk_tokens([0, 0]) == 256
    assert pick_chunk_tokens([100, 90, 7]) == 256          # a handful of short requests: one wave at the smallest split
    assert pick_chunk_tokens([2000] * 200) == 512          # 800 items: 2.7 waves of 512-token items
    lens = [3000] * 60                                     # under 1.4 waves even at 512: the first split with <= 296 items
    c = pick_chunk_tokens(lens)
    assert items(lens, c) <= slots and items(lens, c - 64) > slots
    assert pick_chunk_tokens([8192] * 128, head_groups=4) == 2048


def test_config_generators():
    assert all(64 <= n <= 512 for n in wl.config_lengths(wl.C1))
    l3 = wl.config_lengths(wl.C3)
    assert len(l3) == 256 and min(l3) >= 128 and max(l3) <= 8192
    med = sorted(l3)[128]
    assert 1500 < med < 2800
    w = wl.make_decode_workload(wl.C1)
    assert w.q.shape == (8, 12, 64) and w.k_cache.shape == (512, 16, 12, 64)
    ids = [b for t in w.block_tables.values() for b in t]
    assert len(ids) == len(set(ids))  # non-overlapping
    # algorithmic bytes: K+V per valid token per kv head dominate
    n = wl.decode_algorithmic_bytes([100], 32, 8, 128, 1, 2, 2, True)
    assert n == 2 * 100 * 8 * 128 + 2 * 7 * 8 * 4 + 4 * 7 + 4 + 32 * 128 * 4
    assert wl.prefill_flops(32, 32, 128, 512, 2048) == 4 * 128 * 32 * 32 * (512 * 2048 + 512 * 513 // 2)


class _Recorder(OpExecutor):
    def __init__(self):
        self.calls = []

    def execute(self, op_name, inputs, **kwargs):
        self.calls.append(op_name)
        return "fallback"


def test_backend_dispatch_and_fallback():
    rec = _Recorder()
    be = B200Backend(fallback=rec)
    assert be.execute("matmul", [1, 2]) == "fallback" and rec.calls == ["matmul"]
    assert {"paged_attention", "cache_write", "quantize", "dequantize", "rms_norm", "fused_rms_norm_add"} <= set(be.supported_ops())
    with pytest.raises(ValueError, match="Unknown op"):
        B200Backend().execute("softmax", [torch.zeros(2)])
    with pytest.raises(ValueError, match="fp8"):
        be.execute("quantize", [torch.zeros(2)], dtype="int8")


def test_b200_hardware_spec_has_the_loader_schema():
    """hardware_specs/b200.yaml follows the key set of the reference's hardware_specs/*.yaml (python_runtime/hal/
    hardware_spec.py: ComputeUnit, MemoryLevel, Interconnect fields) and quotes the measured roofline denominators."""
    import json
    import os

    import yaml

    import llm_compileforge_b200 as pkg

    root = os.path.dirname(os.path.abspath(pkg.__file__))
    spec = yaml.safe_load(open(os.path.join(root, "hardware_specs", "b200.yaml")))
    assert set(spec) == {"name", "compute_units", "memory_levels", "interconnects", "op_latency_us"}
    for cu in spec["compute_units"]:
        assert {"name", "fp32_tflops", "fp16_tflops", "bf16_tflops", "int8_tops", "int4_tops"} <= set(cu)
    for ml in spec["memory_levels"]:
        assert set(ml) == {"name", "size_gb", "bandwidth_gbs", "latency_ns"}
    for ic in spec["interconnects"]:
        assert set(ic) == {"name", "bandwidth_gbs", "latency_us", "topology"}
    assert "default" in spec["op_latency_us"] and "paged_attention" in spec["op_latency_us"]
    peaks_path = os.path.join(os.path.dirname(root), "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peaks = json.load(open(peaks_path))
        hbm = [m for m in spec["memory_levels"] if m["name"].startswith("HBM")][0]
        tensor = [c for c in spec["compute_units"] if "Tensor" in c["name"]][0]
        assert abs(hbm["bandwidth_gbs"] - peaks["hbm_gbs"]) < 1 and abs(tensor["bf16_tflops"] - peaks["bf16_tflops_sustained"]) < 1


def test_norm_matmul_plan_follows_the_intake_cost_model():
    """The fused norm-matmul launcher's tile shape (host arithmetic behind ``sfb_fused_rms_norm_matmul_plan``): every
    candidate costs rounds-of-tiles-on-the-busiest-SM x rows taken in per K step; the cluster of two only with a
    workspace for its statistics pre-pass and only when strictly cheaper."""
    from llm_compileforge_b200 import ops

    plan = ops.norm_matmul_plan
    # decode-sized: 64-wide tiles, an SM each (96 tiles on 148 SMs) -> two K steps per stage; the x box holds the rows there are
    assert plan(1, 6144) == dict(pair=0, tile_n=64, stages=4, k_steps_per_stage=2, prepass=0, x_box_rows=8)
    assert plan(100, 6144)["x_box_rows"] == 104 and plan(128, 6144)["x_box_rows"] == 128
    # 256 rows: 64-wide would need two rounds (192 tiles), 256-wide leaves 100 SMs idle: 128-wide, six stages, one launch
    assert plan(256, 6144) == dict(pair=0, tile_n=128, stages=6, k_steps_per_stage=1, prepass=0, x_box_rows=128)
    # more 64-wide tiles than SMs (300 of them, three rounds of 8 + 64 rows against two of 8 + 128 or one of 8 + 256):
    # two thread blocks per SM, one K step per stage
    assert plan(8, 19200) == dict(pair=0, tile_n=64, stages=4, k_steps_per_stage=1, prepass=0, x_box_rows=8)
    # from 512 rows on the cluster of two is cheaper (48 pair tiles: 1 x 256 against 1 x 384) - if there is a workspace
    assert plan(512, 6144) == dict(pair=1, tile_n=256, stages=6, k_steps_per_stage=1, prepass=1, x_box_rows=128)
    assert plan(512, 6144, has_workspace=False) == dict(pair=0, tile_n=256, stages=4, k_steps_per_stage=1, prepass=0, x_box_rows=128)
    assert plan(512, 6144, clusters=0)["pair"] == 0  # a device that cannot co-schedule the pair
    # prefill-sized: pair + pre-pass; without a workspace the single-block kernel with in-kernel statistics
    assert plan(16384, 6144)["pair"] == 1 and plan(16384, 6144)["prepass"] == 1
    big = plan(16384, 6144, has_workspace=False)
    assert (big["pair"], big["tile_n"], big["prepass"]) == (0, 256, 0)
    # ties between widths go to the wider tile: 2 x 384 (256-wide, 165 tiles) = 3 x 256 (128-wide, 315 tiles)
    assert plan(1920, 2568, has_workspace=False)["tile_n"] == 256
    with pytest.raises(ValueError):
        plan(-1, 8)
