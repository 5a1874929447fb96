"""fused_rms_norm_matmul: the oracle restatement against fixtures made by the reference's backend (CPU), and the
tcgen05 kernel against both (GPU).  Tolerance: the output is one bf16 / fp16 rounding of an fp32 result whose inputs
differ from the reference's by one extra rounding of the folded weight, so |diff| <= 2e-2 on unit-variance outputs
and cosine deficit <= 1e-4, the same bounds as the other half-precision operators."""

import numpy as np
import pytest
import torch

from helpers import assert_half_close, from_bits, golden
from llm_compileforge_b200 import workloads as wl
from oracle import reference_port as ref

CASES = {"bf16_a": torch.bfloat16, "bf16_b": torch.bfloat16, "f16_a": torch.float16}


from helpers import assert_half_close_ulp as assert_close_one_ulp  # noqa: E402


def _want(g, name, dtype):
    raw = g[name + ".out"]
    return from_bits(raw, torch.bfloat16) if dtype == torch.bfloat16 else torch.from_numpy(raw)


@pytest.mark.parametrize("name", list(CASES))
def test_oracle_matches_reference_fixture(name):
    g = golden("norm_matmul.npz")
    m, k, n = (int(v) for v in g[name + ".shape"])
    x, rw, w, eps = wl.make_norm_matmul_inputs(m, k, n, CASES[name])
    torch.set_num_threads(1)
    got = ref.fused_rms_norm_matmul(x, rw, w, eps)
    assert got.dtype == CASES[name]
    assert torch.equal(got, _want(g, name, CASES[name]))  # same operators in the same order: bit for bit


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(CASES))
def test_kernel_matches_reference_fixture(name):
    import llm_compileforge_b200 as pkg

    dev = torch.device("cuda:0")
    g = golden("norm_matmul.npz")
    m, k, n = (int(v) for v in g[name + ".shape"])
    x, rw, w, eps = wl.make_norm_matmul_inputs(m, k, n, CASES[name])
    got = pkg.B200Backend(device=dev).execute("fused_rms_norm_matmul", [x.to(dev), rw.to(dev), w.to(dev)], eps=eps)
    assert got.dtype == CASES[name] and tuple(got.shape) == (m, n)
    assert_half_close(got.cpu(), _want(g, name, CASES[name]), what=name)


@pytest.mark.gpu
@pytest.mark.parametrize("m,k,n", [(1, 64, 8), (128, 64, 256), (129, 72, 264), (300, 4096, 1024), (1000, 520, 776), (2048, 1024, 2304),
                                   # 256-wide tiles, several tiles per persistent thread block: statistics pre-pass ...
                                   (4096, 512, 2560),
                                   # ... and statistics inside the kernel (fewer than 2048 rows, but more tiles than SMs)
                                   (1920, 320, 2568),
                                   # 128-wide tiles with the six-stage ring (few rows, wide output): whole and ragged
                                   (256, 4096, 6144), (200, 1000, 9000),
                                   # clusters of two thread blocks on 256 x 256 tiles (pre-pass statistics, enough tiles for every
                                   # cluster): the last row block and the last column block are ragged in the second block's half
                                   (2300, 1000, 2440),
                                   # fewer than 128 rows: the box of x is cut to the rows present (16, 64, 104 of them)
                                   (16, 1024, 3072), (64, 4096, 6144), (100, 520, 776),
                                   # more 64-wide tiles than SMs: two thread blocks share an SM, one K step per stage
                                   (8, 264, 19200)])
def test_kernel_matches_oracle_ragged(m, k, n):
    """Ragged M / N / K (rows past M, columns past N and a partial last K step are zero-filled by TMA and never stored),
    several K rounds of the operand ring, strided input rows; status word stays clean."""
    from llm_compileforge_b200 import ops

    dev = torch.device("cuda:0")
    x, rw, w, eps = wl.make_norm_matmul_inputs(m, k, n, torch.bfloat16, seed=m + k + n)
    wide = torch.zeros((m, k + 8), dtype=torch.bfloat16)
    wide[:, :k] = x
    xs = wide.to(dev)[:, :k]  # row stride k + 8
    ws = torch.empty(ops.norm_matmul_workspace_bytes(m), dtype=torch.uint8, device=dev)
    folded = ops.fold_norm_weight(rw.to(dev), w.to(dev))
    assert torch.equal(folded.cpu(), (rw.float()[:, None] * w.float()).to(torch.bfloat16))
    got = ops.fused_rms_norm_matmul(xs, folded, eps=eps, workspace=ws)
    want = ref.fused_rms_norm_matmul(x, rw, w, eps)
    assert ops.read_status(ws) == 0
    if m >= 2048:  # the statistics pre-pass ran; without a workspace for it the same rows go through the in-kernel statistics
        small = torch.empty(256, dtype=torch.uint8, device=dev)
        assert_close_one_ulp(ops.fused_rms_norm_matmul(xs, folded, eps=eps, workspace=small).cpu(), want, what='in-kernel statistics')
    assert_close_one_ulp(got.cpu(), want, what=f"{m}x{k}x{n}")
    # linearity in the weight: doubling W doubles y exactly (a power of two commutes with every rounding)
    got2 = ops.fused_rms_norm_matmul(xs, ops.fold_norm_weight(rw.to(dev), (w * 2).to(dev)), eps=eps)
    assert torch.equal(got2, got * 2)


@pytest.mark.gpu
def test_fp16_and_empty_shapes():
    from llm_compileforge_b200 import ops

    dev = torch.device("cuda:0")
    x, rw, w, eps = wl.make_norm_matmul_inputs(333, 1032, 520, torch.float16, seed=9)
    got = ops.fused_rms_norm_matmul(x.to(dev), ops.fold_norm_weight(rw.to(dev), w.to(dev)), eps=eps)
    want = ref.fused_rms_norm_matmul(x, rw, w, eps)
    assert got.dtype == torch.float16
    assert_half_close(got.cpu(), want, what="fp16 333x1032x520")
    empty = ops.fused_rms_norm_matmul(x.to(dev)[:0], ops.fold_norm_weight(rw.to(dev), w.to(dev)), eps=eps)
    assert tuple(empty.shape) == (0, 520)
    batched = ops.fused_rms_norm_matmul(x.to(dev)[:330].view(3, 110, 1032), ops.fold_norm_weight(rw.to(dev), w.to(dev)), eps=eps)
    assert tuple(batched.shape) == (3, 110, 520) and torch.equal(batched.view(330, 520), got[:330])
    # fp16 through the two-thread-block kernel (enough 256 x 256 tiles, workspace for the pre-pass); and the two kernels agree:
    # without a workspace the same call runs one thread block per tile with the statistics taken in the kernel
    x, rw, w, eps = wl.make_norm_matmul_inputs(2100, 264, 2600, torch.float16, seed=10)
    folded = ops.fold_norm_weight(rw.to(dev), w.to(dev))
    ws = torch.empty(ops.norm_matmul_workspace_bytes(2100), dtype=torch.uint8, device=dev)
    pair = ops.fused_rms_norm_matmul(x.to(dev), folded, eps=eps, workspace=ws)
    assert ops.read_status(ws) == 0
    want = ref.fused_rms_norm_matmul(x, rw, w, eps)
    assert_half_close(pair.cpu(), want, what="fp16 2100x264x2600, clusters of two")
    single = ops.fused_rms_norm_matmul(x.to(dev), folded, eps=eps, workspace=torch.empty(256, dtype=torch.uint8, device=dev))
    assert_half_close(single.cpu(), want, what="fp16 2100x264x2600, one block per tile")
    assert (pair.float() - single.float()).abs().max().item() <= 2.0 ** -9 * want.abs().max().item()  # at most one rounding apart


@pytest.mark.gpu
def test_fp32_goes_to_the_fallback_or_is_refused():
    import llm_compileforge_b200 as pkg

    dev = torch.device("cuda:0")
    x, rw, w, eps = wl.make_norm_matmul_inputs(4, 64, 8, torch.float32)
    with pytest.raises(ValueError):
        pkg.B200Backend(device=dev).execute("fused_rms_norm_matmul", [x.to(dev), rw.to(dev), w.to(dev)], eps=eps)
