"""RMSNorm on the GPU against the HAL-operator oracle and the reference fixtures."""

import numpy as np
import pytest
import torch

import llm_compileforge_b200 as pkg
from helpers import assert_f32_close, from_bits, golden
from llm_compileforge_b200 import ops
from llm_compileforge_b200 import workloads as wl
from oracle import reference_port as ref

pytestmark = pytest.mark.gpu


def test_hal_rms_norm_bf16_config3(cuda):
    g = golden("rms_norm.npz")
    be = pkg.B200Backend()
    x, w, eps = wl.make_rms_norm_inputs(rows=8, hidden=4096)
    got = be.execute("rms_norm", [x.to(cuda), w.to(cuda)], eps=eps).cpu()
    want = from_bits(g["hal_bf16.out"], torch.bfloat16)
    assert got.dtype == torch.bfloat16
    assert (got.float() - want.float()).abs().max() <= 2e-2
    # float32 arithmetic with one final rounding: at most a rare one-ulp flip
    assert (got != want).float().mean() < 1e-3
    x, w, eps = wl.make_rms_norm_inputs()  # the full [256, 4096]
    got = be.execute("rms_norm", [x.to(cuda), w.to(cuda)], eps=eps).cpu()
    want = ref.rms_norm_hal(x, w, eps)
    assert (got.float() - want.float()).abs().max() <= 2e-2
    assert (got != want).float().mean() < 1e-3


def test_hal_rms_norm_f32_and_odd_width(cuda):
    g = golden("rms_norm.npz")
    be = pkg.B200Backend()
    xf, wf = torch.from_numpy(g["hal_f32.x"]).to(cuda), torch.from_numpy(g["hal_f32.w"]).to(cuda)  # [5, 333]
    assert_f32_close(be.execute("rms_norm", [xf, wf], eps=1e-5).cpu(), torch.from_numpy(g["hal_f32.out"]))
    assert_f32_close(be.execute("rms_norm", [xf], eps=1e-5).cpu(), torch.from_numpy(g["hal_f32_noweight.out"]))
    xs = torch.from_numpy(g["contract_2x4.x"]).to(cuda)
    got = be.execute("rms_norm", [xs, torch.ones(4, device=cuda)]).cpu()
    assert (got - torch.from_numpy(g["contract_2x4.out"])).abs().max() < 1e-6


def test_fused_rms_norm_add(cuda):
    g = golden("rms_norm.npz")
    x, r, w = (torch.from_numpy(g[f"fused_f32.{n}"]) for n in "xrw")
    got = pkg.fused_rms_norm_add(x.to(cuda), r.to(cuda), w.to(cuda), eps=1e-6).cpu()
    assert_f32_close(got, torch.from_numpy(g["fused_f32.out"]))
    # bf16: float32 intermediates; the reference's own bf16 path rounds after every step
    xb, rb, wb = x.bfloat16(), r.bfloat16(), w.bfloat16()
    got = pkg.fused_rms_norm_add(xb.to(cuda), rb.to(cuda), wb.to(cuda), eps=1e-6).cpu()
    want = ref.fused_rms_norm_add_f32_internal(xb, rb, wb, 1e-6)
    assert (got.float() - want.float()).abs().max() <= 2e-2
    ref_bf16 = from_bits(g["fused_bf16.out"], torch.bfloat16)
    assert torch.nn.functional.cosine_similarity(got.float().flatten(), ref_bf16.float().flatten(), dim=0) >= 0.999
    # reference behaviours: batched input keeps its shape, zeros stay finite, eps matters
    y = pkg.fused_rms_norm_add(torch.randn(2, 8, 64, device=cuda), torch.randn(2, 8, 64, device=cuda), torch.randn(64, device=cuda))
    assert y.shape == (2, 8, 64)
    z = pkg.fused_rms_norm_add(torch.zeros(3, 32, device=cuda), torch.zeros(3, 32, device=cuda), torch.ones(32, device=cuda))
    assert torch.isfinite(z).all()
    a = torch.randn(2, 16, device=cuda)
    o = torch.ones(16, device=cuda)
    assert not torch.allclose(pkg.fused_rms_norm_add(a, a, o, eps=1e-3), pkg.fused_rms_norm_add(a, a, o, eps=1e-8))


@pytest.mark.parametrize("shape", [(16384, 4096), (7, 8192), (3, 16384), (1, 128)])
def test_rms_norm_large_and_long_rows(cuda, shape):
    gen = torch.Generator().manual_seed(8)
    x = torch.randn(shape, generator=gen).bfloat16()
    w = (1 + 0.02 * torch.randn(shape[1], generator=gen)).bfloat16()
    got = ops.rms_norm(x.to(cuda), w.to(cuda), 1e-5).cpu()
    rows = slice(0, 64)
    want = ref.rms_norm_hal(x[rows], w, 1e-5)
    assert (got[rows].float() - want.float()).abs().max() <= 2e-2
    # scale invariance up to eps: norm(2x) == norm(x) wherever mean(x^2) >> eps
    got2 = ops.rms_norm((x * 2).to(cuda), w.to(cuda), 1e-5).cpu()
    assert (got2.float() - got.float()).abs().max() <= 2e-2
