"""Shared test helpers: golden fixtures, tolerances, dense-table utilities."""

from __future__ import annotations

import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# Tolerances stated by the benchmark contract:
#   float32 outputs: 1e-5 relative (to the tensor's scale), bf16 / FP8-KV attention
#   outputs: 2e-2 absolute and a cosine-similarity deficit of at most 1e-4;
#   e4m3 codes, scales and slot indices: bit-exact.
F32_REL = 1e-5
HALF_ABS = 2e-2
COS_DEFICIT = 1e-4


def golden(name: str):
    return np.load(os.path.join(GOLDEN, name))


def from_bits(a: np.ndarray, dtype: torch.dtype) -> torch.Tensor:
    """Undo tests/golden/make_golden.py's ``bits``."""
    if dtype == torch.bfloat16:
        return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)
    if dtype == torch.float8_e4m3fn:
        return torch.from_numpy(a.copy()).view(torch.float8_e4m3fn)
    return torch.from_numpy(a.copy())


def tables_to_dict(dense: np.ndarray, table_lens, seq_lens, names=None):
    tables, lens = {}, {}
    for i in range(dense.shape[0]):
        rid = names[i] if names else f"req_{i}"
        tables[rid] = [int(x) for x in dense[i, : int(table_lens[i])]]
        if seq_lens[i] >= 0:
            lens[rid] = int(seq_lens[i])
    return tables, lens


def cos_deficit(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.double().flatten(), b.double().flatten()
    return 1.0 - float(torch.dot(a, b) / (a.norm() * b.norm()))


def assert_f32_close(got: torch.Tensor, ref: torch.Tensor, rel: float = F32_REL, what: str = ""):
    err = (got.double() - ref.double()).abs().max().item()
    scale = ref.double().abs().max().item()
    assert err <= rel * scale, f"{what}: max |diff| {err:.3e} > {rel:g} * max|ref| {scale:.3e}"


def assert_half_close(got: torch.Tensor, ref: torch.Tensor, what: str = ""):
    err = (got.double() - ref.double()).abs().max().item()
    assert err <= HALF_ABS, f"{what}: max |diff| {err:.3e} > {HALF_ABS}"
    cd = cos_deficit(got, ref)
    assert cd <= COS_DEFICIT, f"{what}: cosine deficit {cd:.3e} > {COS_DEFICIT}"


def assert_half_close_ulp(got: torch.Tensor, ref: torch.Tensor, what: str = ""):
    """HALF_ABS plus one bf16 unit in the last place of the reference value (2^-7 relative covers it): a result on a
    rounding boundary may land on either neighbour, and from |y| >= 4 one bf16 step alone is 3.1e-2."""
    g, w = got.double(), ref.double()
    excess = ((g - w).abs() - 2.0 ** -7 * w.abs()).max().item()
    assert excess <= HALF_ABS, f"{what}: |diff| exceeds {HALF_ABS} + 1 ulp by {excess - HALF_ABS:.3e}"
    cd = cos_deficit(got, ref)
    assert cd <= COS_DEFICIT, f"{what}: cosine deficit {cd:.3e} > {COS_DEFICIT}"


def stack_outputs(out: dict, rids) -> torch.Tensor:
    return torch.stack([out[r] for r in rids])


def assert_same(got: torch.Tensor, ref: torch.Tensor):
    """The torch-CPU restatement runs the same operators as the reference, so on
    the machine that made the fixtures it is bit-identical.  A different CPU
    (vector width, thread count) may reorder float sums inside those operators;
    then results must still agree to rounding: 2e-6 relative for float32, one
    unit in the last place for bfloat16."""
    if torch.equal(got, ref):
        return
    assert got.dtype == ref.dtype and got.shape == ref.shape
    scale = ref.double().abs().max().item()
    err = (got.double() - ref.double()).abs().max().item()
    tol = 2e-6 if got.dtype == torch.float32 else 2.0 ** -7
    assert err <= tol * scale, f"restatement differs from the reference fixture: {err:.3e} (scale {scale:.3e})"
