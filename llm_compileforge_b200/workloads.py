"""Seeded synthetic inputs with the shapes and value distributions of the five
benchmark configurations (stand-ins for serving traces; no dataset involved).

Host-side only: every generator returns CPU tensors and plain Python lists, the
layouts the reference's callers use (``k_cache [NB, block_size, Hkv, D]``,
``block_tables: dict[str, list[int]]``, ``seq_lens: dict[str, int]``, see
kernels/paged_attention.py:200-214 of the reference).  Large pools are filled on
the device by the benchmark itself; the length / table logic is shared.

Seeds: one ``torch.Generator`` per tensor class (Q 1001, K 1002, V 1003,
lengths 1004, tables 1005, norm 1006), each offset by the config index.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

BLOCK_SIZE = 16


@dataclass
class DecodeShape:
    name: str
    index: int
    batch: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    dtype: torch.dtype
    kv_fp8: bool = False
    block_size: int = BLOCK_SIZE


C1 = DecodeShape("c1-opt125m-fp32", 1, 8, 12, 12, 64, torch.float32)
C2 = DecodeShape("c2-tinyllama-bf16", 2, 64, 32, 4, 64, torch.bfloat16)
C3 = DecodeShape("c3-llama3-8b-fp8", 3, 256, 32, 8, 128, torch.bfloat16, kv_fp8=True)
C5 = DecodeShape("c5-llama3-70b-fp8", 5, 2048, 64, 8, 128, torch.bfloat16, kv_fp8=True)


def _gen(seed: int) -> torch.Generator:
    return torch.Generator(device="cpu").manual_seed(seed)


def uniform_lengths(batch: int, lo: int, hi: int, seed: int) -> list[int]:
    """``L_i ~ U{lo..hi}`` inclusive."""
    return torch.randint(lo, hi + 1, (batch,), generator=_gen(seed)).tolist()


def lognormal_lengths(batch: int, median: int, lo: int, hi: int, seed: int, sigma: float = 0.75) -> list[int]:
    """``L_i = clip(round(exp(ln median + sigma z)), lo, hi)``; sigma 0.75 is this
    project's documented choice (the configs give median and clip only)."""
    z = torch.randn(batch, generator=_gen(seed), dtype=torch.float64)
    val = torch.exp(math.log(median) + sigma * z).round().clamp(lo, hi)
    return [int(v) for v in val.tolist()]


def config_lengths(shape: DecodeShape, batch: int | None = None) -> list[int]:
    b = shape.batch if batch is None else batch
    seed = 1004 + shape.index
    if shape.index == 1:
        return uniform_lengths(b, 64, 512, seed)
    if shape.index == 2:
        return uniform_lengths(b, 1024, 4096, seed)
    if shape.index == 3:
        return lognormal_lengths(b, 2048, 128, 8192, seed)
    if shape.index == 5:
        return lognormal_lengths(b, 4096, 256, 32768, seed)
    raise ValueError(shape.name)


def blocks_for(length: int, block_size: int = BLOCK_SIZE) -> int:
    return -(-length // block_size)


def random_tables(
    lengths: list[int], n_pool_blocks: int, seed: int, block_size: int = BLOCK_SIZE, extra_blocks: int = 0
) -> dict[str, list[int]]:
    """Non-overlapping consecutive slices of one seeded permutation of the pool
    (config 1: "a seeded random permutation slice of the pool")."""
    need = sum(blocks_for(n, block_size) + extra_blocks for n in lengths)
    if need > n_pool_blocks:
        raise ValueError(f"pool of {n_pool_blocks} blocks cannot hold {need}")
    perm = torch.randperm(n_pool_blocks, generator=_gen(seed)).tolist()
    tables: dict[str, list[int]] = {}
    at = 0
    for i, n in enumerate(lengths):
        nb = blocks_for(n, block_size) + extra_blocks
        tables[f"req_{i}"] = perm[at : at + nb]
        at += nb
    return tables


def pool_blocks_for(shape: DecodeShape, lengths: list[int], extra_blocks: int = 0) -> int:
    if shape.index == 1:
        return 512
    if shape.index == 2 and len(lengths) == shape.batch:
        return 20000
    need = sum(blocks_for(n, shape.block_size) + extra_blocks for n in lengths)
    return need + max(1, need // 10)  # 10 % slack, like a live block manager


@dataclass
class DecodeWorkload:
    shape: DecodeShape
    q: torch.Tensor
    k_cache: torch.Tensor  # source-dtype pool [NB, bs, Hkv, D]
    v_cache: torch.Tensor
    block_tables: dict[str, list[int]]
    seq_lens: dict[str, int]
    scale: float
    lengths: list[int] = field(default_factory=list)


def make_decode_workload(
    shape: DecodeShape, batch: int | None = None, max_len: int | None = None, extra_blocks: int = 0
) -> DecodeWorkload:
    """Full CPU instance of a decode configuration (optionally with a smaller
    batch / clipped lengths so that CPU checkers finish in seconds).

    For the FP8 configurations ``k_cache`` / ``v_cache`` hold the *unquantised*
    bf16 values ``N(0,1)*2``; quantise-on-append turns them into codes.
    Unused pool blocks and the slots past each request's length stay zero."""
    lengths = config_lengths(shape, batch)
    if max_len is not None:
        lengths = [min(n, max_len) for n in lengths]
    b = len(lengths)
    nb = pool_blocks_for(shape, lengths, extra_blocks)
    tables = random_tables(lengths, nb, 1005 + shape.index, shape.block_size, extra_blocks)
    hkv, d, bs = shape.n_kv_heads, shape.head_dim, shape.block_size
    q = torch.randn((b, shape.n_heads, d), generator=_gen(1001 + shape.index)).to(shape.dtype)
    gain = 2.0 if shape.kv_fp8 else 1.0
    if shape.index == 1:
        # config 1 fills the whole 512-block pool
        k = torch.randn((nb, bs, hkv, d), generator=_gen(1002 + shape.index)).to(shape.dtype)
        v = torch.randn((nb, bs, hkv, d), generator=_gen(1003 + shape.index)).to(shape.dtype)
    else:
        k = torch.zeros((nb, bs, hkv, d), dtype=shape.dtype)
        v = torch.zeros((nb, bs, hkv, d), dtype=shape.dtype)
        gk, gv = _gen(1002 + shape.index), _gen(1003 + shape.index)
        for i, n in enumerate(lengths):
            ids = torch.as_tensor(tables[f"req_{i}"][: blocks_for(n, bs)])
            kk = torch.zeros((len(ids) * bs, hkv, d))
            vv = torch.zeros((len(ids) * bs, hkv, d))
            kk[:n] = torch.randn((n, hkv, d), generator=gk) * gain
            vv[:n] = torch.randn((n, hkv, d), generator=gv) * gain
            k[ids] = kk.view(len(ids), bs, hkv, d).to(shape.dtype)
            v[ids] = vv.view(len(ids), bs, hkv, d).to(shape.dtype)
    seq_lens = {f"req_{i}": n for i, n in enumerate(lengths)}
    return DecodeWorkload(shape, q, k, v, tables, seq_lens, 1.0 / math.sqrt(d), lengths)


# ---------------------------------------------------------------------------
# Algorithmic bytes (the roofline numerators)
# ---------------------------------------------------------------------------
def decode_algorithmic_bytes(
    lengths: list[int], n_heads: int, n_kv_heads: int, head_dim: int, kv_elem: int, q_elem: int, out_elem: int,
    fp8_scales: bool, block_size: int = BLOCK_SIZE,
) -> int:
    """K and V counted once per kv head for valid tokens only, plus scales,
    Q in, O out, and the block-table / length words actually dereferenced.
    Split-K partials are not counted."""
    total = 0
    for n in lengths:
        nb = blocks_for(n, block_size)
        total += 2 * n * n_kv_heads * head_dim * kv_elem
        if fp8_scales:
            total += 2 * nb * n_kv_heads * 4
        total += 4 * nb + 4
    total += len(lengths) * n_heads * head_dim * (q_elem + out_elem)
    return total


def append_algorithmic_bytes(n_tokens: int, n_kv_heads: int, head_dim: int, src_elem: int = 2,
                             block_size: int = BLOCK_SIZE) -> int:
    """Quantise-on-append of ``n_tokens`` tokens of K and V: source read, codes
    written, one fp32 scale per (block, kv_head)."""
    return 2 * n_tokens * n_kv_heads * head_dim * (src_elem + 1) + 2 * blocks_for(n_tokens, block_size) * n_kv_heads * 4


def rms_norm_algorithmic_bytes(rows: int, hidden: int, elem: int, residual: bool = False) -> int:
    return rows * hidden * elem * (3 if residual else 2) + hidden * elem


def prefill_flops(n_requests: int, n_heads: int, head_dim: int, n_q: int, prefix: int) -> int:
    """QK^T and PV multiply-adds over the causal region only:
    ``4*D*H*R*(Sq*P + Sq*(Sq+1)/2)``."""
    return 4 * head_dim * n_heads * n_requests * (n_q * prefix + n_q * (n_q + 1) // 2)


# ---------------------------------------------------------------------------
# Config 4: shared-prefix chunked prefill
# ---------------------------------------------------------------------------
@dataclass
class PrefillWorkload:
    n_heads: int
    n_kv_heads: int
    head_dim: int
    prefix_len: int
    chunk_len: int
    q: torch.Tensor  # [R*chunk, H, D] packed by request
    k_cache: torch.Tensor
    v_cache: torch.Tensor
    block_tables: dict[str, list[int]]
    ctx_lens: dict[str, int]
    scale: float


def make_prefill_workload(
    n_requests: int = 32, prefix_len: int = 2048, chunk_len: int = 512, n_heads: int = 32, n_kv_heads: int = 8,
    head_dim: int = 128, dtype: torch.dtype = torch.bfloat16, block_size: int = BLOCK_SIZE,
) -> PrefillWorkload:
    """All requests map the same ``prefix_len`` tokens to identical physical
    blocks (radix prefix sharing: the shared ids head every table), followed by
    a private chunk.  ``prefix_len`` must be block aligned, as full radix hits
    are (python_runtime/engine/cache/radix_cache.py:91-95)."""
    if prefix_len % block_size:
        raise ValueError("shared prefix must be a whole number of blocks")
    pb = prefix_len // block_size
    cb = blocks_for(chunk_len, block_size)
    nb = pb + n_requests * cb
    nb += max(1, nb // 10)
    perm = torch.randperm(nb, generator=_gen(1005 + 4)).tolist()
    shared = perm[:pb]
    tables = {f"req_{i}": shared + perm[pb + i * cb : pb + (i + 1) * cb] for i in range(n_requests)}
    k = torch.zeros((nb, block_size, n_kv_heads, head_dim), dtype=dtype)
    v = torch.zeros_like(k)
    gk, gv = _gen(1002 + 4), _gen(1003 + 4)
    used = torch.as_tensor(perm[: pb + n_requests * cb])
    k[used] = torch.randn((len(used), block_size, n_kv_heads, head_dim), generator=gk).to(dtype)
    v[used] = torch.randn((len(used), block_size, n_kv_heads, head_dim), generator=gv).to(dtype)
    q = torch.randn((n_requests * chunk_len, n_heads, head_dim), generator=_gen(1001 + 4)).to(dtype)
    ctx = {f"req_{i}": prefix_len + chunk_len for i in range(n_requests)}
    return PrefillWorkload(n_heads, n_kv_heads, head_dim, prefix_len, chunk_len, q, k, v, tables, ctx,
                           1.0 / math.sqrt(head_dim))


def make_rms_norm_inputs(rows: int = 256, hidden: int = 4096, dtype: torch.dtype = torch.bfloat16):
    """Config 3's norm: x N(0,1), w N(1, 0.02), eps 1e-5."""
    g = _gen(1006 + 3)
    x = torch.randn((rows, hidden), generator=g).to(dtype)
    w = (1.0 + 0.02 * torch.randn((hidden,), generator=g)).to(dtype)
    return x, w, 1e-5


def make_norm_matmul_inputs(m: int, k: int, n: int, dtype: torch.dtype = torch.bfloat16, seed: int = 1007):
    """Inputs of ``fused_rms_norm_matmul``: activations N(0,1), norm weight N(1, 0.02), matrix N(0, 1/K) (a projection
    with unit-variance outputs); eps 1e-5 as in the reference's operator default."""
    g = _gen(seed)
    x = torch.randn((m, k), generator=g).to(dtype)
    rms_w = (1.0 + 0.02 * torch.randn((k,), generator=g)).to(dtype)
    mat_w = (torch.randn((k, n), generator=g) / math.sqrt(k)).to(dtype)
    return x, rms_w, mat_w, 1e-5


SDPA_MASK_CASES = ("positions_bf16", "ties_f32", "rank5_batch_slice_bf16", "expanded_f32", "causal_drops_mask_bf16")


def make_sdpa_mask_case(name: str):
    """Seeded inputs for the dense-attention operator with the reference backend's mask conventions
    (python_runtime/hal/pytorch_backend/_ops_attention.py:13-53).  Returns ``(inputs, kwargs)`` for
    ``execute("scaled_dot_product_attention", inputs, **kwargs)``; the mask is the fourth input."""
    g = _gen(2000 + SDPA_MASK_CASES.index(name))
    if name == "positions_bf16":  # the compiled model's prefill call: positions 0..S-1 as a [B,1,S,1] column
        b, h, s, d, dt = 2, 2, 144, 128, torch.bfloat16
        mask = torch.arange(s, dtype=torch.float32).view(1, 1, s, 1).expand(b, 1, s, 1).contiguous()
        kw = {}
    elif name == "ties_f32":  # equal positions see one another: blocks of three tokens, offset 5
        b, h, s, d, dt = 1, 3, 77, 64, torch.float32
        mask = (torch.arange(s) // 3 + 5).to(torch.float32).view(1, 1, s, 1)
        kw = {"scale": 0.2}
    elif name == "rank5_batch_slice_bf16":  # [B,B,1,S,1]: dimension 2 squeezed, then the first entry of dimension 1 kept
        b, h, s, d, dt = 2, 2, 40, 128, torch.bfloat16
        pos = torch.stack([torch.arange(s), torch.arange(s) // 2]).to(torch.float32)  # per batch entry
        mask = pos.view(b, 1, 1, s, 1).expand(b, b, 1, s, 1).contiguous()
        kw = {}
    elif name == "expanded_f32":  # the column already expanded to [B,1,S,S]
        b, h, s, d, dt = 2, 1, 33, 32, torch.float32
        mask = (torch.arange(s, dtype=torch.float32) * 2.0).view(1, 1, s, 1).expand(b, 1, s, s)
        kw = {}
    elif name == "causal_drops_mask_bf16":  # is_causal=True: the floating-point mask is ignored
        b, h, s, d, dt = 1, 2, 130, 128, torch.bfloat16
        mask = torch.zeros((b, 1, s, 1), dtype=torch.float32)
        kw = {"is_causal": True}
    else:
        raise KeyError(name)
    q = torch.randn((b, h, s, d), generator=g).to(dt)
    k = torch.randn((b, h, s, d), generator=g).to(dt)
    v = torch.randn((b, h, s, d), generator=g).to(dt)
    return [q, k, v, mask], kw
