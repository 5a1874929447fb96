"""Decode through the entry point that brings its own scratch memory.

``sfb_paged_attention_decode_static`` is for hosts that cannot allocate device
memory when they reach the decode call (all free HBM already belongs to the KV
block pool, or the host has no allocator binding).  It must give exactly what
``sfb_paged_attention_decode`` gives with a caller workspace, call after call,
even though all calls share one built-in array that still holds the previous
call's partial results.  This file is collected last so that a failure here
cannot hide another test's result in a run that stops at the first failure.
"""

import ctypes

import pytest
import torch

from llm_compileforge_b200 import _lib, ops
from llm_compileforge_b200._lib import desc, dtype_code

pytestmark = pytest.mark.gpu


def _static_decode(q, k, v, tables, lens, chunk, k_scale=None, v_scale=None, kv_code=None):
    lib = _lib.load()
    fn = lib.sfb_paged_attention_decode_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.POINTER(_lib.SFBTensor)] * 9 + [ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_int64, ctypes.c_void_p]
    out = torch.empty_like(q)
    rc = fn(desc(q), desc(k), desc(v), desc(k_scale), desc(v_scale), desc(tables), desc(lens), None, desc(out),
            dtype_code(q.dtype), kv_code if kv_code is not None else dtype_code(k.dtype), 0.0, chunk,
            torch.cuda.current_stream().cuda_stream)
    return rc, out


def _case(cuda, seed, batch, heads, kv_heads, dim, max_len, dtype):
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(1, max_len + 1, (batch,), generator=g, dtype=torch.int32)
    width = (max_len + 15) // 16
    nb = batch * width
    tables = torch.randperm(nb, generator=g).to(torch.int32).view(batch, width)
    q = torch.randn((batch, heads, dim), generator=g).to(dtype)
    k = torch.randn((nb, 16, kv_heads, dim), generator=g).to(dtype)
    v = torch.randn((nb, 16, kv_heads, dim), generator=g).to(dtype)
    return [t.to(cuda) for t in (q, k, v, tables, lens)]


def test_static_scratch_decode_matches_workspace_decode_twice(cuda):
    lib = _lib.load()
    # call 1: float32, 5 chunks per request -> partials go through the built-in array
    q, k, v, tables, lens = _case(cuda, 1, batch=6, heads=8, kv_heads=2, dim=64, max_len=300, dtype=torch.float32)
    want = ops.paged_attention_decode(q, k, v, tables, lens, chunk_tokens=64)
    rc, got = _static_decode(q, k, v, tables, lens, 64)
    assert rc == 0, lib.sfb_last_error()
    assert torch.equal(got, want)
    # call 2, straight after, other shapes and dtype: the array still holds call 1's partials
    q2, k2, v2, tables2, lens2 = _case(cuda, 2, batch=9, heads=16, kv_heads=4, dim=128, max_len=200, dtype=torch.bfloat16)
    want2 = ops.paged_attention_decode(q2, k2, v2, tables2, lens2, chunk_tokens=32)
    rc, got2 = _static_decode(q2, k2, v2, tables2, lens2, 32)
    assert rc == 0, lib.sfb_last_error()
    assert torch.equal(got2, want2)
    # and call 1 again gives call 1's answer again
    rc, again = _static_decode(q, k, v, tables, lens, 64)
    assert rc == 0 and torch.equal(again, want)
    bits = ctypes.c_int32(-1)
    rs = lib.sfb_read_status_static
    rs.restype = ctypes.c_int
    rs.argtypes = [ctypes.POINTER(ctypes.c_int32), ctypes.c_void_p]
    assert rs(ctypes.byref(bits), torch.cuda.current_stream().cuda_stream) == 0 and bits.value == 0


def test_static_scratch_rejects_oversized_split(cuda):
    lib = _lib.load()
    # 4096 requests x 64 heads x 128 dims x 2 chunks of float32 partials is far beyond the built-in 16 MiB
    q = torch.zeros((4096, 64, 128), dtype=torch.bfloat16, device=cuda)
    k = torch.zeros((4, 16, 8, 128), dtype=torch.bfloat16, device=cuda)
    tables = torch.zeros((4096, 2), dtype=torch.int32, device=cuda)
    lens = torch.ones(4096, dtype=torch.int32, device=cuda)
    rc, _ = _static_decode(q, k, k, tables, lens, 16)
    assert rc == _lib.SFB_ERR_WORKSPACE
    text = lib.sfb_last_error().decode()
    assert "built-in array" in text and "16777216" in text
