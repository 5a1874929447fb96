"""The `_mlir_ciface_*` shim against the reference's own golden C kernel
(tests/data/golden/rms_norm.c of the reference, compiled by oracle/build_ref.py)."""

import ctypes
import os

import numpy as np
import pytest
import torch

from llm_compileforge_b200 import _lib

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "librms_norm_golden.so")


def _memref2(ptr, rows, cols):
    m = _lib.SFBMemRef2()
    m.allocated = m.aligned = ptr
    m.offset = 0
    m.sizes[0], m.sizes[1] = rows, cols
    m.strides[0], m.strides[1] = cols, 1
    return m


def _memref1(ptr, n):
    m = _lib.SFBMemRef1()
    m.allocated = m.aligned = ptr
    m.offset = 0
    m.sizes[0], m.strides[0] = n, 1
    return m


@pytest.mark.parametrize("shape", [(2, 4), (7, 333), (64, 4096)])
def test_ciface_rms_norm_matches_reference_golden_kernel(cuda, shape):
    if not os.path.exists(GOLDEN):
        pytest.skip("reference golden kernel was not built (oracle/build_ref.py)")
    rows, hidden = shape
    g = torch.Generator().manual_seed(rows * 31 + hidden)
    x = torch.randn((rows, hidden), generator=g)
    w = torch.randn((hidden,), generator=g)
    # reference kernel: host pointers, output written behind the descriptor inside sret
    gold = ctypes.CDLL(GOLDEN)
    sret = ctypes.create_string_buffer(56 + rows * hidden * 4 + 64)
    xm, wm = _memref2(x.data_ptr(), rows, hidden), _memref1(w.data_ptr(), hidden)
    gold._mlir_ciface_rms_norm_f32(sret, ctypes.byref(xm), ctypes.byref(wm))
    od = _lib.SFBMemRef2.from_buffer(sret)
    assert (od.sizes[0], od.sizes[1]) == (rows, hidden)
    want = np.ctypeslib.as_array(ctypes.cast(od.aligned, ctypes.POINTER(ctypes.c_float)), shape=(rows, hidden)).copy()
    # this library: device pointers, callee-allocated output, freed through serveforge_free
    lib = _lib.load()
    lib._mlir_ciface_sfb_rms_norm_f32.restype = None
    lib.serveforge_free.restype = None
    lib.serveforge_free.argtypes = [ctypes.c_void_p]
    xd, wd = x.to(cuda), w.to(cuda)
    sret2 = ctypes.create_string_buffer(4096)
    xm2, wm2 = _memref2(xd.data_ptr(), rows, hidden), _memref1(wd.data_ptr(), hidden)
    lib._mlir_ciface_sfb_rms_norm_f32(sret2, ctypes.byref(xm2), ctypes.byref(wm2))
    od2 = _lib.SFBMemRef2.from_buffer(sret2)
    assert od2.allocated, lib.sfb_last_error()
    assert (od2.sizes[0], od2.sizes[1], od2.strides[0], od2.strides[1]) == (rows, hidden, hidden, 1)
    got = torch.empty((rows, hidden), dtype=torch.float32)
    cudart = ctypes.CDLL("libcudart.so.12")  # already loaded by torch
    cudart.cudaMemcpy.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
    assert cudart.cudaMemcpy(got.data_ptr(), od2.allocated, rows * hidden * 4, 2) == 0  # device -> host
    lib.serveforge_free(od2.allocated)
    err = np.abs(got.numpy() - want).max()
    assert err <= 1e-5 * np.abs(want).max(), err


def _memref(t):
    m = {1: _lib.SFBMemRef1, 2: _lib.SFBMemRef2, 3: _lib.SFBMemRef3, 4: _lib.SFBMemRef4}[t.dim()]()
    m.allocated = m.aligned = t.data_ptr()
    m.offset = 0
    for i in range(t.dim()):
        m.sizes[i], m.strides[i] = t.shape[i], t.stride(i)
    return m


def _take(lib, sret, offset, rank, dtype, device):
    """The output descriptor at `offset` of an sret buffer as a tensor (copied), its buffer released through serveforge_free."""
    cls = {2: _lib.SFBMemRef2, 3: _lib.SFBMemRef3, 4: _lib.SFBMemRef4}[rank]
    od = cls.from_buffer(sret, offset)
    assert od.allocated, lib.sfb_last_error()
    shape = [od.sizes[i] for i in range(rank)]
    out = torch.empty(shape, dtype=dtype, device=device)
    cudart = ctypes.CDLL("libcudart.so.12")
    cudart.cudaMemcpy.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
    assert cudart.cudaMemcpy(out.data_ptr(), od.allocated, out.numel() * out.element_size(), 3) == 0  # device -> device
    lib.serveforge_free(od.allocated)
    return out


def _call(lib, name, sret, *tensors):
    fn = getattr(lib, name)
    fn.restype = None
    refs = [_memref(t) for t in tensors]
    fn(sret, *[ctypes.byref(r) for r in refs])


def test_ciface_attention_operators(cuda):
    """paged_attention, cache_write, cache_read, quantize, dequantize and dense attention in the loader's calling
    convention (runtime/src/hal/cpu/executable.rs:151-200): callee-allocated outputs described in sret, freed through
    serveforge_free; results equal the status-returning entry points'."""
    from llm_compileforge_b200 import ops

    lib = _lib.load()
    lib.serveforge_free.restype = None
    lib.serveforge_free.argtypes = [ctypes.c_void_p]
    g = torch.Generator().manual_seed(4)
    nb, bs, hkv, h, d, b = 20, 16, 2, 4, 128, 3
    kc = torch.zeros((nb, bs, hkv, d), dtype=torch.bfloat16, device=cuda)
    vc = torch.zeros_like(kc)
    tables = torch.randperm(nb, generator=g)[: 6 * b].view(b, 6).to(torch.int32).to(cuda)  # no block in two tables: the writes do not race
    counts = [40, 96, 7]
    cu = torch.tensor([0, 40, 136, 143], dtype=torch.int32, device=cuda)
    start = torch.zeros(b, dtype=torch.int32, device=cuda)
    knew = torch.randn((143, hkv, d), generator=g).to(torch.bfloat16).to(cuda)
    vnew = torch.randn((143, hkv, d), generator=g).to(torch.bfloat16).to(cuda)
    sret = ctypes.create_string_buffer(4096)
    _call(lib, "_mlir_ciface_sfb_cache_write_bf16", sret, knew, vnew, cu, start, tables, kc, vc)
    kc2, vc2 = torch.zeros_like(kc), torch.zeros_like(vc)
    ops.cache_write(knew, vnew, cu, start, tables, kc2, vc2, max_new_tokens=96)
    assert torch.equal(kc, kc2) and torch.equal(vc, vc2) and kc.any()

    lens = torch.tensor(counts, dtype=torch.int32, device=cuda)
    q = torch.randn((b, h, d), generator=g).to(torch.bfloat16).to(cuda)
    _call(lib, "_mlir_ciface_sfb_paged_attention_bf16", sret, q, kc, vc, tables, lens)
    got = _take(lib, sret, 0, 3, torch.bfloat16, cuda)
    assert torch.equal(got, ops.paged_attention_decode(q, kc, vc, tables, lens))

    _call(lib, "_mlir_ciface_sfb_cache_read_bf16", sret, tables, lens, kc, vc)
    key = _take(lib, sret, 0, 4, torch.bfloat16, cuda)
    value = _take(lib, sret, ctypes.sizeof(_lib.SFBMemRef4), 4, torch.bfloat16, cuda)
    assert key.shape == (b, 6 * bs, hkv, d)
    assert torch.equal(key, ops.cache_read(kc, tables, lens, 6 * bs)) and torch.equal(value, ops.cache_read(vc, tables, lens, 6 * bs))
    assert torch.equal(key[1, :96], knew[40:136])

    _call(lib, "_mlir_ciface_sfb_quantize_bf16", sret, kc)
    codes = _take(lib, sret, 0, 4, torch.uint8, cuda)
    scales = _take(lib, sret, ctypes.sizeof(_lib.SFBMemRef4), 2, torch.float32, cuda)
    want_codes, want_scales = ops.quantize_fp8(kc, per_block_head=True)
    assert torch.equal(codes, want_codes.view(torch.uint8)) and torch.equal(scales, want_scales)
    _call(lib, "_mlir_ciface_sfb_dequantize_f32", sret, codes, scales)
    deq = _take(lib, sret, 0, 4, torch.float32, cuda)
    assert torch.equal(deq, ops.dequantize_fp8(want_codes, want_scales, torch.float32))

    qd = torch.randn((2, 4, 50, 64), generator=g).to(cuda)
    kd = torch.randn((2, 2, 50, 64), generator=g).to(cuda)
    vd = torch.randn((2, 2, 50, 64), generator=g).to(cuda)
    for name, mask in (("_mlir_ciface_sfb_scaled_dot_product_attention_f32", "none"), ("_mlir_ciface_sfb_causal_attention_f32", "causal")):
        _call(lib, name, sret, qd, kd, vd)
        dense = _take(lib, sret, 0, 4, torch.float32, cuda)
        assert torch.equal(dense, ops.attention_dense(qd, kd, vd, mask=mask))
        want = torch.nn.functional.scaled_dot_product_attention(qd.cpu(), kd.cpu().repeat_interleave(2, 1), vd.cpu().repeat_interleave(2, 1),
                                                                is_causal=mask == "causal")
        assert (dense.cpu() - want).abs().max().item() <= 1e-5 * want.abs().max().item()
