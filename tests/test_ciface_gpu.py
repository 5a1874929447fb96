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
