"""C-ABI checks that need no GPU: the library loads, exports every symbol the
header declares, descriptor layouts match the reference's memref contract, and
argument validation rejects bad calls before any kernel launch."""

import ctypes
import os
import re

import pytest
import torch

from llm_compileforge_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    """Every function the headers declare, after the preprocessor has expanded the per-type declaration macros."""
    import subprocess

    names = []
    inc = os.path.join(ROOT, "include")
    for f in os.listdir(inc):
        if f.endswith(".h"):
            text = subprocess.run(["gcc", "-E", "-P", os.path.join(inc, f)], capture_output=True, text=True, check=True).stdout
            text = text.replace('__attribute__((visibility("default")))', "SFB_API")
            names += re.findall(r"SFB_API\s+[\w\s\*]+?\b(\w+)\s*\(", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = declared_symbols()
    assert "sfb_paged_attention_decode" in names and "_mlir_ciface_sfb_paged_attention_bf16" in names and len(names) >= 60
    for n in names:
        assert hasattr(lib, n), f"libsfb.so does not export {n}"
    assert lib.sfb_abi_version() == 1


def test_descriptor_layout_matches_memref_contract():
    # tests/contract/memref_3way.c:26-36 of the reference: 40/56/72/88 bytes, fields at 0/8/16
    for cls, size in ((_lib.SFBMemRef1, 40), (_lib.SFBMemRef2, 56), (_lib.SFBMemRef3, 72), (_lib.SFBMemRef4, 88)):
        assert ctypes.sizeof(cls) == size
        assert (cls.allocated.offset, cls.aligned.offset, cls.offset.offset, cls.sizes.offset) == (0, 8, 16, 24)
    assert ctypes.sizeof(_lib.SFBTensor) == 104
    assert _lib.SFBTensor.raw.offset == 16


def _fake_desc(shape, elem, device=_lib.SFB_DEVICE_CUDA, ptr=0x1000, strides=None):
    d = _lib.SFBTensor()
    d.device, d.rank, d.elem_size = device, len(shape), elem
    raw = getattr(d, f"r{len(shape)}")
    raw.allocated = raw.aligned = ptr
    st = strides
    if st is None:
        st, acc = [], 1
        for s in reversed(shape):
            st.insert(0, acc)
            acc *= s
    for i, s in enumerate(shape):
        raw.sizes[i] = s
        raw.strides[i] = st[i]
    return d


def _decode(lib, q, k, v, t, l, o, qd=_lib.SFB_BF16, kvd=_lib.SFB_BF16, ks=None, vs=None, ws=None, ws_bytes=0):
    r = lambda x: None if x is None else ctypes.byref(x)
    return lib.sfb_paged_attention_decode(r(q), r(k), r(v), r(ks), r(vs), r(t), r(l), None, r(o), qd, kvd, 0.0, 0, ws, ws_bytes, None)


def test_decode_argument_validation():
    lib = _lib.load()
    q = _fake_desc((2, 8, 64), 2)
    o = _fake_desc((2, 8, 64), 2)
    k = _fake_desc((10, 16, 2, 64), 2)
    t = _fake_desc((2, 4), 4)
    l = _fake_desc((2,), 4)
    assert _decode(lib, None, k, k, t, l, o) == _lib.SFB_ERR_INVALID_ARG
    assert b"NULL" in lib.sfb_last_error()
    cpu_q = _fake_desc((2, 8, 64), 2, device=_lib.SFB_DEVICE_CPU)
    assert _decode(lib, cpu_q, k, k, t, l, o) == _lib.SFB_ERR_INVALID_ARG
    assert b"no CPU path" in lib.sfb_last_error()
    assert _decode(lib, q, k, k, t, l, o, qd=_lib.SFB_F32) == _lib.SFB_ERR_INVALID_ARG  # elem_size 2 != 4
    bad_heads = _fake_desc((10, 16, 3, 64), 2)
    assert _decode(lib, q, bad_heads, bad_heads, t, l, o) == _lib.SFB_ERR_INVALID_ARG
    assert _decode(lib, q, k, _fake_desc((11, 16, 2, 64), 2), t, l, o) == _lib.SFB_ERR_INVALID_ARG
    assert _decode(lib, q, k, k, _fake_desc((3, 4), 4), l, o) == _lib.SFB_ERR_INVALID_ARG
    strided = _fake_desc((2, 8, 64), 2, strides=[1024, 128, 2])
    assert _decode(lib, strided, k, k, t, l, o) == _lib.SFB_ERR_INVALID_ARG
    # e4m3 pool without scales
    k8 = _fake_desc((10, 16, 2, 64), 1)
    assert _decode(lib, q, k8, k8, t, l, o, kvd=_lib.SFB_F8E4M3) == _lib.SFB_ERR_INVALID_ARG
    # split needs a workspace: 4 blocks * 16 = 64 tokens > chunk 16
    r = ctypes.byref
    rc = lib.sfb_paged_attention_decode(r(q), r(k), r(k), None, None, r(t), r(l), None, r(o), _lib.SFB_BF16, _lib.SFB_BF16,
                                        0.0, 16, None, 0, None)
    assert rc == _lib.SFB_ERR_WORKSPACE
    assert lib.sfb_status_string(rc) == b"workspace missing or too small"


def test_workspace_size_query():
    lib = _lib.load()
    one = lib.sfb_paged_attention_workspace_bytes(8, 12, 64, 32, 16, 512)
    assert one == 256  # 32 blocks * 16 = 512 tokens: a single chunk, status word only
    two = lib.sfb_paged_attention_workspace_bytes(8, 12, 64, 33, 16, 512)
    assert two >= 256 + 8 * 2 * 12 * (64 + 2) * 4
    assert lib.sfb_paged_attention_workspace_bytes(8, 0, 64, 33, 16, 512) < 0


def test_other_entry_points_validate():
    lib = _lib.load()
    r = ctypes.byref
    x = _fake_desc((4, 128), 2)
    w = _fake_desc((64,), 2)
    assert lib.sfb_rms_norm(r(x), None, r(w), r(x), _lib.SFB_BF16, 1e-5, None) == _lib.SFB_ERR_INVALID_ARG
    assert lib.sfb_rms_norm(r(x), None, None, r(x), 7, 1e-5, None) == _lib.SFB_ERR_INVALID_ARG
    xs = _fake_desc((3, 16, 2, 32), 2)
    c = _fake_desc((3, 16, 2, 32), 1)
    s = _fake_desc((3, 3), 4)
    assert lib.sfb_quantize_fp8(r(xs), r(c), r(s), _lib.SFB_BF16, _lib.SFB_QUANT_PER_BLOCK_HEAD, None) == _lib.SFB_ERR_INVALID_ARG
    assert lib.sfb_quantize_fp8(r(xs), r(c), r(s), _lib.SFB_BF16, 9, None) == _lib.SFB_ERR_INVALID_ARG


def test_python_layer_refuses_cpu_tensors():
    import llm_compileforge_b200 as pkg

    q = torch.zeros(1, 4, 32)
    kv = torch.zeros(4, 16, 4, 32)
    with pytest.raises(ValueError, match="CUDA"):
        pkg.paged_attention(q, kv, kv, {"a": [0]}, {"a": 3})
    with pytest.raises(ValueError, match="CUDA"):
        pkg.fused_rms_norm_add(torch.zeros(2, 8), torch.zeros(2, 8), torch.ones(8))
    with pytest.raises(ValueError, match="zero tokens"):
        pkg.paged_attention(q, kv, kv, {"a": [0]}, {"a": 0})
    with pytest.raises(ValueError, match="outside the pool"):
        pkg.paged_attention(q, kv, kv, {"a": [9]}, {"a": 3})
    with pytest.raises(ValueError, match="Unknown op"):
        pkg.B200Backend().execute("matmul", [q, q])


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "libsfb.so"))
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.load()


def test_prefill_and_shared_prefix_validation():
    lib = _lib.load()
    r = ctypes.byref
    lib.sfb_prefill_paged.restype = ctypes.c_int
    q = _fake_desc((40, 8, 128), 2)
    k = _fake_desc((12, 16, 2, 128), 2)
    t = _fake_desc((3, 4), 4)
    cu = _fake_desc((4,), 4)
    ctx = _fake_desc((3,), 4)
    args = lambda **o: [r(o.get("q", q)), r(k), r(k), r(o.get("t", t)), r(o.get("cu", cu)), r(ctx), r(o.get("q", q)), o.get("dt", _lib.SFB_BF16),
                        ctypes.c_float(0.0), 1, 40, None, 0, None]
    assert lib.sfb_prefill_paged(*args(cu=_fake_desc((3,), 4))) == _lib.SFB_ERR_INVALID_ARG      # cu_q needs R+1 entries
    assert lib.sfb_prefill_paged(*args(t=_fake_desc((2, 4), 4))) == _lib.SFB_ERR_INVALID_ARG      # one table row per request
    assert lib.sfb_prefill_paged(*args(dt=_lib.SFB_F8E4M3)) == _lib.SFB_ERR_INVALID_ARG
    assert lib.sfb_prefill_paged(*args(q=_fake_desc((40, 7, 128), 2))) == _lib.SFB_ERR_INVALID_ARG  # 7 heads over 2 kv heads
    assert lib.sfb_prefill_workspace_bytes(1000) == 256 + 8192
    # shared-prefix decode
    fn = lib.sfb_paged_attention_decode_shared_prefix
    dq = _fake_desc((3, 8, 128), 2)
    lens = _fake_desc((3,), 4)
    call = lambda blocks, dt=_lib.SFB_BF16, ws=None, wsb=0: fn(r(dq), r(k), r(k), r(t), r(lens), r(dq), dt, ctypes.c_float(0.0), blocks, 0, ws, wsb, None)
    assert call(0) == _lib.SFB_ERR_INVALID_ARG and call(4) == _lib.SFB_ERR_INVALID_ARG   # prefix must leave room for own tokens
    assert call(2, dt=_lib.SFB_F32) in (_lib.SFB_ERR_UNSUPPORTED, _lib.SFB_ERR_INVALID_ARG)
    assert call(2) == _lib.SFB_ERR_WORKSPACE
    need = lib.sfb_shared_prefix_workspace_bytes(3, 8, 128, 4, 16, 0, 2)
    assert need > 256 + 3 * 2 * 8 * (128 + 2) * 4  # own chunk + the prefix partial slot
    assert lib.sfb_shared_prefix_workspace_bytes(3, 8, 128, 4, 16, 0, 5) < 0


def test_static_scratch_size_check_needs_no_gpu():
    lib = _lib.load()
    fn = lib.sfb_paged_attention_decode_static
    fn.restype = ctypes.c_int
    r = ctypes.byref
    q = _fake_desc((4096, 64, 128), 2)
    k = _fake_desc((4, 16, 8, 128), 2)
    t = _fake_desc((4096, 2), 4)
    lens = _fake_desc((4096,), 4)
    rc = fn(r(q), r(k), r(k), None, None, r(t), r(lens), None, r(q), _lib.SFB_BF16, _lib.SFB_BF16, ctypes.c_float(0.0), ctypes.c_int64(16), None)
    assert rc == _lib.SFB_ERR_WORKSPACE and b"built-in array" in lib.sfb_last_error()


def test_gather_signal_and_norm_matmul_validate_arguments():
    """The newer entry points reject bad calls before touching the device."""
    lib = _lib.load()
    r = ctypes.byref
    q = _fake_desc((2, 8, 128), 2)
    k = _fake_desc((4, 16, 2, 128), 2)
    t = _fake_desc((2, 2), 4)
    lens = _fake_desc((2,), 4)
    out_all = _fake_desc((2, 16, 128), 2)
    two = (ctypes.c_void_p * 2)(0x2000, 0x3000)
    # world outside 1..8, rank outside the world, missing peer table, misaligned peer
    common = (r(q), r(k), r(k), None, None, r(t), r(lens), None, r(out_all))
    tail = (_lib.SFB_BF16, _lib.SFB_BF16, 0.0, 16, None, 0, None)
    assert lib.sfb_paged_attention_decode_gather(*common, two, 9, 0, *tail) == _lib.SFB_ERR_INVALID_ARG
    assert lib.sfb_paged_attention_decode_gather(*common, two, 2, 2, *tail) == _lib.SFB_ERR_INVALID_ARG
    assert lib.sfb_paged_attention_decode_gather(*common, None, 2, 0, *tail) == _lib.SFB_ERR_INVALID_ARG
    odd = (ctypes.c_void_p * 2)(0x2000, 0x3004)
    assert lib.sfb_paged_attention_decode_gather(*common, odd, 2, 0, *tail) == _lib.SFB_ERR_INVALID_ARG
    # the whole output must have world * H heads
    small = _fake_desc((2, 8, 128), 2)
    assert lib.sfb_paged_attention_decode_gather(r(q), r(k), r(k), None, None, r(t), r(lens), None, r(small), two, 2, 0, *tail) == _lib.SFB_ERR_INVALID_ARG
    assert b"out must be" in lib.sfb_last_error()
    assert lib.sfb_peer_signal_wait(two, 0, 0, 1, 3, None, None) == _lib.SFB_ERR_INVALID_ARG
    assert lib.sfb_peer_signal_wait(two, 2, 0, 1, 4, None, None) == _lib.SFB_ERR_INVALID_ARG
    assert lib.sfb_peer_signal_wait(None, 2, 0, 1, 3, None, None) == _lib.SFB_ERR_INVALID_ARG

    x = _fake_desc((64, 256), 2)
    w = _fake_desc((256, 512), 2)
    y = _fake_desc((64, 512), 2)
    g = _fake_desc((256,), 2)
    assert lib.sfb_fused_rms_norm_matmul(r(x), r(w), r(y), _lib.SFB_F32, 1e-5, None, 0, None) == _lib.SFB_ERR_UNSUPPORTED
    assert lib.sfb_fused_rms_norm_matmul(r(x), r(_fake_desc((128, 512), 2)), r(y), _lib.SFB_BF16, 1e-5, None, 0, None) == _lib.SFB_ERR_INVALID_ARG
    assert lib.sfb_fused_rms_norm_matmul(r(x), r(_fake_desc((256, 516), 2)), r(_fake_desc((64, 516), 2)), _lib.SFB_BF16, 1e-5, None, 0, None) == _lib.SFB_ERR_UNSUPPORTED
    assert lib.sfb_fold_norm_weight(r(_fake_desc((255,), 2)), r(w), r(w), _lib.SFB_BF16, None) == _lib.SFB_ERR_INVALID_ARG
    assert lib.sfb_fold_norm_weight(r(g), r(w), r(w), _lib.SFB_F32, None) == _lib.SFB_ERR_UNSUPPORTED
    assert lib.sfb_fused_rms_norm_matmul_workspace_bytes(1000) == 256 + 4096
    assert lib.sfb_fused_rms_norm_matmul_workspace_bytes(-1) == _lib.SFB_ERR_INVALID_ARG


def test_block_manager_rejects_bad_handles_and_arguments():
    lib = _lib.load()
    assert not lib.sfb_bm_create(0, 16) and not lib.sfb_bm_create(16, 0)
    bm = lib.sfb_bm_create(8, 4)
    try:
        assert lib.sfb_bm_allocate(bm, b"a", -1, None, 0) == _lib.SFB_ERR_INVALID_ARG
        assert lib.sfb_bm_allocate(bm, b"a", 100, None, 0) == _lib.SFB_ERR_OUT_OF_BLOCKS
        assert lib.sfb_bm_get_blocks(bm, b"nobody", None, 0) == _lib.SFB_ERR_INVALID_ARG
        assert lib.sfb_bm_row(bm, b"nobody") == -1
        assert lib.sfb_bm_sync(bm, None) == _lib.SFB_ERR_INVALID_ARG  # no device tables attached
        assert lib.sfb_bm_attach_device_tables(bm, None, 4, 4) == _lib.SFB_ERR_INVALID_ARG
        assert lib.sfb_bm_ref_count(bm, 99) == -1
        assert lib.sfb_bm_allocate(bm, b"a", 6, None, 0) == 2 and lib.sfb_bm_num_free_blocks(bm) == 6
    finally:
        lib.sfb_bm_destroy(bm)


def test_trace_line_per_operator_call():
    """SFB_TRACE=1: one stderr line per operator call (the call here fails validation; the line is printed all the same)."""
    import subprocess
    import sys

    code = ("import ctypes; from llm_compileforge_b200 import _lib; lib = _lib.load(); "
            "rc = lib.sfb_rms_norm(None, None, None, None, 0, ctypes.c_float(1e-5), None); print('rc', rc)")
    env = dict(os.environ, SFB_TRACE="1", PYTHONPATH=ROOT)
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, cwd=ROOT)
    assert "rc -1" in res.stdout, res.stdout + res.stderr
    lines = [ln for ln in res.stderr.splitlines() if ln.startswith("[sfb] rms_norm")]
    assert len(lines) == 1 and "us" in lines[0] and "(enqueue)" in lines[0], res.stderr
    quiet = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=dict(os.environ, PYTHONPATH=ROOT), cwd=ROOT)
    assert "[sfb]" not in quiet.stderr
