"""ctypes front-end of the plain-C oracle (TEST INFRASTRUCTURE ONLY).

Wraps ``oracle/sfb_oracle.c`` for numpy/torch-CPU arrays.  The shipped package
never imports this module.
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, c_float, c_int, c_int32, c_int64, c_uint8, c_void_p

import numpy as np

from . import build_oracle

_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build_oracle.build())
        _lib.sfbo_e4m3_encode_array.argtypes = [c_void_p, c_void_p, c_int64]
        _lib.sfbo_e4m3_decode_array.argtypes = [c_void_p, c_void_p, c_int64]
        _lib.sfbo_quantize_pool.argtypes = [c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p]
        _lib.sfbo_paged_decode.argtypes = [
            c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
            c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_float, c_void_p,
        ]
        _lib.sfbo_paged_decode.restype = c_int
        _lib.sfbo_rms_norm.argtypes = [c_void_p, c_void_p, c_void_p, c_float, c_int64, c_int64, c_void_p]
        _lib.sfbo_chunk_prefill.argtypes = [
            c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
            c_float, c_void_p,
        ]
    return _lib


def _ptr(a: np.ndarray | None) -> int | None:
    return None if a is None else a.ctypes.data


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint8)
    lib().sfbo_e4m3_encode_array(_ptr(x), _ptr(out), x.size)
    return out


def e4m3_decode(c: np.ndarray) -> np.ndarray:
    c = np.ascontiguousarray(c, dtype=np.uint8)
    out = np.empty(c.shape, dtype=np.float32)
    lib().sfbo_e4m3_decode_array(_ptr(c), _ptr(out), c.size)
    return out


def quantize_pool(pool: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    pool = np.ascontiguousarray(pool, dtype=np.float32)
    nb, bs, hkv, d = pool.shape
    codes = np.empty(pool.shape, dtype=np.uint8)
    scales = np.empty((nb, hkv), dtype=np.float32)
    lib().sfbo_quantize_pool(_ptr(pool), nb, bs, hkv, d, _ptr(codes), _ptr(scales))
    return codes, scales


def paged_decode(
    q: np.ndarray,
    k_pool: np.ndarray,
    v_pool: np.ndarray,
    tables: np.ndarray,
    seq_lens: np.ndarray,
    scale: float,
    k_scale: np.ndarray | None = None,
    v_scale: np.ndarray | None = None,
) -> np.ndarray:
    """q float32 [B,H,D]; pools [NB,bs,Hkv,D] float32, uint16 (bf16 bits) or uint8
    (e4m3 codes, then k_scale/v_scale float32 [NB,Hkv] are required)."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    kind = {np.dtype(np.float32): 0, np.dtype(np.uint16): 1, np.dtype(np.uint8): 2}[k_pool.dtype]
    k_pool = np.ascontiguousarray(k_pool)
    v_pool = np.ascontiguousarray(v_pool)
    tables = np.ascontiguousarray(tables, dtype=np.int32)
    seq_lens = np.ascontiguousarray(seq_lens, dtype=np.int32)
    if kind == 2:
        k_scale = np.ascontiguousarray(k_scale, dtype=np.float32)
        v_scale = np.ascontiguousarray(v_scale, dtype=np.float32)
    b, h, d = q.shape
    nb, bs, hkv, _ = k_pool.shape
    out = np.empty((b, h, d), dtype=np.float32)
    rc = lib().sfbo_paged_decode(
        _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(k_scale), _ptr(v_scale), kind, _ptr(tables), _ptr(seq_lens),
        b, h, hkv, d, bs, tables.shape[1], nb, float(scale), _ptr(out),
    )
    if rc != 0:
        raise ValueError("oracle: empty request or block id out of range")
    return out


def rms_norm(x: np.ndarray, w: np.ndarray | None, eps: float, residual: np.ndarray | None = None) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, hidden = x.reshape(-1, x.shape[-1]).shape
    w = None if w is None else np.ascontiguousarray(w, dtype=np.float32)
    residual = None if residual is None else np.ascontiguousarray(residual, dtype=np.float32)
    out = np.empty_like(x)
    lib().sfbo_rms_norm(_ptr(x), _ptr(residual), _ptr(w), float(eps), rows, hidden, _ptr(out))
    return out


def chunk_prefill(
    q: np.ndarray, k_pool: np.ndarray, v_pool: np.ndarray, table: np.ndarray, ctx_len: int, scale: float
) -> np.ndarray:
    q = np.ascontiguousarray(q, dtype=np.float32)
    k_pool = np.ascontiguousarray(k_pool, dtype=np.float32)
    v_pool = np.ascontiguousarray(v_pool, dtype=np.float32)
    table = np.ascontiguousarray(table, dtype=np.int32)
    n_q, h, d = q.shape
    _, bs, hkv, _ = k_pool.shape
    out = np.empty_like(q)
    lib().sfbo_chunk_prefill(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(table), n_q, ctx_len, h, hkv, d, bs,
                             float(scale), _ptr(out))
    return out
