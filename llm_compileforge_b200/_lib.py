"""ctypes binding of libsfb.so (the C ABI declared in include/sfb.h).

The Python layer holds no compute of its own: every operator call ends in one
of the ``sfb_*`` entry points below.  There is no CPU or PyTorch fallback; if the
library is missing, or a tensor is not on a CUDA device, the call raises.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, Union, byref, c_char_p, c_float, c_int, c_int32, c_int64, c_void_p

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
# SFB_LIBRARY points at another build of the same library (same ABI), e.g. a system-wide install
LIB_PATH = os.environ.get("SFB_LIBRARY") or os.path.join(_PKG, "libsfb.so")

SFB_DEVICE_CPU, SFB_DEVICE_CUDA = 1, 2

# SFBStatus
SFB_OK = 0
SFB_ERR_INVALID_ARG = -1
SFB_ERR_UNSUPPORTED = -2
SFB_ERR_WORKSPACE = -3
SFB_ERR_CUDA = -4
SFB_ERR_DEVICE_STATUS = -5
SFB_ERR_OUT_OF_BLOCKS = -6
SFB_PEER_SIGNAL, SFB_PEER_WAIT = 1, 2

# SFBDType
SFB_F32, SFB_BF16, SFB_F16, SFB_F8E4M3 = 0, 1, 2, 3

SFB_QUANT_PER_TENSOR, SFB_QUANT_PER_BLOCK_HEAD = 0, 1

SFB_STATUS_BAD_BLOCK_ID, SFB_STATUS_EMPTY_REQUEST, SFB_STATUS_WAIT_TIMEOUT, SFB_STATUS_UNSORTED_POSITIONS = 1, 2, 4, 8
SFB_MASK_NONE, SFB_MASK_CAUSAL_TOP_LEFT, SFB_MASK_CAUSAL_BOTTOM_RIGHT, SFB_MASK_POSITIONS = 0, 1, 2, 3

_DTYPES = {
    torch.float32: SFB_F32,
    torch.bfloat16: SFB_BF16,
    torch.float16: SFB_F16,
    torch.float8_e4m3fn: SFB_F8E4M3,
}


def _memref(rank: int):
    class MemRef(Structure):
        _fields_ = [
            ("allocated", c_void_p),
            ("aligned", c_void_p),
            ("offset", c_int64),
            ("sizes", c_int64 * rank),
            ("strides", c_int64 * rank),
        ]

    MemRef.__name__ = f"SFBMemRef{rank}"
    return MemRef


SFBMemRef1, SFBMemRef2, SFBMemRef3, SFBMemRef4 = (_memref(r) for r in (1, 2, 3, 4))


class _Raw(Union):
    _fields_ = [("r1", SFBMemRef1), ("r2", SFBMemRef2), ("r3", SFBMemRef3), ("r4", SFBMemRef4)]


class SFBTensor(Structure):
    """Mirror of ``SFBTensor`` (= the reference's ``SFATensor``, include/sfa.h:88-99)."""

    _anonymous_ = ("raw",)
    _fields_ = [("device", c_int32), ("rank", c_int32), ("elem_size", c_int32), ("raw", _Raw)]


class SfbError(RuntimeError):
    def __init__(self, status: int, text: str):
        super().__init__(f"libsfb status {status}: {text}")
        self.status = status


_lib: ctypes.CDLL | None = None

_T = POINTER(SFBTensor)


def load() -> ctypes.CDLL:
    """Load libsfb.so; raises ``RuntimeError`` when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m llm_compileforge_b200.build` "
            "(there is no fallback implementation)"
        )
    lib = ctypes.CDLL(LIB_PATH)
    lib.sfb_abi_version.restype = c_int
    lib.sfb_last_error.restype = c_char_p
    lib.sfb_status_string.restype = c_char_p
    lib.sfb_status_string.argtypes = [c_int]
    lib.sfb_paged_attention_workspace_bytes.restype = c_int64
    lib.sfb_paged_attention_workspace_bytes.argtypes = [c_int64] * 6
    lib.sfb_paged_attention_decode.restype = c_int
    lib.sfb_paged_attention_decode.argtypes = [_T] * 9 + [c_int, c_int, c_float, c_int64, c_void_p, c_int64, c_void_p]
    lib.sfb_read_status.restype = c_int
    lib.sfb_read_status.argtypes = [c_void_p, POINTER(c_int32), c_void_p]
    lib.sfb_cache_write.restype = c_int
    lib.sfb_cache_write.argtypes = [_T] * 13 + [c_int, c_int, c_int64, c_void_p]
    lib.sfb_quantize_fp8.restype = c_int
    lib.sfb_quantize_fp8.argtypes = [_T, _T, _T, c_int, c_int, c_void_p]
    lib.sfb_dequantize_fp8.restype = c_int
    lib.sfb_dequantize_fp8.argtypes = [_T, _T, _T, c_int, c_int, c_void_p]
    lib.sfb_rms_norm.restype = c_int
    lib.sfb_rms_norm.argtypes = [_T, _T, _T, _T, c_int, c_float, c_void_p]
    _optional(lib)
    _shared_prefix_protos(lib)
    _block_manager_protos(lib)
    lib.sfb_paged_attention_decode_gather.restype = c_int
    lib.sfb_paged_attention_decode_gather.argtypes = [_T] * 9 + [POINTER(c_void_p), c_int, c_int, c_int, c_int, c_float, c_int64,
                                                                c_void_p, c_int64, c_void_p]
    lib.sfb_prefill_fp8_workspace_bytes.restype = c_int64
    lib.sfb_prefill_fp8_workspace_bytes.argtypes = [c_int64] * 5
    lib.sfb_prefill_paged_fp8.restype = c_int
    lib.sfb_prefill_paged_fp8.argtypes = [_T] * 9 + [c_int, c_float, c_int, c_int64, c_void_p, c_int64, c_void_p]
    lib.sfb_fold_norm_weight.restype = c_int
    lib.sfb_fold_norm_weight.argtypes = [_T, _T, _T, c_int, c_void_p]
    lib.sfb_fused_rms_norm_matmul.restype = c_int
    lib.sfb_fused_rms_norm_matmul.argtypes = [_T, _T, _T, c_int, c_float, c_void_p, c_int64, c_void_p]
    lib.sfb_fused_rms_norm_matmul_workspace_bytes.restype = c_int64
    lib.sfb_fused_rms_norm_matmul_workspace_bytes.argtypes = [c_int64]
    lib.sfb_fused_rms_norm_matmul_plan.restype = ctypes.c_int
    lib.sfb_fused_rms_norm_matmul_plan.argtypes = [c_int64, c_int64, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_int32)]
    lib.sfb_peer_signal_wait.restype = c_int
    lib.sfb_peer_signal_wait.argtypes = [POINTER(c_void_p), c_int, c_int, ctypes.c_uint32, c_int, c_void_p, c_void_p]
    _lib = lib
    return lib


def _optional(lib: ctypes.CDLL) -> None:
    """Prototypes of entry points added after ABI version 1's first set."""
    if hasattr(lib, "sfb_prefill_paged"):
        lib.sfb_prefill_paged.restype = c_int
        lib.sfb_prefill_paged.argtypes = [_T] * 7 + [c_int, c_float, c_int, c_int64, c_void_p, c_int64, c_void_p]
        lib.sfb_prefill_workspace_bytes.restype = c_int64
        lib.sfb_prefill_workspace_bytes.argtypes = [c_int64]
    lib.sfb_prefill_paged_rows.restype = c_int
    lib.sfb_prefill_paged_rows.argtypes = [_T] * 8 + [c_int, c_float, c_int64, c_void_p, c_int64, c_void_p]
    lib.sfb_attention_dense_workspace_bytes.restype = c_int64
    lib.sfb_attention_dense_workspace_bytes.argtypes = [c_int64] * 6 + [c_int]
    lib.sfb_attention_dense.restype = c_int
    lib.sfb_attention_dense.argtypes = [_T] * 5 + [c_int, c_float, c_int, c_void_p, c_int64, c_void_p]
    lib.sfb_cache_read.restype = c_int
    lib.sfb_cache_read.argtypes = [_T] * 5 + [c_int, c_int, c_void_p, c_void_p]


def _block_manager_protos(lib: ctypes.CDLL) -> None:
    h, s, i32p = c_void_p, c_char_p, POINTER(c_int32)
    protos = {
        "sfb_bm_create": (c_void_p, [c_int64, c_int64]),
        "sfb_bm_destroy": (None, [h]),
        "sfb_bm_attach_device_tables": (c_int, [h, c_void_p, c_int64, c_int64]),
        "sfb_bm_allocate": (c_int64, [h, s, c_int64, i32p, c_int64]),
        "sfb_bm_free": (None, [h, s]),
        "sfb_bm_free_block": (None, [h, c_int64]),
        "sfb_bm_assign_cached_blocks": (c_int, [h, s, i32p, c_int64]),
        "sfb_bm_ensure_blocks": (c_int, [h, s, c_int64]),
        "sfb_bm_ensure_blocks_batch": (c_int, [h, POINTER(c_char_p), POINTER(c_int64), c_int64]),
        "sfb_bm_share_prefix": (c_int64, [h, s, s, c_int64]),
        "sfb_bm_increment_ref_count": (None, [h, c_int64]),
        "sfb_bm_ref_count": (c_int64, [h, c_int64]),
        "sfb_bm_num_free_blocks": (c_int64, [h]),
        "sfb_bm_get_blocks": (c_int64, [h, s, i32p, c_int64]),
        "sfb_bm_row": (c_int64, [h, s]),
        "sfb_bm_sync": (c_int64, [h, c_void_p]),
    }
    for name, (res, args) in protos.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args


def _shared_prefix_protos(lib: ctypes.CDLL) -> None:
    lib.sfb_shared_prefix_workspace_bytes.restype = c_int64
    lib.sfb_shared_prefix_workspace_bytes.argtypes = [c_int64] * 7
    lib.sfb_paged_attention_decode_shared_prefix.restype = c_int
    lib.sfb_paged_attention_decode_shared_prefix.argtypes = [_T] * 6 + [c_int, c_float, c_int64, c_int64, c_void_p, c_int64, c_void_p]


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype {dtype} is not supported by libsfb") from None


def desc(t: torch.Tensor | None, what: str = "tensor"):
    """``byref`` descriptor of a CUDA tensor (``None`` passes a NULL pointer).

    The descriptor only borrows the tensor's memory; the caller keeps the tensor
    alive until the stream has consumed it."""
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError(f"{what} must live on a CUDA device (libsfb has no CPU path), got {t.device}")
    if not 1 <= t.dim() <= 4:
        raise ValueError(f"{what}: rank {t.dim()} outside 1..4")
    d = SFBTensor()
    d.device = SFB_DEVICE_CUDA
    d.rank = t.dim()
    d.elem_size = t.element_size()
    raw = getattr(d, f"r{t.dim()}")
    raw.allocated = t.data_ptr()
    raw.aligned = t.data_ptr()
    raw.offset = 0
    for i in range(t.dim()):
        raw.sizes[i] = t.shape[i]
        raw.strides[i] = t.stride(i)
    return byref(d)


def check(status: int) -> None:
    """Map a negative status to the exception type the reference's callers see:
    ``ValueError`` for bad arguments (python_runtime/hal/pytorch_backend/__init__.py:112-119
    raises ValueError for bad op calls), ``RuntimeError`` otherwise."""
    if status == SFB_OK:
        return
    text = load().sfb_last_error().decode("utf-8", "replace")
    if status in (SFB_ERR_INVALID_ARG, SFB_ERR_UNSUPPORTED):
        raise ValueError(f"libsfb: {text}")
    raise SfbError(status, text)


def current_stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream
