"""HAL backend: the reference's ``OpExecutor`` surface over libsfb.

``OpExecutor.execute(op_name, inputs, **kwargs)`` is the seam the reference's
engine calls (python_runtime/hal/interface.py:51-61; caller
python_runtime/engine/mlir_executor.py:358).  ``B200Backend`` serves the
attention hot-path operators on the GPU and forwards every other operator name
to an optional fallback executor, the way the reference's ``TritonBackend``
chains to the PyTorch backend (python_runtime/hal/triton_backend.py:48-65).

Operator names: ``rms_norm`` is the live HAL name
(pytorch_backend/_ops_norm.py:70); ``paged_attention``, ``cache_write``,
``quantize`` and ``dequantize`` are the names sf-dialect/include/Sf/HALOps.td:184-211
reserves; ``fused_rms_norm_add`` is the kernels-package name.
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from collections.abc import Callable
from typing import Any

import torch

from . import _lib, kernels_api, ops

try:  # the reference's own ABC when its package is importable, else a local twin
    from python_runtime.hal.interface import OpExecutor  # type: ignore
except Exception:  # noqa: BLE001

    class OpExecutor(ABC):  # type: ignore[no-redef]
        """Same contract as python_runtime/hal/interface.py:45-74."""

        @abstractmethod
        def execute(self, op_name: str, inputs: list[Any], **kwargs: Any) -> torch.Tensor: ...

        def async_copy(self, src: Any, dst: Any, byte_count: int) -> None:
            raise NotImplementedError("async_copy not supported")

        def memory_retrieve(self, key: Any, table: Any) -> torch.Tensor:
            raise NotImplementedError("memory_retrieve not supported")

        def send_kv_cache(self, blocks: Any, target_device: str) -> None:
            raise NotImplementedError("send_kv_cache not supported")


class B200Backend(OpExecutor):
    """Attention hot-path operators on one B200.

    Args:
        fallback: executor for every operator name this backend does not own
            (for the reference: ``PyTorchBackend("cuda")``).  Without one an
            unknown name raises ``ValueError`` like the reference backend does
            (pytorch_backend/__init__.py:112-119).
        device: CUDA device the inputs are expected on.
    """

    def __init__(self, fallback: OpExecutor | None = None, device: str | torch.device = "cuda") -> None:
        self._fallback = fallback
        self.device = torch.device(device)
        self._ops: dict[str, Callable[..., Any]] = {
            "paged_attention": self._op_paged_attention,
            "cache_write": self._op_cache_write,
            "cache_read": self._op_cache_read,
            "attention_forward": self._op_attention_forward,
            "quantize": self._op_quantize,
            "dequantize": self._op_dequantize,
            "rms_norm": self._op_rms_norm,
            "fused_rms_norm_add": self._op_fused_rms_norm_add,
            "flash_attention": self._op_flash_attention,
            "scaled_dot_product_attention": self._op_scaled_dot_product_attention,
            "chunked_prefill": self._op_chunked_prefill,
            "fused_rms_norm_matmul": self._op_fused_rms_norm_matmul,
        }
        self._folded: dict[tuple, torch.Tensor] = {}

    def supported_ops(self) -> list[str]:
        return sorted(self._ops)

    def execute(self, op_name: str, inputs: list[Any], **kwargs: Any) -> Any:
        handler = self._ops.get(op_name)
        if handler is not None:
            return handler(inputs, **kwargs)
        if self._fallback is not None:
            return self._fallback.execute(op_name, inputs, **kwargs)
        raise ValueError(f"Unknown op: '{op_name}'")

    # ── handlers ────────────────────────────────────────────────────────────
    def _op_paged_attention(self, inputs: list[Any], **kw: Any) -> Any:
        """inputs: ``[query, key_cache, value_cache, block_table]`` (HALOps.td:186-187).

        ``block_table`` is either the reference's dict (then ``seq_lens`` is a
        dict keyword and the result is a dict, like kernels.paged_attention) or a
        dense int32 tensor ``[B,max_blocks]`` (then ``seq_lens`` is an int32
        tensor and the result is ``[B,H,D]``; ``shared_prefix_blocks=n`` selects the
        shared-prefix route for tables whose first n entries are identical in every row)."""
        q, k_cache, v_cache, table = inputs[:4]
        seq_lens = kw.get("seq_lens", inputs[4] if len(inputs) > 4 else None)
        common = dict(k_scale=kw.get("k_scale"), v_scale=kw.get("v_scale"), scale=kw.get("scale"),
                      chunk_tokens=kw.get("chunk_tokens", 0))
        if isinstance(table, dict):
            return kernels_api.paged_attention(q, k_cache, v_cache, table, seq_lens or {},
                                               block_size=kw.get("block_size", k_cache.shape[1]), **common)
        if seq_lens is None:
            raise ValueError("paged_attention with a dense block table needs seq_lens")
        if kw.get("shared_prefix_blocks"):
            return ops.paged_attention_decode_shared_prefix(q, k_cache, v_cache, table, seq_lens, int(kw["shared_prefix_blocks"]),
                                                            scale=kw.get("scale"), chunk_tokens=kw.get("chunk_tokens", 0),
                                                            workspace=kw.get("workspace"))
        return ops.paged_attention_decode(q, k_cache, v_cache, table, seq_lens, workspace=kw.get("workspace"), **common)

    def _op_cache_write(self, inputs: list[Any], **kw: Any) -> None:
        """inputs: ``[key, value, positions]`` (HALOps.td:197-198) with keywords
        ``k_cache, v_cache, block_tables`` (dense int32) and, for an e4m3 pool,
        ``k_scale, v_scale, k_tail, v_tail``.  ``positions`` is either an int32
        tensor ``[B]`` of start positions plus ``cu_tokens [B+1]``, or - for the
        one-token-per-request decode step - just ``[B]`` positions."""
        key, value, positions = inputs[:3]
        b = positions.shape[0]
        cu = kw.get("cu_tokens")
        if cu is None:
            cu = torch.arange(b + 1, dtype=torch.int32, device=key.device)
            max_new = 1
        else:
            max_new = int(kw["max_new_tokens"])
        ops.cache_write(key, value, cu, positions, kw["block_tables"], kw["k_cache"], kw["v_cache"],
                        max_new_tokens=max_new, k_scale=kw.get("k_scale"), v_scale=kw.get("v_scale"),
                        k_tail=kw.get("k_tail"), v_tail=kw.get("v_tail"), tail_rows=kw.get("tail_rows"))

    def _op_quantize(self, inputs: list[Any], **kw: Any) -> Any:
        """``quantize(input, dtype="fp8")`` -> ``(codes, scale)`` (HALOps.td:202-206)."""
        dtype = kw.get("dtype", "fp8")
        if dtype not in ("fp8", "fp8_e4m3", "float8_e4m3fn"):
            raise ValueError(f"quantize: dtype {dtype!r} not supported (fp8 e4m3 only)")
        return ops.quantize_fp8(inputs[0], per_block_head=bool(kw.get("per_block_head", False)))

    def _op_dequantize(self, inputs: list[Any], **kw: Any) -> torch.Tensor:
        return ops.dequantize_fp8(inputs[0], inputs[1], kw.get("out_dtype", torch.float32))

    def _op_rms_norm(self, inputs: list[Any], **kw: Any) -> torch.Tensor:
        """Same arguments as pytorch_backend/_ops_norm.py:30-45 (eps default 1e-5)."""
        weight = inputs[1] if len(inputs) > 1 else None
        return ops.rms_norm(inputs[0], weight, eps=kw.get("eps", 1e-5))

    def _op_fused_rms_norm_add(self, inputs: list[Any], **kw: Any) -> torch.Tensor:
        return ops.rms_norm(inputs[0], inputs[2], eps=kw.get("eps", 1e-6), residual=inputs[1])


    def _op_flash_attention(self, inputs: list[Any], **kw: Any) -> torch.Tensor:
        """Dense attention ``[q, k, v]`` each ``[B,H,S,D]`` with the keywords of
        kernels.flash_attention_fwd (``scale``, ``causal`` default True)."""
        return kernels_api.flash_attention_fwd(inputs[0], inputs[1], inputs[2], scale=kw.get("scale"),
                                               causal=kw.get("causal", kw.get("is_causal", True)))

    def _op_scaled_dot_product_attention(self, inputs: list[Any], **kw: Any) -> torch.Tensor:
        """Dense SDPA with the reference backend's keywords and mask conventions
        (pytorch_backend/_ops_attention.py:13-53): ``[q, k, v(, attn_mask)]`` each ``[B,H,S,D]``, ``is_causal`` default
        False, ``scale``, ``dropout_p``.  As there:

        * a mask of more than four dimensions loses dimension 2, and a mask ``[B, B, S, ...]`` keeps its first entry of
          dimension 1 (``:17-22``);
        * a floating-point mask together with ``is_causal=True`` is dropped (``:33-35``);
        * a floating-point mask with ``is_causal=False`` holds POSITION VALUES, ``[B,1,S,1]`` (or that expanded to
          ``[B,1,S,S]``): key j is visible to query i iff ``pos[i] >= pos[j]`` (``:36-43``) - the call the compiled model
          makes for prefill (python_runtime/engine/mlir_executor.py:358).  It runs on the prefill kernels with one visible
          length per query row; the positions must not decrease along the sequence (the kernel reports it otherwise and
          the call goes to the fallback executor, ``ValueError`` without one).

        Boolean / additive masks of other kinds, dropout, and ``is_causal=True`` with different query and key lengths go
        to the fallback executor."""
        q, k, v = inputs[:3]
        mask = kw.get("attn_mask")
        if mask is None and len(inputs) > 3:
            mask = inputs[3]
        if mask is not None and mask.dim() > 4:
            mask = mask.squeeze(2)
        if mask is not None and mask.dim() == 4 and mask.shape[1] > 1 and mask.shape[1] == q.shape[0]:
            mask = mask[:, :1, :, :]
        causal = bool(kw.get("is_causal", False))
        if mask is not None and mask.dtype.is_floating_point and causal:
            mask = None
        positions = None
        if mask is not None and mask.dtype.is_floating_point and mask.dim() == 4 and mask.shape[1] == 1 and mask.shape[-2] > 1:
            s_len = mask.shape[-2]
            fits = q.shape[2] == s_len and k.shape[2] == s_len and mask.shape[0] in (1, q.shape[0])
            # [B,1,S,1], or that column expanded to [B,1,S,S] (a view, or a copy whose rows are constant: one device check)
            column = mask.shape[-1] == 1 or (mask.shape[-1] == s_len and fits and
                                             (mask.stride(-1) == 0 or bool((mask == mask[..., :1]).all().item())))
            if column and fits:
                positions = mask[:, 0, :, 0]
        basic = (float(kw.get("dropout_p", 0.0)) == 0.0 and q.dim() == 4 and q.is_cuda and q.shape[1] % k.shape[1] == 0
                 and not (causal and q.shape[2] != k.shape[2]))
        if basic and positions is not None:
            out, ws = ops.attention_dense(q, k, v, mask="positions", positions=positions, scale=kw.get("scale"), return_workspace=True)
            if not ops.read_status(ws) & _lib.SFB_STATUS_UNSORTED_POSITIONS:
                return out
        elif basic and mask is None:
            return ops.attention_dense(q, k, v, mask="causal" if causal else "none", scale=kw.get("scale"))
        if self._fallback is None:
            raise ValueError("scaled_dot_product_attention: this mask / dropout combination needs a fallback executor")
        return self._fallback.execute("scaled_dot_product_attention", inputs, **kw)

    def _op_attention_forward(self, inputs: list[Any], **kw: Any) -> torch.Tensor:
        """The Rust runtime's dense attention (runtime/src/engine/kernels.rs:97-302) as an operator: ``[q [H,S,D], k, v
        [H,Skv,D]]`` head-major float32 with q already scaled, ``is_decode`` (no mask) or prefill (row i sees keys 0..i);
        the result is position-major ``[S, H*D]`` like its ``ctx_flat``."""
        q, k, v = inputs[:3]
        h, s_len, d = q.shape
        out = torch.empty((s_len, h, d), dtype=q.dtype, device=q.device)
        ops.attention_dense(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), mask="none" if kw.get("is_decode", s_len == 1) else "causal",
                            scale=1.0, out=out.permute(1, 0, 2).unsqueeze(0))
        return out.view(s_len, h * d)

    def _op_cache_read(self, inputs: list[Any], **kw: Any) -> Any:
        """``cache_read(block_table [R,max_blocks])`` -> ``(key, value)`` each ``[R, max_seq_len, Hkv, D]``
        (sf-dialect/include/Sf/HALOps.td:190-194; CacheManager.read_paged, python_runtime/engine/cache_manager.py:173-197).
        Keywords: ``k_cache``, ``v_cache``, ``max_seq_len``, optional ``seq_lens`` (default: every table entry is read,
        as read_paged does), ``k_scale`` / ``v_scale`` for an e4m3 pool, ``out_dtype``."""
        table = inputs[0]
        bs = kw["k_cache"].shape[1]
        max_len = int(kw.get("max_seq_len", table.shape[1] * bs))
        lens = kw.get("seq_lens")
        if lens is None:
            lens = torch.full((table.shape[0],), table.shape[1] * bs, dtype=torch.int32, device=table.device)
        key = ops.cache_read(kw["k_cache"], table, lens, max_len, scale=kw.get("k_scale"), out_dtype=kw.get("out_dtype"))
        value = ops.cache_read(kw["v_cache"], table, lens, max_len, scale=kw.get("v_scale"), out_dtype=kw.get("out_dtype"))
        return key, value

    def _op_fused_rms_norm_matmul(self, inputs: list[Any], **kw: Any) -> torch.Tensor:
        """``[x, rms_weight, mat_weight]`` with ``eps`` (default 1e-5), as pytorch_backend/_ops_norm.py:47-65:
        ``rms_norm(x) * rms_weight @ mat_weight``, result in x's dtype.  The folded weight ``diag(rms_weight) mat_weight``
        is built on first use of a weight pair and kept (keyed by the two tensors' storage and version counters; the entry
        keeps both tensors alive so that their addresses cannot be reused).
        fp32 and unaligned shapes go to the fallback executor."""
        x, g, w = inputs[0], inputs[1], inputs[-1]
        own = (x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and w.dtype == x.dtype and g.dtype == x.dtype and w.dim() == 2
               and w.shape[0] == x.shape[-1] and w.shape[0] % 8 == 0 and w.shape[1] % 8 == 0 and w.stride(1) == 1 and x.stride(-1) == 1)
        if not own:
            if self._fallback is None:
                raise ValueError("fused_rms_norm_matmul: bf16 / fp16 with K and N multiples of 8, or a fallback executor")
            return self._fallback.execute("fused_rms_norm_matmul", inputs, **kw)
        key = (g.data_ptr(), g._version, w.data_ptr(), w._version, tuple(w.shape))
        entry = self._folded.get(key)
        if entry is None:
            if len(self._folded) >= 256:
                self._folded.clear()
            # the entry holds g and w: while it lives their storage cannot be freed and handed to other tensors that
            # would then match the key with different contents
            entry = self._folded[key] = (ops.fold_norm_weight(g.contiguous(), w), g, w)
        return ops.fused_rms_norm_matmul(x, entry[0], eps=kw.get("eps", 1e-5))

    def _op_chunked_prefill(self, inputs: list[Any], **kw: Any) -> torch.Tensor:
        """inputs ``[query [T,H,D], key_cache, value_cache, block_table [R,max_blocks]]``
        with keywords ``cu_q [R+1]``, ``ctx_lens [R]`` (int32, device) and ``max_q_tokens``."""
        q, k_cache, v_cache, table = inputs[:4]
        return ops.prefill_paged(q, k_cache, v_cache, table, kw["cu_q"], kw["ctx_lens"], max_q_tokens=int(kw["max_q_tokens"]),
                                 scale=kw.get("scale"), causal=kw.get("causal", True), workspace=kw.get("workspace"))


def register(name: str = "b200") -> None:
    """Register the backend factory with the reference's registry
    (python_runtime/hal/registry.py:13-21) when that package is importable."""
    from python_runtime.hal import registry  # type: ignore

    registry.register(name, lambda **kwargs: B200Backend(**kwargs))
