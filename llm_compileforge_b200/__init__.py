"""B200-native attention hot path for LLM-CompileForge.

Paged-attention decode, FP8-e4m3 KV quantise-on-append / dequantise-in-attention,
chunked prefill and RMSNorm as hand-written sm_100a kernels behind one C ABI
(``include/sfb.h`` -> ``libsfb.so``), exposed to Python through the reference's
operator surface:

    from llm_compileforge_b200 import B200Backend, paged_attention

The CUDA library is loaded on first use; there is no CPU fallback.
"""

from .cache import PagedKVCache
from .hal import B200Backend, OpExecutor
from .kernels_api import FP8KVCacheQuantizer, chunked_prefill, flash_attention_fwd, fused_rms_norm_add, paged_attention

__all__ = ["B200Backend", "OpExecutor", "PagedKVCache", "FP8KVCacheQuantizer", "chunked_prefill", "flash_attention_fwd",
           "fused_rms_norm_add", "paged_attention"]
__version__ = "0.1.0"
