"""B200-native sparse-MLA kernels behind the op surface of leavelet/sparse_mla_sm120.

``sparse_mla_decode_fwd`` / ``sparse_mla_prefill_fwd`` / ``sparse_mla_fwd`` are the legacy
surface (bf16 output only); ``flash_ops`` holds the current surface (tuples with LSE) and the
raw scheduler / split-KV / combine entry points; ``indexer`` the FP8 MQA-logits indexer, top-k
and cache writer; ``pipeline`` the indexer -> top-k -> attention chain as one call;
``interface`` the FlashMLA-shaped surface; ``cp`` the multi-GPU paths.  Everything runs through libsmla_b200.so.
"""
from .ops import sparse_mla_decode_fwd, sparse_mla_fwd, sparse_mla_prefill_fwd
from . import flash_ops, indexer  # noqa: F401

__all__ = ["sparse_mla_decode_fwd", "sparse_mla_prefill_fwd", "sparse_mla_fwd", "flash_ops", "indexer"]
