"""Import-name shim: the legacy ``sparse_mla_sm120`` package of the reference
(sparse_mla_sm120/__init__.py, ops.py:100-189), served by the B200 kernels."""
from .ops import sparse_mla_decode_fwd, sparse_mla_fwd, sparse_mla_prefill_fwd

__all__ = ["sparse_mla_decode_fwd", "sparse_mla_prefill_fwd", "sparse_mla_fwd"]
