"""Import-name shim: ``flash_mla_sm120`` of the reference project, served by the B200 kernels.

A caller of the reference (``import flash_mla_sm120``, ``flash_mla_sm120.ops``,
``flash_mla_sm120.interface``, ``flash_mla_sm120.cuda``) finds the same names, argument orders and
return values here (flash_mla_sm120/__init__.py:1-16 of the reference); the work is done by
``sparse_mla_sm120_b200``."""
from .ops import sparse_mla_decode_fwd, sparse_mla_prefill_fwd
from .interface import (
    FlashMLASchedMeta,
    get_mla_metadata,
    flash_mla_with_kvcache,
    flash_mla_sparse_fwd,
)

__all__ = [
    "sparse_mla_decode_fwd",
    "sparse_mla_prefill_fwd",
    "FlashMLASchedMeta",
    "get_mla_metadata",
    "flash_mla_with_kvcache",
    "flash_mla_sparse_fwd",
]
