"""``flash_mla_sm120.interface`` of the reference (flash_mla_sm120/interface.py:13-194) on the B200 kernels."""
from sparse_mla_sm120_b200.interface import (  # noqa: F401
    FlashMLASchedMeta,
    flash_mla_sparse_fwd,
    flash_mla_with_kvcache,
    get_mla_metadata,
)
