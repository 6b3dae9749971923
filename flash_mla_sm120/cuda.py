"""``flash_mla_sm120.cuda`` of the reference: the four raw entry points of csrc/binding.cpp:250-292,
with the same positional and keyword arguments, on the B200 kernels (through the C ABI of
libsmla_b200.so)."""
from sparse_mla_sm120_b200.flash_ops import (  # noqa: F401
    get_decode_metadata,
    sparse_mla_combine_v2_fwd,
    sparse_mla_splitkv_v2_fwd,
)
from sparse_mla_sm120_b200.flash_ops import sparse_mla_prefill_raw as sparse_mla_prefill_fwd  # noqa: F401
