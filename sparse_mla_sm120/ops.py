"""``sparse_mla_sm120.ops`` of the reference (sparse_mla_sm120/ops.py:100-189) on the B200 kernels."""
from sparse_mla_sm120_b200.ops import sparse_mla_decode_fwd, sparse_mla_fwd, sparse_mla_prefill_fwd  # noqa: F401
