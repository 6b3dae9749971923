"""``flash_mla_sm120.ops`` of the reference (flash_mla_sm120/ops.py:48-165) on the B200 kernels."""
import torch

from sparse_mla_sm120_b200.flash_ops import sparse_mla_decode_fwd, sparse_mla_prefill_fwd  # noqa: F401


def _effective_stride_kv_row(kv_cache: torch.Tensor) -> int:
    """Bytes per token such that ``page_block_size * result`` is the distance between two pages,
    also for caches whose pages are padded (the helper of flash_mla_sm120/ops.py:23-45, which
    callers and the reference's tests/test_nan_safe.py:105-131 import from here).  The B200 ops
    take the page stride from the tensor themselves; this is for code that calls the raw entries."""
    row_bytes = kv_cache.stride(-2) * kv_cache.element_size()
    if kv_cache.dim() < 3:
        return row_bytes
    rows_per_page = kv_cache.shape[-3]
    page_bytes = kv_cache.stride(0) * kv_cache.element_size()
    if page_bytes == rows_per_page * row_bytes:
        return row_bytes
    if page_bytes % rows_per_page:
        raise AssertionError(f"kv_cache block stride {page_bytes} not divisible by page_block_size {rows_per_page}")
    return page_bytes // rows_per_page
