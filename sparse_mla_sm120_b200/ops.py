"""The legacy op surface of the reference (sparse_mla_sm120/ops.py:100-189), on B200 kernels.

``sparse_mla_decode_fwd``, ``sparse_mla_prefill_fwd`` and ``sparse_mla_fwd`` take
(q [T, H, 576] bf16, kv_cache [pool, 1, 656] uint8, indices [T, topk] int32, sm_scale, d_v) and
return the bf16 output only, exactly as the legacy package does.  The legacy limits that came
from its fixed workspace (decode <= 64 tokens, topk == 2048) do not apply here.
"""
from __future__ import annotations

import torch

from . import flash_ops

_DECODE_THRESHOLD = 64


def _validate_common_inputs(q, kv_cache, indices, d_v=512):
    assert q.dtype == torch.bfloat16, f"q must be bf16, got {q.dtype}"
    assert q.is_contiguous(), "q must be contiguous"
    assert kv_cache.is_contiguous(), "kv_cache must be contiguous"
    assert indices.dtype == torch.int32, f"indices must be int32, got {indices.dtype}"
    assert indices.is_contiguous(), "indices must be contiguous"
    num_tokens, num_heads, dim = q.shape
    return num_tokens, num_heads, dim, dim - d_v, indices.shape[-1]


def sparse_mla_decode_fwd(q, kv_cache, indices, sm_scale, d_v: int = 512) -> torch.Tensor:
    """sparse_mla_sm120/ops.py:100-147: decode, returns output [T, H, d_v] bf16."""
    _validate_common_inputs(q, kv_cache, indices, d_v)
    return flash_ops.sparse_mla_decode_fwd(q, kv_cache, indices, sm_scale, d_v)[0]


def sparse_mla_prefill_fwd(q, kv_cache, indices, sm_scale, d_v: int = 512) -> torch.Tensor:
    """sparse_mla_sm120/ops.py:150-175: prefill, returns output [T, H, d_v] bf16."""
    _validate_common_inputs(q, kv_cache, indices, d_v)
    return flash_ops.sparse_mla_prefill_fwd(q, kv_cache, indices, sm_scale, d_v)[0]


def sparse_mla_fwd(q, kv_cache, indices, sm_scale, d_v: int = 512) -> torch.Tensor:
    """sparse_mla_sm120/ops.py:178-189: decode for <= 64 tokens, prefill above."""
    if q.shape[0] <= _DECODE_THRESHOLD:
        return sparse_mla_decode_fwd(q, kv_cache, indices, sm_scale, d_v)
    return sparse_mla_prefill_fwd(q, kv_cache, indices, sm_scale, d_v)
