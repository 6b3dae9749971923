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


def _check_inputs(q, kv_cache, indices, d_v):
    """The legacy surface takes contiguous bf16 queries, a contiguous byte cache and int32 indices
    (sparse_mla_sm120/ops.py:82-97 asserts the same); anything else is a ValueError here."""
    problems = []
    if q.dtype != torch.bfloat16:
        problems.append(f"q must be bf16, got {q.dtype}")
    if indices.dtype != torch.int32:
        problems.append(f"indices must be int32, got {indices.dtype}")
    for name, t in (("q", q), ("kv_cache", kv_cache), ("indices", indices)):
        if not t.is_contiguous():
            problems.append(f"{name} must be contiguous")
    if q.dim() != 3 or q.shape[-1] - d_v != 64:
        problems.append(f"q must be [num_tokens, num_heads, d_v + 64], got {tuple(q.shape)} with d_v={d_v}")
    if problems:
        raise ValueError("; ".join(problems))


def sparse_mla_decode_fwd(q, kv_cache, indices, sm_scale, d_v: int = 512) -> torch.Tensor:
    """sparse_mla_sm120/ops.py:100-147: decode, returns output [T, H, d_v] bf16."""
    _check_inputs(q, kv_cache, indices, d_v)
    return flash_ops.sparse_mla_decode_fwd(q, kv_cache, indices, sm_scale, d_v)[0]


def sparse_mla_prefill_fwd(q, kv_cache, indices, sm_scale, d_v: int = 512) -> torch.Tensor:
    """sparse_mla_sm120/ops.py:150-175: prefill, returns output [T, H, d_v] bf16."""
    _check_inputs(q, kv_cache, indices, d_v)
    return flash_ops.sparse_mla_prefill_fwd(q, kv_cache, indices, sm_scale, d_v)[0]


def sparse_mla_fwd(q, kv_cache, indices, sm_scale, d_v: int = 512) -> torch.Tensor:
    """sparse_mla_sm120/ops.py:178-189: decode for <= 64 tokens, prefill above."""
    if q.shape[0] <= _DECODE_THRESHOLD:
        return sparse_mla_decode_fwd(q, kv_cache, indices, sm_scale, d_v)
    return sparse_mla_prefill_fwd(q, kv_cache, indices, sm_scale, d_v)
