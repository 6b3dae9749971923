"""FP8 MQA-logits indexer, top-k selection and the KV-cache writer.

None of these has a counterpart in the reference project: its indices come from an external
indexer (flash_mla_sm120/interface.py:39-58) and its cache is written by the serving engine;
the cache row format is the one of tests/test_decode.py:33-57.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from ._lib import IMPL_AUTO, check
from ._runtime import ptr, require_cuda, status_buffer, stream_ptr


def fp8_mqa_logits(q: torch.Tensor, k: torch.Tensor, k_scale: torch.Tensor, weights: torch.Tensor,
                   ks: torch.Tensor, ke: torch.Tensor, out: Optional[torch.Tensor] = None,
                   impl: int = IMPL_AUTO) -> torch.Tensor:
    """logits[i, j] = k_scale[j] * sum_h weights[i, h] * relu(q[i, h] . k[j]); -inf outside [ks_i, ke_i).

    q [s_q, H, 128] float8_e4m3fn, k [s_k, 128] float8_e4m3fn, k_scale [s_k] fp32,
    weights [s_q, H] fp32, ks / ke [s_q] int32 -> logits [s_q, s_k] fp32."""
    require_cuda(q, k, k_scale, weights, ks, ke, out)
    if q.dtype != torch.float8_e4m3fn or k.dtype != torch.float8_e4m3fn:
        raise ValueError("q and k must be float8_e4m3fn")
    if q.dim() != 3 or k.dim() != 2 or q.shape[-1] != 128 or k.shape[-1] != 128:
        raise ValueError("q must be [s_q, H, 128] and k [s_k, 128]")
    assert q.is_contiguous() and k.is_contiguous() and weights.is_contiguous() and k_scale.is_contiguous()
    assert ks.dtype == torch.int32 and ke.dtype == torch.int32
    s_q, h, _ = q.shape
    s_k = k.shape[0]
    if out is None:
        out = torch.empty((s_q, s_k), dtype=torch.float32, device=q.device)
    check(_lib.load().smla_mqa_logits(ptr(q), ptr(k), ptr(k_scale), ptr(weights), ptr(ks), ptr(ke), ptr(out),
                                      s_q, h, s_k, out.stride(0), impl, ptr(status_buffer(q.device)),
                                      stream_ptr(q.device)))
    return out


def topk_indices(logits: torch.Tensor, ks: Optional[torch.Tensor], ke: Optional[torch.Tensor],
                 k: int = 2048) -> torch.Tensor:
    """Per row, the column numbers of the k largest logits inside [ks, ke) as int32 [rows, k],
    padded with -1 when fewer than k candidates exist.  Ties at the k-th value go to the lowest
    columns.  The order inside a row is a fixed function of the input but not ascending, and not
    part of the contract.  Rows of any width."""
    require_cuda(logits, ks, ke)
    assert logits.dim() == 2 and logits.dtype == torch.float32 and logits.stride(1) == 1
    rows, cols = logits.shape
    out = torch.empty((rows, k), dtype=torch.int32, device=logits.device)
    check(_lib.load().smla_topk(ptr(logits), ptr(ks), ptr(ke), ptr(out), rows, cols, logits.stride(0), k,
                                stream_ptr(logits.device)))
    return out


def pack_kv_cache(kv_bf16: torch.Tensor) -> torch.Tensor:
    """bf16 [..., 576] -> packed uint8 [..., 656] (512 e4m3 | 4 fp32 power-of-two scales | 64 bf16)."""
    require_cuda(kv_bf16)
    assert kv_bf16.dtype == torch.bfloat16 and kv_bf16.shape[-1] == 576 and kv_bf16.is_contiguous()
    rows = kv_bf16.numel() // 576
    out = torch.empty(kv_bf16.shape[:-1] + (656,), dtype=torch.uint8, device=kv_bf16.device)
    check(_lib.load().smla_pack_kv(ptr(kv_bf16), ptr(out), rows, stream_ptr(kv_bf16.device)))
    return out
