"""Indexer -> top-k -> sparse attention as one call (one GPU).

The reference ships the three kernels separately (the attention ops in sparse_mla_sm120/ops.py,
the indexer benchmarked by benchmarks/bench_lighting_indexer.py) and a serving stack chains them
per layer.  Here the chain is one function on one stream with no host synchronisation in between,
so it can be captured into a CUDA graph as a whole."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import indexer
from ._lib import IMPL_AUTO
from .flash_ops import sparse_mla_decode_fwd


def positions_to_rows(positions: torch.Tensor, block_table: torch.Tensor, page_block_size: int) -> torch.Tensor:
    """Logical token positions [T, k] (-1 = none) -> physical cache rows through the page table
    ``block_table`` [T, max_pages] int32 (row t is the table of the request token t belongs to)."""
    valid = positions >= 0
    p = positions.clamp(min=0).long()
    page = torch.gather(block_table.long(), 1, p // page_block_size)
    rows = page * page_block_size + p % page_block_size
    return torch.where(valid, rows, torch.full_like(rows, -1)).to(torch.int32)


def sparse_mla_indexed_decode_fwd(q: torch.Tensor, kv_cache: torch.Tensor, qi: torch.Tensor, ki: torch.Tensor,
                                  k_scale: torch.Tensor, weights: torch.Tensor, ks: torch.Tensor, ke: torch.Tensor,
                                  sm_scale: float, topk: int = 2048, block_table: Optional[torch.Tensor] = None,
                                  attn_sink: Optional[torch.Tensor] = None, impl: int = IMPL_AUTO,
                                  ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``q`` [T, H, 576] bf16 attention queries, ``qi`` [T, H_i, 128] e4m3 / ``weights`` [T, H_i]
    indexer queries, ``ki`` [s_k, 128] e4m3 / ``k_scale`` [s_k] indexer keys, ``ks`` / ``ke`` [T]
    the window of each token.  Returns (out [T, H, 512] bf16, lse [T, H], rows [T, topk] int32)."""
    logits = indexer.fp8_mqa_logits(qi, ki, k_scale, weights, ks, ke)
    rows = indexer.topk_indices(logits, ks, ke, topk)
    if block_table is not None:
        rows = positions_to_rows(rows, block_table, kv_cache.shape[1])
    out, lse = sparse_mla_decode_fwd(q, kv_cache, rows, sm_scale, attn_sink=attn_sink, impl=impl)
    return out, lse, rows
