"""Indexer -> top-k -> sparse attention as one call (one GPU).

The reference has the attention ops only (sparse_mla_sm120/ops.py, flash_mla_sm120/ops.py); the
indices they consume come from an indexer outside it (flash_mla_sm120/interface.py:39-58), and a
serving stack chains the steps per layer.  Here the chain is one function on one stream with no
host synchronisation in between, so it can be captured into a CUDA graph as a whole."""
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


class GraphedIndexedDecode:
    """The indexer -> top-k -> decode chain of one decoding step captured into a CUDA graph.

    Shapes are fixed at construction (tokens, heads, context length, top-k); the caches are bound
    by reference (a serving stack appends to them in place between steps), the per-step inputs
    are copied into static buffers before every replay.  One graph launch replaces about ten
    kernel launches and their host-side argument handling."""

    def __init__(self, kv_cache: torch.Tensor, ki: torch.Tensor, k_scale: torch.Tensor, num_tokens: int,
                 num_heads: int, indexer_heads: int, sm_scale: float, topk: int = 2048,
                 block_table: Optional[torch.Tensor] = None, attn_sink: Optional[torch.Tensor] = None,
                 impl: int = IMPL_AUTO):
        dev = kv_cache.device
        # the graph holds raw pointers into these: they must live as long as it does
        self.kv_cache, self.ki, self.k_scale, self.block_table, self.attn_sink = kv_cache, ki, k_scale, block_table, attn_sink
        self.q = torch.zeros((num_tokens, num_heads, 576), dtype=torch.bfloat16, device=dev)
        self.qi = torch.zeros((num_tokens, indexer_heads, 128), dtype=torch.float8_e4m3fn, device=dev)
        self.weights = torch.zeros((num_tokens, indexer_heads), dtype=torch.float32, device=dev)
        self.ks = torch.zeros(num_tokens, dtype=torch.int32, device=dev)
        self.ke = torch.zeros(num_tokens, dtype=torch.int32, device=dev)

        def step():
            return sparse_mla_indexed_decode_fwd(self.q, kv_cache, self.qi, ki, k_scale, self.weights, self.ks, self.ke,
                                                 sm_scale, topk=topk, block_table=block_table, attn_sink=attn_sink,
                                                 impl=impl)

        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            step()                                   # warm-up: library load, scratch buffers, kernel attributes
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=side):
                self.out, self.lse, self.rows = step()
        torch.cuda.current_stream(dev).wait_stream(side)

    def __call__(self, q, qi, weights, ks, ke) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """Returns (out, lse, rows): static tensors, overwritten by the next call."""
        self.q.copy_(q)
        self.qi.copy_(qi)
        self.weights.copy_(weights)
        self.ks.copy_(ks)
        self.ke.copy_(ke)
        return self.replay()

    def replay(self) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """For callers that write the step's inputs straight into ``self.q``, ``self.qi``,
        ``self.weights``, ``self.ks``, ``self.ke``: one graph launch, nothing else."""
        self.graph.replay()
        return self.out, self.lse, self.rows
