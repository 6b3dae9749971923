"""FlashMLA-shaped calling surface (flash_mla_sm120/interface.py:13-194) on the B200 kernels.

Same names, arguments and return shapes as the reference module, so that a serving stack that
drives FlashMLA (``get_mla_metadata`` once per decoding step, ``flash_mla_with_kvcache`` once per
layer with the same metadata object) can switch over:

* ``q`` is ``[b, s_q, h_q, d]`` (or ``[tokens, h_q, d]``), ``indices`` ``[b, s_q, topk]``; the
  ``s_q`` query tokens of a request are flattened into tokens, as the reference does
  (interface.py:80-82).
* returns ``out [b, s_q, h_q, d_v]`` bf16 and ``lse [b, h_q, s_q]`` fp32 (base 2).
* the scheduler metadata lives in the ``FlashMLASchedMeta`` object: it is computed by the first
  call that uses the object and reused, after checking that the configuration is the same, by
  the later ones.  Here the object also keeps the split-KV scratch, and when every request gets
  its own partition there is nothing to schedule: the attention kernel runs alone.

Only sparse attention over an FP8 cache is served (as in the reference).  Both cache layouts and the
second ("extra") cache are taken; see flash_ops for which kernel serves which.
"""
from __future__ import annotations

import dataclasses
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import IMPL_AUTO, IMPL_SCALAR, LAYOUT_V32, check
from ._runtime import (BLOCK_N, FIXED_OVERHEAD, kv_geometry, num_sms, pick_num_sm_parts_fp32, pick_split, ptr,
                       require_cuda, resolve_impl, status_buffer, stream_ptr, tc_aligned)
from .flash_ops import _check_q, _Extra, _layout, sparse_mla_prefill_fwd


@dataclasses.dataclass
class FlashMLASchedMeta:
    """Persistent per-step scheduling state (interface.py:13-32)."""

    @dataclasses.dataclass
    class Config:
        b: int
        s_q: int
        h_q: int
        page_block_size: int
        h_k: int
        causal: bool
        is_fp8_kvcache: bool
        topk: Optional[int]
        extra_page_block_size: Optional[int]
        extra_topk: Optional[int]

    have_initialized: bool = False
    config: Optional[Config] = None
    tile_scheduler_metadata: Optional[torch.Tensor] = None
    num_splits: Optional[torch.Tensor] = None
    num_sm_parts: int = 0
    max_nsplits: int = 0
    # split-KV scratch, kept with the metadata so that the layers of a step share it
    o_accum: Optional[torch.Tensor] = None
    lse_accum: Optional[torch.Tensor] = None
    uniform_k: int = 0     # > 1: equally long requests in this many equal partitions each, no scheduler records needed


def get_mla_metadata(*args, **kwargs) -> Tuple[FlashMLASchedMeta, None]:
    """interface.py:35-36: the metadata is filled in lazily by the first attention call."""
    return FlashMLASchedMeta(), None


def flash_mla_with_kvcache(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    block_table: Optional[torch.Tensor],
    cache_seqlens: Optional[torch.Tensor],
    head_dim_v: int,
    tile_scheduler_metadata: FlashMLASchedMeta,
    num_splits: None = None,
    softmax_scale: Optional[float] = None,
    causal: bool = False,
    is_fp8_kvcache: bool = False,
    indices: Optional[torch.Tensor] = None,
    attn_sink: Optional[torch.Tensor] = None,
    extra_k_cache: Optional[torch.Tensor] = None,
    extra_indices_in_kvcache: Optional[torch.Tensor] = None,
    topk_length: Optional[torch.Tensor] = None,
    extra_topk_length: Optional[torch.Tensor] = None,
    bf16_qk: bool = False,
    out: Optional[torch.Tensor] = None,
    impl: int = IMPL_AUTO,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Sparse decode over a paged FP8 cache (interface.py:39-171).  ``block_table`` and
    ``cache_seqlens`` are accepted and unused, as in the reference: ``indices`` are physical rows."""
    meta = tile_scheduler_metadata
    if not isinstance(meta, FlashMLASchedMeta):
        raise TypeError("tile_scheduler_metadata must come from get_mla_metadata()")
    if num_splits is not None:
        raise ValueError("num_splits must be None (the metadata object carries it)")
    if indices is None:
        raise ValueError("only sparse attention is served: indices is required")
    if not is_fp8_kvcache:
        raise ValueError("an FP8 KV cache is required")
    if head_dim_v != 512:
        raise ValueError(f"head_dim_v must be 512, got {head_dim_v}")
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** (-0.5)

    batch = q.shape[0]
    s_q = q.shape[1] if q.dim() == 4 else 1
    q_in = q.reshape(-1, q.shape[-2], q.shape[-1])
    _check_q(q_in)
    num_tokens, num_heads, _ = q_in.shape
    topk = indices.shape[-1]
    idx_in = indices.reshape(num_tokens, topk)
    layout = _layout(q_in, k_cache)
    impl = resolve_impl(impl, layout)
    page_block_size, page_stride = kv_geometry(k_cache)
    require_cuda(q_in, k_cache, idx_in)
    assert idx_in.dtype == torch.int32 and idx_in.is_contiguous()
    extra_topk = extra_indices_in_kvcache.shape[-1] if extra_indices_in_kvcache is not None else 0
    extra_idx = None if extra_indices_in_kvcache is None else extra_indices_in_kvcache.reshape(num_tokens, -1)
    ex = _Extra(layout, num_tokens, extra_k_cache, extra_idx, extra_topk, extra_topk_length)
    use_ext = layout != LAYOUT_V32 or ex.topk > 0
    blocks = max(-(-topk // BLOCK_N), 1) + -(-ex.topk // BLOCK_N)

    cfg = FlashMLASchedMeta.Config(b=batch, s_q=s_q, h_q=num_heads, page_block_size=k_cache.shape[1],
                                   h_k=k_cache.shape[2], causal=causal, is_fp8_kvcache=is_fp8_kvcache, topk=topk,
                                   extra_page_block_size=extra_k_cache.shape[1] if extra_k_cache is not None else None,
                                   extra_topk=ex.topk if ex.topk > 0 else None)
    lib = _lib.load()
    stream = stream_ptr(q.device)
    if not meta.have_initialized:
        meta.have_initialized = True
        meta.config = cfg
        fp32 = use_ext and (impl == IMPL_SCALAR or not tc_aligned(k_cache, ex.kv))
        fixed_overhead = FIXED_OVERHEAD
        if fp32:
            meta.num_sm_parts = pick_num_sm_parts_fp32(num_tokens, num_heads, num_sms(q.device))
        else:
            meta.num_sm_parts, fixed_overhead = pick_split(num_tokens, num_sms(q.device), blocks,
                                                           uniform=topk_length is None and ex.topk == 0)
        meta.max_nsplits = min(blocks, meta.num_sm_parts)
        if (not use_ext and fixed_overhead == 0 and impl != IMPL_SCALAR and meta.num_sm_parts > num_tokens
                and meta.num_sm_parts % num_tokens == 0 and blocks % (meta.num_sm_parts // num_tokens) == 0):
            meta.uniform_k = meta.num_sm_parts // num_tokens
        if meta.num_sm_parts != num_tokens:
            meta.tile_scheduler_metadata = torch.empty(meta.num_sm_parts * 8, dtype=torch.int32, device=q.device)
            meta.num_splits = torch.empty(num_tokens + 1, dtype=torch.int32, device=q.device)
            check(lib.smla_sched_meta(num_tokens, topk, ex.topk, meta.num_sm_parts, fixed_overhead, ptr(topk_length),
                                      ptr(ex.length), ptr(meta.tile_scheduler_metadata), ptr(meta.num_splits), stream))
            records = num_tokens + meta.num_sm_parts
            meta.o_accum = torch.empty((records, 1, num_heads, head_dim_v), dtype=torch.float32, device=q.device)
            meta.lse_accum = torch.empty((records, 1, num_heads), dtype=torch.float32, device=q.device)
    elif meta.config != cfg:
        raise ValueError(f"the metadata object was initialised for {meta.config}, this call has {cfg}")

    if out is not None:
        output = out.view(num_tokens, num_heads, head_dim_v)
    else:
        output = torch.empty((num_tokens, num_heads, head_dim_v), dtype=torch.bfloat16, device=q.device)
    out_lse = torch.empty((num_tokens, num_heads), dtype=torch.float32, device=q.device)
    st = status_buffer(q.device)
    if use_ext and meta.num_sm_parts == num_tokens:
        check(lib.smla_prefill_ext(
            ptr(q_in), ptr(k_cache), ptr(idx_in), ptr(ex.kv), ptr(ex.indices), ptr(output), ptr(out_lse), None,
            num_tokens, num_heads, topk, ex.topk, float(softmax_scale), layout, page_block_size, page_stride,
            ex.block, ex.stride, ptr(attn_sink), ptr(topk_length), ptr(ex.length), impl, ptr(st), stream))
    elif use_ext:
        check(lib.smla_decode_splitkv_ext(
            ptr(q_in), ptr(k_cache), ptr(idx_in), ptr(ex.kv), ptr(ex.indices), ptr(meta.o_accum), ptr(meta.lse_accum),
            ptr(output), ptr(out_lse), ptr(meta.tile_scheduler_metadata), ptr(meta.num_splits), num_tokens, num_heads,
            topk, ex.topk, float(softmax_scale), layout, page_block_size, page_stride, ex.block, ex.stride,
            meta.num_sm_parts, ptr(attn_sink), ptr(topk_length), ptr(ex.length), impl, ptr(st), stream))
        check(lib.smla_combine(ptr(meta.o_accum), ptr(meta.lse_accum), ptr(output), ptr(out_lse), ptr(meta.num_splits),
                               num_tokens, num_heads, meta.max_nsplits, ptr(attn_sink), stream))
    elif meta.num_sm_parts == num_tokens:
        check(lib.smla_prefill(ptr(q_in), ptr(k_cache), ptr(idx_in), ptr(output), ptr(out_lse), None, num_tokens,
                               num_heads, topk, float(softmax_scale), page_block_size, page_stride, ptr(attn_sink),
                               ptr(topk_length), impl, ptr(st), stream))
    elif meta.uniform_k > 1 and impl != IMPL_SCALAR and topk_length is None:
        check(lib.smla_decode_uniform(
            ptr(q_in), ptr(k_cache), ptr(idx_in), ptr(meta.o_accum), ptr(meta.lse_accum), ptr(output), ptr(out_lse),
            num_tokens, num_heads, topk, float(softmax_scale), page_block_size, page_stride, meta.uniform_k,
            ptr(attn_sink), impl, ptr(st), stream))
    else:
        check(lib.smla_decode_splitkv(
            ptr(q_in), ptr(k_cache), ptr(idx_in), ptr(meta.o_accum), ptr(meta.lse_accum), ptr(output), ptr(out_lse),
            ptr(meta.tile_scheduler_metadata), ptr(meta.num_splits), num_tokens, num_heads, topk,
            float(softmax_scale), page_block_size, page_stride, meta.num_sm_parts, ptr(attn_sink), ptr(topk_length),
            impl, ptr(st), stream))
        check(lib.smla_combine(ptr(meta.o_accum), ptr(meta.lse_accum), ptr(output), ptr(out_lse), ptr(meta.num_splits),
                               num_tokens, num_heads, meta.max_nsplits, ptr(attn_sink), stream))
    output = output.reshape(batch, s_q, num_heads, head_dim_v)
    lse = out_lse.reshape(batch, s_q, num_heads).permute(0, 2, 1).contiguous()
    return output, lse


def flash_mla_sparse_fwd(
    q: torch.Tensor,
    kv: torch.Tensor,
    indices: torch.Tensor,
    sm_scale: float,
    d_v: int = 512,
    attn_sink: Optional[torch.Tensor] = None,
    topk_length: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    extra_k_cache: Optional[torch.Tensor] = None,
    extra_indices_in_kvcache: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Sparse prefill (interface.py:174-194): ``indices`` may carry a singleton middle dimension.
    Returns (out, max_logits, lse)."""
    idx = indices.squeeze(1) if indices.dim() == 3 else indices
    extra_topk = extra_indices_in_kvcache.shape[-1] if extra_indices_in_kvcache is not None else 0
    return sparse_mla_prefill_fwd(q, kv, idx, sm_scale, d_v, attn_sink=attn_sink, topk_length=topk_length, out=out,
                                  extra_k_cache=extra_k_cache, extra_indices=extra_indices_in_kvcache,
                                  extra_topk=extra_topk)
