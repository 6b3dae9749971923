"""The current op surface of the reference (flash_mla_sm120/ops.py:48-165), on B200 kernels.

Same names, argument order, argument meaning and return tuples; the raw entry points that the
reference exposes as ``flash_mla_sm120.cuda`` (csrc/binding.cpp:250-292) are the functions
``get_decode_metadata``, ``sparse_mla_splitkv_v2_fwd``, ``sparse_mla_combine_v2_fwd`` and
``sparse_mla_prefill_raw`` below.

Two cache layouts are served, told apart as the reference does by the width of q and of a cache row:
V32 (q 576 wide, 656-byte rows) and MODEL1 (q 512 wide, 584 bytes per token with the scales in a footer
of the page; V is the whole row).  V32 without a second cache runs on the tcgen05 kernels; MODEL1 and the
second ("extra") cache run on the exact fp32 kernel.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import IMPL_AUTO, IMPL_SCALAR, LAYOUT_MODEL1, LAYOUT_V32, check
from ._runtime import (BLOCK_N, FIXED_OVERHEAD, kv_geometry, kv_layout, num_sms, pick_num_sm_parts_fp32, pick_split, ptr,
                       require_cuda, resolve_impl, scratch, status_buffer, stream_ptr, tc_aligned)


def _check_q(q: torch.Tensor):
    if q.dim() != 3:
        raise ValueError(f"q must be [num_tokens, num_heads, d_qk], got {tuple(q.shape)}")
    if q.dtype != torch.bfloat16:
        raise ValueError(f"q must be bf16, got {q.dtype}")
    if q.shape[-1] not in (576, 512):
        raise ValueError(f"Unsupported d_qk={q.shape[-1]}; expected 576 (V32) or 512 (MODEL1)")
    assert q.is_contiguous()


def _layout(q: torch.Tensor, kv_cache: torch.Tensor) -> int:
    """Cache layout of a call (csrc/binding.cpp:117-133 dispatches on d_qk in the same way)."""
    layout = kv_layout(kv_cache)
    want = LAYOUT_MODEL1 if q.shape[-1] == 512 else LAYOUT_V32
    if layout != want:
        raise ValueError(f"q with {q.shape[-1]} dims does not go with cache rows of {kv_cache.shape[-1]} bytes")
    return layout


class _Extra:
    """The second cache of a call: pointers and page geometry, all zero when there is none."""

    def __init__(self, layout, num_tokens, extra_k_cache, extra_indices, extra_topk, extra_topk_length=None):
        self.topk = int(extra_topk or 0)
        self.kv = self.indices = self.length = None
        self.block, self.stride = 0, 0
        if self.topk <= 0:
            self.topk = 0
            return
        if extra_k_cache is None or extra_indices is None:
            raise ValueError(f"extra_topk={extra_topk} needs extra_k_cache and extra_indices")
        if kv_layout(extra_k_cache) != layout:
            raise ValueError("the extra cache must have the layout of the main cache")
        require_cuda(extra_k_cache, extra_indices, extra_topk_length)
        if extra_indices.dtype != torch.int32 or not extra_indices.is_contiguous() or \
                extra_indices.numel() != num_tokens * self.topk:
            raise ValueError(f"extra_indices must be contiguous int32 [{num_tokens}, {self.topk}]")
        self.block, self.stride = kv_geometry(extra_k_cache)
        self.kv, self.indices, self.length = extra_k_cache, extra_indices, extra_topk_length


# ------------------------------------------------------------------ raw entry points
def get_decode_metadata(b, topk, extra_topk, num_sm_parts, fixed_overhead, topk_length, extra_topk_length,
                        sched_meta, num_splits):
    """csrc/binding.cpp:281-286."""
    require_cuda(sched_meta, num_splits, topk_length, extra_topk_length)
    check(_lib.load().smla_sched_meta(b, topk, extra_topk, num_sm_parts, fixed_overhead, ptr(topk_length),
                                      ptr(extra_topk_length), ptr(sched_meta), ptr(num_splits),
                                      stream_ptr(sched_meta.device)))


def sparse_mla_splitkv_v2_fwd(Q, KV_cache, indices, o_accum, lse_accum, output, out_lse, sched_meta, num_splits,
                              sm_scale, topk, stride_kv_row, page_block_size, num_sm_parts, attn_sink=None,
                              extra_k_cache=None, extra_indices=None, topk_length=None, extra_topk=0,
                              extra_topk_length=None, bf16_qk=True, impl=IMPL_AUTO):
    """csrc/binding.cpp:96-164.  ``stride_kv_row * page_block_size`` is the page stride."""
    _check_q(Q)
    require_cuda(Q, KV_cache, indices, o_accum, lse_accum, output, out_lse, sched_meta, num_splits)
    if attn_sink is not None and attn_sink.dtype != torch.float32:
        raise ValueError("attn_sink must be float32")
    num_tokens, num_heads, _ = Q.shape
    st = status_buffer(Q.device)
    layout = _layout(Q, KV_cache)
    impl = resolve_impl(impl, layout)
    ex = _Extra(layout, num_tokens, extra_k_cache, extra_indices, extra_topk, extra_topk_length)
    if layout != LAYOUT_V32 or ex.topk:
        check(_lib.load().smla_decode_splitkv_ext(
            ptr(Q), ptr(KV_cache), ptr(indices), ptr(ex.kv), ptr(ex.indices), ptr(o_accum), ptr(lse_accum),
            ptr(output), ptr(out_lse), ptr(sched_meta), ptr(num_splits), num_tokens, num_heads, topk, ex.topk,
            float(sm_scale), layout, page_block_size, int(stride_kv_row) * int(page_block_size), ex.block, ex.stride,
            num_sm_parts, ptr(attn_sink), ptr(topk_length), ptr(ex.length), impl, ptr(st), stream_ptr(Q.device)))
        return
    check(_lib.load().smla_decode_splitkv(
        ptr(Q), ptr(KV_cache), ptr(indices), ptr(o_accum), ptr(lse_accum), ptr(output), ptr(out_lse),
        ptr(sched_meta), ptr(num_splits), num_tokens, num_heads, topk, float(sm_scale), page_block_size,
        int(stride_kv_row) * int(page_block_size), num_sm_parts, ptr(attn_sink), ptr(topk_length), impl,
        ptr(st), stream_ptr(Q.device)))


def sparse_mla_combine_v2_fwd(o_accum, lse_accum, output, out_lse, num_splits_ptr, batch, max_nsplits,
                              attn_sink=None):
    """csrc/binding.cpp:166-183."""
    require_cuda(o_accum, lse_accum, output, out_lse, num_splits_ptr)
    num_heads = o_accum.shape[2]
    check(_lib.load().smla_combine(ptr(o_accum), ptr(lse_accum), ptr(output), ptr(out_lse), ptr(num_splits_ptr),
                                   batch, num_heads, max_nsplits, ptr(attn_sink), stream_ptr(o_accum.device)))


def sparse_mla_prefill_raw(Q, KV_cache, indices, output, out_lse, sm_scale, topk, stride_kv_row, page_block_size,
                           attn_sink=None, topk_length=None, bf16_qk=True, out_max_logits=None,
                           extra_k_cache=None, extra_indices=None, extra_topk=0, impl=IMPL_AUTO):
    """csrc/binding.cpp:185-247 (there named sparse_mla_prefill_fwd)."""
    _check_q(Q)
    require_cuda(Q, KV_cache, indices, output, out_lse)
    if output.dtype != torch.bfloat16:
        raise ValueError("output must be bf16")
    if out_lse.dtype != torch.float32:
        raise ValueError("out_lse must be float32")
    num_tokens, num_heads, _ = Q.shape
    st = status_buffer(Q.device)
    layout = _layout(Q, KV_cache)
    impl = resolve_impl(impl, layout)
    ex = _Extra(layout, num_tokens, extra_k_cache, extra_indices, extra_topk)
    if layout != LAYOUT_V32 or ex.topk:
        check(_lib.load().smla_prefill_ext(
            ptr(Q), ptr(KV_cache), ptr(indices), ptr(ex.kv), ptr(ex.indices), ptr(output), ptr(out_lse),
            ptr(out_max_logits), num_tokens, num_heads, topk, ex.topk, float(sm_scale), layout, page_block_size,
            int(stride_kv_row) * int(page_block_size), ex.block, ex.stride, ptr(attn_sink), ptr(topk_length), None,
            impl, ptr(st), stream_ptr(Q.device)))
        return
    check(_lib.load().smla_prefill(
        ptr(Q), ptr(KV_cache), ptr(indices), ptr(output), ptr(out_lse), ptr(out_max_logits), num_tokens,
        num_heads, topk, float(sm_scale), page_block_size, int(stride_kv_row) * int(page_block_size),
        ptr(attn_sink), ptr(topk_length), impl, ptr(st), stream_ptr(Q.device)))


# ------------------------------------------------------------------ op surface
def sparse_mla_decode_fwd(
    q: torch.Tensor,
    kv_cache: torch.Tensor,
    indices: torch.Tensor,
    sm_scale: float,
    d_v: int = 512,
    attn_sink: Optional[torch.Tensor] = None,
    bf16_qk: bool = True,
    extra_k_cache: Optional[torch.Tensor] = None,
    extra_indices: Optional[torch.Tensor] = None,
    topk_length: Optional[torch.Tensor] = None,
    extra_topk_length: Optional[torch.Tensor] = None,
    extra_topk: int = 0,
    out: Optional[torch.Tensor] = None,
    impl: int = IMPL_AUTO,
    num_sm_parts: Optional[int] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Split-KV sparse-MLA decode: scheduler -> attention -> combine (attention alone when the
    partition count equals the number of requests, i.e. when nothing is split).

    q [T, H, 576] bf16 over packed 656-byte rows, or q [T, H, 512] over the 584-byte MODEL1 layout;
    indices [T, topk] int32 (-1 = no entry); extra_k_cache / extra_indices [T, extra_topk] /
    extra_topk_length name a second cache whose rows join the same softmax.
    Returns (out [T, H, 512] bf16, lse [T, H] fp32, base-2 LSE of the scaled logits).
    Signature and results follow flash_mla_sm120/ops.py:48-119."""
    _check_q(q)
    layout = _layout(q, kv_cache)
    impl = resolve_impl(impl, layout)
    page_block_size, page_stride = kv_geometry(kv_cache)
    if d_v != 512:
        raise ValueError(f"d_v must be 512, got {d_v}")
    num_tokens, num_heads, _ = q.shape
    topk = indices.shape[-1]
    assert indices.dtype == torch.int32 and indices.is_contiguous()
    ex = _Extra(layout, num_tokens, extra_k_cache, extra_indices, extra_topk, extra_topk_length)
    require_cuda(q, kv_cache, indices)
    use_ext = layout != LAYOUT_V32 or ex.topk > 0
    blocks = max(-(-topk // BLOCK_N), 1) + -(-ex.topk // BLOCK_N)

    fixed_overhead = FIXED_OVERHEAD
    if num_sm_parts is None:
        fp32 = use_ext and (impl == IMPL_SCALAR or not tc_aligned(kv_cache, ex.kv))
        if fp32:
            num_sm_parts = pick_num_sm_parts_fp32(num_tokens, num_heads, num_sms(q.device))
        else:   # requests of equal length (no topk_length, no second cache) may be cut into equal partitions
            num_sm_parts, fixed_overhead = pick_split(num_tokens, num_sms(q.device), blocks,
                                                      uniform=topk_length is None and ex.topk == 0)
    lib = _lib.load()
    stream = stream_ptr(q.device)
    if out is not None:
        output = out.view(num_tokens, num_heads, d_v)
    else:
        output = torch.empty((num_tokens, num_heads, d_v), dtype=torch.bfloat16, device=q.device)
    out_lse = torch.empty((num_tokens, num_heads), dtype=torch.float32, device=q.device)
    if use_ext:
        st = ptr(status_buffer(q.device))
        if num_sm_parts == num_tokens:
            check(lib.smla_prefill_ext(
                ptr(q), ptr(kv_cache), ptr(indices), ptr(ex.kv), ptr(ex.indices), ptr(output), ptr(out_lse), None,
                num_tokens, num_heads, topk, ex.topk, float(sm_scale), layout, page_block_size, page_stride,
                ex.block, ex.stride, ptr(attn_sink), ptr(topk_length), ptr(ex.length), impl, st, stream))
            return output, out_lse
        ws = scratch(q.device, num_tokens + num_sm_parts, num_heads, num_tokens, num_sm_parts)
        check(lib.smla_sched_meta(num_tokens, topk, ex.topk, num_sm_parts, fixed_overhead, ptr(topk_length),
                                  ptr(ex.length), ptr(ws["sched_meta"]), ptr(ws["num_splits"]), stream))
        check(lib.smla_decode_splitkv_ext(
            ptr(q), ptr(kv_cache), ptr(indices), ptr(ex.kv), ptr(ex.indices), ptr(ws["o_accum"]),
            ptr(ws["lse_accum"]), ptr(output), ptr(out_lse), ptr(ws["sched_meta"]), ptr(ws["num_splits"]),
            num_tokens, num_heads, topk, ex.topk, float(sm_scale), layout, page_block_size, page_stride,
            ex.block, ex.stride, num_sm_parts, ptr(attn_sink), ptr(topk_length), ptr(ex.length), impl, st, stream))
        check(lib.smla_combine(ptr(ws["o_accum"]), ptr(ws["lse_accum"]), ptr(output), ptr(out_lse),
                               ptr(ws["num_splits"]), num_tokens, num_heads, min(blocks, num_sm_parts),
                               ptr(attn_sink), stream))
        return output, out_lse
    if num_sm_parts == num_tokens:
        # One partition per request: nothing is split, so neither the scheduler nor the combine
        # has anything to decide; the attention kernel derives the trivial schedule itself.
        check(lib.smla_prefill(
            ptr(q), ptr(kv_cache), ptr(indices), ptr(output), ptr(out_lse), None, num_tokens, num_heads,
            topk, float(sm_scale), page_block_size, page_stride, ptr(attn_sink), ptr(topk_length), impl,
            ptr(status_buffer(q.device)), stream))
        return output, out_lse
    total_splits = num_tokens + num_sm_parts
    ws = scratch(q.device, total_splits, num_heads, num_tokens, num_sm_parts)
    if (fixed_overhead == 0 and topk_length is None and impl != IMPL_SCALAR and num_sm_parts % num_tokens == 0
            and blocks % (num_sm_parts // num_tokens) == 0):
        # requests of equal length in equal partitions: the attention kernel derives the schedule itself, the step is
        # two launches (attention, combine)
        check(lib.smla_decode_uniform(
            ptr(q), ptr(kv_cache), ptr(indices), ptr(ws["o_accum"]), ptr(ws["lse_accum"]), ptr(output), ptr(out_lse),
            num_tokens, num_heads, topk, float(sm_scale), page_block_size, page_stride, num_sm_parts // num_tokens,
            ptr(attn_sink), impl, ptr(status_buffer(q.device)), stream))
        return output, out_lse
    check(lib.smla_sched_meta(num_tokens, topk, 0, num_sm_parts, fixed_overhead, ptr(topk_length), None,
                              ptr(ws["sched_meta"]), ptr(ws["num_splits"]), stream))
    check(lib.smla_decode_splitkv(
        ptr(q), ptr(kv_cache), ptr(indices), ptr(ws["o_accum"]), ptr(ws["lse_accum"]), ptr(output), ptr(out_lse),
        ptr(ws["sched_meta"]), ptr(ws["num_splits"]), num_tokens, num_heads, topk, float(sm_scale),
        page_block_size, page_stride, num_sm_parts, ptr(attn_sink), ptr(topk_length), impl,
        ptr(status_buffer(q.device)), stream))
    max_nsplits = min(max(-(-topk // BLOCK_N), 1), num_sm_parts)
    check(lib.smla_combine(ptr(ws["o_accum"]), ptr(ws["lse_accum"]), ptr(output), ptr(out_lse),
                           ptr(ws["num_splits"]), num_tokens, num_heads, max_nsplits, ptr(attn_sink), stream))
    return output, out_lse


def sparse_mla_prefill_fwd(
    q: torch.Tensor,
    kv_cache: torch.Tensor,
    indices: torch.Tensor,
    sm_scale: float,
    d_v: int = 512,
    attn_sink: Optional[torch.Tensor] = None,
    topk_length: Optional[torch.Tensor] = None,
    bf16_qk: bool = True,
    out: Optional[torch.Tensor] = None,
    extra_k_cache: Optional[torch.Tensor] = None,
    extra_indices: Optional[torch.Tensor] = None,
    extra_topk: int = 0,
    impl: int = IMPL_AUTO,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Single-pass sparse-MLA attention for many query tokens.

    Returns (out [T, H, 512] bf16, max_logits [T, H] fp32, lse [T, H] fp32), as
    flash_mla_sm120/ops.py:122-165."""
    _check_q(q)
    layout = _layout(q, kv_cache)
    impl = resolve_impl(impl, layout)
    page_block_size, page_stride = kv_geometry(kv_cache)
    require_cuda(q, kv_cache, indices)
    if d_v != 512:
        raise ValueError(f"d_v must be 512, got {d_v}")
    num_tokens, num_heads, _ = q.shape
    topk = indices.shape[-1]
    assert indices.dtype == torch.int32 and indices.is_contiguous()
    if out is not None:
        output = out.view(num_tokens, num_heads, d_v)
    else:
        output = torch.empty((num_tokens, num_heads, d_v), dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((num_tokens, num_heads), dtype=torch.float32, device=q.device)
    max_logits = torch.empty((num_tokens, num_heads), dtype=torch.float32, device=q.device)
    ex = _Extra(layout, num_tokens, extra_k_cache, extra_indices, extra_topk)
    if layout != LAYOUT_V32 or ex.topk:
        check(_lib.load().smla_prefill_ext(
            ptr(q), ptr(kv_cache), ptr(indices), ptr(ex.kv), ptr(ex.indices), ptr(output), ptr(lse), ptr(max_logits),
            num_tokens, num_heads, topk, ex.topk, float(sm_scale), layout, page_block_size, page_stride, ex.block,
            ex.stride, ptr(attn_sink), ptr(topk_length), None, impl, ptr(status_buffer(q.device)), stream_ptr(q.device)))
        return output, max_logits, lse
    check(_lib.load().smla_prefill(
        ptr(q), ptr(kv_cache), ptr(indices), ptr(output), ptr(lse), ptr(max_logits), num_tokens, num_heads,
        topk, float(sm_scale), page_block_size, page_stride, ptr(attn_sink), ptr(topk_length), impl,
        ptr(status_buffer(q.device)), stream_ptr(q.device)))
    return output, max_logits, lse
