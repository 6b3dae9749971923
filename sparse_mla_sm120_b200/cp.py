"""Multi-GPU paths: one process per GPU, torch.distributed (NCCL over NVLink) for the exchange.

The reference has no multi-GPU code.  Two shardings are offered:

* decode batches shard by sequence: every rank calls ``flash_ops.sparse_mla_decode_fwd`` on its
  own requests, nothing is exchanged (``shard_requests`` gives the slice of a rank);
* long-context decode shards the KV context: rank g holds rows [g*L/G, (g+1)*L/G) of every
  sequence.  Each rank keeps the entries of the global index list that fall into its shard
  (``partition_indices``), runs split-KV decode over them to one fp32 partial + base-2 LSE per
  token, and the partials are merged with the same LSE-weighted combine that merges split-KV
  partials (``sparse_mla_decode_cp_fwd``).  The exchange costs every rank the same whatever the
  number of ranks G: an all-to-all by head slice (rank d receives, from everybody, the partials of
  heads [d*H/G, (d+1)*H/G)), a merge of those H/G heads, and an all-gather of the bf16 result
  (about 4 MB in and 2 MB out per rank at 16 tokens x 128 heads).  When the heads do not divide by
  G the partials are all-gathered whole instead.  A token with no entry on a rank contributes
  LSE = -1e30 and drops out of the merge exactly.  ``sparse_mla_prefill_cp_fwd`` runs the same
  step over chunks of query tokens; ``GraphedCpDecode`` replays it as one CUDA graph.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from . import _lib
from ._lib import IMPL_AUTO, check
from ._runtime import (FIXED_OVERHEAD, kv_geometry, num_sms, pick_num_sm_parts, ptr, require_cuda, scratch,
                       status_buffer, stream_ptr)


# Below this many bytes received per rank the partials of all ranks are simply all-gathered and merged (one
# collective, (G-1) x T x H x 2052 bytes in); above it the exchange is all-to-all by head slice + all-gather of
# the bf16 result (two collectives, traffic independent of G).  Both collectives cost 10-20 us of latency at
# these sizes, which is what the limit weighs against the bytes.
ALL_GATHER_LIMIT_BYTES = 8 << 20


def shard_requests(num_requests: int, rank: int, world: int) -> Tuple[int, int]:
    """[begin, end) of the requests rank serves when a decode batch is sharded by sequence."""
    per, rem = divmod(num_requests, world)
    begin = rank * per + min(rank, rem)
    return begin, begin + per + (1 if rank < rem else 0)


def shard_context(context_len: int, rank: int, world: int, align: int = 64) -> Tuple[int, int]:
    """[lo, hi) of the token positions rank holds; shards are contiguous and page aligned."""
    per = -(-context_len // world)
    per = -(-per // align) * align
    lo = min(rank * per, context_len)
    return lo, min(lo + per, context_len)


def partition_indices(indices: torch.Tensor, lo: int, hi: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Stable compaction of the entries of each row inside [lo, hi), rebased to lo, -1 padded.
    Returns (local_indices [T, topk] int32, local_length [T] int32)."""
    require_cuda(indices)
    assert indices.dim() == 2 and indices.dtype == torch.int32 and indices.is_contiguous()
    T, topk = indices.shape
    local = torch.empty_like(indices)
    length = torch.empty(T, dtype=torch.int32, device=indices.device)
    check(_lib.load().smla_cp_partition_indices(ptr(indices), ptr(local), ptr(length), T, topk, lo, hi,
                                                stream_ptr(indices.device)))
    return local, length


_gather_bufs: Dict[Tuple, Tuple[torch.Tensor, torch.Tensor]] = {}


def _gather_buffers(device, world, T, H):
    """(packed, o_all, lse_all): one fp32 buffer [world, T*H*513 rounded up to 4] and its views o_all [world, T, H, 512],
    lse_all [world, T, H].  A rank's partials and LSEs are adjacent, so ONE all-gather of ``packed``
    exchanges both."""
    key = (device.index, world, T, H)
    if key not in _gather_bufs:
        per = (T * H * 513 + 3) & ~3                      # a rank's share, kept 16-byte aligned
        packed = torch.empty((world, per), dtype=torch.float32, device=device)
        if len(_gather_bufs) >= 16:
            _gather_bufs.pop(next(iter(_gather_bufs)))
        _gather_bufs[key] = (packed, packed[:, :T * H * 512].view(world, T, H, 512),
                             packed[:, T * H * 512:T * H * 513].view(world, T, H))
    return _gather_bufs[key]


def decode_partial(q, kv_local, local_indices, local_length, sm_scale, o_part=None, lse_part=None,
                   impl: int = IMPL_AUTO, num_sm_parts: Optional[int] = None):
    """Local step: fp32 partial [T, H, 512] and base-2 LSE [T, H] over this rank's entries."""
    require_cuda(q, kv_local, local_indices, local_length)
    T, H, _ = q.shape
    topk = local_indices.shape[-1]
    pbs, stride = kv_geometry(kv_local)
    if num_sm_parts is None:
        num_sm_parts = pick_num_sm_parts(T, num_sms(q.device))
    ws = scratch(q.device, T + num_sm_parts, H, T, num_sm_parts)
    if o_part is None:
        o_part = torch.empty((T, H, 512), dtype=torch.float32, device=q.device)
        lse_part = torch.empty((T, H), dtype=torch.float32, device=q.device)
    lib, stream = _lib.load(), stream_ptr(q.device)
    check(lib.smla_sched_meta(T, topk, 0, num_sm_parts, FIXED_OVERHEAD, ptr(local_length), None,
                              ptr(ws["sched_meta"]), ptr(ws["num_splits"]), stream))
    check(lib.smla_decode_partial(ptr(q), ptr(kv_local), ptr(local_indices), ptr(ws["o_accum"]),
                                  ptr(ws["lse_accum"]), ptr(o_part), ptr(lse_part), ptr(ws["sched_meta"]),
                                  ptr(ws["num_splits"]), T, H, topk, float(sm_scale), pbs, stride, num_sm_parts,
                                  ptr(local_length), impl, ptr(status_buffer(q.device)), stream))
    return o_part, lse_part


def combine_parts(o_parts, lse_parts, attn_sink=None, out=None):
    """Merge [G, T, H, 512] fp32 partials and [G, T, H] base-2 LSEs -> (out bf16, lse).  The parts
    of a rank must be contiguous; the ranks may lie any (4-float aligned) distance apart."""
    require_cuda(o_parts, lse_parts)
    G, T, H, _ = o_parts.shape
    assert o_parts[0].is_contiguous() and lse_parts[0].is_contiguous()
    if out is None:
        out = torch.empty((T, H, 512), dtype=torch.bfloat16, device=o_parts.device)
    lse = torch.empty((T, H), dtype=torch.float32, device=o_parts.device)
    o_stride = o_parts.stride(0) if G > 1 else T * H * 512
    l_stride = lse_parts.stride(0) if G > 1 else T * H
    check(_lib.load().smla_combine_parts_strided(ptr(o_parts), ptr(lse_parts), ptr(out), ptr(lse), G, T, H, o_stride,
                                                 l_stride, ptr(attn_sink), stream_ptr(o_parts.device)))
    return out, lse


_a2a_bufs: Dict[Tuple, Dict[str, torch.Tensor]] = {}


def _a2a_buffers(device, world, T, H):
    """Exchange buffers of the head-sliced path, cached per (device, stream, shape): ``send`` / ``recv``
    [world, c] fp32 with c = T*(H/world)*513 rounded up to a multiple of 512 floats (a slice's partials, then its
    LSEs), ``mine`` the merged bf16 slice followed by its fp32 LSEs as bytes, ``gathered`` [world, bytes]."""
    stream = torch.cuda.current_stream(device).cuda_stream
    key = (device.index, stream, world, T, H)
    b = _a2a_bufs.get(key)
    if b is None:
        hs = H // world
        c = -(-(T * hs * 513) // 512) * 512
        chunk_bytes = -(-(T * hs * (1024 + 4)) // 16) * 16
        b = {"send": torch.empty((world, c), dtype=torch.float32, device=device),
             "recv": torch.empty((world, c), dtype=torch.float32, device=device),
             "mine": torch.empty(chunk_bytes, dtype=torch.uint8, device=device),
             "gathered": torch.empty((world, chunk_bytes), dtype=torch.uint8, device=device),
             "c": c, "chunk_bytes": chunk_bytes}
        if len(_a2a_bufs) >= 16:                 # a serving process uses a handful of shapes: drop the oldest
            _a2a_bufs.pop(next(iter(_a2a_bufs)))
        _a2a_bufs[key] = b
    return b


def decode_partial_sliced(q, kv_local, local_indices, local_length, sm_scale, send, slices: int, slice_stride: int,
                          impl: int = IMPL_AUTO, num_sm_parts: Optional[int] = None):
    """Local step of the head-sliced exchange: like ``decode_partial``, the result written as
    ``slices`` head slices into ``send`` (see smla_decode_partial_sliced)."""
    require_cuda(q, kv_local, local_indices, local_length, send)
    T, H, _ = q.shape
    topk = local_indices.shape[-1]
    pbs, stride = kv_geometry(kv_local)
    if num_sm_parts is None:
        num_sm_parts = pick_num_sm_parts(T, num_sms(q.device))
    ws = scratch(q.device, T + num_sm_parts, H, T, num_sm_parts)
    lib, stream = _lib.load(), stream_ptr(q.device)
    check(lib.smla_sched_meta(T, topk, 0, num_sm_parts, FIXED_OVERHEAD, ptr(local_length), None,
                              ptr(ws["sched_meta"]), ptr(ws["num_splits"]), stream))
    check(lib.smla_decode_partial_sliced(ptr(q), ptr(kv_local), ptr(local_indices), ptr(ws["o_accum"]),
                                         ptr(ws["lse_accum"]), ptr(send), slices, slice_stride, ptr(ws["sched_meta"]),
                                         ptr(ws["num_splits"]), T, H, topk, float(sm_scale), pbs, stride, num_sm_parts,
                                         ptr(local_length), impl, ptr(status_buffer(q.device)), stream))


def merge_head_slice(recv: torch.Tensor, mine: torch.Tensor, world: int, T: int, hs: int, c: int, attn_sink_slice=None):
    """Merge the ``world`` partials of this rank's head slice (``recv`` [world, c] fp32 as received) into
    ``mine``: [T, hs, 512] bf16 followed by [T, hs] fp32 base-2 LSEs."""
    out_b = mine[:T * hs * 1024].view(torch.bfloat16)
    lse_b = mine[T * hs * 1024:T * hs * 1028].view(torch.float32)
    check(_lib.load().smla_combine_parts_strided(ptr(recv), recv.data_ptr() + T * hs * 512 * 4, ptr(out_b), ptr(lse_b), world,
                                                 T, hs, c, c, ptr(attn_sink_slice), stream_ptr(recv.device)))


def unslice(gathered: torch.Tensor, world: int, T: int, hs: int, chunk_bytes: int, out=None):
    """[world] chunks of (bf16 [T, hs, 512], fp32 [T, hs]) -> (out [T, world*hs, 512] bf16, lse [T, world*hs])."""
    dev = gathered.device
    if out is None:
        out = torch.empty((T, world * hs, 512), dtype=torch.bfloat16, device=dev)
    lse = torch.empty((T, world * hs), dtype=torch.float32, device=dev)
    check(_lib.load().smla_cp_unslice(ptr(gathered), ptr(out), ptr(lse), world, T, hs, chunk_bytes, stream_ptr(dev)))
    return out, lse


def sparse_mla_decode_cp_fwd(q, kv_local, indices, sm_scale, shard_lo: int, shard_hi: int, group=None,
                             attn_sink=None, impl: int = IMPL_AUTO, out=None):
    """Context-parallel decode.  ``indices`` [T, topk] are global row numbers of the full context
    (identical on every rank), ``kv_local`` holds rows [shard_lo, shard_hi) of it.
    Returns (out [T, H, 512] bf16, lse [T, H] fp32 base-2), identical on every rank."""
    import torch.distributed as dist
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    T, H, _ = q.shape
    local_idx, local_len = partition_indices(indices, shard_lo, shard_hi)
    if world > 1 and H % world == 0 and (world - 1) * T * H * 2052 > ALL_GATHER_LIMIT_BYTES:
        # head-sliced exchange: per-rank traffic does not grow with the number of ranks
        b = _a2a_buffers(q.device, world, T, H)
        hs = H // world
        decode_partial_sliced(q, kv_local, local_idx, local_len, sm_scale, b["send"], world, b["c"], impl=impl)
        dist.all_to_all_single(b["recv"], b["send"], group=group)
        sink = attn_sink[rank * hs:(rank + 1) * hs] if attn_sink is not None else None
        merge_head_slice(b["recv"], b["mine"], world, T, hs, b["c"], sink)
        dist.all_gather_into_tensor(b["gathered"], b["mine"], group=group)
        return unslice(b["gathered"], world, T, hs, b["chunk_bytes"], out)
    packed, o_all, lse_all = _gather_buffers(q.device, world, T, H)
    decode_partial(q, kv_local, local_idx, local_len, sm_scale, o_all[rank], lse_all[rank], impl=impl)
    if world > 1:
        dist.all_gather_into_tensor(packed, packed[rank], group=group)       # partials and LSEs in one exchange
    return combine_parts(o_all, lse_all, attn_sink, out)


def sparse_mla_prefill_cp_fwd(q, kv_local, indices, sm_scale, shard_lo: int, shard_hi: int, group=None,
                              attn_sink=None, impl: int = IMPL_AUTO, chunk_tokens: int = 256):
    """Context-parallel prefill: the KV context is sharded as for decode, every rank holds all the
    query tokens.  The tokens are processed in chunks (the fp32 partials of a chunk are what is
    exchanged: chunk_tokens x H x 2 KB per rank) through the same partition -> partial -> exchange ->
    merge step.  Returns (out [T, H, 512] bf16, lse [T, H] fp32 base-2), identical on every rank."""
    T, H, _ = q.shape
    out = torch.empty((T, H, 512), dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((T, H), dtype=torch.float32, device=q.device)
    for t0 in range(0, T, chunk_tokens):
        t1 = min(t0 + chunk_tokens, T)
        o, l = sparse_mla_decode_cp_fwd(q[t0:t1], kv_local, indices[t0:t1], sm_scale, shard_lo, shard_hi, group,
                                        attn_sink, impl, out=out[t0:t1])
        lse[t0:t1] = l
    return out, lse


class GraphedCpDecode:
    """One context-parallel decode step (index partition, local decode, exchange, merge) captured
    into a CUDA graph, collectives included: one graph launch per step instead of about ten
    launches and two collectives issued from the host.  Shapes are fixed at construction, the cache
    shard is bound by reference, q and the indices are copied into static buffers before a replay.
    If the capture fails (a process-group backend that cannot be captured) the object runs the
    step eagerly and ``self.graph`` is None."""

    def __init__(self, kv_local, num_tokens: int, num_heads: int, topk: int, sm_scale: float, shard_lo: int,
                 shard_hi: int, group=None, attn_sink=None, impl: int = IMPL_AUTO):
        dev = kv_local.device
        self.kv_local, self.attn_sink = kv_local, attn_sink
        self.q = torch.zeros((num_tokens, num_heads, 576), dtype=torch.bfloat16, device=dev)
        self.indices = torch.full((num_tokens, topk), -1, dtype=torch.int32, device=dev)
        self.out = torch.empty((num_tokens, num_heads, 512), dtype=torch.bfloat16, device=dev)

        def step():
            return sparse_mla_decode_cp_fwd(self.q, kv_local, self.indices, sm_scale, shard_lo, shard_hi, group, attn_sink,
                                            impl, out=self.out)

        self._step = step
        self.graph = None
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):
                step()                               # warm-up: library load, buffers, communicator set-up
            side.synchronize()
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    _, self.lse = step()
                self.graph = graph
            except Exception:                        # noqa: BLE001 - any capture failure means: run eagerly
                self.graph = None
        torch.cuda.current_stream(dev).wait_stream(side)

    def __call__(self, q, indices):
        self.q.copy_(q)
        self.indices.copy_(indices)
        return self.replay()

    def close(self):
        """Drops the captured graph.  Call it before the process group is destroyed: a communicator whose
        collectives are still referenced by a live CUDA graph may not shut down."""
        torch.cuda.synchronize(self.q.device)
        self.graph = None
        self._step = None

    def replay(self):
        if self.graph is None:
            _, self.lse = self._step()
        else:
            self.graph.replay()
        return self.out, self.lse


# ----------------------------------------------------------------------------------------------
# Indexer under context parallelism: every rank scores its own shard of the context, keeps its k
# best candidates per query, and the ranks merge the G*k candidates to the global k best.  The
# global k best of a row are a subset of the union of the per-shard k best, so the merge is exact
# (up to the choice among equal logits at the k-th value).
# ----------------------------------------------------------------------------------------------

def local_window(ks: torch.Tensor, ke: torch.Tensor, shard_lo: int, shard_hi: int):
    """The part of each query's window [ks, ke) (global positions) that falls into the shard, in
    shard-local positions; empty windows come out as ks == ke.  On CUDA tensors one kernel; on CPU
    tensors (the host-side tests) plain torch."""
    if not ks.is_cuda:
        n_local = shard_hi - shard_lo
        return ((ks - shard_lo).clamp(0, n_local).to(torch.int32), (ke - shard_lo).clamp(0, n_local).to(torch.int32))
    assert ks.dtype == torch.int32 and ke.dtype == torch.int32 and ks.is_contiguous() and ke.is_contiguous()
    ks_l, ke_l = torch.empty_like(ks), torch.empty_like(ke)
    check(_lib.load().smla_cp_local_window(ptr(ks), ptr(ke), ptr(ks_l), ptr(ke_l), ks.numel(), shard_lo, shard_hi,
                                           stream_ptr(ks.device)))
    return ks_l, ke_l


def local_candidates(qi, ki_local, k_scale_local, weights, ks, ke, shard_lo: int, shard_hi: int, k: int,
                     out: Optional[torch.Tensor] = None):
    """Score the shard's keys and keep the k best per query.

    ``qi`` [T, H_i, 128] e4m3 and ``weights`` [T, H_i] are the indexer queries (identical on every
    rank), ``ki_local`` [shard_hi - shard_lo, 128] e4m3 with ``k_scale_local`` the shard's keys,
    ``ks`` / ``ke`` [T] int32 the visible window of each query in GLOBAL positions.
    Returns (values [T, k] fp32 with -inf padding, positions [T, k] int32 global with -1 padding);
    ``out`` [2, T, k] int32, when given, receives both (values as their bit patterns)."""
    from . import indexer
    T = qi.shape[0]
    ks_l, ke_l = local_window(ks, ke, shard_lo, shard_hi)
    logits = indexer.fp8_mqa_logits(qi, ki_local, k_scale_local, weights, ks_l, ke_l)
    picked = indexer.topk_indices(logits, ks_l, ke_l, k)
    if out is None:
        out = torch.empty((2, T, k), dtype=torch.int32, device=qi.device)
    vals, pos = out[0].view(torch.float32), out[1]
    check(_lib.load().smla_cp_candidates(ptr(logits), logits.stride(0), ptr(picked), ptr(vals), ptr(pos), T, k, shard_lo,
                                         stream_ptr(qi.device)))
    return vals, pos


def merge_candidates(vals: torch.Tensor, pos: torch.Tensor, k: int) -> torch.Tensor:
    """``vals`` / ``pos`` [T, G*k]: the candidates of all shards side by side.  Returns the global
    positions of the k best per row as int32 [T, k], -1 padded."""
    from . import indexer
    vals, pos = vals.contiguous(), pos.contiguous()
    pick = indexer.topk_indices(vals, None, None, k)                     # columns of the candidate list
    out = torch.empty_like(pick)
    check(_lib.load().smla_cp_pick_positions(ptr(pos), ptr(pick), ptr(out), vals.shape[0], k, vals.shape[1],
                                             stream_ptr(vals.device)))
    return out


def interleave_candidates(gathered: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``gathered`` [G, 2, T, k] int32 (every rank's values and positions as all-gathered) ->
    (values [T, G*k] fp32, positions [T, G*k] int32): the candidates of a token side by side."""
    world, _, T, k = gathered.shape
    vals_all = torch.empty((T, world * k), dtype=torch.float32, device=gathered.device)
    pos_all = torch.empty((T, world * k), dtype=torch.int32, device=gathered.device)
    check(_lib.load().smla_cp_interleave_candidates(ptr(gathered), ptr(vals_all), ptr(pos_all), world, T, k,
                                                    stream_ptr(gathered.device)))
    return vals_all, pos_all


def select_indices_cp(qi, ki_local, k_scale_local, weights, ks, ke, shard_lo: int, shard_hi: int, k: int = 2048,
                      group=None) -> torch.Tensor:
    """Distributed top-k of the indexer logits over a context sharded across the ranks of
    ``group``.  Returns the same [T, k] int32 global positions on every rank.  Exchanged per
    query token: G * k * 8 bytes, in one all-gather."""
    import torch.distributed as dist
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    T = qi.shape[0]
    gathered = torch.empty((world, 2, T, k), dtype=torch.int32, device=qi.device)
    _, pos = local_candidates(qi, ki_local, k_scale_local, weights, ks, ke, shard_lo, shard_hi, k, out=gathered[rank])
    if world == 1:
        return pos
    dist.all_gather_into_tensor(gathered, gathered[rank], group=group)
    return merge_candidates(*interleave_candidates(gathered), k)


def sparse_mla_indexed_decode_cp_fwd(q, kv_local, qi, ki_local, k_scale_local, weights, ks, ke, sm_scale,
                                     shard_lo: int, shard_hi: int, topk: int = 2048, group=None, attn_sink=None,
                                     impl: int = IMPL_AUTO):
    """One decode step of a long sequence whose context (attention cache and indexer keys alike)
    is sharded across the ranks: indexer logits -> distributed top-k -> context-parallel sparse
    attention.  Positions are rows of the flat cache.  Returns (out, lse, indices)."""
    indices = select_indices_cp(qi, ki_local, k_scale_local, weights, ks, ke, shard_lo, shard_hi, topk, group)
    out, lse = sparse_mla_decode_cp_fwd(q, kv_local, indices, sm_scale, shard_lo, shard_hi, group, attn_sink, impl)
    return out, lse, indices


class GraphedIndexedCpDecode:
    """``sparse_mla_indexed_decode_cp_fwd`` (indexer logits over the shard, local top-k, candidate all-gather,
    global top-k, index partition, local decode, exchange, merge) captured into one CUDA graph, its three
    collectives included: one graph launch per step instead of about twenty launches issued from the host.
    Shapes are fixed at construction; the cache shard and the shard's indexer keys are bound by reference; the
    step's inputs are copied into static buffers before a replay.  ``close()`` before the process group goes, as
    for GraphedCpDecode.  If the capture fails the object runs the step eagerly and ``self.graph`` is None."""

    def __init__(self, kv_local, ki_local, k_scale_local, num_tokens: int, num_heads: int, indexer_heads: int,
                 sm_scale: float, shard_lo: int, shard_hi: int, topk: int = 2048, group=None, attn_sink=None,
                 impl: int = IMPL_AUTO):
        dev = kv_local.device
        self.kv_local, self.ki_local, self.k_scale_local, self.attn_sink = kv_local, ki_local, k_scale_local, attn_sink
        self.q = torch.zeros((num_tokens, num_heads, 576), dtype=torch.bfloat16, device=dev)
        self.qi = torch.zeros((num_tokens, indexer_heads, 128), dtype=torch.float8_e4m3fn, device=dev)
        self.weights = torch.zeros((num_tokens, indexer_heads), dtype=torch.float32, device=dev)
        self.ks = torch.zeros(num_tokens, dtype=torch.int32, device=dev)
        self.ke = torch.zeros(num_tokens, dtype=torch.int32, device=dev)

        def step():
            return sparse_mla_indexed_decode_cp_fwd(self.q, kv_local, self.qi, ki_local, k_scale_local, self.weights,
                                                    self.ks, self.ke, sm_scale, shard_lo, shard_hi, topk, group,
                                                    attn_sink, impl)

        self._step = step
        self.graph = None
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):
                self.out, self.lse, self.indices = step()   # warm-up: library load, buffers, communicator set-up
            side.synchronize()
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    self.out, self.lse, self.indices = step()
                self.graph = graph
            except Exception:                        # noqa: BLE001 - any capture failure means: run eagerly
                self.graph = None
        torch.cuda.current_stream(dev).wait_stream(side)

    def __call__(self, q, qi, weights, ks, ke):
        self.q.copy_(q)
        self.qi.copy_(qi)
        self.weights.copy_(weights)
        self.ks.copy_(ks)
        self.ke.copy_(ke)
        return self.replay()

    def close(self):
        torch.cuda.synchronize(self.q.device)
        self.graph = None
        self._step = None

    def replay(self):
        """(out, lse, indices): static tensors, overwritten by the next replay."""
        if self.graph is None:
            self.out, self.lse, self.indices = self._step()
        else:
            self.graph.replay()
        return self.out, self.lse, self.indices

