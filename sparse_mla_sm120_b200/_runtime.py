"""Host-side glue shared by the op modules: pointers, streams, cached scratch, split policy."""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional, Tuple

import torch

from . import _lib

HEADS_PER_TILE = 128     # one CTA covers every head of a query token
CTAS_PER_PART = 2        # two CTAs (one per half of d_v) share a partition
FIXED_OVERHEAD = 5       # scheduler cost of starting a request, in 64-token blocks
BLOCK_N = 64

_scratch: Dict[Tuple, Dict[str, torch.Tensor]] = {}
_num_sms: Dict[int, int] = {}


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def num_sms(device: torch.device) -> int:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _num_sms:
        _num_sms[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _num_sms[idx]


def require_cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("sparse_mla_sm120_b200 runs on CUDA tensors only (there is no CPU path)")


def kv_layout(kv_cache: torch.Tensor) -> int:
    """LAYOUT_V32 for 656-byte rows, LAYOUT_MODEL1 for 584-byte rows."""
    if kv_cache.dtype not in (torch.uint8, torch.int8, torch.float8_e4m3fn):
        raise ValueError(f"kv_cache must be a byte tensor, got {kv_cache.dtype}")
    row = kv_cache.shape[-1]
    if row == 656:
        return _lib.LAYOUT_V32
    if row == 584:
        return _lib.LAYOUT_MODEL1
    raise ValueError(f"kv_cache rows must be 656 bytes (V32) or 584 bytes (MODEL1), got {row}")


def kv_geometry(kv_cache: torch.Tensor) -> Tuple[int, int]:
    """(page_block_size, bytes between pages) of a packed cache tensor.

    V32 (656-byte rows): accepts [num_blocks, block, 1, 656], the legacy flat [pool, 1, 656] and
    [pool, 656].  MODEL1 (584 bytes per token, scales in a footer of the page): [num_blocks, block, 1, 584]
    only, since the position of the footer depends on the page size.  A page stride larger than
    block * row (a padded allocation) is honoured; flash_mla_sm120/ops.py:23-45 computes the same quantity."""
    layout = kv_layout(kv_cache)
    row = kv_cache.shape[-1]
    if kv_cache.stride(-1) != 1:
        raise ValueError("kv_cache rows must be contiguous")
    if kv_cache.dim() == 4:
        block = kv_cache.shape[1]
        if kv_cache.shape[2] != 1 or kv_cache.stride(1) != row:
            raise ValueError(f"kv_cache must be [num_blocks, block, 1, {row}] with {row}-byte rows")
        return block, kv_cache.stride(0)
    if layout != _lib.LAYOUT_V32:
        raise ValueError("a MODEL1 cache must be [num_blocks, block, 1, 584]")
    if kv_cache.dim() == 3:
        if kv_cache.shape[1] != 1 or kv_cache.stride(0) != 656:
            raise ValueError("kv_cache must be [pool, 1, 656] with 656-byte rows")
        pool = max(kv_cache.shape[0], 1)
        return pool, pool * 656
    if kv_cache.dim() == 2:
        if kv_cache.stride(0) != 656:
            raise ValueError("kv_cache must be [pool, 656] with 656-byte rows")
        pool = max(kv_cache.shape[0], 1)
        return pool, pool * 656
    raise ValueError(f"unsupported kv_cache rank {kv_cache.dim()}")


# What IMPL_AUTO means for a MODEL1 cache.  The tensor-core kernel rounds V's RoPE columns to e4m3 (the reference
# keeps them in bf16), which costs up to about 2e-3 on rows with few entries and fails some of the reference's own
# V4 tests by a small margin; the default is therefore the exact fp32 kernel.  A deployment that accepts FP8-class
# error in those 64 columns sets SMLA_MODEL1_IMPL=tc in the environment (or assigns _lib.IMPL_TC here) and gets the
# tensor-core kernel, about two orders of magnitude faster.
MODEL1_DEFAULT_IMPL = _lib.IMPL_TC if os.environ.get("SMLA_MODEL1_IMPL", "").lower() in ("tc", "2") else _lib.IMPL_SCALAR


def resolve_impl(impl: int, layout: int) -> int:
    """IMPL_AUTO for a MODEL1 cache -> MODEL1_DEFAULT_IMPL; everything else unchanged."""
    if impl == _lib.IMPL_AUTO and layout == _lib.LAYOUT_MODEL1:
        return MODEL1_DEFAULT_IMPL
    return impl


def tc_aligned(kv_cache: torch.Tensor, extra_kv: Optional[torch.Tensor] = None) -> bool:
    """What the tensor-core kernel's bulk copies need of the caches of an `_ext` call: base addresses and page
    strides that are multiples of 16 bytes (the library checks the same and falls back to the fp32 kernel)."""
    for t in (kv_cache, extra_kv):
        if t is not None and (t.data_ptr() % 16 != 0 or kv_geometry(t)[1] % 16 != 0):
            return False
    return True


def pick_num_sm_parts_fp32(num_tokens: int, num_heads: int, sms: int) -> int:
    """Partitions for the fp32 kernel, which runs ceil(heads / 8) CTAs per partition: requests stay
    whole when they already give two CTAs per SM, otherwise the work is cut so that they do."""
    tiles = -(-num_heads // 8)
    if num_tokens * tiles >= 2 * sms:
        return num_tokens
    return max(2 * sms // tiles, 1)


BLOCKS_PER_PARTITION = 4  # a partition should be worth at least two 128-token tiles: below that the partials cost more than the split gains


def pick_num_sm_parts(num_tokens: int, sms: int, blocks_per_token: Optional[int] = None) -> int:
    """Partitions for the split-KV scheduler when nothing is known about the requests' lengths (or they differ).

    A partition is served by two CTAs, so at most sms // 2 partitions run at once.  When whole requests already
    fill half of the machine in full waves they are left unsplit (one partition per token: no partial outputs, no
    combine traffic; 40 requests of top-k 2048: 48 us unsplit, 64 us cut into 74 partitions that mostly straddle two
    requests).  Otherwise the work is cut into up to sms // 2 partitions, but not into partitions of fewer than
    BLOCKS_PER_PARTITION 64-token blocks (every extra partition is a partial output that the combine has to read
    back: one request of top-k 2048 is fastest in 8 partitions, 27 us, against 38 us in 74)."""
    max_parts = max(sms // CTAS_PER_PART, 1)
    ctas = num_tokens * CTAS_PER_PART
    waves = -(-ctas // sms)
    if ctas / (waves * sms) >= 0.5:
        return num_tokens
    if blocks_per_token is None:
        return max_parts
    want = -(-(num_tokens * max(blocks_per_token, 1)) // BLOCKS_PER_PARTITION)
    return max(num_tokens, min(max_parts, want))


# Cost model of a decode step at 128 heads on a B200, microseconds (fitted to measurements of 4 to 48 requests of
# top-k 2048 in 1, 2, 4 and 8 equal partitions each; it reproduces them to about 1 us): a partition pays a fixed part
# (set-up, Q quantisation, epilogue) and its 128-token tiles; a split step pays for every partial record, which is
# written and read back once, and at least the latency of the combine launch.
_US_FIXED, _US_TILE, _US_RECORD, _US_SPLIT_MIN = 11.3, 2.3, 0.15, 8.0


def pick_split(num_tokens: int, sms: int, blocks_per_token: Optional[int] = None, uniform: bool = False) -> Tuple[int, int]:
    """(partitions, fixed overhead) to give the scheduler.

    When every request has the same number of blocks (no ``topk_length``), the requests can be cut into k equal
    partitions each, k a divisor of the block count, by asking the scheduler for k * tokens partitions with a fixed
    overhead of 0: no partition then straddles two requests, i.e. none pays the fixed part of a partition twice.
    k is chosen by the cost model above (k = 1: nothing is split, the attention kernel runs alone).  Otherwise
    (lengths differ or are unknown) the choice is pick_num_sm_parts with the reference's fixed overhead."""
    if not uniform or blocks_per_token is None:
        return pick_num_sm_parts(num_tokens, sms, blocks_per_token), FIXED_OVERHEAD
    max_parts = max(sms // CTAS_PER_PART, 1)
    n = max(blocks_per_token, 1)
    waves = -(-num_tokens // max_parts)
    best = (waves * (_US_FIXED + -(-n // 2) * _US_TILE), num_tokens, FIXED_OVERHEAD)
    cuts = 0
    for k in range(2, n + 1):
        if n % k or k * num_tokens > max_parts or n // k < BLOCKS_PER_PARTITION:
            continue
        cuts += 1
        t = _US_FIXED + -(-(n // k) // 2) * _US_TILE + max(_US_SPLIT_MIN, _US_RECORD * k * num_tokens)
        if t < best[0]:
            best = (t, k * num_tokens, 0)
    if cuts == 0 and n >= 2 * BLOCKS_PER_PARTITION:
        # no equal cut exists although the requests are long enough to be worth cutting (a block count without a
        # suitable divisor, or too many requests for two partitions each): the general rule
        return pick_num_sm_parts(num_tokens, sms, blocks_per_token), FIXED_OVERHEAD
    return best[1], best[2]


_SCRATCH_LIMIT = 64      # cached call shapes per process before the least recently used one is dropped


def scratch(device: torch.device, total_splits: int, num_heads: int, num_tokens: int, num_parts: int):
    """Cached scratch for one decode call shape on the current stream (the reference allocates
    these on every call, flash_mla_sm120/ops.py:78-99).

    The key includes the stream: two calls of the same shape on different streams get different
    buffers, so they cannot race on ``o_accum``.  An entry that is handed out while its stream is
    being captured into a CUDA graph is pinned: the graph keeps raw pointers into it, so it is
    never evicted.  Past _SCRATCH_LIMIT entries the least recently used unpinned one is dropped
    (it was allocated on, and only ever used on, its own stream, so the caching allocator may
    reuse it in stream order)."""
    stream = torch.cuda.current_stream(device)
    key = (device.index, stream.cuda_stream, total_splits, num_heads, num_tokens, num_parts)
    ws = _scratch.pop(key, None)
    if ws is None:
        ws = {
            "o_accum": torch.empty((total_splits, 1, num_heads, 512), dtype=torch.float32, device=device),
            "lse_accum": torch.empty((total_splits, 1, num_heads), dtype=torch.float32, device=device),
            "sched_meta": torch.empty(num_parts * 8, dtype=torch.int32, device=device),
            "num_splits": torch.empty(num_tokens + 1, dtype=torch.int32, device=device),
            "pinned": False,
        }
    if torch.cuda.is_current_stream_capturing():
        ws["pinned"] = True
    _scratch[key] = ws                      # most recently used last
    if len(_scratch) > _SCRATCH_LIMIT:
        for old in list(_scratch):
            if not _scratch[old]["pinned"] and old != key:
                del _scratch[old]
                break
    return ws


_status: Dict[int, torch.Tensor] = {}


def status_buffer(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _status:
        _status[idx] = torch.zeros(4, dtype=torch.int32, device=device)
    return _status[idx]


def check_status(device: Optional[torch.device] = None) -> None:
    """Synchronises and raises if a kernel recorded a bounded wait that gave up.  Not called on
    the hot path (it reads device memory); tests and the benchmark call it."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    st = status_buffer(device)
    host = (ctypes.c_int32 * 4)()
    rc = _lib.load().smla_device_status(ptr(st), ctypes.addressof(host), stream_ptr(device))
    if rc != 0:
        raise _lib.SmlaError(_lib.load().smla_last_error().decode())
