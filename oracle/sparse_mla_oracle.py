"""CPU oracle for the sparse-MLA hot path.  TEST INFRASTRUCTURE ONLY.

This module is a restatement, in plain CPU PyTorch / Python, of the reference's own
PyTorch reference path and of the integer algorithms of its scheduler.  It is the
checker used by the tests, by the smoke check and by the benchmark's CPU-baseline leg;
the library itself never imports it (the product path is CUDA only and fails loudly
when the CUDA library is missing).

Parity pin: every function that has a counterpart in the reference is checked against
the reference's own function on the committed fixtures under ``tests/golden/`` (made by
``tests/golden/make_golden.py``, which imports the reference's test modules).  The two
functions at the end (``mqa_logits_ref``/``topk_ref`` and ``cp_partition_ref``) have no
counterpart in the reference at all: their parity is UNPINNED, they restate the formula
of the benchmark configuration only.

Reference citations are paths inside the reference project.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch

D_NOPE = 512
D_ROPE = 64
D_QK = D_NOPE + D_ROPE
D_V = 512
QUANT_TILE = 128
NUM_TILES = 4
ROW_BYTES = D_NOPE + NUM_TILES * 4 + D_ROPE * 2  # 656
BLOCK_N = 64  # tokens per scheduling block
LOG2E = 1.4426950408889634
LN2 = 0.6931471805599453


# --------------------------------------------------------------------------- KV row format
def pow2_scale(scales_inv: torch.Tensor) -> torch.Tensor:
    """Round a positive scale up to a power of two, floor 1e-4.

    Follows tests/test_decode.py:20-22 (_cast_scale_inv_to_ue8m0)."""
    return torch.pow(2, torch.clamp_min(scales_inv, 1e-4).log2().ceil())


def quantize_kv_v32(kv_bf16: torch.Tensor) -> torch.Tensor:
    """bf16 [num_blocks, block, 1, 576] -> packed uint8 [num_blocks, block, 1, 656].

    Row = 512 e4m3 bytes | 4 fp32 power-of-two scales (one per 128 values) | 64 bf16 RoPE.
    Follows tests/test_decode.py:33-57."""
    nb, bs, hk, d = kv_bf16.shape
    assert d == D_QK and hk == 1
    kv = kv_bf16.squeeze(2)
    out = torch.zeros(nb, bs, ROW_BYTES, dtype=torch.uint8)
    for ti in range(NUM_TILES):
        tile = kv[..., ti * QUANT_TILE:(ti + 1) * QUANT_TILE].float()
        amax = tile.abs().amax(dim=-1).clamp(min=1e-4)
        scale = pow2_scale(amax / 448.0)
        fp8 = (tile / scale.unsqueeze(-1)).clamp(-448, 448).to(torch.float8_e4m3fn)
        out[..., ti * QUANT_TILE:(ti + 1) * QUANT_TILE] = fp8.view(torch.uint8)
        sb = scale.to(torch.float32).contiguous().view(torch.uint8).reshape(nb, bs, 4)
        out[..., D_NOPE + ti * 4:D_NOPE + (ti + 1) * 4] = sb
    rope = kv[..., D_NOPE:].to(torch.bfloat16).contiguous().view(torch.uint8).reshape(nb, bs, D_ROPE * 2)
    out[..., D_NOPE + NUM_TILES * 4:] = rope
    return out.view(nb, bs, 1, ROW_BYTES)


def dequantize_kv_v32(packed: torch.Tensor) -> torch.Tensor:
    """packed uint8 [num_blocks, block, 1, 656] -> bf16 [num_blocks, block, 1, 576].

    The dequantised value fp8*scale is rounded to bf16.  Follows tests/test_decode.py:60-71."""
    nb, bs, hk, bpt = packed.shape
    assert bpt == ROW_BYTES
    p = packed.reshape(nb, bs, bpt)
    out = torch.zeros(nb, bs, D_QK, dtype=torch.bfloat16)
    for ti in range(NUM_TILES):
        fp8 = p[..., ti * QUANT_TILE:(ti + 1) * QUANT_TILE].contiguous().view(torch.float8_e4m3fn).float()
        sc = p[..., D_NOPE + ti * 4:D_NOPE + (ti + 1) * 4].contiguous().view(torch.float32).squeeze(-1)
        out[..., ti * QUANT_TILE:(ti + 1) * QUANT_TILE] = (fp8 * sc.unsqueeze(-1)).to(torch.bfloat16)
    out[..., D_NOPE:] = p[..., D_NOPE + NUM_TILES * 4:].contiguous().view(torch.bfloat16).reshape(nb, bs, D_ROPE)
    return out.view(nb, bs, 1, D_QK)


# --------------------------------------------------------------------------- MODEL1 row format
M1_D_NOPE = 448
M1_D_QK = 512
M1_TILE = 64
M1_NUM_TILES = 7
M1_DATA_BYTES = M1_D_NOPE + D_ROPE * 2     # 576: e4m3 values + bf16 RoPE of one token
M1_SCALE_BYTES = 8                         # 7 UE8M0 scales + 1 pad
M1_ROW_BYTES = M1_DATA_BYTES + M1_SCALE_BYTES  # 584 logical bytes per token


def quantize_kv_model1(kv_bf16: torch.Tensor) -> torch.Tensor:
    """bf16 [num_blocks, block, 1, 512] -> uint8 [num_blocks, block, 1, 584], footer-ordered.

    The bytes of a page are NOT token-major: first block x 576 data bytes (per token 448 e4m3 |
    64 bf16 RoPE), then block x 8 footer bytes (per token 7 UE8M0 exponents, one per 64 values, and a
    pad byte).  Follows tests/test_decode.py:76-116."""
    nb, bs, hk, d = kv_bf16.shape
    assert d == M1_D_QK and hk == 1
    kv = kv_bf16.squeeze(2)
    tiles = kv[..., :M1_D_NOPE].float().reshape(nb, bs, M1_NUM_TILES, M1_TILE)
    scale = pow2_scale(tiles.abs().amax(dim=-1).clamp(min=1e-4) / 448.0)          # [nb, bs, 7]
    fp8 = (tiles / scale.unsqueeze(-1)).clamp(-448, 448).to(torch.float8_e4m3fn)
    data = torch.zeros(nb, bs, M1_DATA_BYTES, dtype=torch.uint8)
    data[..., :M1_D_NOPE] = fp8.view(torch.uint8).reshape(nb, bs, M1_D_NOPE)
    data[..., M1_D_NOPE:] = kv[..., M1_D_NOPE:].to(torch.bfloat16).contiguous().view(torch.uint8).reshape(nb, bs, D_ROPE * 2)
    footer = torch.zeros(nb, bs, M1_SCALE_BYTES, dtype=torch.uint8)
    footer[..., :M1_NUM_TILES] = ((scale.to(torch.float32).contiguous().view(torch.int32) >> 23) & 0xFF).to(torch.uint8)
    page = torch.cat([data.reshape(nb, bs * M1_DATA_BYTES), footer.reshape(nb, bs * M1_SCALE_BYTES)], dim=1)
    return page.contiguous().view(nb, bs, 1, M1_ROW_BYTES)


def dequantize_kv_model1(packed: torch.Tensor) -> torch.Tensor:
    """uint8 [num_blocks, block, 1, 584] (footer-ordered pages) -> bf16 [num_blocks, block, 1, 512].

    value = bf16(e4m3 * 2^(ue8m0 - 127)); RoPE verbatim.  Follows tests/test_decode.py:119-147."""
    nb, bs, hk, bpt = packed.shape
    assert bpt == M1_ROW_BYTES and hk == 1
    page = packed.reshape(nb, bs * bpt)
    data = page[:, :bs * M1_DATA_BYTES].reshape(nb, bs, M1_DATA_BYTES)
    footer = page[:, bs * M1_DATA_BYTES:].reshape(nb, bs, M1_SCALE_BYTES)
    fp8 = data[..., :M1_D_NOPE].contiguous().view(torch.float8_e4m3fn).float().reshape(nb, bs, M1_NUM_TILES, M1_TILE)
    scale = torch.pow(2.0, footer[..., :M1_NUM_TILES].float() - 127.0)
    out = torch.zeros(nb, bs, M1_D_QK, dtype=torch.bfloat16)
    out[..., :M1_D_NOPE] = (fp8 * scale.unsqueeze(-1)).to(torch.bfloat16).reshape(nb, bs, M1_D_NOPE)
    out[..., M1_D_NOPE:] = data[..., M1_D_NOPE:].contiguous().view(torch.bfloat16).reshape(nb, bs, D_ROPE)
    return out.view(nb, bs, 1, M1_D_QK)


# --------------------------------------------------------------------------- attention
def ref_sparse_attn(q: torch.Tensor, kv_dequant: torch.Tensor, indices: torch.Tensor,
                    sm_scale: float, d_v: int = D_V,
                    topk_length: Optional[torch.Tensor] = None
                    ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Sparse attention over gathered rows, fp32.

    q [b, s_q, h, 576] bf16; kv_dequant [..., 576] bf16 (flattened to rows);
    indices [b, s_q, topk] int32 (physical row, -1 = invalid).
    Returns (out bf16 [b, s_q, h, d_v], lse fp32 natural log [b, s_q, h]; -inf for a row
    with no valid index, whose output is 0).
    Follows tests/test_decode.py:151-176 (ref_sparse_attn_decode); ``topk_length`` [b]
    additionally masks positions >= length as the kernels do
    (csrc/kernel/decode/decode_v2_kernel.cuh:346-362)."""
    b, s_q, h_q, d_qk = q.shape
    topk = indices.shape[-1]
    kv_flat = kv_dequant.reshape(-1, d_qk).float()
    q_f = q.float()
    idx_fixed = indices.clamp(min=0)
    invalid = indices < 0
    if topk_length is not None:
        pos = torch.arange(topk).view(1, 1, topk)
        invalid = invalid | (pos >= topk_length.view(b, 1, 1))
    gathered = kv_flat.index_select(0, idx_fixed.reshape(-1).long()).view(b, s_q, topk, d_qk)
    P = torch.einsum("bshd,bstd->bsht", q_f, gathered) * sm_scale
    P[invalid.unsqueeze(2).expand_as(P)] = float("-inf")
    lse = torch.logsumexp(P, dim=-1)
    lse_safe = lse.clone()
    lse_safe[lse_safe == float("-inf")] = float("+inf")
    weights = torch.exp(P - lse_safe.unsqueeze(-1))
    # NaN-safety as in the kernels: an invalid entry contributes an exact zero even when
    # the row it was clamped to holds NaN (decode_v2_kernel.cuh:262-278).
    vals = gathered[..., :d_v].clone()
    vals[invalid.unsqueeze(-1).expand_as(vals)] = 0.0
    out = torch.einsum("bsht,bstd->bshd", weights, vals)
    return out.to(torch.bfloat16), lse


def ref_sparse_attn_dual(q: torch.Tensor, kv_dequant: torch.Tensor, indices: torch.Tensor, sm_scale: float,
                         d_v: int = D_V, topk_length: Optional[torch.Tensor] = None,
                         extra_kv_dequant: Optional[torch.Tensor] = None,
                         extra_indices: Optional[torch.Tensor] = None,
                         extra_topk_length: Optional[torch.Tensor] = None,
                         attn_sink: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Sparse attention over the rows of a main cache and, optionally, of a second cache, fp32.

    q [b, s_q, h, d_qk] bf16; the rows named by ``indices`` [b, s_q, topk] (masked past ``topk_length``
    [b]) and by ``extra_indices`` [b, s_q, extra_topk] (masked past ``extra_topk_length`` [b]) enter ONE
    softmax; V is the first d_v values of a row.  ``attn_sink`` [h] (natural-log logit, +-inf allowed)
    scales the output by 1 / (1 + exp(sink - lse)) BEFORE the rounding to bf16; the returned LSE does not
    include the sink.  A row without any valid entry gives output 0 and LSE -inf.
    Follows tests/test_v4_features.py:50-101 (ref_v4_decode)."""
    b, s_q, h_q, d_qk = q.shape

    def scope(kv, idx, length):
        n = idx.shape[-1]
        bad = idx < 0
        if length is not None:
            bad = bad | (torch.arange(n).view(1, 1, n) >= length.view(b, 1, 1))
        rows = kv.reshape(-1, d_qk).float().index_select(0, idx.clamp(min=0).reshape(-1).long())
        return rows.view(b, s_q, n, d_qk), bad

    gathered, invalid = scope(kv_dequant, indices, topk_length)
    if extra_kv_dequant is not None and extra_indices is not None:
        g2, i2 = scope(extra_kv_dequant, extra_indices, extra_topk_length)
        gathered, invalid = torch.cat([gathered, g2], dim=2), torch.cat([invalid, i2], dim=2)
    gathered = torch.nan_to_num(gathered, nan=0.0, posinf=float("inf"), neginf=float("-inf"))
    P = torch.einsum("bshd,bstd->bsht", q.float(), gathered) * sm_scale
    P[invalid.unsqueeze(2).expand_as(P)] = float("-inf")
    lse = torch.logsumexp(P, dim=-1)
    lse_safe = lse.masked_fill(lse == float("-inf"), float("inf"))
    out = torch.einsum("bsht,bstd->bshd", torch.exp(P - lse_safe.unsqueeze(-1)), gathered[..., :d_v])
    if attn_sink is not None:
        out = out * (1.0 / (1.0 + torch.exp(attn_sink.view(1, 1, h_q).float() - lse))).unsqueeze(-1)
    out[(lse == float("-inf")).unsqueeze(-1).expand_as(out)] = 0.0
    return out.to(torch.bfloat16), lse


def apply_attn_sink(out: torch.Tensor, lse: torch.Tensor, attn_sink: torch.Tensor
                    ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Fold a per-head sink logit (natural-log units) into output and LSE.

    out *= 1/(1+exp(sink-lse)) follows tests/test_decode.py:316-320; the merged LSE
    lse' = lse + log(1+exp(sink-lse)) follows decode_v2_kernel.cuh:582-595 (there in base 2)."""
    sink = attn_sink.view(*([1] * (lse.dim() - 1)), -1).float()
    lse_f = lse.float()
    empty = torch.isinf(lse_f) & (lse_f < 0)          # no valid entry: the output is 0 whatever the sink
    scale = torch.where(empty, torch.zeros_like(lse_f), 1.0 / (1.0 + torch.exp(sink - lse_f.masked_fill(empty, 0.0))))
    out2 = (out.float() * scale.unsqueeze(-1)).to(torch.bfloat16)
    lse2 = torch.where(empty, sink.expand_as(lse_f),
                       lse_f + torch.log1p(torch.exp(sink - lse_f)))
    return out2, lse2


# --------------------------------------------------------------------------- combine
def combine_ref(o_accum: torch.Tensor, lse_accum: torch.Tensor, num_splits: Sequence[int],
                batch: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """LSE-weighted merge of split partials, base-2, float64.

    o_accum [S, 1, H, d_v] fp32 (each partial normalised by its own sum), lse_accum
    [S, 1, H] fp32 base-2, num_splits[b+1] prefix sum.  Requests with <=1 split pass
    through.  Follows tests/test_combine.py:20-50 (combine_v2_ref)."""
    outs, lses = [], []
    for b in range(batch):
        start, end = int(num_splits[b]), int(num_splits[b + 1])
        if end - start <= 1:
            outs.append(o_accum[start, 0].to(torch.bfloat16))
            lses.append(lse_accum[start, 0])
            continue
        po = o_accum[start:end, 0].double()
        pl = lse_accum[start:end, 0].double()
        max_lse = pl.max(dim=0).values
        scales = torch.pow(2.0, pl - max_lse.unsqueeze(0))
        scale_sum = scales.sum(dim=0)
        weighted = (po * scales.unsqueeze(-1)).sum(dim=0)
        inv = torch.where(scale_sum > 0, 1.0 / scale_sum, torch.zeros_like(scale_sum))
        outs.append((weighted * inv.unsqueeze(-1)).float().to(torch.bfloat16))
        lses.append(torch.where(scale_sum > 0, torch.log2(scale_sum) + max_lse,
                                torch.full_like(max_lse, -1e30)).float())
    return torch.stack(outs), torch.stack(lses)


# --------------------------------------------------------------------------- scheduler
def sched_meta_ref(b: int, topk: int, extra_topk: int, num_sm_parts: int, fixed_overhead: int,
                   topk_length: Optional[Sequence[int]] = None,
                   extra_topk_length: Optional[Sequence[int]] = None,
                   block_n: int = BLOCK_N) -> Tuple[List[List[int]], List[int]]:
    """Greedy block partition of split-KV decode work over ``num_sm_parts`` partitions.

    Returns (meta, num_splits): meta[p] = [begin_req, end_req, begin_block, end_block,
    begin_split_idx, first_req_is_split, last_req_is_split, 0]; num_splits[b+1] prefix sum.
    Integer-exact restatement of csrc/kernel/sched/get_sched_meta.cu:25-125 with the record
    layout of csrc/kernel/sched/sched_params.h:8-18."""
    num_blocks, last_block = [], []
    total = 0
    for i in range(b):
        cur = int(topk_length[i]) if topk_length is not None else topk
        if cur == 0:
            cur = 1
        if extra_topk > 0:
            cur = (cur + block_n - 1) // block_n * block_n
            cur += int(extra_topk_length[i]) if extra_topk_length is not None else extra_topk
        lb = (cur - 1) // block_n if cur > 0 else 0
        num_blocks.append(lb + 1)
        last_block.append(lb)
        total += lb + 1 + fixed_overhead
    payload = (total + num_sm_parts - 1) // num_sm_parts + fixed_overhead
    now_req = now_block = now_n_split = cum = 0
    num_splits = [0] * (b + 1)
    meta = []
    for _ in range(num_sm_parts):
        begin_req = now_req
        begin_block = now_block if now_req < b else 0
        begin_split = now_n_split
        first_split = 1 if now_block != 0 else 0
        remain = payload
        while now_req < b:
            rb = num_blocks[now_req] - now_block
            if remain >= rb + fixed_overhead:
                cum += now_n_split + 1
                num_splits[now_req + 1] = cum
                remain -= rb + fixed_overhead
                now_req += 1
                now_block = 0
                now_n_split = 0
            else:
                if remain > fixed_overhead:
                    now_block += remain - fixed_overhead
                    now_n_split += 1
                remain = 0
                break
        end_req = now_req if now_block > 0 else now_req - 1
        if now_block > 0:
            end_block = now_block
        elif now_req > 0:
            end_block = last_block[now_req - 1] + 1
        else:
            end_block = 0
        # end_req == -1 cannot index in the reference either: the comparison is guarded
        # by end_req < b and reads last_block_sh[-1]; only reachable when b == 0.
        last_split = 1 if (0 <= end_req < b and end_block != last_block[end_req] + 1) else 0
        if begin_req == end_req:
            f = first_split | last_split
            first_split = last_split = f
        meta.append([begin_req, end_req, begin_block, end_block, begin_split, first_split, last_split, 0])
    return meta, num_splits


def expected_blocks(b, topk, extra_topk, topk_length, extra_topk_length, block_n=BLOCK_N):
    """Blocks per request as the scheduler counts them (tests/test_scheduler.py:52-64)."""
    blocks = []
    for i in range(b):
        cur = topk_length[i] if topk_length is not None else topk
        if cur == 0:
            cur = 1
        if extra_topk > 0:
            cur = math.ceil(cur / block_n) * block_n
            cur += extra_topk_length[i] if extra_topk_length is not None else extra_topk
        blocks.append(math.ceil(cur / block_n))
    return blocks


def verify_schedule(meta: List[List[int]], num_splits: Sequence[int], blocks: Sequence[int], b: int) -> None:
    """Coverage (each block exactly once), prefix-sum consistency and monotonic order.

    The three invariants of tests/test_scheduler.py:67-129 in one pass."""
    assigned = {i: set() for i in range(b)}
    per_req = [0] * b
    last_req, last_blk = -1, -1
    for pi, m in enumerate(meta):
        br, er, bb, eb = m[0], m[1], m[2], m[3]
        if br >= b:
            continue
        assert br >= last_req, f"partition {pi} goes backwards"
        if br == last_req:
            assert bb >= last_blk, f"partition {pi} overlaps previous"
        for req in range(br, er + 1):
            if req >= b:
                break
            per_req[req] += 1
            s = bb if req == br else 0
            e = eb if req == er else blocks[req]
            for blk in range(s, e):
                assert blk not in assigned[req], f"block {blk} of request {req} assigned twice"
                assigned[req].add(blk)
        last_req, last_blk = er, eb
    for i in range(b):
        assert assigned[i] == set(range(blocks[i])), f"request {i}: got {sorted(assigned[i])}"
    assert num_splits[0] == 0
    cum = 0
    for i in range(b):
        cum += per_req[i]
        assert num_splits[i + 1] == cum, f"num_splits[{i + 1}]={num_splits[i + 1]} expected {cum}"


# --------------------------------------------------------------------------- tolerance form
def allclose_report(actual: torch.Tensor, expected: torch.Tensor, abs_tol: float, rel_tol: float):
    """|a-e| <= abs_tol + rel_tol*max(|a|,|e|) elementwise (tests/test_v4_features.py:34-47)."""
    a, e = actual.float(), expected.float()
    diff = (a - e).abs()
    tol = abs_tol + rel_tol * torch.maximum(a.abs(), e.abs())
    bad = diff > tol
    return (not bool(bad.any())), float(diff.max()), int(bad.sum())


def cos_diff(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.double().flatten(), b.double().flatten()
    denom = (a * a).sum() + (b * b).sum()
    if float(denom) == 0.0:
        return 0.0
    return float(1.0 - 2.0 * (a * b).sum() / denom)


# --------------------------------------------------------------------------- no reference counterpart
def mqa_logits_ref(q_fp8: torch.Tensor, k_fp8: torch.Tensor, k_scale: torch.Tensor,
                   weights: torch.Tensor, ks: torch.Tensor, ke: torch.Tensor) -> torch.Tensor:
    """logits[i,j] = sum_h w[i,h] * relu(q[i,h,:] . k[j,:]) * k_scale[j], -inf outside [ks_i, ke_i).

    q_fp8 [s_q, H, 128] float8_e4m3fn, k_fp8 [s_k, 128] float8_e4m3fn, k_scale [s_k] fp32,
    weights [s_q, H] fp32.  PARITY UNPINNED: the reference has no indexer; this restates the
    formula of the benchmark configuration in fp32."""
    q = q_fp8.float()
    k = k_fp8.float()
    s = torch.einsum("ihd,jd->ihj", q, k).relu_()
    logits = torch.einsum("ihj,ih->ij", s, weights.float()) * k_scale.float().unsqueeze(0)
    j = torch.arange(k.shape[0]).unsqueeze(0)
    mask = (j >= ks.view(-1, 1)) & (j < ke.view(-1, 1))
    return logits.masked_fill(~mask, float("-inf"))


def topk_ref(logits: torch.Tensor, k: int) -> torch.Tensor:
    """Indices of the k largest finite-or-not logits per row, -1 padded where a row has
    fewer than k entries above -inf.  PARITY UNPINNED (no reference counterpart)."""
    kk = min(k, logits.shape[1])
    vals, idx = torch.topk(logits, kk, dim=1)
    idx = idx.to(torch.int32)
    idx[vals == float("-inf")] = -1
    if kk < k:
        idx = torch.cat([idx, torch.full((logits.shape[0], k - kk), -1, dtype=torch.int32)], dim=1)
    return idx


def cp_partition_ref(indices: torch.Tensor, lo: int, hi: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Stable compaction of the indices that fall in [lo, hi), rebased to lo, -1 padded.

    indices [T, topk] int32 -> (local [T, topk] int32, length [T] int32).
    PARITY UNPINNED (the reference has no multi-GPU path)."""
    T, topk = indices.shape
    local = torch.full_like(indices, -1)
    length = torch.zeros(T, dtype=torch.int32)
    for t in range(T):
        row = indices[t]
        keep = row[(row >= lo) & (row < hi)] - lo
        local[t, :keep.numel()] = keep
        length[t] = keep.numel()
    return local, length


# --------------------------------------------------------------------------- FP8-class numerics
def emulate_fp8_attention(q: torch.Tensor, packed: torch.Tensor, indices: torch.Tensor, sm_scale: float,
                          topk_length: Optional[torch.Tensor] = None, p_shift: int = 5
                          ) -> Tuple[torch.Tensor, torch.Tensor]:
    """The attention of ``ref_sparse_attn`` with the roundings a kernel of the FP8 class makes, in
    fp32 on the CPU: used to DERIVE the tolerances of the tensor-core kernels instead of fitting
    them to a kernel's output.  It restates numerics, not an implementation:

      * Q no-PE -> e4m3 with one power-of-two scale per head, amax floor 1e-4 (the reference
        quantises Q the same way, per 128-value tile: csrc/kernel/common/fp8_quant.cuh:44-103);
        Q RoPE and K RoPE stay bf16;
      * K / V are the stored e4m3 bytes times their power-of-two scales, exactly (no bf16
        rounding of the dequantised value, unlike ``dequantize_kv_v32``: the tensor core reads the bytes);
      * logits and softmax statistics in fp32;
      * the softmax weight times the row's V scale is rounded to e4m3 (scaled by 2**p_shift against
        the row maximum) before it multiplies V, as the reference's kernels round P
        (csrc/kernel/decode/decode_v2_kernel.cuh:414-493); the denominator uses the unrounded weights.

    q [T, H, 576] bf16, packed [..., 656] uint8 rows, indices [T, topk] int32.
    Returns (out bf16 [T, H, 512], lse natural log [T, H])."""
    T, H, _ = q.shape
    rows = packed.reshape(-1, ROW_BYTES)
    fp8 = rows[:, :D_NOPE].contiguous().view(torch.float8_e4m3fn).float().view(-1, NUM_TILES, QUANT_TILE)
    sc = rows[:, D_NOPE:D_NOPE + 16].contiguous().view(torch.float32).view(-1, NUM_TILES)
    k_nope = (fp8 * sc.unsqueeze(-1)).view(-1, D_NOPE)                       # exact: scales are powers of two
    k_rope = rows[:, D_NOPE + 16:].contiguous().view(torch.bfloat16).float()
    s_row = sc.amax(dim=1)                                                  # the row's largest scale
    qf = q.float()
    amax = qf[..., :D_NOPE].abs().amax(dim=-1).clamp(min=1e-4)
    sq = pow2_scale(amax / 448.0)
    q8 = (qf[..., :D_NOPE] / sq.unsqueeze(-1)).clamp(-448, 448).to(torch.float8_e4m3fn).float() * sq.unsqueeze(-1)
    topk = indices.shape[-1]
    invalid = indices < 0
    if topk_length is not None:
        invalid = invalid | (torch.arange(topk).view(1, topk) >= topk_length.view(T, 1))
    idx = indices.clamp(min=0).long()
    out = torch.zeros(T, H, D_V)
    lse = torch.full((T, H), float("-inf"))
    for t in range(T):
        kn, kr, st = k_nope[idx[t]], k_rope[idx[t]], s_row[idx[t]]
        x = (q8[t] @ kn.T + qf[t, :, D_NOPE:] @ kr.T) * (sm_scale * LOG2E)        # [H, topk], base-2 logits
        x[:, invalid[t]] = float("-inf")
        z = x + st.clamp(min=1e-38).log2().unsqueeze(0)                           # the row's V scale rides in the exponent
        z[:, invalid[t]] = float("-inf")
        m = z.amax(dim=1, keepdim=True)
        live = torch.isfinite(m.squeeze(1))
        m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
        p = torch.exp2(z - m + p_shift)
        p8 = p.clamp(max=448).to(torch.float8_e4m3fn).float()
        v_raw = kn / st.clamp(min=1e-38).unsqueeze(1)                             # V in units of its row scale
        v_raw[invalid[t]] = 0.0
        l = (p / st.clamp(min=1e-38).unsqueeze(0)).sum(dim=1)
        o = (p8 @ v_raw) / l.clamp(min=1e-38).unsqueeze(1)
        out[t] = torch.where(live.unsqueeze(1), o, torch.zeros_like(o))
        lse[t] = torch.where(live, (l.clamp(min=1e-38).log2() + m.squeeze(1) - p_shift) * LN2, torch.full_like(l, float("-inf")))
    return out.to(torch.bfloat16), lse


def _fp8_class_rows(packed: torch.Tensor):
    """What a kernel of the FP8 class sees of every row of a cache, for either layout (told apart by the row size):
    (k_nope exact fp32 [N, nope], k_rope fp32 [N, 64], s_row [N], v_raw [N, 512] in units of s_row).

    V32: s_row is the row's largest scale and V its no-PE values.  MODEL1: V is the whole row, so its RoPE
    part is rounded to e4m3 as well, against a scale s_row that covers both the row's scales and its RoPE
    (2^ceil(log2(amax / 448)))."""
    if packed.shape[-1] == ROW_BYTES:
        rows = packed.reshape(-1, ROW_BYTES)
        fp8 = rows[:, :D_NOPE].contiguous().view(torch.float8_e4m3fn).float().view(-1, NUM_TILES, QUANT_TILE)
        sc = rows[:, D_NOPE:D_NOPE + 16].contiguous().view(torch.float32).view(-1, NUM_TILES)
        k_nope = (fp8 * sc.unsqueeze(-1)).view(-1, D_NOPE)
        k_rope = rows[:, D_NOPE + 16:].contiguous().view(torch.bfloat16).float()
        s_row = sc.amax(dim=1)
        return k_nope, k_rope, s_row, k_nope / s_row.clamp(min=1e-38).unsqueeze(1)
    nb, bs, hk, bpt = packed.shape
    assert bpt == M1_ROW_BYTES and hk == 1
    page = packed.reshape(nb, bs * bpt)
    data = page[:, :bs * M1_DATA_BYTES].reshape(nb * bs, M1_DATA_BYTES)
    footer = page[:, bs * M1_DATA_BYTES:].reshape(nb * bs, M1_SCALE_BYTES)
    fp8 = data[:, :M1_D_NOPE].contiguous().view(torch.float8_e4m3fn).float().view(-1, M1_NUM_TILES, M1_TILE)
    sc = torch.pow(2.0, footer[:, :M1_NUM_TILES].float() - 127.0)
    k_nope = (fp8 * sc.unsqueeze(-1)).view(-1, M1_D_NOPE)
    k_rope = data[:, M1_D_NOPE:].contiguous().view(torch.bfloat16).float()
    need = k_rope.abs().amax(dim=1) / 448.0
    s_rope = torch.where(need > 0, torch.pow(2.0, need.clamp(min=1e-38).log2().ceil()), torch.zeros_like(need))
    s_row = torch.maximum(sc.amax(dim=1), s_rope)
    inv = 1.0 / s_row.clamp(min=1e-38).unsqueeze(1)
    v_rope = (k_rope * inv).clamp(-448, 448).to(torch.float8_e4m3fn).float()
    return k_nope, k_rope, s_row, torch.cat([k_nope * inv, v_rope], dim=1)


def emulate_fp8_attention_dual(q: torch.Tensor, packed: torch.Tensor, indices: torch.Tensor, sm_scale: float,
                               topk_length: Optional[torch.Tensor] = None,
                               extra_packed: Optional[torch.Tensor] = None,
                               extra_indices: Optional[torch.Tensor] = None,
                               extra_topk_length: Optional[torch.Tensor] = None,
                               attn_sink: Optional[torch.Tensor] = None, p_shift: int = 5
                               ) -> Tuple[torch.Tensor, torch.Tensor]:
    """``emulate_fp8_attention`` for everything ``ref_sparse_attn_dual`` takes: either cache layout, a
    second cache whose rows join the same softmax, and a sink (applied as there: the output is scaled, the
    LSE is not).  Same roundings, same purpose: the distance of this function to the fp32 oracle is what a
    tensor-core kernel is allowed, it restates no kernel.

    q [T, H, 576 | 512] bf16, indices [T, topk], extra_indices [T, extra_topk].
    Returns (out bf16 [T, H, 512], lse natural log [T, H])."""
    T, H, d_qk = q.shape
    nope = D_NOPE if packed.shape[-1] == ROW_BYTES else M1_D_NOPE
    assert d_qk == nope + D_ROPE
    caches = [(_fp8_class_rows(packed), indices, topk_length)]
    if extra_packed is not None and extra_indices is not None:
        caches.append((_fp8_class_rows(extra_packed), extra_indices, extra_topk_length))
    qf = q.float()
    amax = qf[..., :nope].abs().amax(dim=-1).clamp(min=1e-4)
    sq = pow2_scale(amax / 448.0)
    q8 = (qf[..., :nope] / sq.unsqueeze(-1)).clamp(-448, 448).to(torch.float8_e4m3fn).float() * sq.unsqueeze(-1)
    out = torch.zeros(T, H, D_V)
    lse = torch.full((T, H), float("-inf"))
    for t in range(T):
        kn, kr, st, vr, bad = [], [], [], [], []
        for (c_nope, c_rope, c_s, c_v), idx, length in caches:
            n = idx.shape[-1]
            b = idx[t] < 0
            if length is not None:
                b = b | (torch.arange(n) >= int(length[t]))
            i = idx[t].clamp(min=0).long()
            kn.append(c_nope[i]); kr.append(c_rope[i]); st.append(c_s[i]); vr.append(c_v[i]); bad.append(b)
        kn, kr, st, vr, bad = torch.cat(kn), torch.cat(kr), torch.cat(st), torch.cat(vr), torch.cat(bad)
        x = (q8[t] @ kn.T + qf[t, :, nope:] @ kr.T) * (sm_scale * LOG2E)
        z = x + st.clamp(min=1e-38).log2().unsqueeze(0)
        z[:, bad] = float("-inf")
        m = z.amax(dim=1, keepdim=True)
        live = torch.isfinite(m.squeeze(1))
        m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
        p = torch.exp2(z - m + p_shift)
        p8 = p.clamp(max=448).to(torch.float8_e4m3fn).float()
        vr = vr.clone()
        vr[bad] = 0.0
        l = (p / st.clamp(min=1e-38).unsqueeze(0)).sum(dim=1)
        o = (p8 @ vr) / l.clamp(min=1e-38).unsqueeze(1)
        row_lse = torch.where(live, (l.clamp(min=1e-38).log2() + m.squeeze(1) - p_shift) * LN2, torch.full_like(l, float("-inf")))
        if attn_sink is not None:
            o = o * (1.0 / (1.0 + torch.exp(attn_sink.float() - row_lse))).unsqueeze(1)
        out[t] = torch.where(live.unsqueeze(1), o, torch.zeros_like(o))
        lse[t] = row_lse
    return out.to(torch.bfloat16), lse

