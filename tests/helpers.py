"""Seeded input builders and comparison helpers shared by the tests.

Inputs are generated on the CPU from torch.manual_seed so that the oracle and the GPU kernels
see the same bytes; the GPU side receives copies.
"""
from __future__ import annotations

import math
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from oracle import sparse_mla_oracle as orc  # noqa: E402

LN2 = math.log(2.0)

# Tolerances.  The exact fp32 kernel must agree with the fp32 oracle to bf16 rounding of the
# output.  The tensor-core kernel quantises Q and the softmax weights to e4m3 (3 mantissa bits),
# as the reference's V32 kernels do; its bounds are the FlashMLA-style form the reference uses
# for its own FP8 paths (tests/test_v4_features.py:28-31) plus a cosine bound.
# e4m3 rounding is up to 2^-4 relative (3.6 % rms) per softmax weight; over the top-k sum the
# errors are independent, so the output error is noise of about 3 % of the output's own rms
# magnitude (measured: mean |d| 2.7 % of rms, 1 - cos 4e-4).  The elementwise bound therefore
# carries a term proportional to rms(reference) (6 sigma of that noise) besides the FlashMLA form.
SCALAR_ABS, SCALAR_REL, SCALAR_LSE = 2e-5, 2.0 ** -7, 2e-4
TC_ABS, TC_REL, TC_COS, TC_LSE = 1e-3, 2.01 / 128, 1e-3, 1e-2
TC_PREFILL_ABS, TC_PREFILL_REL = 8e-4, 3.01 / 128
TC_NOISE = 0.2       # x rms(reference output)


def bf16_from_bits(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.astype(np.uint16)).view(torch.bfloat16)


def make_case(seed, num_tokens, num_heads, topk, num_blocks, kv_std=1.0, q_std=0.5, invalid_tail=0.1,
              block=64, clamp=None, unique=True):
    """Random packed cache + queries + indices.  Returns a dict of CPU tensors."""
    g = torch.Generator().manual_seed(seed)
    kv = torch.randn(num_blocks, block, 1, 576, generator=g).mul_(kv_std)
    if clamp is not None:
        kv.clamp_(-clamp, clamp)
    kv = kv.to(torch.bfloat16)
    packed = orc.quantize_kv_v32(kv)
    q = torch.randn(num_tokens, num_heads, 576, generator=g).mul_(q_std)
    if clamp is not None:
        q.clamp_(-clamp, clamp)
    q = q.to(torch.bfloat16)
    pool = num_blocks * block
    if unique and topk <= pool:
        idx = torch.stack([torch.randperm(pool, generator=g)[:topk] for _ in range(num_tokens)]).to(torch.int32)
    else:
        idx = torch.randint(0, pool, (num_tokens, topk), generator=g, dtype=torch.int32)
    n_inv = int(topk * invalid_tail)
    if n_inv:
        idx[:, -n_inv:] = -1
    return {"kv_bf16": kv, "packed": packed, "q": q, "indices": idx, "sm_scale": 576 ** -0.5}


def oracle_attn(case, topk_length=None):
    """(out bf16 [T,H,512], lse natural-log [T,H]) from the CPU oracle."""
    deq = orc.dequantize_kv_v32(case["packed"])
    q4 = case["q"].unsqueeze(1)
    idx3 = case["indices"].unsqueeze(1)
    out, lse = orc.ref_sparse_attn(q4, deq, idx3, case["sm_scale"], 512, topk_length=topk_length)
    return out.squeeze(1), lse.squeeze(1)


def lse2_to_nat(lse2: torch.Tensor) -> torch.Tensor:
    """Kernel LSE (base 2, -1e30 for an empty row) -> natural log with -inf for empty rows."""
    out = lse2.double() * LN2
    out[lse2 < -1e20] = float("-inf")
    return out


def compare_lse(lse2_kernel: torch.Tensor, lse_ref: torch.Tensor, tol: float):
    k = lse2_to_nat(lse2_kernel.cpu())
    r = lse_ref.double()
    empty_r = torch.isinf(r) & (r < 0)
    empty_k = torch.isinf(k) & (k < 0)
    assert torch.equal(empty_r, empty_k), "rows without a valid entry differ"
    d = (k - r)[~empty_r].abs()
    err = float(d.max()) if d.numel() else 0.0
    assert err <= tol, f"LSE error {err} > {tol}"
    return err


def compare_out(out_kernel: torch.Tensor, out_ref: torch.Tensor, abs_tol, rel_tol, cos_tol=None, noise=1.0):
    """|d| <= abs_tol + rel_tol*max(|a|,|b|) elementwise; when cos_tol is given (FP8 kernel) the
    absolute term grows by TC_NOISE * rms(reference) and 1 - cos must stay below cos_tol."""
    if cos_tol is not None:
        abs_tol = abs_tol + noise * TC_NOISE * float(out_ref.float().pow(2).mean().sqrt())
        cos_tol = cos_tol * noise * noise
    ok, max_diff, nbad = orc.allclose_report(out_kernel.cpu(), out_ref, abs_tol, rel_tol)
    assert ok, f"{nbad} elements outside |d| <= {abs_tol} + {rel_tol}*max(|a|,|b|); max diff {max_diff}"
    if cos_tol is not None:
        cd = orc.cos_diff(out_kernel.cpu(), out_ref)
        assert cd <= cos_tol, f"1 - cos = {cd} > {cos_tol}"
    return max_diff
