"""The allocation-free decode entry point against the regular one.

smla_decode_splitkv_noalloc keeps its scratch in an array inside the library, for hosts that
cannot hand the library device memory when they call it (their own pool owns the device, or the
call site must not enter the CUDA allocator).  The test drives it through the C ABI twice in a
row, since the second call finds the first call's leftovers in the shared array, and compares
each result with the regular scheduler + decode + combine path on the same inputs.  This file
sorts last on purpose: a run that stops at the first failure has then covered everything else.
"""
import pytest
import torch

import helpers as H
from helpers import make_case

pytestmark = pytest.mark.gpu


def _noalloc(lib, q, kv, idx, sm_scale, parts, sink=None, tl=None):
    from sparse_mla_sm120_b200._lib import check
    from sparse_mla_sm120_b200._runtime import ptr, stream_ptr
    T, Hh, _ = q.shape
    out = torch.empty((T, Hh, 512), dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((T, Hh), dtype=torch.float32, device=q.device)
    check(lib.smla_decode_splitkv_noalloc(ptr(q), ptr(kv), ptr(idx), ptr(out), ptr(lse), T, Hh, idx.shape[1],
                                          float(sm_scale), 64, 64 * 656, parts, ptr(sink), ptr(tl), 0, None,
                                          stream_ptr(q.device)))
    return out, lse


def test_noalloc_matches_regular_entry_point_twice():
    from sparse_mla_sm120_b200 import _lib, flash_ops
    lib = _lib.load()
    dev = torch.device("cuda:0")
    # two different requests, so that the second call really has to overwrite the first call's scratch
    cases = [make_case(31, 5, 128, 1024, 32, invalid_tail=0.1), make_case(32, 3, 64, 512, 16, invalid_tail=0.0)]
    sink = torch.linspace(-2, 2, 128)
    for rep, (case, parts) in enumerate(zip(cases, (20, 7))):
        q, kv, idx = case["q"].to(dev), case["packed"].to(dev), case["indices"].to(dev)
        s = sink[:q.shape[1]].contiguous().to(dev) if rep == 0 else None
        assert lib.smla_noalloc_scratch_need(q.shape[0], q.shape[1], parts) <= (16 << 20)
        ref_out, ref_lse = flash_ops.sparse_mla_decode_fwd(q, kv, idx, case["sm_scale"], attn_sink=s, num_sm_parts=parts)
        out, lse = _noalloc(lib, q, kv, idx, case["sm_scale"], parts, sink=s)
        torch.cuda.synchronize()
        # same kernels on the same inputs: the tolerance of the other decode tests is far from needed
        H.compare_out(out, ref_out.cpu(), H.TC_ABS, H.TC_REL, H.TC_COS)
        assert float((lse.cpu() - ref_lse.cpu()).abs().max()) <= H.TC_LSE
        assert torch.equal(out, ref_out) and torch.equal(lse, ref_lse)


def test_noalloc_rejects_what_does_not_fit():
    from sparse_mla_sm120_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda:0")
    case = make_case(33, 64, 128, 64, 2)
    q, kv, idx = case["q"].to(dev), case["packed"].to(dev), case["indices"].to(dev)
    assert lib.smla_noalloc_scratch_need(64, 128, 74) > (16 << 20)
    with pytest.raises(ValueError, match="scratch"):
        _noalloc(lib, q, kv, idx, case["sm_scale"], 74)


def test_noalloc_refuses_bad_arguments_before_launching_anything():
    """An unknown kernel selector or a misaligned q is refused by the argument checks; the scheduler, which
    runs first, must not have been launched (the scratch keeps the previous call's records)."""
    from sparse_mla_sm120_b200 import _lib
    from sparse_mla_sm120_b200._runtime import ptr, stream_ptr
    lib = _lib.load()
    dev = torch.device("cuda:0")
    case = make_case(34, 2, 16, 128, 2)
    q, kv, idx = case["q"].to(dev), case["packed"].to(dev), case["indices"].to(dev)
    _noalloc(lib, q, kv, idx, case["sm_scale"], 3)
    torch.cuda.synchronize()
    out = torch.empty(2, 16, 512, dtype=torch.bfloat16, device=dev)
    lse = torch.empty(2, 16, dtype=torch.float32, device=dev)
    for impl, q_ptr in ((77, ptr(q)), (0, ptr(q) + 2)):
        rc = lib.smla_decode_splitkv_noalloc(q_ptr, ptr(kv), ptr(idx), ptr(out), ptr(lse), 2, 16, 128,
                                             float(case["sm_scale"]), 64, 64 * 656, 3, None, None, impl, None,
                                             stream_ptr(dev))
        assert rc < 0, lib.smla_last_error()
