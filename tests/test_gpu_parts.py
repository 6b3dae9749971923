"""Parity of the scheduler, combine, cache writer, indexer, top-k and index partition kernels."""
import numpy as np
import pytest
import torch

from helpers import bf16_from_bits, orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


# ------------------------------------------------------------------ scheduler: integer-exact
@pytest.mark.parametrize("b,topk,parts", [(1, 512, 4), (1, 2048, 32), (4, 1024, 16), (8, 2048, 32), (16, 512, 4),
                                          (32, 512, 64), (64, 2048, 74), (64, 2048, 64), (128, 2048, 74),
                                          (5, 2048, 148), (4096, 2048, 74)])
def test_scheduler_matches_oracle(b, topk, parts):
    from sparse_mla_sm120_b200 import flash_ops
    meta = torch.empty(parts * 8, dtype=torch.int32, device=DEV)
    ns = torch.empty(b + 1, dtype=torch.int32, device=DEV)
    flash_ops.get_decode_metadata(b, topk, 0, parts, 5, None, None, meta, ns)
    ref_meta, ref_ns = orc.sched_meta_ref(b, topk, 0, parts, 5)
    got = meta.view(parts, 8).cpu().tolist()
    assert got == ref_meta
    assert ns.cpu().tolist() == ref_ns
    orc.verify_schedule(got, ns.cpu().tolist(), orc.expected_blocks(b, topk, 0, None, None), b)


def test_scheduler_lengths_and_extra():
    from sparse_mla_sm120_b200 import flash_ops
    for tl, etl, topk, extra, parts in [([256, 512, 128, 512], None, 512, 0, 8), ([0, 512], None, 512, 0, 4),
                                        ([100, 200, 300], None, 512, 0, 4),
                                        ([256, 512, 128, 512], [128, 64, 256, 0], 512, 256, 8)]:
        b = len(tl)
        meta = torch.empty(parts * 8, dtype=torch.int32, device=DEV)
        ns = torch.empty(b + 1, dtype=torch.int32, device=DEV)
        tl_d = torch.tensor(tl, dtype=torch.int32, device=DEV)
        etl_d = None if etl is None else torch.tensor(etl, dtype=torch.int32, device=DEV)
        flash_ops.get_decode_metadata(b, topk, extra, parts, 5, tl_d, etl_d, meta, ns)
        ref_meta, ref_ns = orc.sched_meta_ref(b, topk, extra, parts, 5, tl, etl)
        assert meta.view(parts, 8).cpu().tolist() == ref_meta and ns.cpu().tolist() == ref_ns


# ------------------------------------------------------------------ combine
def _combine(o_accum, lse_accum, num_splits, batch, h, sink=None):
    from sparse_mla_sm120_b200 import flash_ops
    out = torch.zeros(batch, h, 512, dtype=torch.bfloat16, device=DEV)
    lse = torch.zeros(batch, h, dtype=torch.float32, device=DEV)
    ns = torch.as_tensor(num_splits, dtype=torch.int32).to(DEV)
    mx = int(max(num_splits[i + 1] - num_splits[i] for i in range(batch)))
    flash_ops.sparse_mla_combine_v2_fwd(o_accum.to(DEV), lse_accum.to(DEV), out, lse, ns, batch, mx,
                                        None if sink is None else sink.to(DEV))
    torch.cuda.synchronize()
    return out.cpu(), lse.cpu()


def test_combine_golden(golden_dir):
    g = np.load(f"{golden_dir}/combine.npz")
    ns = g["num_splits"].tolist()
    b = len(ns) - 1
    out, lse = _combine(torch.from_numpy(g["o_accum"]), torch.from_numpy(g["lse_accum"]), ns, b, 16)
    ref_out, ref_lse = bf16_from_bits(g["out_bf16"]), torch.from_numpy(g["lse"])
    multi = [i for i in range(b) if ns[i + 1] - ns[i] > 1]   # single-split requests are not touched
    assert float((out[multi].float() - ref_out[multi].float()).abs().max()) < 2e-3
    assert float((lse[multi] - ref_lse[multi]).abs().max()) < 1e-4
    single = [i for i in range(b) if ns[i + 1] - ns[i] <= 1]
    assert not out[single].any()


@pytest.mark.parametrize("nsplits", [2, 4, 8, 16, 32, 74])
@pytest.mark.parametrize("num_heads", [8, 64, 128])
def test_combine_grid(nsplits, num_heads):
    """tests/test_combine.py:60-93: bounds 1e-2 on output and LSE (ours: 2e-3 / 1e-4)."""
    torch.manual_seed(42)
    batch = 4
    o = torch.randn(batch * nsplits, 1, num_heads, 512) * 0.1
    l = torch.randn(batch * nsplits, 1, num_heads) * 3.0
    l[0, 0, :] = 100.0
    l[1:nsplits, 0, :] = -100.0
    ns = [i * nsplits for i in range(batch + 1)]
    out, lse = _combine(o, l, ns, batch, num_heads)
    ref_out, ref_lse = orc.combine_ref(o, l, ns, batch)
    assert float((out.float() - ref_out.float()).abs().max()) < 2e-3
    assert float((lse - ref_lse).abs().max()) < 1e-4
    assert torch.isfinite(out.float()).all()


# ------------------------------------------------------------------ cache writer: byte-exact
def test_pack_kv_bytes(golden_dir):
    from sparse_mla_sm120_b200 import indexer
    g = np.load(f"{golden_dir}/kv_format.npz")
    kv = bf16_from_bits(g["kv_bf16"])
    packed = indexer.pack_kv_cache(kv.to(DEV)).cpu()
    assert np.array_equal(packed.numpy(), g["packed"])
    torch.manual_seed(1)
    kv = (torch.randn(1000, 576) * torch.logspace(-6, 4, 1000).unsqueeze(1)).to(torch.bfloat16)
    kv[17] = 0
    ref = orc.quantize_kv_v32(kv.view(1000, 1, 1, 576)).view(1000, 656)
    got = indexer.pack_kv_cache(kv.to(DEV)).cpu()
    assert torch.equal(got, ref)


# ------------------------------------------------------------------ indexer + top-k + partition
def _indexer_case(seed, s_q, h, s_k):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(s_q, h, 128, generator=g).to(torch.float8_e4m3fn)
    kf = torch.randn(s_k, 128, generator=g)
    k_scale = kf.abs().amax(dim=1) / 448.0
    k = (kf / k_scale.unsqueeze(1)).to(torch.float8_e4m3fn)
    w = torch.randn(s_q, h, generator=g) * 0.1
    ks = torch.zeros(s_q, dtype=torch.int32)
    ke = (s_k - s_q + torch.arange(s_q)).to(torch.int32).clamp(min=1)
    return q, k, k_scale, w, ks, ke


@pytest.mark.parametrize("impl", [1, 2])
@pytest.mark.parametrize("s_q,h,s_k", [(8, 64, 1000), (130, 64, 4096), (5, 32, 257)])
def test_mqa_logits(s_q, h, s_k, impl):
    from sparse_mla_sm120_b200 import indexer
    q, k, k_scale, w, ks, ke = _indexer_case(3, s_q, h, s_k)
    ks[1 % s_q] = 7
    ref = orc.mqa_logits_ref(q, k, k_scale, w, ks, ke)
    got = indexer.fp8_mqa_logits(q.to(DEV), k.to(DEV), k_scale.to(DEV), w.to(DEV), ks.to(DEV), ke.to(DEV),
                                 impl=impl).cpu()
    assert torch.equal(torch.isinf(got), torch.isinf(ref)), "range mask differs"
    fin = ~torch.isinf(ref)
    # products of e4m3 values are exact in fp32; only the summation order differs
    assert float((got[fin] - ref[fin]).abs().max()) <= 1e-4 * float(ref[fin].abs().max())


def test_mqa_logits_short_then_long_items():
    """Causal windows over a long key range: the first work items of a CTA need one or two key tiles, later ones
    five or six.  (A group of one or two tiles needs nothing from the epilogue warps, so the loader could once
    arm two groups before a slow epilogue warp had waited for the first; the status word must stay clear.)"""
    from sparse_mla_sm120_b200 import indexer
    from sparse_mla_sm120_b200._runtime import check_status
    s_q, h, s_k = 800, 64, 2048
    q, k, k_scale, w, _, _ = _indexer_case(11, s_q, h, s_k)
    ks = torch.zeros(s_q, dtype=torch.int32)
    ke = (torch.arange(s_q, dtype=torch.int32) + 1)
    ref = orc.mqa_logits_ref(q, k, k_scale, w, ks, ke)
    for _ in range(3):
        got = indexer.fp8_mqa_logits(q.to(DEV), k.to(DEV), k_scale.to(DEV), w.to(DEV), ks.to(DEV), ke.to(DEV)).cpu()
        check_status(torch.device(DEV))
        assert torch.equal(torch.isinf(got), torch.isinf(ref)), "range mask differs"
        fin = ~torch.isinf(ref)
        assert float((got[fin] - ref[fin]).abs().max()) <= 1e-4 * float(ref[fin].abs().max())


def test_topk_sets():
    from sparse_mla_sm120_b200 import indexer
    torch.manual_seed(5)
    rows, cols, k = 6, 5000, 512
    logits = torch.randn(rows, cols)
    logits[2, 100:400] = 1.3            # a run of ties across the threshold
    ks = torch.tensor([0, 10, 0, 0, 4000, 0], dtype=torch.int32)
    ke = torch.tensor([cols, 4000, cols, 300, cols, 0], dtype=torch.int32)
    masked = logits.clone()
    j = torch.arange(cols).unsqueeze(0)
    masked[(j < ks.view(-1, 1)) | (j >= ke.view(-1, 1))] = float("-inf")
    got = indexer.topk_indices(masked.to(DEV), ks.to(DEV), ke.to(DEV), k).cpu()
    for r in range(rows):
        g = got[r][got[r] >= 0]
        n = int(min(k, max(int(ke[r]) - int(ks[r]), 0)))
        assert g.numel() == n and torch.all(got[r][n:] == -1)
        assert torch.unique(g).numel() == n                      # no duplicates
        if n:
            thr = torch.topk(masked[r], n).values[-1]
            vals = masked[r][g.long()]
            assert float(vals.min()) >= float(thr)
            assert int((masked[r] > thr).sum()) == int((vals > thr).sum())   # every strictly-greater one taken
    # ties go to the lower column
    r = 2
    thr = torch.topk(masked[r], k).values[-1]
    assert abs(float(thr) - 1.3) < 1e-6
    tied = got[r][(masked[r][got[r].long()] == masked[r][100])]
    assert int(tied.max()) - int(tied.min()) + 1 == tied.numel() and int(tied.min()) == 100


def test_topk_many_ties_and_wide_rows():
    """More ties at the threshold than the two-read kernel keeps as candidates (the row is redone
    by the multi-pass kernel), and rows wider than its 65536-column limit."""
    from sparse_mla_sm120_b200 import indexer
    torch.manual_seed(6)
    for rows, cols, k, tie_lo, tie_hi in [(3, 9000, 1024, 2000, 6000), (2, 70000, 2048, 100, 400)]:
        logits = torch.randn(rows, cols)
        logits[1, tie_lo:tie_hi] = 0.75
        got = indexer.topk_indices(logits.to(DEV), None, None, k).cpu()
        for r in range(rows):
            g = got[r]
            assert int((g < 0).sum()) == 0 and torch.unique(g).numel() == k
            thr = torch.topk(logits[r], k).values[-1]
            vals = logits[r][g.long()]
            assert float(vals.min()) >= float(thr)
            assert int((logits[r] > thr).sum()) == int((vals > thr).sum())
            tied = g[vals == thr]
            if tied.numel() > 1 and r == 1 and float(thr) == 0.75:      # ties go to the lowest columns
                all_tied = torch.nonzero(logits[r] == thr).flatten()
                assert torch.equal(torch.sort(tied).values, all_tied[:tied.numel()].to(torch.int32))


def _check_topk_rows(got, masked, k):
    for r in range(masked.shape[0]):
        g = got[r][got[r] >= 0]
        n = int(min(k, int(torch.isfinite(masked[r]).sum())))
        assert g.numel() == n and torch.all(got[r][n:] == -1), (r, g.numel(), n)
        assert torch.unique(g).numel() == n
        if n:
            thr = torch.topk(masked[r], n).values[-1]
            vals = masked[r][g.long()]
            assert float(vals.min()) >= float(thr)
            assert int((masked[r] > thr).sum()) == int((vals > thr).sum())


def test_topk_one_read_paths():
    """The one-read kernel's branches: several stretches of 65536 columns with ragged window
    edges, logits clustered at the end of the row, -inf inside the window (so many that the
    sampled guess fails and the multi-pass kernel takes over), a row pointer that is not
    16-byte aligned, and the same input twice (the order of the output is reproducible)."""
    from sparse_mla_sm120_b200 import indexer
    torch.manual_seed(9)
    rows, cols, k = 5, 200000, 2048
    logits = torch.randn(rows, cols)
    logits[1, -5000:] += 3.0                                     # the recent tokens dominate
    logits[2, torch.rand(cols) < 0.5] = float("-inf")            # half of the window is masked inside
    logits[3, torch.rand(cols) < 0.995] = float("-inf")          # fewer than k finite entries
    logits[4] = torch.linspace(-1.0, 1.0, cols)                  # monotone: the top-k is the tail
    ks = torch.tensor([777, 0, 13, 0, 5], dtype=torch.int32)
    ke = torch.tensor([199001, cols, cols - 1, cols, cols - 3], dtype=torch.int32)
    masked = logits.clone()
    j = torch.arange(cols).unsqueeze(0)
    masked[(j < ks.view(-1, 1)) | (j >= ke.view(-1, 1))] = float("-inf")
    dev_logits = masked.to(DEV)
    got = indexer.topk_indices(dev_logits, ks.to(DEV), ke.to(DEV), k)
    again = indexer.topk_indices(dev_logits, ks.to(DEV), ke.to(DEV), k)
    assert torch.equal(got, again)
    _check_topk_rows(got.cpu(), masked, k)
    assert int((got[3] >= 0).sum().item()) == int(torch.isfinite(masked[3]).sum())
    # thresholds near zero: the candidates lie on both sides of zero (bins linear in the value)
    near = torch.randn(6, 150000) * 0.03 + torch.tensor([-0.060, -0.066, -0.068, -0.070, -0.075, -0.2]).view(-1, 1)
    near[4, ::7] = 0.0
    near[4, 3::11] = -0.0
    got = indexer.topk_indices(near.to(DEV), None, None, k).cpu()
    _check_topk_rows(got, near, k)
    # misaligned rows: a view that starts one float into the buffer
    shifted = torch.empty(3, 20001, device=DEV)
    shifted[:, 1:] = dev_logits[:3, 50000:70000]
    view = shifted[:, 1:]
    got = indexer.topk_indices(view, None, None, 512).cpu()
    _check_topk_rows(got, masked[:3, 50000:70000], 512)


def test_cp_partition():
    from sparse_mla_sm120_b200 import cp
    torch.manual_seed(8)
    idx = torch.stack([torch.randperm(4096)[:300] for _ in range(9)]).to(torch.int32)
    idx[:, -20:] = -1
    for lo, hi in [(0, 1024), (1024, 2048), (3072, 4096), (100, 100)]:
        ref_local, ref_len = orc.cp_partition_ref(idx, lo, hi)
        local, length = cp.partition_indices(idx.to(DEV), lo, hi)
        assert torch.equal(local.cpu(), ref_local) and torch.equal(length.cpu(), ref_len)


def test_device_status_report_and_clear():
    """The host side of a bounded wait that gave up, without making one give up: a status record is written into
    the device buffer by hand; smla_device_status must report it, name the wait and clear the buffer."""
    import ctypes
    from sparse_mla_sm120_b200 import _lib
    from sparse_mla_sm120_b200._runtime import check_status, ptr, status_buffer, stream_ptr
    dev = torch.device(DEV)
    lib = _lib.load()
    st = status_buffer(dev)
    st.zero_()
    host = (ctypes.c_int32 * 4)()
    assert lib.smla_device_status(ptr(st), ctypes.addressof(host), stream_ptr(dev)) == 0
    st.copy_(torch.tensor([29, 2, 5, 0], dtype=torch.int32))
    rc = lib.smla_device_status(ptr(st), ctypes.addressof(host), stream_ptr(dev))
    assert rc == -6 and list(host) == [29, 2, 5, 0]
    assert b"attention s_free" in lib.smla_last_error()
    torch.cuda.synchronize()
    assert st.tolist() == [0, 0, 0, 0]
    st.copy_(torch.tensor([13, 1, 0, 0], dtype=torch.int32))
    with pytest.raises(_lib.SmlaError, match="indexer k_empty"):
        check_status(dev)
    check_status(dev)       # cleared by the report
