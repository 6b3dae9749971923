"""Context-parallel decode on the GPU.  One-GPU case: the shards are processed one after the
other on cuda:0 and merged with the strided combine (all kernels of the multi-GPU path, no
collective).  Two-GPU case (skipped with fewer devices): two NCCL ranks, all-gather, merge."""
import os
import socket
import subprocess
import sys

import pytest
import torch

import helpers as H
from helpers import make_case, oracle_attn, ROOT

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.mark.parametrize("impl", [1, 2])
@pytest.mark.parametrize("world", [2, 4])
def test_cp_pieces_on_one_gpu(world, impl):
    from sparse_mla_sm120_b200 import cp
    from sparse_mla_sm120_b200._runtime import check_status
    dev = torch.device("cuda:0")
    case = make_case(23, 5, 128, 512, 32, invalid_tail=0.05)
    rows = case["packed"].shape[0] * 64
    case["indices"][4] = torch.where(case["indices"][4] < rows // world, case["indices"][4], -1)   # one-shard token
    ref_out, ref_lse = oracle_attn(case)
    q, idx = case["q"].to(dev), case["indices"].to(dev)
    if world == 4:      # the packed exchange buffer of the multi-GPU path: a rank's partials and LSEs adjacent
        _, o_all, l_all = cp._gather_buffers(dev, world, 5, 128)
    else:
        o_all = torch.empty((world, 5, 128, 512), dtype=torch.float32, device=dev)
        l_all = torch.empty((world, 5, 128), dtype=torch.float32, device=dev)
    for r in range(world):
        lo, hi = cp.shard_context(rows, r, world)
        kv_local = case["packed"].view(-1, 656)[lo:hi].reshape(-1, 64, 1, 656).to(dev)
        local_idx, local_len = cp.partition_indices(idx, lo, hi)
        cp.decode_partial(q, kv_local, local_idx, local_len, case["sm_scale"], o_all[r], l_all[r], impl=impl)
    out, lse = cp.combine_parts(o_all, l_all)
    torch.cuda.synchronize()
    check_status(dev)
    assert bool((l_all[1:, 4] < -1e20).all()), "token 4 has entries on shard 0 only"
    if impl == 1:
        H.compare_out(out, ref_out, H.SCALAR_ABS, H.SCALAR_REL)
        H.compare_lse(lse, ref_lse, H.SCALAR_LSE)
    else:
        H.compare_out(out, ref_out, H.TC_ABS, H.TC_REL, H.TC_COS)
        H.compare_lse(lse, ref_lse, H.TC_LSE)


def _indexer_case(seed, s_q, h, s_k):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(s_q, h, 128, generator=g).to(torch.float8_e4m3fn)
    kf = torch.randn(s_k, 128, generator=g)
    k_scale = kf.abs().amax(dim=1) / 448.0
    k = (kf / k_scale.unsqueeze(1)).to(torch.float8_e4m3fn)
    w = torch.randn(s_q, h, generator=g) * 0.1
    ks = torch.zeros(s_q, dtype=torch.int32)
    ke = (s_k - s_q + 1 + torch.arange(s_q)).to(torch.int32)
    return q, k, k_scale, w, ks, ke


def _check_selection(got, full_logits, k):
    """got [T, k] int32: every row must hold min(k, finite entries) distinct columns whose logits
    are not below the k-th largest, with every strictly larger one present."""
    for r in range(got.shape[0]):
        g = got[r][got[r] >= 0]
        n = int(min(k, int(torch.isfinite(full_logits[r]).sum())))
        assert g.numel() == n and torch.unique(g).numel() == n
        if n:
            thr = torch.topk(full_logits[r], n).values[-1]
            vals = full_logits[r][g.long()]
            assert float(vals.min()) >= float(thr)
            assert int((full_logits[r] > thr).sum()) == int((vals > thr).sum())


@pytest.mark.parametrize("world,s_k,k", [(2, 4096, 256), (4, 4096, 256), (4, 16384, 2048), (8, 32768, 2048)])
def test_indexer_cp_pieces_on_one_gpu(world, s_k, k):
    """Per-shard logits + top-k, candidates side by side, merge: the distributed selection without
    the collective, against the oracle's logits over the whole context."""
    from sparse_mla_sm120_b200 import cp
    dev = torch.device("cuda:0")
    s_q, h = 6, 64
    q, key, k_scale, w, ks, ke = _indexer_case(41, s_q, h, s_k)
    ks[1], ke[1] = 1500, 1700          # fewer than k candidates, inside one shard (world 2) / two shards (world 4)
    ks[2], ke[2] = 900, 3300
    full = H.orc.mqa_logits_ref(q, key, k_scale, w, ks, ke)
    gathered = torch.empty((world, 2, s_q, k), dtype=torch.int32, device=dev)      # what the all-gather would leave
    for r in range(world):
        lo, hi = cp.shard_context(s_k, r, world)
        cp.local_candidates(q.to(dev), key[lo:hi].contiguous().to(dev), k_scale[lo:hi].contiguous().to(dev),
                            w.to(dev), ks.to(dev), ke.to(dev), lo, hi, k, out=gathered[r])
    vals, pos = cp.interleave_candidates(gathered)
    assert torch.equal(vals.view(torch.int32), gathered[:, 0].permute(1, 0, 2).reshape(s_q, world * k))
    assert torch.equal(pos, gathered[:, 1].permute(1, 0, 2).reshape(s_q, world * k))
    got = cp.merge_candidates(vals, pos, k).cpu()
    _check_selection(got, full, k)
    assert int((got[1] >= 0).sum()) == 200


def test_indexed_decode_pipeline_one_gpu():
    """Indexer -> top-k -> attention in one call; the rows it selected are checked against the
    oracle's logits, the attention output against the oracle over those rows."""
    from sparse_mla_sm120_b200 import pipeline
    dev = torch.device("cuda:0")
    case = make_case(43, 6, 128, 256, 48, invalid_tail=0.0)
    s_k = case["packed"].shape[0] * 64
    q, key, k_scale, w, ks, ke = _indexer_case(44, 6, 64, s_k)
    ke[3] = 100                          # fewer candidates than topk: -1 padding reaches the attention
    out, lse, rows = pipeline.sparse_mla_indexed_decode_fwd(
        case["q"].to(dev), case["packed"].to(dev), q.to(dev), key.to(dev), k_scale.to(dev), w.to(dev), ks.to(dev),
        ke.to(dev), case["sm_scale"], topk=256)
    torch.cuda.synchronize()
    _check_selection(rows.cpu(), H.orc.mqa_logits_ref(q, key, k_scale, w, ks, ke), 256)
    case["indices"] = rows.cpu()
    ref_out, ref_lse = oracle_attn(case)
    H.compare_out(out, ref_out, H.TC_ABS, H.TC_REL, H.TC_COS)
    H.compare_lse(lse, ref_lse, H.TC_LSE)
    # the same step as a CUDA-graph replay, twice with different inputs
    graphed = pipeline.GraphedIndexedDecode(case["packed"].to(dev), key.to(dev), k_scale.to(dev), 6, 128, 64,
                                            case["sm_scale"], topk=256)
    ke2 = ke.clone(); ke2[0] = 700
    for ke_i in (ke2, ke):
        g_out, g_lse, g_rows = graphed(case["q"].to(dev), q.to(dev), w.to(dev), ks.to(dev), ke_i.to(dev))
    torch.cuda.synchronize()
    assert torch.equal(g_rows, rows) and torch.equal(g_out, out) and torch.equal(g_lse, lse)
    # through a page table that reverses the pages
    pages = s_k // 64
    table = torch.arange(pages - 1, -1, -1, dtype=torch.int32).repeat(6, 1)
    mapped = pipeline.positions_to_rows(rows, table.to(dev), 64).cpu()
    r = rows.cpu()
    want = torch.where(r >= 0, (pages - 1 - r // 64) * 64 + r % 64, r)
    assert torch.equal(mapped, want.to(torch.int32))


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("tokens", [4, 70])
def test_cp_head_sliced_pieces_on_one_gpu(world, tokens):
    """The head-sliced exchange with the ranks emulated one after the other on cuda:0: every rank's local
    step writes its partials as head slices, the all-to-all is a copy between the emulated ranks' buffers,
    every rank merges its slice, the all-gather is a stack, and the un-slice gives the full output.
    70 tokens stand for a prefill chunk."""
    from sparse_mla_sm120_b200 import cp
    dev = torch.device("cuda:0")
    case = make_case(31, tokens, 128, 512, 64, invalid_tail=0.05)
    rows = case["packed"].shape[0] * 64
    q, idx = case["q"].to(dev), case["indices"].to(dev)
    T, Hh = tokens, 128
    hs = Hh // world
    c = -(-(T * hs * 513) // 512) * 512
    chunk_bytes = -(-(T * hs * 1028) // 16) * 16
    sends = []
    for g in range(world):
        lo, hi = cp.shard_context(rows, g, world)
        kv_local = case["packed"].view(-1, 656)[lo:hi].reshape(-1, 64, 1, 656).to(dev)
        local_idx, local_len = cp.partition_indices(idx, lo, hi)
        send = torch.empty((world, c), dtype=torch.float32, device=dev)
        cp.decode_partial_sliced(q, kv_local, local_idx, local_len, case["sm_scale"], send, world, c)
        sends.append(send)
    sink = torch.linspace(-2.0, 2.0, Hh, device=dev)
    gathered = torch.empty((world, chunk_bytes), dtype=torch.uint8, device=dev)
    for d in range(world):
        recv = torch.stack([sends[g][d] for g in range(world)]).contiguous()      # what the all-to-all delivers to rank d
        cp.merge_head_slice(recv, gathered[d], world, T, hs, c, sink[d * hs:(d + 1) * hs].contiguous())
    out, lse = cp.unslice(gathered, world, T, hs, chunk_bytes)
    torch.cuda.synchronize()
    ref_out, ref_lse = oracle_attn(case)
    ref_out, ref_lse = H.orc.apply_attn_sink(ref_out, ref_lse, sink.cpu())
    H.compare_out(out, ref_out, H.TC_ABS, H.TC_REL, H.TC_COS)
    H.compare_lse(lse, ref_lse, H.TC_LSE)


_RANK_SCRIPT = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["SMLA_ROOT"]); sys.path.insert(0, os.path.join(os.environ["SMLA_ROOT"], "tests"))
import helpers as H
from sparse_mla_sm120_b200 import cp
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank); dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
case = H.make_case(29, 4, 128, 1024, 64, invalid_tail=0.05)
rows = case["packed"].shape[0] * 64
lo, hi = cp.shard_context(rows, rank, world)
kv_local = case["packed"].view(-1, 656)[lo:hi].reshape(-1, 64, 1, 656).to(dev)
out, lse = cp.sparse_mla_decode_cp_fwd(case["q"].to(dev), kv_local, case["indices"].to(dev), case["sm_scale"], lo, hi)
torch.cuda.synchronize()
ref_out, ref_lse = H.oracle_attn(case)
H.compare_out(out, ref_out, H.TC_ABS, H.TC_REL, H.TC_COS)
H.compare_lse(lse, ref_lse, H.TC_LSE)
# the same step captured into one CUDA graph (collectives included), replayed twice on fresh inputs
graphed = cp.GraphedCpDecode(kv_local, 4, 128, 1024, case["sm_scale"], lo, hi)
for _ in range(2):
    g_out, g_lse = graphed(case["q"].to(dev), case["indices"].to(dev))
    torch.cuda.synchronize()
    assert torch.equal(g_out, out) and torch.equal(g_lse, lse), "graph replay differs from the eager step"
graphed.close()
# the head-sliced exchange (the default above a traffic limit), forced for this small case
cp.ALL_GATHER_LIMIT_BYTES = 0
s_out, s_lse = cp.sparse_mla_decode_cp_fwd(case["q"].to(dev), kv_local, case["indices"].to(dev), case["sm_scale"], lo, hi)
torch.cuda.synchronize()
H.compare_out(s_out, ref_out, H.TC_ABS, H.TC_REL, H.TC_COS)
H.compare_lse(s_lse, ref_lse, H.TC_LSE)
# context-parallel prefill: the query tokens in chunks of 3 through the same exchange
p_out, p_lse = cp.sparse_mla_prefill_cp_fwd(case["q"].to(dev), kv_local, case["indices"].to(dev), case["sm_scale"], lo, hi,
                                           chunk_tokens=3)
torch.cuda.synchronize()
H.compare_out(p_out, ref_out, H.TC_ABS, H.TC_REL, H.TC_COS)
H.compare_lse(p_lse, ref_lse, H.TC_LSE)
# indexer -> distributed top-k -> context-parallel attention
g = torch.Generator().manual_seed(47)
qi = torch.randn(4, 64, 128, generator=g).to(torch.float8_e4m3fn)
kf = torch.randn(rows, 128, generator=g)
k_scale = kf.abs().amax(dim=1) / 448.0
ki = (kf / k_scale.unsqueeze(1)).to(torch.float8_e4m3fn)
w = torch.randn(4, 64, generator=g) * 0.1
ks = torch.tensor([0, 100, 0, 3000], dtype=torch.int32); ke = torch.tensor([rows, rows - 5, 700, 3100], dtype=torch.int32)
out, lse, sel = cp.sparse_mla_indexed_decode_cp_fwd(case["q"].to(dev), kv_local, qi.to(dev), ki[lo:hi].contiguous().to(dev),
    k_scale[lo:hi].contiguous().to(dev), w.to(dev), ks.to(dev), ke.to(dev), case["sm_scale"], lo, hi, topk=1024)
torch.cuda.synchronize()
sel = sel.cpu()
full = H.orc.mqa_logits_ref(qi, ki, k_scale, w, ks, ke)
for r in range(4):
    got = sel[r][sel[r] >= 0]
    n = min(1024, int(torch.isfinite(full[r]).sum()))
    assert got.numel() == n and torch.unique(got).numel() == n, (r, got.numel(), n)
    thr = torch.topk(full[r], n).values[-1]
    assert float(full[r][got.long()].min()) >= float(thr)
gathered = [torch.empty_like(sel) for _ in range(world)]
dist.all_gather_object(gathered, sel)
assert all(torch.equal(gathered[0], t) for t in gathered), "ranks disagree on the selection"
case["indices"] = sel
ref_out, ref_lse = H.oracle_attn(case)
H.compare_out(out, ref_out, H.TC_ABS, H.TC_REL, H.TC_COS)
H.compare_lse(lse, ref_lse, H.TC_LSE)
# the same step with the indexer, captured into one CUDA graph (three collectives inside), replayed twice
gi = cp.GraphedIndexedCpDecode(kv_local, ki[lo:hi].contiguous().to(dev), k_scale[lo:hi].contiguous().to(dev), 4, 128, 64,
                               case["sm_scale"], lo, hi, topk=1024)
for _ in range(2):
    g_out, g_lse, g_sel = gi(case["q"].to(dev), qi.to(dev), w.to(dev), ks.to(dev), ke.to(dev))
    torch.cuda.synchronize()
    assert torch.equal(g_sel.cpu(), sel) and torch.equal(g_out, out) and torch.equal(g_lse, lse), \
        "graph replay of the indexed step differs from the eager step"
assert gi.graph is not None
gi.close()
print("rank", rank, "ok", flush=True)
dist.barrier(); torch.cuda.synchronize()
os._exit(0)      # every rank leaves at once; nothing here depends on an orderly shutdown of the communicator
'''


def test_cp_prefill_chunks_without_a_process_group():
    """Context-parallel prefill with a world of one: the chunking of the query tokens and the partition of the
    indices over a shard that is the whole context."""
    from sparse_mla_sm120_b200 import cp
    case = make_case(31, 7, 64, 256, 16, invalid_tail=0.1)
    ref_out, ref_lse = oracle_attn(case)
    rows = case["packed"].shape[0] * 64
    out, lse = cp.sparse_mla_prefill_cp_fwd(case["q"].to(DEV), case["packed"].to(DEV), case["indices"].to(DEV), case["sm_scale"],
                                            0, rows, chunk_tokens=3)
    torch.cuda.synchronize()
    H.compare_out(out.cpu(), ref_out, H.TC_ABS, H.TC_REL, H.TC_COS)
    H.compare_lse(lse.cpu(), ref_lse, H.TC_LSE)


@pytest.mark.parametrize("world", [2, 4])
def test_cp_nccl_ranks(tmp_path, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    script = tmp_path / "rank.py"
    script.write_text(_RANK_SCRIPT)
    env = dict(os.environ, SMLA_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
    # One run on a port that is free now (asked from the kernel); a failure is reported, never re-run: a rank that
    # died of a GPU fault must not be launched again unchanged on shared GPUs.
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = str(sock.getsockname()[1])
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                          "--master-addr", "127.0.0.1", "--master-port", port, str(script)],
                         env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert all(f"rank {r} ok" in res.stdout for r in range(world))
