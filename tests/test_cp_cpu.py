"""Host logic of the multi-GPU paths on CPU: shard arithmetic, and the context-parallel
decomposition run as two gloo ranks (oracle partials per shard, all-gather, LSE merge) against
the single-rank oracle.  No GPU involved."""
import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import make_case, oracle_attn, orc
from sparse_mla_sm120_b200 import cp


def test_shard_arithmetic():
    for n, w in [(64, 8), (10, 4), (3, 8), (128, 2)]:
        spans = [cp.shard_requests(n, r, w) for r in range(w)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert max(e - b for b, e in spans) - min(e - b for b, e in spans) <= 1
    for L, w in [(131072, 8), (100000, 4), (4096, 2), (100, 8)]:
        spans = [cp.shard_context(L, r, w) for r in range(w)]
        assert spans[0][0] == 0 and spans[-1][1] == L
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert all(lo % 64 == 0 or lo == L for lo, _ in spans)


def test_partition_oracle():
    idx = torch.tensor([[5, -1, 70, 64, 3, 127, 128, -1]], dtype=torch.int32)
    local, n = orc.cp_partition_ref(idx, 64, 128)
    assert local.tolist() == [[6, 0, 63, -1, -1, -1, -1, -1]] and n.tolist() == [3]


def _rank_main(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    case = make_case(17, 3, 16, 256, 8, invalid_tail=0.1)          # identical on every rank (seeded)
    case["indices"][2, :] = torch.where(case["indices"][2] < 256, case["indices"][2], -1)  # rank 1 sees nothing of token 2
    rows = case["packed"].shape[0] * 64
    lo, hi = cp.shard_context(rows, rank, world)
    local_idx, local_len = orc.cp_partition_ref(case["indices"], lo, hi)
    shard = {"packed": case["packed"].view(-1, 656)[lo:hi].reshape(-1, 64, 1, 656), "q": case["q"],
             "indices": local_idx, "sm_scale": case["sm_scale"]}
    out, lse = oracle_attn(shard, topk_length=local_len)            # normalised partial + natural-log LSE
    lse2 = torch.where(torch.isinf(lse), torch.full_like(lse, -1e30), lse * orc.LOG2E)
    o_all = [torch.empty_like(out, dtype=torch.float32) for _ in range(world)]
    l_all = [torch.empty_like(lse2) for _ in range(world)]
    dist.all_gather(o_all, out.float())
    dist.all_gather(l_all, lse2)
    merged, mlse = orc.combine_ref(torch.stack(o_all, 1).reshape(-1, 1, 16, 512),   # [T*world, 1, H, 512]: splits of a token adjacent
                                   torch.stack(l_all, 1).reshape(-1, 1, 16), [i * world for i in range(4)], 3)
    if rank == 0:
        ref_out, ref_lse = oracle_attn(case)
        ret["err"] = float((merged.float() - ref_out.float()).abs().max())
        ret["lse_err"] = float((mlse * orc.LN2 - ref_lse).abs().max())
        ret["empty_part"] = bool((l_all[1][2] < -1e20).all())
    dist.barrier()
    dist.destroy_process_group()


def test_context_parallel_decomposition_two_gloo_ranks():
    port = 29500 + os.getpid() % 1000
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_rank_main, args=(2, port, ret), nprocs=2, join=True)
        assert ret["empty_part"], "token 2 has no entry on rank 1: its partial must be empty"
        assert ret["err"] < 2e-2 and ret["lse_err"] < 1e-5, dict(ret)   # bf16 partials: 2^-8 relative


def _indexer_inputs(seed, s_q, h, s_k):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(s_q, h, 128, generator=g).to(torch.float8_e4m3fn)
    kf = torch.randn(s_k, 128, generator=g)
    k_scale = kf.abs().amax(dim=1) / 448.0
    k = (kf / k_scale.unsqueeze(1)).to(torch.float8_e4m3fn)
    w = torch.randn(s_q, h, generator=g) * 0.1
    ks = torch.tensor([0, 40, 300, 0], dtype=torch.int32)[:s_q]
    ke = torch.tensor([s_k, 200, s_k - 3, 100], dtype=torch.int32)[:s_q]
    return q, k, k_scale, w, ks, ke


def test_local_window():
    ks = torch.tensor([0, 40, 300, 0, 500], dtype=torch.int32)
    ke = torch.tensor([512, 200, 509, 100, 500], dtype=torch.int32)
    a, b = cp.local_window(ks, ke, 256, 512)
    assert a.tolist() == [0, 0, 44, 0, 244] and b.tolist() == [256, 0, 253, 0, 244]
    a, b = cp.local_window(ks, ke, 0, 256)
    assert a.tolist() == [0, 40, 256, 0, 256] and b.tolist() == [256, 200, 256, 100, 256]


def _indexer_rank_main(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    s_q, h, s_k, k = 4, 8, 512, 48
    q, key, k_scale, w, ks, ke = _indexer_inputs(31, s_q, h, s_k)
    lo, hi = cp.shard_context(s_k, rank, world)
    ks_l, ke_l = cp.local_window(ks, ke, lo, hi)
    logits = orc.mqa_logits_ref(q, key[lo:hi], k_scale[lo:hi], w, ks_l, ke_l)
    local = orc.topk_ref(logits, k)
    vals = torch.where(local >= 0, torch.gather(logits, 1, local.clamp(min=0).long()), torch.tensor(float("-inf")))
    pos = torch.where(local >= 0, local + lo, local)
    v_all = [torch.empty_like(vals) for _ in range(world)]
    p_all = [torch.empty_like(pos) for _ in range(world)]
    dist.all_gather(v_all, vals)
    dist.all_gather(p_all, pos)
    v, p = torch.cat(v_all, 1), torch.cat(p_all, 1)
    pick = orc.topk_ref(v, k)
    merged = torch.where(pick >= 0, torch.gather(p, 1, pick.clamp(min=0).long()), pick)
    if rank == 0:
        full = orc.mqa_logits_ref(q, key, k_scale, w, ks, ke)
        want = orc.topk_ref(full, k)
        ret["same_sets"] = all(set(merged[i][merged[i] >= 0].tolist()) == set(want[i][want[i] >= 0].tolist())
                               for i in range(s_q))
        ret["counts"] = [int((merged[i] >= 0).sum()) for i in range(s_q)]
    dist.barrier()
    dist.destroy_process_group()


def test_indexer_candidate_merge_two_gloo_ranks():
    """Per-shard top-k + merge of the candidates gives the top-k of the whole context."""
    port = 30500 + os.getpid() % 1000
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_indexer_rank_main, args=(2, port, ret), nprocs=2, join=True)
        assert ret["same_sets"], dict(ret)
        assert ret["counts"] == [48, 48, 48, 48]


def test_positions_to_rows_cpu():
    """Logical positions -> physical cache rows through a page table (pure index arithmetic)."""
    from sparse_mla_sm120_b200.pipeline import positions_to_rows
    table = torch.tensor([[7, 2, 9], [0, 5, 1]], dtype=torch.int32)
    pos = torch.tensor([[0, 63, 64, 130, -1], [191, 1, -1, 65, 128]], dtype=torch.int32)
    rows = positions_to_rows(pos, table, 64)
    assert rows.dtype == torch.int32
    assert rows.tolist() == [[7 * 64, 7 * 64 + 63, 2 * 64, 9 * 64 + 2, -1], [1 * 64 + 63, 1, -1, 5 * 64 + 1, 1 * 64]]
