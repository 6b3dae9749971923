"""Host logic of the multi-GPU paths on CPU: shard arithmetic, and the context-parallel
decomposition run as two gloo ranks (oracle partials per shard, all-gather, LSE merge) against
the single-rank oracle.  No GPU involved."""
import os
import sys

import pytest
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
