"""Context-parallel decode on the GPU.  One-GPU case: the shards are processed one after the
other on cuda:0 and merged with the strided combine (all kernels of the multi-GPU path, no
collective).  Two-GPU case (skipped with fewer devices): two NCCL ranks, all-gather, merge."""
import os
import subprocess
import sys

import pytest
import torch

import helpers as H
from helpers import make_case, oracle_attn, ROOT

pytestmark = pytest.mark.gpu


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
dist.barrier(); dist.destroy_process_group()
print("rank", rank, "ok")
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_cp_two_nccl_ranks(tmp_path):
    script = tmp_path / "rank.py"
    script.write_text(_RANK_SCRIPT)
    env = dict(os.environ, SMLA_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
    # a rendezvous port may still be held by an earlier job on the same box: one retry on another port
    for port in ("29631", "29747"):
        res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                              "--master-addr", "127.0.0.1", "--master-port", port, str(script)],
                             env=env, capture_output=True, text=True, timeout=300)
        if res.returncode == 0:
            break
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "rank 0 ok" in res.stdout and "rank 1 ok" in res.stdout
