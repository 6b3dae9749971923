#!/usr/bin/env python
"""Benchmark of the sparse-MLA hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-extras]

One step = one split-KV decode call (scheduler -> attention -> combine) over one batch of the
DeepSeek-V3.2-shape decode configuration: 64 requests per GPU, 128 query heads, top-k 2048,
per-request KV length uniform in [4096, 32768] in a paged (block 64) pool of packed 656-byte
FP8 rows.  All inputs are synthetic and seeded.  With N > 1 every rank serves its own 64
requests (decode batches shard by sequence, nothing is exchanged), so scaling is weak.

Printed line: ``value`` is the algorithmic HBM traffic of the whole job divided by the step time
with inputs resident on the device (CUDA-graph replay of the public op); ``e2e`` is the same
through the public op with q / indices coming from pinned host memory and the output copied back
every step (the paged KV cache is device-resident state, as in any serving engine).
``--impl reference`` times the reference's CPU PyTorch path (restated in oracle/) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

B_PER_GPU, HEADS, TOPK, D_QK, D_V, ROW = 64, 128, 2048, 576, 512, 656
LEN_LO, LEN_HI, BLOCK = 4096, 32768, 64
NSETS = 8   # rotating (q, indices) sets so that consecutive steps gather different rows
SM_SCALE = D_QK ** -0.5
WORKLOAD = ("V3.2-shape sparse-MLA decode: b=64/GPU, s_q=1, h_q=128, topk=2048, d_qk=576, d_v=512, "
            "KV len U[4096,32768], paged block 64, packed FP8 656 B rows")
# DRAM bytes per launch of the attention kernel from the ncu capture summarised in
# profiles/attn_tc_decode_b64.md (dram__bytes_read.sum + dram__bytes_write.sum of one launch).
NCU_TRAFFIC_BYTES = 113_699_328


def algorithmic_bytes(num_tokens: int, n_valid: int) -> int:
    """Bytes one decode step must move: gathered rows + q + output + indices + LSE."""
    return num_tokens * (n_valid * ROW + HEADS * D_QK * 2 + HEADS * D_V * 2 + TOPK * 4 + HEADS * 4)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 1679.4)), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            parts = [x.strip() for x in s.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx = float(parts[1])
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def build_workload(device, seed: int, batch: int):
    """Paged pool + NSETS rotating (q, indices) sets, all on the device."""
    from sparse_mla_sm120_b200 import indexer
    g = torch.Generator(device="cpu").manual_seed(seed)
    lens = torch.randint(LEN_LO, LEN_HI + 1, (batch,), generator=g)
    nblk = (lens + BLOCK - 1) // BLOCK
    total_blocks = int(nblk.sum())
    perm = torch.randperm(total_blocks, generator=g)          # shuffled block table
    tables, off = [], 0
    for n in nblk.tolist():
        tables.append(perm[off:off + n]); off += n
    gd = torch.Generator(device=device).manual_seed(seed)
    pool = torch.empty((total_blocks, BLOCK, 1, ROW), dtype=torch.uint8, device=device)
    chunk = 2048  # blocks per packing chunk (bounds the bf16 temporary)
    for b0 in range(0, total_blocks, chunk):
        b1 = min(b0 + chunk, total_blocks)
        kv = torch.randn(((b1 - b0) * BLOCK, D_QK), device=device, generator=gd).to(torch.bfloat16)
        pool[b0:b1] = indexer.pack_kv_cache(kv).view(b1 - b0, BLOCK, 1, ROW)
    sets = []
    for s in range(NSETS):
        q = (torch.randn((batch, HEADS, D_QK), device=device, generator=gd) * 0.5).to(torch.bfloat16)
        idx = torch.empty((batch, TOPK), dtype=torch.int32)
        for i, (L, tab) in enumerate(zip(lens.tolist(), tables)):
            pos = torch.randperm(L, generator=g)[:TOPK]
            idx[i] = (tab[pos // BLOCK] * BLOCK + pos % BLOCK).to(torch.int32)
        sets.append((q, idx.to(device)))
    return pool, sets, lens


def time_events(fn, steps, warmup, sync):
    for i in range(warmup):
        fn(i)
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(warmup + i)
    e1.record()
    sync()
    return e0.elapsed_time(e1) / 1e3


def run_ours(args):
    import torch.distributed as dist
    from sparse_mla_sm120_b200 import _lib, flash_ops
    from sparse_mla_sm120_b200._runtime import (FIXED_OVERHEAD, check_status, kv_geometry, pick_num_sm_parts, ptr,
                                                 scratch, status_buffer, stream_ptr)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    hbm_peak, bf16_peak, peak_kind = measured_peaks()

    pool, sets, lens = build_workload(device, 1234 + rank, B_PER_GPU)
    bytes_step = algorithmic_bytes(B_PER_GPU, TOPK)

    def barrier_sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident: CUDA-graph replay of the public op, one graph per input set ----------
    outs, graphs = [], []
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for q, idx in sets:
            for _ in range(2):
                o = flash_ops.sparse_mla_decode_fwd(q, pool, idx, SM_SCALE)
            side.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                o = flash_ops.sparse_mla_decode_fwd(q, pool, idx, SM_SCALE)
            graphs.append(g); outs.append(o)
    torch.cuda.synchronize()
    check_status(device)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier_sync()
    secs = time_events(lambda i: graphs[i % NSETS].replay(), args.steps, args.warmup, barrier_sync)
    t = torch.tensor([secs], device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    secs = float(t.item())
    check_status(device)

    # ---- end to end: pinned host q / indices in, output out, through the public op -------------
    # Every step copies its q and indices from pinned host memory and its O and LSE back.  The three
    # legs run on their own streams over three sets of device buffers, so that the copies of
    # neighbouring steps overlap the kernel (PCIe is full duplex); the time is that of the whole
    # pipeline for `steps` steps.
    NBUF = 3
    host_sets = [(q.cpu().pin_memory(), idx.cpu().pin_memory()) for q, idx in sets]
    host_out = [torch.empty((B_PER_GPU, HEADS, D_V), dtype=torch.bfloat16).pin_memory() for _ in range(NBUF)]
    host_lse = [torch.empty((B_PER_GPU, HEADS), dtype=torch.float32).pin_memory() for _ in range(NBUF)]
    dq = [torch.empty_like(sets[0][0]) for _ in range(NBUF)]
    didx = [torch.empty_like(sets[0][1]) for _ in range(NBUF)]
    dout = [torch.empty((B_PER_GPU, HEADS, D_V), dtype=torch.bfloat16, device=device) for _ in range(NBUF)]
    s_in, s_run, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(NBUF)]
    ev_run = [torch.cuda.Event() for _ in range(NBUF)]
    ev_out = [torch.cuda.Event() for _ in range(NBUF)]
    keep = [None] * NBUF

    def e2e_step(i):
        b = i % NBUF
        hq, hidx = host_sets[i % NSETS]
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_run[b])          # the step that last read these input buffers has run
            dq[b].copy_(hq, non_blocking=True)
            didx[b].copy_(hidx, non_blocking=True)
            ev_in[b].record(s_in)
        with torch.cuda.stream(s_run):
            s_run.wait_event(ev_in[b])
            s_run.wait_event(ev_out[b])         # the previous result in this output buffer has been copied out
            o, lse = flash_ops.sparse_mla_decode_fwd(dq[b], pool, didx[b], SM_SCALE, out=dout[b])
            ev_run[b].record(s_run)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_run[b])
            host_out[b].copy_(o, non_blocking=True)
            host_lse[b].copy_(lse, non_blocking=True)
            lse.record_stream(s_out)
            ev_out[b].record(s_out)
        keep[b] = (o, lse)

    def time_pipeline(steps, warmup):
        for i in range(warmup):
            e2e_step(i)
        barrier_sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s_run)
        for i in range(steps):
            e2e_step(warmup + i)
        s_run.wait_stream(s_in)
        s_run.wait_stream(s_out)
        e1.record(s_run)
        barrier_sync()
        return e0.elapsed_time(e1) / 1e3

    barrier_sync()
    e2e_secs = time_pipeline(args.steps, args.warmup)
    t = torch.tensor([e2e_secs], device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_secs = float(t.item())
    clocks = sampler.stop() if rank == 0 else None

    # ---- the dominant kernel alone (attention): batches of back-to-back launches on the launching
    # stream, CUDA events around each batch, so that the host's launch latency is not counted ------
    T = B_PER_GPU
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    parts = pick_num_sm_parts(T, sms)
    lib, stream = _lib.load(), stream_ptr(device)
    pbs, pstride = kv_geometry(pool)
    out = torch.empty((T, HEADS, D_V), dtype=torch.bfloat16, device=device)
    lse = torch.empty((T, HEADS), dtype=torch.float32, device=device)
    st = status_buffer(device)

    def attention_launcher(nparts):
        """Returns (launch(i), kernels per step) for the attention kernel of a step with nparts partitions."""
        if nparts == T:   # nothing is split: the public op launches the attention kernel alone
            return (lambda i: lib.smla_prefill(ptr(sets[i % NSETS][0]), ptr(pool), ptr(sets[i % NSETS][1]), ptr(out), ptr(lse),
                                               None, T, HEADS, TOPK, SM_SCALE, pbs, pstride, None, None, 0, ptr(st), stream)), 1
        ws = scratch(device, T + nparts, HEADS, T, nparts)
        lib.smla_sched_meta(T, TOPK, 0, nparts, FIXED_OVERHEAD, None, None, ptr(ws["sched_meta"]), ptr(ws["num_splits"]), stream)
        return (lambda i: lib.smla_decode_splitkv(ptr(sets[i % NSETS][0]), ptr(pool), ptr(sets[i % NSETS][1]), ptr(ws["o_accum"]),
                                                  ptr(ws["lse_accum"]), ptr(out), ptr(lse), ptr(ws["sched_meta"]),
                                                  ptr(ws["num_splits"]), T, HEADS, TOPK, SM_SCALE, pbs, pstride, nparts,
                                                  None, None, 0, ptr(st), stream)), 3

    def time_batches(launch, batches=10, per_batch=20):
        for i in range(max(args.warmup, 3)):
            launch(i)
        torch.cuda.synchronize()
        ts = []
        for b in range(batches):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(per_batch):
                launch(b * per_batch + i)
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e-3 / per_batch)
        return statistics.mean(ts)

    attn_launch, launches_per_step = attention_launcher(parts)
    k_secs = time_batches(attn_launch)
    check_status(device)

    # ---- the split-KV form of the same step (scheduler + attention + combine over sms/2 partitions),
    # which the default policy does not pick at this batch size; reported beside the headline -------
    split_extra = None
    if rank == 0 and not args.no_extras:
        sp = max(sms // 2, 1)
        sgraphs = []
        with torch.cuda.stream(side):
            for q, idx in sets:
                for _ in range(2):
                    flash_ops.sparse_mla_decode_fwd(q, pool, idx, SM_SCALE, num_sm_parts=sp)
                side.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    o = flash_ops.sparse_mla_decode_fwd(q, pool, idx, SM_SCALE, num_sm_parts=sp)
                sgraphs.append((g, o))
        torch.cuda.synchronize()
        s_secs = time_events(lambda i: sgraphs[i % NSETS][0].replay(), min(args.steps, 500), max(args.warmup, 3), torch.cuda.synchronize)
        s_launch, _ = attention_launcher(sp)
        split_extra = {"num_sm_parts": sp, "us_per_step": s_secs / min(args.steps, 500) * 1e6,
                       "attention_kernel_us": time_batches(s_launch) * 1e6,
                       "timed": "scheduler + attention + combine, CUDA graph replay"}
        check_status(device)

    extras = {}
    if world > 1 and not args.no_extras:
        try:
            cp_extra = run_cp_extra(device, rank, world)
        except Exception as e:
            cp_extra = {"error": repr(e)}
    else:
        cp_extra = None
    if rank == 0 and not args.no_extras:
        try:
            extras = run_extras(device, bf16_peak)
        except Exception as e:  # the headline line must still print
            extras = {"error": repr(e)}
    if cp_extra is not None:
        extras["cp_decode"] = cp_extra
    if split_extra is not None:
        extras["split_kv_decode"] = split_extra
    cpu = cpu_baseline(pool, sets) if rank == 0 else None

    if rank == 0:
        total_bytes = bytes_step * world
        ms = secs / args.steps * 1e3
        line = {
            "metric": "sparse_mla_decode_algorithmic_hbm_throughput",
            "value": total_bytes * args.steps / secs / 1e9, "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "decode_us_per_step": ms * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "requests_per_gpu": B_PER_GPU, "sharding": "requests across GPUs, no collective",
                       "l2": f"inputs larger than L2: {NSETS} rotating (q, indices) sets gathering from a "
                             f"{pool.numel() / 1e9:.2f} GB pool",
                       "timed": ("attention kernel alone (one partition per request: nothing to schedule or combine)"
                                 if launches_per_step == 1 else "scheduler + attention + combine") + ", CUDA graph replay",
                       "num_sm_parts": parts},
            "e2e": {"value": total_bytes * args.steps / e2e_secs / 1e9, "unit": "GB/s",
                    "us_per_step": e2e_secs / args.steps * 1e6,
                    "h2d_bytes_per_step": int(dq[0].numel() * 2 + didx[0].numel() * 4),
                    "d2h_bytes_per_step": int(host_out[0].numel() * 2 + host_lse[0].numel() * 4),
                    "note": "paged KV cache is device-resident state; q and indices come from pinned host memory, output and LSE go "
                            "back, every step; copies and kernel of neighbouring steps overlap on three streams"},
            "gpu_launches": launches_per_step * args.steps,
            "roofline": {"bound": "hbm", "kernel": "attn_tc_kernel", "achieved": bytes_step / k_secs / 1e9, "peak": hbm_peak,
                         "unit": "GB/s", "frac": bytes_step / k_secs / 1e9 / hbm_peak, "peak_kind": f"of {peak_kind}",
                         "kernel_us": k_secs * 1e6, "traffic": NCU_TRAFFIC_BYTES,
                         "frac_of_8TBs_nominal": bytes_step / k_secs / 8e12},
            "cpu_baseline": cpu, "clocks": clocks, "extras": extras,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_cp_extra(device, rank, world):
    """Context-parallel long-context decode: 16 requests, 131072-token context sharded across the
    ranks, top-k 2048 uniform over the whole context.  Timed per step on the device, max over ranks:
    index partition + scheduler + local split-KV decode + local merge + one NCCL all-gather + final merge.
    (The indexer that would produce the indices is not part of this timing.)"""
    import torch.distributed as dist
    from sparse_mla_sm120_b200 import cp, indexer
    b, ctx = 16, 131072
    lo, hi = cp.shard_context(ctx, rank, world)
    rows = hi - lo
    g = torch.Generator(device=device).manual_seed(99 + rank)
    pools = []
    for _ in range(b):   # one contiguous shard per request; rows of request i live at [i*rows, (i+1)*rows)
        pools.append(indexer.pack_kv_cache(torch.randn((rows, D_QK), device=device, generator=g).to(torch.bfloat16)))
    kv_local = torch.cat(pools).view(-1, BLOCK, 1, ROW)
    gi = torch.Generator(device=device).manual_seed(7)      # same indices on every rank
    q = (torch.randn((b, HEADS, D_QK), device=device, generator=gi) * 0.5).to(torch.bfloat16)
    pos = torch.stack([torch.randperm(ctx, device=device, generator=gi)[:TOPK] for _ in range(b)])
    # global row number = request * ctx + position; the local pool stores request i's shard at i*rows
    in_shard = (pos >= lo) & (pos < hi)
    local = torch.where(in_shard, pos - lo + torch.arange(b, device=device).view(-1, 1) * rows, torch.full_like(pos, -1)).to(torch.int32)

    def step():
        # entries outside the shard are already -1; compaction and the local length come from the partition kernel
        li, ln = cp.partition_indices(local, 0, b * rows)
        packed, o_all, l_all = cp._gather_buffers(device, world, b, HEADS)
        cp.decode_partial(q, kv_local, li, ln, SM_SCALE, o_all[rank], l_all[rank])
        dist.all_gather_into_tensor(packed, packed[rank])       # partials and LSEs of a rank are adjacent
        return cp.combine_parts(o_all, l_all)

    for _ in range(5):
        step()
    dist.barrier(); torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n = 50
    e0.record()
    for _ in range(n):
        step()
    e1.record(); torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / n * 1e3], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    res = {"workload": "b=16, h=128, topk=2048, 131072-token context sharded over the ranks", "us_per_step": float(t.item()),
           "timed": "partition + scheduler + local decode + local merge + one NCCL all-gather + final merge (eager launches)",
           "exchange_bytes_per_rank": b * HEADS * (D_V + 1) * 4}
    # the same step with the indexer in front: 16 tokens of ONE sequence whose 131072-token context
    # (attention cache and indexer keys) is sharded; local logits + local top-k + candidate all-gather
    # + global top-k, then the context-parallel decode
    del kv_local, pools
    kv_one = indexer.pack_kv_cache(torch.randn((rows, D_QK), device=device, generator=g).to(torch.bfloat16)).view(-1, BLOCK, 1, ROW)
    hh = 64
    qi = torch.randn((b, hh, 128), device=device, generator=gi).to(torch.float8_e4m3fn)
    w = torch.randn((b, hh), device=device, generator=gi) * 0.1
    kf = torch.randn((rows, 128), device=device, generator=g)
    k_scale = kf.abs().amax(dim=1) / 448.0
    ki = (kf / k_scale.unsqueeze(1)).to(torch.float8_e4m3fn)
    ks = torch.zeros(b, dtype=torch.int32, device=device)
    ke = (ctx - b + 1 + torch.arange(b, device=device)).to(torch.int32)

    def step_indexed():
        return cp.sparse_mla_indexed_decode_cp_fwd(q, kv_one, qi, ki, k_scale, w, ks, ke, SM_SCALE, lo, hi, topk=TOPK)

    for _ in range(5):
        step_indexed()
    dist.barrier(); torch.cuda.synchronize()
    e0.record()
    for _ in range(n):
        step_indexed()
    e1.record(); torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / n * 1e3], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    res["us_per_step_with_indexer"] = float(t.item())
    res["indexer_exchange_bytes_per_rank"] = b * TOPK * 8
    return res


def run_extras(device, bf16_peak):
    """Secondary measurements of the other kernels on the path (not part of the timed step)."""
    from sparse_mla_sm120_b200 import flash_ops, indexer
    out = {}
    g = torch.Generator(device=device).manual_seed(7)
    # prefill: s_q 4096, H 128, topk 2048 over 8192 rows, causal top-k
    s_q, rows = 4096, 8192
    kv = indexer.pack_kv_cache(torch.randn((rows, D_QK), device=device, generator=g).to(torch.bfloat16)).view(rows // 64, 64, 1, ROW)
    q = torch.randn((s_q, HEADS, D_QK), device=device, generator=g).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(4096 + i, device=device, generator=g)[:TOPK] for i in range(s_q)]).to(torch.int32)
    for _ in range(2):
        flash_ops.sparse_mla_prefill_fwd(q, kv, idx, SM_SCALE)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n = 5
    e0.record()
    for _ in range(n):
        flash_ops.sparse_mla_prefill_fwd(q, kv, idx, SM_SCALE)
    e1.record(); torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / n
    flops = 2.0 * s_q * HEADS * TOPK * (D_QK + D_V)
    out["prefill"] = {"workload": "s_q=4096, h=128, topk=2048, KV 8192 rows", "ms": ms,
                      "tflops": flops / ms / 1e9, "frac_of_bf16_peak": flops / ms / 1e9 / bf16_peak}
    del q, idx, kv
    # indexer: q e4m3 [4096, 64, 128], k e4m3 [65536, 128], ke = 61440 + i, then top-2048 per row
    s_q, s_k, hh = 4096, 65536, 64
    qi = torch.randn((s_q, hh, 128), device=device, generator=g).to(torch.float8_e4m3fn)
    kf = torch.randn((s_k, 128), device=device, generator=g)
    k_scale = kf.abs().amax(dim=1) / 448.0
    ki = (kf / k_scale.unsqueeze(1)).to(torch.float8_e4m3fn)
    w = torch.randn((s_q, hh), device=device, generator=g) * 0.1
    ks = torch.zeros(s_q, dtype=torch.int32, device=device)
    ke = (61440 + torch.arange(s_q, device=device)).to(torch.int32)
    logits = torch.empty((s_q, s_k), dtype=torch.float32, device=device)
    for name, fn in (("mqa_logits", lambda: indexer.fp8_mqa_logits(qi, ki, k_scale, w, ks, ke, out=logits)),
                     ("topk", lambda: indexer.topk_indices(logits, ks, ke, TOPK))):
        fn(); fn()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(3):
            fn()
        e1.record(); torch.cuda.synchronize()
        out[name] = {"ms": e0.elapsed_time(e1) / 3}
    pairs = float(ke.double().sum())
    fl = 2.0 * hh * 128 * pairs
    out["mqa_logits"].update({"workload": "s_q=4096, 64 heads, d=128, s_k=65536, ke=61440+i", "tflops": fl / out["mqa_logits"]["ms"] / 1e9,
                              "frac_of_fp8_peak(2x measured bf16)": fl / out["mqa_logits"]["ms"] / 1e9 / (2 * bf16_peak),
                              "write_gbs": s_q * s_k * 4 / out["mqa_logits"]["ms"] / 1e6})
    out["topk"].update({"workload": "top-2048 of each of 4096 rows of 65536 fp32", "read_gbs": s_q * s_k * 4 / out["topk"]["ms"] / 1e6})
    del logits, qi, ki
    out["indexed_decode"] = run_indexed_decode_extra(device, g)
    return out


def run_indexed_decode_extra(device, g):
    """Indexer -> top-k -> sparse decode as one call: 16 tokens of one long sequence, 131072-token
    context, 64 indexer heads, top-2048, 128 attention heads.  Eager launches and CUDA-graph replay."""
    from sparse_mla_sm120_b200 import indexer, pipeline
    t, ctx, hh = 16, 131072, 64
    kv = indexer.pack_kv_cache(torch.randn((ctx, D_QK), device=device, generator=g).to(torch.bfloat16)).view(ctx // BLOCK, BLOCK, 1, ROW)
    q = (torch.randn((t, HEADS, D_QK), device=device, generator=g) * 0.5).to(torch.bfloat16)
    qi = torch.randn((t, hh, 128), device=device, generator=g).to(torch.float8_e4m3fn)
    kf = torch.randn((ctx, 128), device=device, generator=g)
    k_scale = kf.abs().amax(dim=1) / 448.0
    ki = (kf / k_scale.unsqueeze(1)).to(torch.float8_e4m3fn)
    w = torch.randn((t, hh), device=device, generator=g) * 0.1
    ks = torch.zeros(t, dtype=torch.int32, device=device)
    ke = (ctx - t + 1 + torch.arange(t, device=device)).to(torch.int32)

    def step():
        return pipeline.sparse_mla_indexed_decode_fwd(q, kv, qi, ki, k_scale, w, ks, ke, SM_SCALE, topk=TOPK)

    def timed(fn, n=50):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record(); torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n * 1e3

    res = {"workload": "16 tokens, 131072-token context, 64 indexer heads, top-2048, h=128",
           "timed": "fp8 logits + top-k + scheduler + split-KV decode + combine", "us_per_step_eager": timed(step)}
    try:
        graphed = pipeline.GraphedIndexedDecode(kv, ki, k_scale, t, HEADS, hh, SM_SCALE, topk=TOPK)
        graphed(q, qi, w, ks, ke)                      # inputs into the static buffers
        res["us_per_step_graph"] = timed(graphed.replay)
    except Exception as e:       # capture is an optimisation of the launch path, not a requirement
        res["us_per_step_graph"] = None
        res["graph_error"] = repr(e)
    return res


def cpu_baseline(pool, sets, n_req: int = 16):
    """The reference's CPU PyTorch path (oracle port) on a bounded sample: n_req of the 64
    requests of one step, all host threads."""
    from oracle import sparse_mla_oracle as orc
    q, idx = sets[0]
    rows = pool.view(-1, ROW)[idx[:n_req].reshape(-1).long()].cpu()
    qc = q[:n_req].cpu().unsqueeze(1)
    local_idx = torch.arange(n_req * TOPK, dtype=torch.int32).view(n_req, 1, TOPK)
    torch.set_num_threads(os.cpu_count())
    best = None
    for _ in range(5):
        t0 = time.perf_counter()
        deq = orc.dequantize_kv_v32(rows.view(-1, 64, 1, ROW))
        orc.ref_sparse_attn(qc, deq, local_idx, SM_SCALE, D_V)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return {"value": algorithmic_bytes(n_req, TOPK) / best / 1e9, "unit": "GB/s", "cores": os.cpu_count(),
            "kind": "port", "sample": f"{n_req} of {B_PER_GPU} requests of one step (dequantise gathered rows + fp32 attention), best of 5",
            "seconds": best}


def run_reference(args):
    """The reference's own CPU implementation of the path (its PyTorch reference functions,
    restated in oracle/), timed on the host cores on a bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import sparse_mla_oracle as orc
    torch.set_num_threads(os.cpu_count())
    n_req = 16
    g = torch.Generator().manual_seed(1234)
    kv = torch.randn(n_req * TOPK // 64, 64, 1, D_QK, generator=g).to(torch.bfloat16)
    packed = orc.quantize_kv_v32(kv)
    q = (torch.randn(n_req, 1, HEADS, D_QK, generator=g) * 0.5).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(n_req * TOPK, generator=g)[:TOPK] for _ in range(n_req)]).view(n_req, 1, TOPK).int()

    def step():
        deq = orc.dequantize_kv_v32(packed)
        orc.ref_sparse_attn(q, deq, idx, SM_SCALE, D_V)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    secs = time.perf_counter() - t0
    value = algorithmic_bytes(n_req, TOPK) * args.steps / secs / 1e9
    sample = f"{n_req} of {B_PER_GPU} requests per step on the CPU (the step's unit work scales linearly with requests)"
    print(json.dumps({
        "impl": "reference", "metric": "sparse_mla_decode_algorithmic_hbm_throughput", "value": value, "unit": "GB/s",
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": secs / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": os.cpu_count(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }), flush=True)


def run_small_case(name):
    """Small instances of the secondary kernels, sized for a profiler capture (a few hundred MB on the
    device, kernels of well under a millisecond); prints one informative JSON line, no headline metric."""
    from sparse_mla_sm120_b200 import flash_ops, indexer
    device = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    g = torch.Generator(device=device).manual_seed(11)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if name == "prefill":
        s_q, rows = 512, 8192
        kv = indexer.pack_kv_cache(torch.randn((rows, D_QK), device=device, generator=g).to(torch.bfloat16)).view(rows // 64, 64, 1, ROW)
        q = torch.randn((s_q, HEADS, D_QK), device=device, generator=g).to(torch.bfloat16)
        idx = torch.stack([torch.randperm(4096 + i, device=device, generator=g)[:TOPK] for i in range(s_q)]).to(torch.int32)
        fn = lambda: flash_ops.sparse_mla_prefill_fwd(q, kv, idx, SM_SCALE)
        work = {"flop": 2.0 * s_q * HEADS * TOPK * (D_QK + D_V)}
        desc = f"prefill s_q={s_q}, h=128, topk=2048, KV {rows} rows"
    else:
        s_q, s_k, hh = 512, 65536, 64
        qi = torch.randn((s_q, hh, 128), device=device, generator=g).to(torch.float8_e4m3fn)
        kf = torch.randn((s_k, 128), device=device, generator=g)
        k_scale = kf.abs().amax(dim=1) / 448.0
        ki = (kf / k_scale.unsqueeze(1)).to(torch.float8_e4m3fn)
        w = torch.randn((s_q, hh), device=device, generator=g) * 0.1
        ks = torch.zeros(s_q, dtype=torch.int32, device=device)
        ke = (61440 + torch.arange(s_q, device=device)).to(torch.int32)
        logits = torch.empty((s_q, s_k), dtype=torch.float32, device=device)

        def fn():
            indexer.fp8_mqa_logits(qi, ki, k_scale, w, ks, ke, out=logits)
            indexer.topk_indices(logits, ks, ke, TOPK)
        work = {"flop": 2.0 * s_q * hh * 128 * s_k}
        desc = f"indexer s_q={s_q}, 64 heads, d=128, s_k={s_k}, then top-2048"
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(3):
        fn()
    e1.record(); torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 3
    print(json.dumps({"case": name, "workload": desc, "ms": ms, "tflops": work["flop"] / ms / 1e9}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--case", default=None, choices=["prefill", "indexer"],
                    help="run a small instance of a secondary kernel (for profiler captures) instead of the benchmark")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.case is not None:
        run_small_case(args.case)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
