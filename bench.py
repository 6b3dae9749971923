#!/usr/bin/env python
"""Benchmark of the sparse-MLA hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-extras]

One step = one call of the public decode op (``sparse_mla_decode_fwd``) over one batch of the
DeepSeek-V3.2-shape decode configuration: 64 requests per GPU, 128 query heads, top-k 2048,
per-request KV length uniform in [4096, 32768] in a paged (block 64) pool of packed 656-byte
FP8 rows.  At this batch size the op's policy gives every request its own partition, so the op
is ONE launch, the attention kernel (nothing to schedule or to combine); the split-KV form of the
same step (scheduler + attention + combine) is timed beside it as ``extras.split_kv_decode``.
All inputs are synthetic and seeded.  With N > 1 every rank serves its own 64 requests (decode
batches shard by sequence, nothing is exchanged), so scaling is weak.

Printed line: ``value`` is the algorithmic HBM traffic of the whole job divided by the step time
with inputs resident on the device (CUDA-graph replay of the public op); ``e2e`` is the same
through the public op with q / indices coming from pinned host memory and the output copied back
every step (the paged KV cache is device-resident state, as in any serving engine).
``roofline`` is the attention kernel alone, timed live with CUDA events.
``--impl reference`` times the reference's CPU PyTorch path (restated in oracle/) on the host
cores, on the same seeded sample of the step as this arm's ``cpu_baseline``.
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
# DRAM bytes of one launch of the attention kernel on this workload's shape, from one ncu capture
# (dram__bytes_read.sum + dram__bytes_write.sum); the capture's summary is kept with the other profiles.
NCU_TRAFFIC_BYTES = 90_347_008
CPU_SAMPLE_REQUESTS = 64   # requests of one step that the CPU legs compute: the whole step (about 0.13 s on 16 host threads)


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
            extras = run_extras(device, hbm_peak, bf16_peak, peak_kind)
        except Exception as e:  # the headline line must still print
            extras = {"error": repr(e)}
    if cp_extra is not None:
        extras["cp_decode"] = cp_extra
    if split_extra is not None:
        extras["split_kv_decode"] = split_extra
    cpu = cpu_baseline() if rank == 0 else None

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
            "roofline": {"bound": "hbm", "kernel": "attn_pair_kernel", "achieved": bytes_step / k_secs / 1e9, "peak": hbm_peak,
                         "unit": "GB/s", "frac": bytes_step / k_secs / 1e9 / hbm_peak, "peak_kind": f"of {peak_kind}",
                         "kernel_us": k_secs * 1e6, "traffic": NCU_TRAFFIC_BYTES,
                         "frac_of_8TBs_nominal": bytes_step / k_secs / 8e12},
            "cpu_baseline": cpu, "clocks": clocks, "extras": extras,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        # Every rank leaves together and at once: the line is out, and tearing down a communicator that CUDA graphs
        # have captured collectives of has been seen to wait for ever.
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(0)


def run_cp_extra(device, rank, world):
    """Context-parallel long-context decode: 16 requests, 131072-token context per request sharded across the
    ranks, top-k 2048 uniform over the whole context.  Timed per step on the device, max over ranks: index
    partition + scheduler + local split-KV decode + local merge cut into head slices + all-to-all by head slice +
    merge of H/G heads + all-gather of the bf16 result + reassembly.  Eager launches and the whole step
    captured into one CUDA graph (collectives included).  ``speedup_vs_1gpu`` compares with the same 16
    requests decoded on ONE GPU that holds the whole context (measured on rank 0).
    (The indexer that would produce the indices is not part of this timing.)"""
    import torch.distributed as dist
    from sparse_mla_sm120_b200 import cp, flash_ops, indexer
    b, ctx = 16, 131072
    lo, hi = cp.shard_context(ctx, rank, world)
    rows = hi - lo
    assert rows * world == ctx
    g = torch.Generator(device=device).manual_seed(99 + rank)
    pools = []
    for _ in range(b):   # one contiguous shard per request; rows of request i live at [i*rows, (i+1)*rows) of the local pool
        pools.append(indexer.pack_kv_cache(torch.randn((rows, D_QK), device=device, generator=g).to(torch.bfloat16)))
    kv_local = torch.cat(pools).view(-1, BLOCK, 1, ROW)
    del pools
    gi = torch.Generator(device=device).manual_seed(7)      # same indices on every rank
    q = (torch.randn((b, HEADS, D_QK), device=device, generator=gi) * 0.5).to(torch.bfloat16)
    pos = torch.stack([torch.randperm(ctx, device=device, generator=gi)[:TOPK] for _ in range(b)])
    # One global row numbering in which every rank's rows are one range: rank g holds [g*b*rows, (g+1)*b*rows),
    # request i's position p lives at (p // rows) * b * rows + i * rows + p % rows.
    req = torch.arange(b, device=device).view(-1, 1)
    indices = ((pos // rows) * (b * rows) + req * rows + pos % rows).to(torch.int32)
    s_lo, s_hi = rank * b * rows, (rank + 1) * b * rows

    def timed(fn, n=50):
        for _ in range(5):
            fn()
        dist.barrier(); torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record(); torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / n * 1e3], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    hs = HEADS // world
    res = {"workload": "b=16, h=128, topk=2048, 131072-token context per request sharded over the ranks",
           "timed": "partition + scheduler + local decode + local merge + exchange (see `exchange`) + final merge",
           "us_per_step": timed(lambda: cp.sparse_mla_decode_cp_fwd(q, kv_local, indices, SM_SCALE, s_lo, s_hi)),
           }
    sliced = HEADS % world == 0 and (world - 1) * b * HEADS * 2052 > cp.ALL_GATHER_LIMIT_BYTES
    res["exchange"] = ("all-to-all by head slice + all-gather of the bf16 result" if sliced
                       else "one all-gather of the fp32 partials (below the traffic limit)")
    res["exchange_bytes_in_per_rank"] = ((world - 1) * b * hs * ((D_V + 1) * 4 + D_V * 2 + 4) if sliced
                                         else (world - 1) * b * HEADS * (D_V + 1) * 4)
    try:
        graphed = cp.GraphedCpDecode(kv_local, b, HEADS, TOPK, SM_SCALE, s_lo, s_hi)
        graphed(q, indices)
        res["us_per_step_graph"] = timed(graphed.replay)
        res["graph_captured"] = graphed.graph is not None
        graphed.close()          # the graph references the communicator: drop it before the process group goes
        del graphed
    except Exception as e:       # noqa: BLE001 - capture is an optimisation of the launch path, not a requirement
        res["us_per_step_graph"] = None
        res["graph_error"] = repr(e)
    # the same 16 requests on ONE GPU holding all 16 x 131072 rows (1.4 GB), on rank 0
    one = None
    if rank == 0:
        full = torch.empty((b * ctx // BLOCK, BLOCK, 1, ROW), dtype=torch.uint8, device=device)
        g1 = torch.Generator(device=device).manual_seed(5)
        step_rows = 1 << 18
        for r0 in range(0, b * ctx, step_rows):
            full.view(-1, ROW)[r0:r0 + step_rows] = indexer.pack_kv_cache(
                torch.randn((step_rows, D_QK), device=device, generator=g1).to(torch.bfloat16))
        idx1 = (pos + req * ctx).to(torch.int32)
        for _ in range(3):
            flash_ops.sparse_mla_decode_fwd(q, full, idx1, SM_SCALE)
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            flash_ops.sparse_mla_decode_fwd(q, full, idx1, SM_SCALE); side.synchronize()
            with torch.cuda.graph(gr, stream=side):
                flash_ops.sparse_mla_decode_fwd(q, full, idx1, SM_SCALE)
        torch.cuda.synchronize()
        one = _time_cuda(gr.replay, 100, warm=5) * 1e3
        del full, gr
    t1 = torch.tensor([one if one is not None else 0.0], device=device)
    dist.broadcast(t1, 0)
    res["one_gpu_us_per_step"] = float(t1.item())
    best = min(x for x in (res["us_per_step"], res.get("us_per_step_graph")) if x)
    res["speedup_vs_1gpu"] = float(t1.item()) / best
    # the same step with the indexer in front: 16 tokens of ONE sequence whose 131072-token context
    # (attention cache and indexer keys) is sharded; local logits + local top-k + candidate all-gather
    # + global top-k, then the context-parallel decode
    del kv_local
    kv_one = indexer.pack_kv_cache(torch.randn((rows, D_QK), device=device, generator=g).to(torch.bfloat16)).view(-1, BLOCK, 1, ROW)
    hh = 64
    qi = torch.randn((b, hh, 128), device=device, generator=gi).to(torch.float8_e4m3fn)
    w = torch.randn((b, hh), device=device, generator=gi) * 0.1
    kf = torch.randn((rows, 128), device=device, generator=g)
    k_scale = kf.abs().amax(dim=1) / 448.0
    ki = (kf / k_scale.unsqueeze(1)).to(torch.float8_e4m3fn)
    ks = torch.zeros(b, dtype=torch.int32, device=device)
    ke = (ctx - b + 1 + torch.arange(b, device=device)).to(torch.int32)
    res["us_per_step_with_indexer"] = timed(
        lambda: cp.sparse_mla_indexed_decode_cp_fwd(q, kv_one, qi, ki, k_scale, w, ks, ke, SM_SCALE, lo, hi, topk=TOPK))
    res["indexer_exchange_bytes_per_rank"] = b * TOPK * 8
    try:
        gi2 = cp.GraphedIndexedCpDecode(kv_one, ki, k_scale, b, HEADS, hh, SM_SCALE, lo, hi, topk=TOPK)
        gi2(q, qi, w, ks, ke)
        res["us_per_step_with_indexer_graph"] = timed(gi2.replay)
        res["indexer_graph_captured"] = gi2.graph is not None
        gi2.close()
        del gi2
    except Exception as e:       # noqa: BLE001
        res["us_per_step_with_indexer_graph"] = None
        res["indexer_graph_error"] = repr(e)
    return res


def _time_cuda(fn, n, warm=2):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        fn()
    e1.record(); torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n          # ms


def _cpu_attention_slice(q, kv_packed, idx, tokens):
    """The reference's CPU path (oracle port) on the first `tokens` query tokens of a GPU case, best of 3."""
    from oracle import sparse_mla_oracle as orc
    torch.set_num_threads(os.cpu_count())
    qc, ic = q[:tokens].cpu().unsqueeze(1), idx[:tokens].cpu().unsqueeze(1)
    packed = kv_packed.cpu()
    best = None
    for _ in range(3):
        t0 = time.perf_counter()
        orc.ref_sparse_attn(qc, orc.dequantize_kv_v32(packed), ic, SM_SCALE, D_V)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return best


def run_extras(device, hbm_peak, bf16_peak, peak_kind):
    """Secondary measurements of the other kernels and shapes on the path (not part of the timed step)."""
    from sparse_mla_sm120_b200 import flash_ops, indexer
    out = {}
    g = torch.Generator(device=device).manual_seed(7)
    # ---- prefill: s_q 4096, H 128, topk 2048 over 8192 rows, causal top-k (token i sees 4096 + i keys)
    s_q, rows = 4096, 8192
    kv = indexer.pack_kv_cache(torch.randn((rows, D_QK), device=device, generator=g).to(torch.bfloat16)).view(rows // 64, 64, 1, ROW)
    q = torch.randn((s_q, HEADS, D_QK), device=device, generator=g).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(4096 + i, device=device, generator=g)[:TOPK] for i in range(s_q)]).to(torch.int32)
    ms = _time_cuda(lambda: flash_ops.sparse_mla_prefill_fwd(q, kv, idx, SM_SCALE), 5)
    flops = 2.0 * s_q * HEADS * TOPK * (D_QK + D_V)
    cpu_tokens = 8
    cpu_s = _cpu_attention_slice(q, kv, idx, cpu_tokens)
    out["prefill"] = {
        "workload": "s_q=4096, h=128, topk=2048, KV 8192 rows, causal top-k", "ms": ms, "tflops": flops / ms / 1e9,
        "roofline": {"bound": "tensor", "kernel": "attn_pair_kernel", "achieved": flops / ms / 1e9, "peak": bf16_peak, "unit": "TFLOP/s",
                     "frac": flops / ms / 1e9 / bf16_peak, "peak_kind": f"of {peak_kind} (dense BF16; the kernel's MMAs are FP8)",
                     "traffic": None},
        "cpu_baseline": {"value": flops * cpu_tokens / s_q / cpu_s / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port",
                         "sample": f"first {cpu_tokens} of {s_q} query tokens, best of 3", "seconds": cpu_s}}
    # ---- the same prefill with the start of a sequence in it: token i sees i + 1 keys, and its index list is
    # padded with -1 once they run out (tokens 0..2047), as a serving engine hands it over
    idx_c = torch.full((s_q, TOPK), -1, dtype=torch.int32, device=device)
    for i in range(s_q):
        n = min(i + 1, TOPK)
        idx_c[i, :n] = torch.randperm(i + 1, device=device, generator=g)[:n].to(torch.int32)
    ms_c = _time_cuda(lambda: flash_ops.sparse_mla_prefill_fwd(q, kv, idx_c, SM_SCALE), 5)
    valid = float((idx_c >= 0).sum())
    fl_c = 2.0 * HEADS * valid * (D_QK + D_V)
    out["prefill_causal_padded"] = {
        "workload": "s_q=4096 from the start of a sequence: token i has min(i+1, 2048) entries, the rest of its list is -1",
        "ms": ms_c, "valid_entries": valid, "tflops": fl_c / ms_c / 1e9,
        "roofline": {"bound": "tensor", "kernel": "attn_pair_kernel", "achieved": fl_c / ms_c / 1e9, "peak": bf16_peak, "unit": "TFLOP/s",
                     "frac": fl_c / ms_c / 1e9 / bf16_peak, "peak_kind": f"of {peak_kind} (dense BF16; flops of valid entries only)",
                     "traffic": None}}
    del q, idx, idx_c, kv
    # ---- decode with two query tokens per request (multi-token prediction): the workload of the headline
    # with s_q = 2, i.e. 128 query tokens, each with its own index list
    try:
        pool, sets, _ = build_workload(device, 4321, B_PER_GPU)
        q2 = (torch.randn((B_PER_GPU, 2, HEADS, D_QK), device=device, generator=g) * 0.5).to(torch.bfloat16)
        i2 = torch.stack([sets[0][1], sets[1][1]], dim=1).contiguous()               # [b, 2, topk]
        from sparse_mla_sm120_b200 import interface
        meta, _ = interface.get_mla_metadata()
        run2 = lambda: interface.flash_mla_with_kvcache(q2, pool, None, None, D_V, meta, None, SM_SCALE, False, True, indices=i2)
        run2(); torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            run2(); side.synchronize()
            with torch.cuda.graph(gr, stream=side):
                run2()
        torch.cuda.synchronize()
        ms2 = _time_cuda(gr.replay, 200, warm=5)
        by2 = algorithmic_bytes(2 * B_PER_GPU, TOPK)
        out["decode_mtp_sq2"] = {
            "workload": "the headline's decode with s_q=2: 64 requests x 2 query tokens, h=128, topk=2048, through flash_mla_with_kvcache",
            "us_per_step": ms2 * 1e3, "num_sm_parts": meta.num_sm_parts,
            "roofline": {"bound": "hbm", "kernel": "attn_pair_kernel", "achieved": by2 / ms2 / 1e6, "peak": hbm_peak, "unit": "GB/s",
                         "frac": by2 / ms2 / 1e6 / hbm_peak, "peak_kind": f"of {peak_kind}", "traffic": None,
                         "note": "whole step (CUDA graph replay), algorithmic bytes count each token's gathered rows"}}
        # ---- small decode batches of the same shape (the split-KV path: scheduler + attention + combine as
        # dependent launches), CUDA-graph replay
        small = {}
        for bsz in (1, 8, 16, 32, 48):
            qs_, is_ = sets[0][0][:bsz].contiguous(), sets[0][1][:bsz].contiguous()
            runb = lambda: flash_ops.sparse_mla_decode_fwd(qs_, pool, is_, SM_SCALE)
            runb(); torch.cuda.synchronize()
            gb = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                runb(); side.synchronize()
                with torch.cuda.graph(gb, stream=side):
                    runb()
            torch.cuda.synchronize()
            us = _time_cuda(gb.replay, 200, warm=5) * 1e3
            small[f"b{bsz}"] = {"us_per_step": us, "gbs": algorithmic_bytes(bsz, TOPK) / us / 1e3}
            del gb
        out["decode_small_batches"] = {"workload": "the headline's decode shape at 1, 8, 16, 32 and 48 requests (rows of the first input set); "
                                                   "the op's own split policy: k equal partitions per request without a scheduler launch up to 37 requests, unsplit beyond",
                                       **small}
        del pool, sets, q2, i2
    except Exception as e:           # noqa: BLE001 - a secondary measurement must not take the others down
        out["decode_mtp_sq2"] = {"error": repr(e)}
    # ---- the headline's decode shape over the second cache layout (MODEL1: 584 bytes per token, 448 e4m3 + 64 bf16
    # RoPE + 7 UE8M0 scales in the page footer; q is 512 wide), alone and with a second cache of 512 more entries
    try:
        pages, blk = 4096, 64                                   # 262144 tokens, 153 MB: larger than L2
        def m1_pool(npages):
            nope = (torch.randn((npages * blk, 448), device=device, generator=g) * 60).clamp(-448, 448).to(torch.float8_e4m3fn)
            rope = torch.randn((npages * blk, 64), device=device, generator=g).to(torch.bfloat16)
            data = torch.cat([nope.view(torch.uint8), rope.view(torch.uint8)], dim=1).view(npages, blk * 576)
            footer = torch.full((npages, blk, 8), 120, dtype=torch.uint8, device=device)   # 2^-7 for every block of 64 values
            footer[..., :7] += torch.randint(0, 3, (npages, blk, 7), device=device, generator=g, dtype=torch.uint8)
            footer[..., 7] = 0
            return torch.cat([data, footer.view(npages, blk * 8)], dim=1).view(npages, blk, 1, 584)
        pool1 = m1_pool(pages)
        qm = (torch.randn((B_PER_GPU, HEADS, 512), device=device, generator=g) * 0.5).to(torch.bfloat16)
        im = torch.stack([torch.randperm(pages * blk, device=device, generator=g)[:TOPK] for _ in range(B_PER_GPU)]).to(torch.int32)
        epool = m1_pool(256)
        ie = torch.stack([torch.randperm(256 * blk, device=device, generator=g)[:512] for _ in range(B_PER_GPU)]).to(torch.int32)
        side = torch.cuda.Stream()
        res = {}
        for name, kw, entries in (("main_cache_only", {}, TOPK),
                                  ("with_extra_cache_512", {"extra_k_cache": epool, "extra_indices": ie, "extra_topk": 512}, TOPK + 512)):
            runm = lambda: flash_ops.sparse_mla_decode_fwd(qm, pool1, im, 512 ** -0.5, impl=2, **kw)   # 2 = the tensor-core kernel
            runm(); torch.cuda.synchronize()
            gm = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                runm(); side.synchronize()
                with torch.cuda.graph(gm, stream=side):
                    runm()
            torch.cuda.synchronize()
            us = _time_cuda(gm.replay, 200, warm=5) * 1e3
            bym = B_PER_GPU * (entries * 584 + HEADS * 512 * 2 + HEADS * D_V * 2 + entries * 4 + HEADS * 4)
            res[name] = {"us_per_step": us, "entries_per_request": entries,
                         "roofline": {"bound": "hbm", "kernel": "attn_pair_kernel", "achieved": bym / us / 1e3, "peak": hbm_peak,
                                      "unit": "GB/s", "frac": bym / us / 1e3 / hbm_peak, "peak_kind": f"of {peak_kind}", "traffic": None}}
            del gm
        exact_ms = _time_cuda(lambda: flash_ops.sparse_mla_decode_fwd(qm, pool1, im, 512 ** -0.5, impl=1), 3, warm=1)
        out["decode_model1"] = {"workload": "64 requests, h=128, topk=2048 over a MODEL1 cache (584 bytes per token, q 512 wide), "
                                            "262144-token pool; CUDA graph replay of the whole step on the tensor-core kernel "
                                            "(impl=IMPL_TC; the default for this layout is the exact fp32 kernel)",
                                "exact_fp32_kernel_us_per_step": exact_ms * 1e3, **res}
        # prefill of the C3 shape over the same layout: 4096 query tokens, causal top-k over 8192 rows
        pool_p = m1_pool(128)
        qp = torch.randn((4096, HEADS, 512), device=device, generator=g).to(torch.bfloat16)
        ip = torch.stack([torch.randperm(4096 + i, device=device, generator=g)[:TOPK] for i in range(4096)]).to(torch.int32)
        ms_p = _time_cuda(lambda: flash_ops.sparse_mla_prefill_fwd(qp, pool_p, ip, 512 ** -0.5, impl=2), 5)
        fl_p = 2.0 * 4096 * HEADS * TOPK * (512 + D_V)
        out["prefill_model1"] = {
            "workload": "s_q=4096, h=128, topk=2048 over a MODEL1 cache of 8192 rows, causal top-k; tensor-core kernel (impl=IMPL_TC)",
            "ms": ms_p, "tflops": fl_p / ms_p / 1e9,
            "roofline": {"bound": "tensor", "kernel": "attn_pair_kernel", "achieved": fl_p / ms_p / 1e9, "peak": bf16_peak,
                         "unit": "TFLOP/s", "frac": fl_p / ms_p / 1e9 / bf16_peak, "peak_kind": f"of {peak_kind} (dense BF16)",
                         "traffic": None}}
        del pool1, epool, qm, im, ie, pool_p, qp, ip
    except Exception as e:           # noqa: BLE001
        out["decode_model1"] = {"error": repr(e)}
    # ---- indexer: q e4m3 [4096, 64, 128], k e4m3 [65536, 128], ke = 61440 + i, then top-2048 per row
    s_q, s_k, hh = 4096, 65536, 64
    qi = torch.randn((s_q, hh, 128), device=device, generator=g).to(torch.float8_e4m3fn)
    kf = torch.randn((s_k, 128), device=device, generator=g)
    k_scale = kf.abs().amax(dim=1) / 448.0
    ki = (kf / k_scale.unsqueeze(1)).to(torch.float8_e4m3fn)
    w = torch.randn((s_q, hh), device=device, generator=g) * 0.1
    ks = torch.zeros(s_q, dtype=torch.int32, device=device)
    ke = (61440 + torch.arange(s_q, device=device)).to(torch.int32)
    logits = torch.empty((s_q, s_k), dtype=torch.float32, device=device)
    out["mqa_logits"] = {"ms": _time_cuda(lambda: indexer.fp8_mqa_logits(qi, ki, k_scale, w, ks, ke, out=logits), 3)}
    out["topk"] = {"ms": _time_cuda(lambda: indexer.topk_indices(logits, ks, ke, TOPK), 3)}
    pairs = float(ke.double().sum())
    fl = 2.0 * hh * 128 * pairs
    mq = out["mqa_logits"]
    # CPU slice: the oracle's formula on the first 32 query rows against the first 8192 keys
    from oracle import sparse_mla_oracle as orc
    cq, ck = 32, 8192
    qs_, kc_, kss_, ws_ = qi[:cq].cpu(), ki[:ck].cpu(), k_scale[:ck].cpu(), w[:cq].cpu()
    z0, z1 = torch.zeros(cq, dtype=torch.int32), torch.full((cq,), ck, dtype=torch.int32)
    best = None
    for _ in range(3):
        t0 = time.perf_counter()
        orc.mqa_logits_ref(qs_, kc_, kss_, ws_, z0, z1)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    mq.update({"workload": "s_q=4096, 64 heads, d=128, s_k=65536, ke=61440+i", "tflops": fl / mq["ms"] / 1e9,
               "write_gbs": s_q * s_k * 4 / mq["ms"] / 1e6,
               "roofline": {"bound": "tensor", "kernel": "mqa_logits_tc_kernel", "achieved": fl / mq["ms"] / 1e9, "peak": 2 * bf16_peak,
                            "unit": "TFLOP/s", "frac": fl / mq["ms"] / 1e9 / (2 * bf16_peak),
                            "peak_kind": f"2 x the {peak_kind} dense BF16 rate (the kernel's MMAs are FP8)", "traffic": None,
                            "hbm_write_frac": s_q * s_k * 4 / mq["ms"] / 1e6 / hbm_peak},
               "cpu_baseline": {"value": 2.0 * hh * 128 * cq * ck / best / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port",
                                "sample": f"first {cq} query rows x first {ck} keys, best of 3", "seconds": best}})
    out["topk"].update({"workload": "top-2048 of each of 4096 rows of 65536 fp32", "read_gbs": s_q * s_k * 4 / out["topk"]["ms"] / 1e6,
                        "roofline": {"bound": "hbm", "kernel": "topk_kernel", "achieved": s_q * s_k * 4 / out["topk"]["ms"] / 1e6,
                                     "peak": hbm_peak, "unit": "GB/s", "frac": s_q * s_k * 4 / out["topk"]["ms"] / 1e6 / hbm_peak,
                                     "peak_kind": f"of {peak_kind}", "traffic": None}})
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


def cpu_sample_step(n_req: int = CPU_SAMPLE_REQUESTS):
    """The CPU sample of one decode step that BOTH arms time: n_req of the step's 64 requests (all of them by
    default; a request's work does not depend on the others), seeded, built on the host.  The rows that a step
    gathers are generated directly (n_req x 2048 rows) instead of a whole paged pool, which the CPU path would
    only index into.  Returns (step function, algorithmic bytes of the sample, description)."""
    from oracle import sparse_mla_oracle as orc
    torch.set_num_threads(os.cpu_count())
    g = torch.Generator().manual_seed(1234)
    kv = torch.randn(n_req * TOPK // 64, 64, 1, D_QK, generator=g).to(torch.bfloat16)
    packed = orc.quantize_kv_v32(kv)
    q = (torch.randn(n_req, 1, HEADS, D_QK, generator=g) * 0.5).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(n_req * TOPK, generator=g)[:TOPK] for _ in range(n_req)]).view(n_req, 1, TOPK).int()

    def step():
        deq = orc.dequantize_kv_v32(packed)          # the reference's CPU path dequantises, then attends in fp32
        orc.ref_sparse_attn(q, deq, idx, SM_SCALE, D_V)

    sample = (f"{n_req} of the {B_PER_GPU} requests of one step (dequantise the gathered rows + fp32 attention), seed 1234, "
              f"{os.cpu_count()} host threads")
    return step, algorithmic_bytes(n_req, TOPK), sample


def cpu_baseline():
    """The reference's CPU PyTorch path (oracle port) on the bounded sample, best of 5."""
    step, nbytes, sample = cpu_sample_step()
    best = None
    for _ in range(5):
        t0 = time.perf_counter()
        step()
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return {"value": nbytes / best / 1e9, "unit": "GB/s", "cores": os.cpu_count(), "kind": "port",
            "sample": sample + ", best of 5", "seconds": best}


def run_reference(args):
    """The reference's own CPU implementation of the path (its PyTorch reference functions, restated in
    oracle/), timed on the host cores.  One timed step computes the bounded sample (the same one as the
    other arm's cpu_baseline); ``ms_per_step`` is scaled to the whole 64-request step, ``ms_per_sample``
    is what was measured."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    step, nbytes, sample = cpu_sample_step()
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    secs = time.perf_counter() - t0
    value = nbytes * args.steps / secs / 1e9
    world = int(os.environ.get("WORLD_SIZE", "1"))
    print(json.dumps({
        "impl": "reference", "metric": "sparse_mla_decode_algorithmic_hbm_throughput", "value": value, "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": secs / args.steps * 1e3 * (B_PER_GPU / CPU_SAMPLE_REQUESTS),
        "ms_per_sample": secs / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample,
                   "note": "one host runs this arm whatever N is: a ratio against the N-GPU arm divides N GPUs by one host"},
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
    if name == "decode":
        # the headline's shape over a 172 MB pool (larger than L2, small enough for a profiler's save and restore)
        pages = 4096
        kv = indexer.pack_kv_cache(torch.randn((pages * 64, D_QK), device=device, generator=g).to(torch.bfloat16)).view(pages, 64, 1, ROW)
        q = (torch.randn((B_PER_GPU, HEADS, D_QK), device=device, generator=g) * 0.5).to(torch.bfloat16)
        idx = torch.stack([torch.randperm(pages * 64, device=device, generator=g)[:TOPK] for _ in range(B_PER_GPU)]).to(torch.int32)
        fn = lambda: flash_ops.sparse_mla_decode_fwd(q, kv, idx, SM_SCALE)
        work = {"flop": 2.0 * B_PER_GPU * HEADS * TOPK * (D_QK + D_V)}
        desc = f"decode b={B_PER_GPU}, h=128, topk=2048, KV pool of {pages * 64} rows (172 MB)"
    elif name == "prefill":
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
    ap.add_argument("--steps", type=int, default=None, help="timed steps (default 3000; 20 for --impl reference)")
    ap.add_argument("--warmup", type=int, default=None, help="untimed steps before them (default 50; 3 for --impl reference)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--case", default=None, choices=["decode", "prefill", "indexer"],
                    help="run a small instance of a secondary kernel (for profiler captures) instead of the benchmark")
    args = ap.parse_args()
    # a step of the reference arm is about 0.13 s of host work: its default run is 20 steps, so that both arms finish
    # within minutes when called without flags
    if args.steps is None:
        args.steps = 20 if args.impl == "reference" else 3000
    if args.warmup is None:
        args.warmup = 3 if args.impl == "reference" else 50
    args.warmup = max(args.warmup, 3)
    if args.case is not None:
        run_small_case(args.case)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
