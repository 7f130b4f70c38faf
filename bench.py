#!/usr/bin/env python
"""Benchmark of the joint-attention forward: attention TFLOP/s (4*B*H*Sq*Sk*D per call).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload c2_image1024|c3_image2048|c4_video480p|c5_video768p]
                    [--mode auto|local|ulysses|ring] [--fixed-m]

A step is one DiT forward's worth of attention: ``layers`` (60 for the image workloads) independent
seeded layer calls, each on its own q/k/v/o buffers, so consecutive calls never find their inputs in
L2.  ``value`` is timed with CUDA events with inputs resident in HBM; ``e2e`` times the same calls
through the public API from pinned host buffers, with the host->device copies of q, k, v and the
device->host copy of the output inside the timed region.

Under ``torchrun`` (N > 1) the default placement is the reference's head-parallel one with CFG halves
on chip halves: batch elements first, then heads, are dealt to ranks and every rank runs the local
kernel on its resident shard (no collective on the data path).  ``--mode ulysses`` starts and ends
sequence-sharded with an all-to-all either side; ``--mode ring`` rotates K/V shards between ranks.

Besides the headline line every run also measures, in the same process and on the same GPUs, the collective
placements on the long shapes (``workloads`` in the JSON line): the 48,872-token video shape head-parallel with
the exchange either side of the kernel (Ulysses), the 351,296-token shape as a ring over K/V shards, and the
2048 x 2048 image shape with CFG halves on chip halves - each with this library's peer-memory kernels and, beside
it, over NCCL collectives, and each with the one-GPU time of the same call measured in the same run (every rank
runs the whole call as a replica) so that the scaling efficiency needs no number from another run.

``--impl reference`` times the CPU restatement of the reference's own CPU attention (fp32 softmax)
on the host cores for the same workload and metric, on a bounded sample per step.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "diffusers-tpu_b200"))

import torch  # noqa: E402

METRIC = "attention_tflops"
UNIT = "TFLOP/s"
LAYERS = {"c1_image512_cpu": 60, "c2_image1024": 60, "c3_image2048": 20, "c4_video480p": 4, "c5_video768p": 1}
PROFILE_SUMMARY = os.path.join(ROOT, "profiles", "attn_fwd_kernel_c2_image1024.md")


def profiled_traffic_bytes():
    """DRAM bytes per launch of the attention kernel on the c2 workload as the committed ncu summary records them
    (``dram__bytes_read.sum`` + ``dram__bytes_write.sum`` of its last captured launch), or None."""
    try:
        text = open(PROFILE_SUMMARY).read()
    except OSError:
        return None
    total = 0.0
    for key in ("dram__bytes_read.sum", "dram__bytes_write.sum"):
        row = next((ln for ln in text.splitlines() if ln.startswith("| " + key)), None)
        if row is None:
            return None
        cell = [c.strip() for c in row.strip("|").split("|")][-1]
        try:
            total += float(cell.split()[0]) * {"MB": 1e6, "GB": 1e9, "KB": 1e3}[cell.split()[1]]
        except (ValueError, KeyError, IndexError):
            return None
    return total


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    return 1590.0, 1400.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        exe = shutil.which("nvidia-smi")
        if exe is None:
            return
        fd, self.path = tempfile.mkstemp(suffix=".csv")
        os.close(fd)
        self.proc = subprocess.Popen(
            [exe, f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
            stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)

    def stop(self):
        if self.proc is None:
            return None
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, max_clock, reasons, power = [], None, set(), []
        with open(self.path) as f:
            for line in f:
                parts = [x.strip() for x in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    clocks.append(float(parts[1]))
                    max_clock = float(parts[2])
                    power.append(float(parts[3]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                     parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        os.unlink(self.path)
        if not clocks:
            return None
        # keep the samples taken under load (upper half), the first ones may predate the first launch
        busy = sorted(clocks)[len(clocks) // 2:]
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max_clock, "reasons": sorted(reasons),
                "samples": len(clocks), "power_w_max": max(power) if power else None}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


# --------------------------------------------------------------------------------------------
# reference arm: the oracle's fp32-softmax attention on the host cores
# --------------------------------------------------------------------------------------------
def cpu_attention_sample(cfg, sample_heads: int, min_seconds: float, max_reps: int):
    from dtb200.inputs import make_inputs
    from oracle import attn_oracle

    torch.set_num_threads(os.cpu_count() or 1)
    q, k, v, kv_len = make_inputs(cfg, 0, heads=sample_heads)
    q, k, v, kv_len = q[:1], k[:1], v[:1], kv_len[:1]
    # long sequences: a strided sample of query rows against all keys bounds time and memory
    rows = None if cfg.seq <= 8192 else torch.arange(0, cfg.seq, cfg.seq // 2048)
    n_rows = cfg.seq if rows is None else len(rows)
    flops = 4.0 * 1 * sample_heads * n_rows * cfg.seq * cfg.head_dim
    attn_oracle.attention_fp32(q[:, :1, :256], k[:, :1, :256], v[:, :1, :256])  # warm the thread pool
    times = []
    t_all = time.perf_counter()
    while len(times) < max_reps and (time.perf_counter() - t_all < min_seconds or not times):
        t0 = time.perf_counter()
        attn_oracle.attention_fp32(q, k, v, kv_len=kv_len, rows=rows)
        times.append(time.perf_counter() - t0)
    best = min(times)
    return {"value": flops / best / 1e12, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{n_rows} of {cfg.seq} query rows x all keys, {sample_heads} of {cfg.heads} heads of batch "
                      f"element 0 of one {cfg.name} layer call, fp32 softmax on CPU, best of {len(times)}"}, times


def run_reference(args, cfg):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    sample_heads = min(cfg.heads, 8 if cfg.seq <= 8192 else 1)
    step_times = []
    base = None
    for i in range(args.warmup + args.steps):
        base, times = cpu_attention_sample(cfg, sample_heads, 0.0, 1)
        if i >= args.warmup:
            step_times.append(times[0])
    n_rows = cfg.seq if cfg.seq <= 8192 else len(range(0, cfg.seq, cfg.seq // 2048))
    flops = 4.0 * sample_heads * n_rows * cfg.seq * cfg.head_dim
    total = sum(step_times)
    value = flops * len(step_times) / total / 1e12
    base["value"] = value
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * total / len(step_times), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": cfg.name, "B": cfg.batch, "H": cfg.heads, "S": cfg.seq, "D": cfg.head_dim,
                   "step": base["sample"]},
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------------
def run_ours(args, cfg):
    import torch.distributed as dist

    import dtb200
    from dtb200.inputs import make_inputs

    rank, world, local = dist_env()
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    mode = args.mode
    if mode == "auto":
        mode = "local"
    layers = args.layers or LAYERS[cfg.name]
    from dtb200 import parallel

    # --shard-of N on one GPU: time rank 0's resident shard of an N-GPU placement (what one rank of that run computes)
    place_world = args.shard_of if (args.shard_of and world == 1 and mode == "local") else world
    bg, hg = parallel.placement(cfg.batch, cfg.heads, place_world) if mode == "local" else (1, 1)
    b_local = cfg.batch // bg
    h_local = cfg.heads // hg
    my_b = (rank // hg) * b_local
    my_h = (rank % hg) * h_local

    # Ulysses with CFG halves on chip halves: every batch element gets its own sub-group of ranks.
    group = None
    cfg_groups = 1
    if mode == "ulysses" and args.cfg_halves and cfg.batch > 1 and world % cfg.batch == 0 and world > cfg.batch:
        cfg_groups = cfg.batch
        for ranks in parallel.cfg_subgroups(world, cfg_groups):
            g = dist.new_group(ranks)
            if rank in ranks:
                group = g
    sub_world = world // cfg_groups
    sub_rank = rank % sub_world
    my_cfg = rank // sub_world

    # Resident inputs: one buffer set per layer call.
    sets = []
    for i in range(layers):
        if mode == "local":
            q, k, v, kv_len = make_inputs(cfg, i, device="cuda", heads=cfg.heads)
            q = q[my_b:my_b + b_local, my_h:my_h + h_local].contiguous()
            k = k[my_b:my_b + b_local, my_h:my_h + h_local].contiguous()
            v = v[my_b:my_b + b_local, my_h:my_h + h_local].contiguous()
            kv_len = kv_len[my_b:my_b + b_local].contiguous()
        else:
            q, k, v, kv_len = parallel.make_sequence_shard(cfg, i, sub_rank, sub_world, dev)
            if cfg_groups > 1:   # this half owns one batch element
                q, k, v = (t[my_cfg:my_cfg + 1].contiguous() for t in (q, k, v))
                kv_len = kv_len[my_cfg:my_cfg + 1].contiguous()
        sets.append((q, k, v, kv_len, torch.empty_like(q)))
    torch.cuda.synchronize()

    mk = None
    launches_per_call = 1
    fused = None
    if mode != "local" and args.transport == "p2p" and sub_world > 1:
        from dtb200 import symm

        shp = sets[0][0].shape
        cls = symm.UlyssesP2P if mode == "ulysses" else symm.RingPull
        fused = cls(shp[0], shp[1], shp[2], group=group, device=dev)

    def layer_call(s):
        q, k, v, kv_len, o = s
        if mode == "local":
            dtb200.attention(q, k, v, kv_len=kv_len, use_fixed_m=args.fixed_m, mk=mk, out=o)
        elif fused is not None and mode == "ulysses":
            fused(q, k, v, kv_len=kv_len)
        elif fused is not None:
            fused(q, k, v, kv_len=kv_len, out=o)
        elif mode == "ulysses":
            parallel.ulysses_attention(q, k, v, kv_len=kv_len, out=o, group=group)
        else:
            parallel.ring_attention(q, k, v, kv_len=kv_len, out=o)

    balanced = False
    if mode == "local":
        # does the automatic mode balance the last wave of this rank's launch (a sweep kernel + a merge kernel)?
        import ctypes

        from dtb200 import _lib, ops

        q0, k0, v0, n0, o0 = sets[0]
        probe = ops._fill_params(q0, k0, v0, o0, n0, None, None, 0, 0, None)
        balanced = _lib.load().dtb_attn_workspace_bytes(ctypes.byref(probe)) > 0
        launches_per_call = 2 if balanced else 1
    if args.fixed_m:
        launches_per_call += 3  # two row-norm reductions and the operand kernel in front of the attention kernel
    if mode == "ring":
        launches_per_call = world + 1  # one residual kernel per ring step and the final normalisation
    launches_per_call *= world         # every rank launches its own

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        for s in sets:
            layer_call(s)
    barrier()
    dtb200.check_device_status(dev)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        for s in sets:
            layer_call(s)
    e1.record()
    barrier()
    ms_total = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    dtb200.check_device_status(dev)

    # ---- the same calls with the bounded-logit softmax on a statically calibrated operand (the reference's fastest
    # configuration keeps the operand off the per-call path: fixed_m_bound.py:300-408), reported beside the headline
    bounded = None
    if mode == "local" and not args.fixed_m and not args.no_bounded:
        from dtb200 import fixed_m as fm

        qn, kn = dtb200.ops.row_norm_maxima(sets[0][0], sets[0][1])
        if kn.numel() != qn.numel():
            kn = kn.repeat_interleave(qn.numel() // kn.numel())
        mk_static = torch.from_numpy(fm.static_fixed_m_operands(
            qn.cpu().numpy(), kn.cpu().numpy(), margin_log2=1.0, gate=fm.FIXED_M_RING_SAFE_BOUND)).to(dev)
        for s in sets[:min(len(sets), 6)]:
            dtb200.attention(s[0], s[1], s[2], kv_len=s[3], use_fixed_m=True, mk=mk_static, out=s[4])
        barrier()
        b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        b0.record()
        for _ in range(args.steps):
            for s in sets:
                dtb200.attention(s[0], s[1], s[2], kv_len=s[3], use_fixed_m=True, mk=mk_static, out=s[4])
        b1.record()
        barrier()
        bounded_ms = b0.elapsed_time(b1)
        if world > 1:
            t = torch.tensor([bounded_ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            bounded_ms = t.item()
        dtb200.check_device_status(dev)
        bounded = {"ms_total": bounded_ms, "eligible_heads": int(mk_static[1].sum().item()), "heads": int(mk_static.shape[1])}

    # ---- an on-box comparator, not the reference: torch's SDPA on the cuDNN backend over the same buffers, without
    # the padding mask (it attends all keys, which is the same arithmetic per call), timed like the headline
    comparator = None
    if mode == "local" and world == 1 and not args.no_comparator and not args.shard_of:
        try:
            from torch.nn.attention import SDPBackend, sdpa_kernel

            with sdpa_kernel(SDPBackend.CUDNN_ATTENTION):
                for s in sets[:min(len(sets), 6)]:
                    torch.nn.functional.scaled_dot_product_attention(s[0], s[1], s[2])
                barrier()
                c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                c0.record()
                for _ in range(args.steps):
                    for s in sets:
                        torch.nn.functional.scaled_dot_product_attention(s[0], s[1], s[2])
                c1.record()
                barrier()
            comparator = {"ms_total": c0.elapsed_time(c1)}
        except Exception as e:  # a torch build without the cuDNN backend: say so, the headline does not depend on it
            comparator = {"unavailable": f"{type(e).__name__}: {e}"[:200]}

    # ---- end to end: pinned host buffers -> device -> kernel -> pinned host result, double buffered
    e2e_ms, e2e_steps, h2d_bytes, d2h_bytes = None, 0, 0, 0
    if not args.no_e2e:
        e2e_ms, e2e_steps, h2d_bytes, d2h_bytes = run_e2e(args, mode, layers, sets, world, dev, group, barrier, fused)
    dtb200.check_device_status(dev)

    h2d_rates = None
    if e2e_ms is not None:
        # host->device rate this rank saw (its share of the step's input bytes over its own elapsed time)
        mine = torch.tensor([h2d_bytes / world * e2e_steps / (e2e_ms * 1e-3) / 1e9], device=dev, dtype=torch.float64)
        if world > 1:
            allr = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(allr, mine)
            h2d_rates = [round(x.item(), 1) for x in allr]
        else:
            h2d_rates = [round(mine.item(), 1)]
    if world > 1:
        t = torch.tensor([ms_total, e2e_ms or 0.0], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = t[0].item()
        e2e_ms = t[1].item() if e2e_ms is not None else None
    del fused
    sets_info = (len(sets), 3 * sets[0][0].numel() * 2 / 1e6)
    sets.clear()
    torch.cuda.empty_cache()
    workloads = None
    if not args.no_workloads and args.workload == "c2_image1024" and mode == "local" and not args.shard_of:
        workloads = run_workloads(args, world, rank, local, dev)
    finish(args, cfg, mode, layers, sets_info, world, rank, bg, hg, cfg_groups, sub_world, ms_total, e2e_ms, e2e_steps,
           h2d_bytes, d2h_bytes, launches_per_call, clocks, workloads, h2d_rates, balanced, bounded, comparator)
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------------------------
# collective placements on the long shapes, with the one-GPU time of the same call measured beside them
# --------------------------------------------------------------------------------------------
WORKLOAD_CALLS = {"c3_image2048": (3, 12), "c4_video480p": (3, 4), "c5_video768p": (3, 2)}   # (warm-up, timed)


def _timed_calls(fn, sets, warmup, calls, world, rank, local, dev):
    """ms per call (max over ranks, CUDA events on the launching stream) and the SM clock sampled meanwhile."""
    import torch.distributed as dist

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(warmup):
        fn(sets[i % len(sets)])
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(calls):
        fn(sets[i % len(sets)])
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / calls
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
    return ms, clocks


def _n_sets(bytes_per_set):
    """Rotating input sets so that consecutive calls do not find their inputs in the 126 MB L2."""
    return int(max(1, min(6, -(-300e6 // max(bytes_per_set, 1)))))


def run_workloads(args, world, rank, local, dev):
    """The collective placements, each as ``{ms_per_call, tflops, frac_of_burst_per_gpu, n1_ms_per_call,
    efficiency_vs_n1, sm_mhz, ...}``; at one GPU only the local kernel on the whole call."""
    import torch.distributed as dist

    import dtb200
    from dtb200 import parallel
    from dtb200.inputs import CONFIGS, make_inputs

    burst, _, _ = measured_peaks()
    plan = [("c4_video480p", "ulysses", False), ("c5_video768p", "ring", False), ("c3_image2048", "ulysses", True)]
    if world == 8:
        plan.append(("c5_video768p", "ulysses", False))
    results = {}
    n1_cache = {}
    subgroups = {}

    def record(key, cfg, ms, clocks, extra):
        tf = cfg.flops() / (ms * 1e-3) / 1e12
        entry = {"ms_per_call": ms, "tflops": tf, "frac_of_burst_per_gpu": tf / (burst * world),
                 "sm_mhz": clocks["sm_mhz"] if clocks else None,
                 "clock_reasons": clocks["reasons"] if clocks else None}
        entry.update(extra)
        results[key] = entry
        return entry

    for name, mode, cfg_halves in plan:
        cfg = CONFIGS[name]
        warmup, calls = WORKLOAD_CALLS[name]
        # ---- one GPU: every rank runs the whole call on its own GPU (replicas), max over ranks
        if name not in n1_cache:
            q, k, v, kv_len = make_inputs(cfg, 0, device="cuda")
            o = torch.empty_like(q)
            ms1, clk1 = _timed_calls(lambda s: dtb200.attention(s[0], s[1], s[2], kv_len=s[3], out=s[4]),
                                     [(q, k, v, kv_len, o)], warmup, calls, world, rank, local, dev)
            dtb200.check_device_status(dev)
            n1_cache[name] = ms1
            record(f"{name}/1gpu", cfg, ms1, clk1,
                   {"n_gpus_used": 1, "parallelism": "local kernel on the whole call" +
                    (f" ({world} replicas, slowest)" if world > 1 else ""),
                    "frac_of_burst_per_gpu": cfg.flops() / (ms1 * 1e-3) / 1e12 / burst,
                    "l2": "one input set; q/k/v of a call are larger than L2"})
            del q, k, v, o
            torch.cuda.empty_cache()
        if world == 1:
            continue
        ms1 = n1_cache[name]
        # ---- N GPUs, sequence-sharded in and out
        group, groups, sub_world, sub_rank, my_cfg = None, 1, world, rank, 0
        if cfg_halves and cfg.batch > 1 and world % cfg.batch == 0 and world > cfg.batch:
            groups = cfg.batch
            if groups not in subgroups:
                for ranks in parallel.cfg_subgroups(world, groups):
                    g = dist.new_group(ranks)
                    if rank in ranks:
                        subgroups[groups] = g
            group = subgroups[groups]
            sub_world = world // groups
            sub_rank, my_cfg = rank % sub_world, rank // sub_world
        if cfg.heads % sub_world and mode == "ulysses":
            continue
        shard_bytes = 3 * (cfg.batch // groups) * cfg.heads * (cfg.seq // sub_world) * 256
        sets = []
        for i in range(_n_sets(shard_bytes)):
            q, k, v, kv_len = parallel.make_sequence_shard(cfg, i, sub_rank, sub_world, dev)
            if groups > 1:
                q, k, v = (t[my_cfg:my_cfg + 1].contiguous() for t in (q, k, v))
                kv_len = kv_len[my_cfg:my_cfg + 1].contiguous()
            sets.append((q, k, v, kv_len, torch.empty_like(q)))
        shp = sets[0][0].shape
        placement = (f"cfg{groups} x " if groups > 1 else "") + f"{mode}{sub_world}"
        for transport in ("p2p", "nccl"):
            if transport == "p2p":
                from dtb200 import symm

                cls = symm.UlyssesP2P if mode == "ulysses" else symm.RingPull
                op = cls(shp[0], shp[1], shp[2], group=group, device=dev)
                if mode == "ulysses":
                    fn = lambda s: op(s[0], s[1], s[2], kv_len=s[3])
                else:
                    fn = lambda s: op(s[0], s[1], s[2], kv_len=s[3], out=s[4])
                how = ("peer-store exchange fused into the scatter and attention kernels" if mode == "ulysses"
                       else "copy-engine pulls of K/V shards under the residual kernel")
            else:
                op = None
                if mode == "ulysses":
                    fn = lambda s: parallel.ulysses_attention(s[0], s[1], s[2], kv_len=s[3], out=s[4], group=group)
                    how = "NCCL all-to-all either side of the kernel"
                else:
                    fn = lambda s: parallel.ring_attention(s[0], s[1], s[2], kv_len=s[3], out=s[4], group=group)
                    how = "NCCL send/recv rotation of K/V shards"
            ms, clk = _timed_calls(fn, sets, warmup, calls, world, rank, local, dev)
            dtb200.check_device_status(dev)
            record(f"{name}/{placement}/{transport}", cfg, ms, clk,
                   {"n_gpus_used": world, "parallelism": f"{placement}: {how}", "n1_ms_per_call": ms1,
                    "efficiency_vs_n1": ms1 / (world * ms),
                    "l2": f"{len(sets)} rotating input sets of {shard_bytes / 1e6:.0f} MB per rank"})
            del op, fn
            torch.cuda.empty_cache()
        del sets
        torch.cuda.empty_cache()
    # ---- the projection behind keep-heads attention on the C2 shapes: GEMM with the reduce-scatter over the head
    # shards fused into its epilogue (peer reductions) against GEMM + NCCL reduce-scatter
    cfg = CONFIGS["c2_image1024"]
    if world > 1 and cfg.heads % world == 0 and (cfg.batch * cfg.seq) % world == 0:
        from dtb200 import symm

        B, S, H, N = cfg.batch, cfg.seq, cfg.heads, cfg.heads * 128
        Hl = H // world
        g = torch.Generator(device=dev).manual_seed(900 + rank)
        n_sets = 4
        os_ = [torch.randn(B, Hl, S, 128, generator=g, device=dev).to(torch.bfloat16) for _ in range(n_sets)]
        w_local = (torch.randn(Hl * 128, N, generator=g, device=dev) * (H * 128) ** -0.5).to(torch.bfloat16)
        flops = 2.0 * B * S * (H * 128) * N
        rows = B * S // world
        op = symm.OutProjReduceScatter(B, S, N, device=dev)
        op_exact = symm.OutProjReduceScatter(B, S, N, device=dev, exact=True)
        part = torch.empty(B, S, N, dtype=torch.bfloat16, device=dev)
        shard = torch.empty(rows, N, dtype=torch.bfloat16, device=dev)

        def nccl_call(o):
            dtb200.out_proj(o, w_local, out=part)
            dist.reduce_scatter_tensor(shard, part.view(B * S, N))

        nvlink_bytes = (world - 1) / world * B * S * N * 4            # f32 partial sums that leave this GPU
        for name, fn, how in (("p2p", lambda o: op(o, w_local), "bf16 partial rows stored into the owners' staging slots by the GEMM's epilogue, summed there"),
                              ("p2p_f32_reductions", lambda o: op_exact(o, w_local), "f32 partial sums added into the owners' shards by the GEMM's epilogue"),
                              ("nccl", nccl_call, "bf16 GEMM, then NCCL reduce-scatter of the bf16 partial sums")):
            ms, clk = _timed_calls(fn, os_, 3, 20, world, rank, local, dev)
            dtb200.check_device_status(dev)
            results[f"c2_image1024_out_proj/reduce_scatter{world}/{name}"] = {
                "ms_per_call": ms, "tflops": flops / (ms * 1e-3) / 1e12, "n_gpus_used": world,
                "sm_mhz": clk["sm_mhz"] if clk else None, "parallelism": f"head shards x {world}: {how}",
                "nvlink_gbs_per_gpu": (nvlink_bytes if "f32" in name else nvlink_bytes / 2) / (ms * 1e-3) / 1e9,
                "frac_of_nvlink_770": (nvlink_bytes if "f32" in name else nvlink_bytes / 2) / (ms * 1e-3) / 1e9 / 770.0}
        del op, op_exact
    return results


def run_e2e(args, mode, layers, sets, world, dev, group, barrier, fused):
    import dtb200
    from dtb200 import parallel

    n_host = min(layers, 4)
    host_sets = []
    for i in range(n_host):
        q, k, v, kv_len, o = sets[i]
        host_sets.append((q.cpu().pin_memory(), k.cpu().pin_memory(), v.cpu().pin_memory(), kv_len,
                          torch.empty(o.shape, dtype=o.dtype).pin_memory()))
    copy_in, copy_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    compute = torch.cuda.current_stream(dev)
    dev_bufs = [tuple(torch.empty_like(t) for t in sets[0][:3]) + (torch.empty_like(sets[0][4]),) for _ in range(2)]
    in_ready = [torch.cuda.Event() for _ in range(2)]
    out_ready = [torch.cuda.Event() for _ in range(2)]
    buf_free = [torch.cuda.Event() for _ in range(2)]
    h2d_bytes = sum(t.numel() * t.element_size() for t in host_sets[0][:3]) * layers * world
    d2h_bytes = host_sets[0][4].numel() * host_sets[0][4].element_size() * layers * world

    def e2e_step():
        for i in range(layers):
            hq, hk, hv, kv_len, ho = host_sets[i % n_host]
            dq, dk, dv, do = dev_bufs[i % 2]
            with torch.cuda.stream(copy_in):
                copy_in.wait_event(buf_free[i % 2])
                dq.copy_(hq, non_blocking=True)
                dk.copy_(hk, non_blocking=True)
                dv.copy_(hv, non_blocking=True)
                in_ready[i % 2].record(copy_in)
            compute.wait_event(in_ready[i % 2])
            if mode == "local":
                dtb200.attention(dq, dk, dv, kv_len=kv_len, use_fixed_m=args.fixed_m, out=do)
            elif fused is not None and mode == "ulysses":
                do = fused(dq, dk, dv, kv_len=kv_len)
            elif fused is not None:
                fused(dq, dk, dv, kv_len=kv_len, out=do)
            elif mode == "ulysses":
                parallel.ulysses_attention(dq, dk, dv, kv_len=kv_len, out=do, group=group)
            else:
                parallel.ring_attention(dq, dk, dv, kv_len=kv_len, out=do)
            out_ready[i % 2].record(compute)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(out_ready[i % 2])
                ho.copy_(do, non_blocking=True)
                buf_free[i % 2].record(copy_out)
        compute.wait_stream(copy_out)

    for ev in buf_free:
        ev.record(compute)
    e2e_steps = max(1, min(args.steps, 3))
    e2e_step()
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(e2e_steps):
        e2e_step()
    f1.record()
    barrier()
    return f0.elapsed_time(f1), e2e_steps, h2d_bytes, d2h_bytes


def dtb200_describe(cfg, bg, hg):
    """The library's one-line account of how it launches one rank's call of this placement."""
    import dtb200

    return dtb200.describe_launch(cfg.batch // bg, cfg.heads // hg, cfg.seq)


def finish(args, cfg, mode, layers, sets_info, world, rank, bg, hg, cfg_groups, sub_world, ms_total, e2e_ms, e2e_steps,
           h2d_bytes, d2h_bytes, launches_per_call, clocks, workloads, h2d_rates, balanced=False, bounded=None,
           comparator=None):
    flops_call = cfg.flops() / (bg * hg) * world if (args.shard_of and world == 1) else cfg.flops()
    flops_step = flops_call * layers
    value = flops_step * args.steps / (ms_total * 1e-3) / 1e12
    e2e_value = flops_step * e2e_steps / (e2e_ms * 1e-3) / 1e12 if e2e_ms else None
    burst, sustained, src = measured_peaks()
    # dominant kernel: attn_fwd_kernel, one launch per layer call per rank; its share of the call's FLOPs
    flops_launch = flops_call / world
    launch_ms = ms_total / (args.steps * layers)
    achieved = flops_launch / (launch_ms * 1e-3) / 1e12

    cpu_base = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_base, _ = cpu_attention_sample(cfg, min(cfg.heads, 8 if cfg.seq <= 8192 else 1), 10.0, 12)

    # The denominator follows the conditions of this run: the burst GEMM figure when the timed region is short
    # or the SM clock stayed near its maximum, the sustained (power-capped) figure otherwise.
    timed_s = ms_total * 1e-3
    near_max = bool(clocks and clocks.get("sm_max_mhz") and clocks["sm_mhz"] >= 0.95 * clocks["sm_max_mhz"])
    use_burst = timed_s < 2.0 or near_max
    peak = burst if use_burst else sustained
    traffic = profiled_traffic_bytes() if (cfg.name == "c2_image1024" and world == 1 and mode == "local") else None
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "frac_of_burst": achieved / burst, "frac_of_sustained": achieved / sustained,
                "peak_burst": burst, "peak_sustained": sustained,
                "peak_source": f"{src} {'burst' if use_burst else 'sustained'} bf16 GEMM: timed region {timed_s:.2f} s, "
                               f"median SM clock {clocks['sm_mhz'] if clocks else 'n/a'} MHz",
                "kernel": "attn_fwd_kernel", "flops_per_launch": flops_launch, "traffic": traffic,
                "traffic_source": None if traffic is None else
                "ncu capture of this kernel on this workload, read from the summary committed under profiles/ "
                "(not measured in this run)"}
    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_total / args.steps, "ms_per_layer_call": launch_ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {
                "workload": cfg.name, "B": cfg.batch, "H": cfg.heads, "S": cfg.seq, "D": cfg.head_dim,
                "layer_calls_per_step": layers, "softmax": "bounded-logit (fixed-m)" if args.fixed_m else "online",
                "launch": dtb200_describe(cfg, bg, hg),
                "parallelism": {"local": f"cfg{bg}xheads{hg} (resident head-parallel shards, no collective)",
                                "ulysses": f"cfg{cfg_groups} x ulysses{sub_world} ({'peer-store exchange fused into the kernels' if args.transport == 'p2p' else 'NCCL all-to-all'})",
                                "ring": f"ring{world} ({'copy-engine pulls of K/V shards' if args.transport == 'p2p' else 'NCCL send/recv rotation'})"}[mode],
                "l2": "inputs larger than L2: every layer call reads its own q/k/v buffers "
                      f"({sets_info[0]} sets, {sets_info[1]:.0f} MB each per rank)",
                "inputs": "N(0,1) q,k,v with unit-weight qk-RMSNorm, bf16, trailing text padding 0-300 keys per batch element",
            },
            "pct_of_peak": {"of_measured_sustained": 100 * value / (sustained * world),
                            "of_measured_burst": 100 * value / (burst * world),
                            "of_nominal_2250": 100 * value / (2250.0 * world)},
            "roofline": roofline,
            "e2e": None if e2e_ms is None else {
                    "value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes,
                    "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps, "h2d_gbs_per_rank": h2d_rates,
                    "how": "pinned host q,k,v -> device (double buffered, copy streams) -> dtb200.attention -> pinned host o"},
            "gpu_launches": args.steps * layers * launches_per_call,
            "clocks": clocks,
            "cpu_baseline": cpu_base,
            "bounded_logit": None if bounded is None else {
                "value": flops_step * args.steps / (bounded["ms_total"] * 1e-3) / 1e12, "unit": UNIT,
                "ms_per_layer_call": bounded["ms_total"] / (args.steps * layers),
                "frac_of_burst": flops_launch / (bounded["ms_total"] / (args.steps * layers) * 1e-3) / 1e12 / burst,
                "eligible_heads": f"{bounded['eligible_heads']} of {bounded['heads']}",
                "how": "same calls, per-head constant softmax offset from a statically calibrated operand (norms of the "
                       "first call, margin 1 log2 unit, gate 106.5 because the keys are not k-smoothed); not the headline"},
            "comparator": None if comparator is None else comparator if "unavailable" in comparator else {
                "name": "torch.nn.functional.scaled_dot_product_attention, cuDNN backend (a library kernel on this "
                        "box, not the reference)",
                "value": flops_step * args.steps / (comparator["ms_total"] * 1e-3) / 1e12, "unit": UNIT,
                "ms_per_layer_call": comparator["ms_total"] / (args.steps * layers),
                "how": "same buffers and call count as the headline, timed right after it in the same process; no "
                       "padding mask (all keys attended)"},
            "workloads": workloads,
        }
        print(json.dumps(line))


def run_prepass(args, cfg):
    """HBM-bound pre-pass (q/k RMSNorm + rotary + layout) on the workload's shapes: GB/s against the copy peak."""
    import dtb200

    dev = torch.device("cuda", 0)
    B, S, H = cfg.batch, cfg.seq, cfg.heads
    n_sets = max(2, min(8, int(2e9 // (6 * B * S * H * 256))))      # rotate buffer sets larger than L2
    g = torch.Generator(device="cuda").manual_seed(0)
    sets = [tuple(torch.randn(B, S, H, 128, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
                  for _ in range(3)) for _ in range(n_sets)]
    ang = torch.arange(S, device=dev, dtype=torch.float32)[:, None] * torch.linspace(1e-4, 1.0, 48, device=dev)[None, :]
    rope = (torch.cat([ang.cos()] * 2, -1), torch.cat([ang.sin()] * 2, -1))
    w = torch.ones(128, device=dev)
    kv_len = torch.full((B,), S - 100, dtype=torch.int32, device=dev)
    call = lambda i: dtb200.qk_prepass(*sets[i % n_sets], q_weight=w, k_weight=w, rope=rope, kv_len=kv_len, want_mk=True)
    for i in range(max(args.warmup, 3) * n_sets):
        call(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n = args.steps * n_sets
    e0.record()
    for i in range(n):
        call(i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / n
    algo_bytes = 3 * 2 * B * S * H * 256
    hbm = 6549.1
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        hbm = float(json.load(open(path))["hbm_gbs"])
    gbs = algo_bytes / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "qk_prepass_gbs", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms * n_sets, "ms_per_call": ms, "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": cfg.name + " pre-pass", "B": B, "S": S, "H": H, "D": 128, "rotary": 96,
                   "l2": f"{n_sets} rotating buffer sets of {algo_bytes / 2e6:.0f} MB inputs"},
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm, "unit": "GB/s", "frac": gbs / hbm,
                     "algorithmic_bytes_per_launch": algo_bytes, "kernel": "qk_prepass_kernel", "traffic": None},
        "gpu_launches": 2 * n,
    }))


def run_smooth_k(args, cfg):
    """HBM-bound k-smoothing (column means over the valid rows, then subtract and zero the pads) on the workload's
    key tensor: GB/s against the copy peak.  Algorithmic bytes: K read by each of the two passes and written once."""
    import dtb200

    dev = torch.device("cuda", 0)
    B, S, H = cfg.batch, cfg.seq, cfg.heads
    n_sets = max(2, min(8, int(1.5e9 // (B * S * H * 256))))      # rotate buffers larger than L2
    g = torch.Generator(device="cuda").manual_seed(0)
    ks = [torch.randn(B, H, S, 128, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16) for _ in range(n_sets)]
    outs = [torch.empty_like(k) for k in ks]
    kv_len = torch.full((B,), S - 100, dtype=torch.int32, device=dev)
    call = lambda i: dtb200.smooth_k(ks[i % n_sets], kv_len=kv_len, out=outs[i % n_sets], want_norms=True)
    for i in range(max(args.warmup, 3) * n_sets):
        call(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n = args.steps * n_sets
    e0.record()
    for i in range(n):
        call(i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / n
    algo_bytes = 3 * B * S * H * 256
    hbm = 6549.1
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        hbm = float(json.load(open(path))["hbm_gbs"])
    gbs = algo_bytes / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "smooth_k_gbs", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms * n_sets, "ms_per_call": ms, "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": cfg.name + " k-smoothing", "B": B, "S": S, "H": H, "D": 128,
                   "l2": f"{n_sets} rotating key tensors of {B * S * H * 256 / 1e6:.0f} MB"},
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm, "unit": "GB/s", "frac": gbs / hbm,
                     "algorithmic_bytes_per_launch": algo_bytes, "kernel": "k_colsum_kernel + k_smooth_kernel",
                     "traffic": None},
        "gpu_launches": 2 * n,
    }))


def run_out_proj(args, cfg):
    """The projection behind the attention call on the workload's shapes (all heads on one GPU, N = heads * 128):
    TFLOP/s (2 * B * S * K * N per call) against the measured bf16 GEMM peak."""
    import dtb200

    dev = torch.device("cuda", 0)
    B, S, H = cfg.batch, cfg.seq, cfg.heads
    N = H * 128
    n_sets = max(2, min(8, int(1.0e9 // (B * S * H * 256))))
    g = torch.Generator(device="cuda").manual_seed(0)
    os_ = [torch.randn(B, H, S, 128, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16) for _ in range(n_sets)]
    w = (torch.randn(H * 128, N, generator=g, device=dev, dtype=torch.float32) * (H * 128) ** -0.5).to(torch.bfloat16)
    outs = [torch.empty(B, S, N, dtype=torch.bfloat16, device=dev) for _ in range(n_sets)]
    call = lambda i: dtb200.out_proj(os_[i % n_sets], w, out=outs[i % n_sets])
    for i in range(max(args.warmup, 3) * n_sets):
        call(i)
    torch.cuda.synchronize()
    dtb200.check_device_status(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n = args.steps * n_sets
    e0.record()
    for i in range(n):
        call(i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / n
    flops = 2.0 * B * S * (H * 128) * N
    burst, sustained, src = measured_peaks()
    tf = flops / (ms * 1e-3) / 1e12
    print(json.dumps({
        "metric": "out_proj_tflops", "value": tf, "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms * n_sets, "ms_per_call": ms, "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": cfg.name + " output projection", "B": B, "S": S, "K": H * 128, "N": N,
                   "l2": f"{n_sets} rotating attention outputs of {B * S * H * 256 / 1e6:.0f} MB"},
        "roofline": {"bound": "tensor", "achieved": tf, "peak": burst, "unit": UNIT, "frac": tf / burst,
                     "peak_source": f"{src} burst bf16 GEMM", "flops_per_launch": flops, "kernel": "out_proj_kernel",
                     "traffic": None},
        "gpu_launches": n,
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2_image1024")
    ap.add_argument("--mode", default="auto", choices=["auto", "local", "ulysses", "ring"])
    ap.add_argument("--transport", default="p2p", choices=["p2p", "nccl"],
                    help="ulysses/ring: this library's peer-memory kernels (p2p) or NCCL collectives")
    ap.add_argument("--layers", type=int, default=0, help="layer calls per step (default: per workload)")
    ap.add_argument("--fixed-m", action="store_true", help="bounded-logit softmax, operand derived per call")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cfg-halves", action="store_true", help="ulysses: one sub-group of ranks per batch element")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--shard-of", type=int, default=0,
                    help="one GPU only: run rank 0's shard of an N-GPU resident placement (kernel studies)")
    ap.add_argument("--no-comparator", action="store_true", help="skip the cuDNN SDPA comparator timed beside the headline")
    ap.add_argument("--no-bounded", action="store_true", help="skip the bounded-logit (fixed-m) figure beside the headline")
    ap.add_argument("--no-workloads", action="store_true",
                    help="skip the collective placements on the long shapes (the workloads entry of the line)")
    ap.add_argument("--kernel", default="attention", choices=["attention", "prepass", "smooth_k", "out_proj"],
                    help="attention (the metric's kernel), one of the HBM-bound kernels in front of it, or the projection behind it")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    from dtb200.inputs import CONFIGS

    cfg = CONFIGS[args.workload]
    if args.impl == "reference":
        run_reference(args, cfg)
    elif args.kernel == "prepass":
        run_prepass(args, cfg)
    elif args.kernel == "smooth_k":
        run_smooth_k(args, cfg)
    elif args.kernel == "out_proj":
        run_out_proj(args, cfg)
    else:
        run_ours(args, cfg)


if __name__ == "__main__":
    main()
