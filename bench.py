#!/usr/bin/env python
"""Benchmark of the quantized-matmul path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload: the MoE grouped slice-M W8A8 matmul (64 experts, K=7168, N=4096, 131072 routed rows,
Zipf(1.1) expert loads), expert/row-sharded over the N ranks with no collective on the data path.
One step = one pass over all routed rows.  Prints ONE JSON line on rank 0.

The line's `value` is timed over exactly K steps.  Next to it the line carries
  sustained   the same launch repeated for >= 2 s (power-capped clocks), with the clock samples of that region
  secondary   (1 GPU only) the other workloads of the metric - decode_a, decode_b, prefill, w4a8, w4a8_per_tensor,
              mxfp8, mxfp4, mx_swiglu, mx_routing, quant_int8, quant_mx -
              each replayed from a CUDA graph for >= 1.5 s so that its clock record holds >= 10 samples
  verify      the shard outputs of all ranks assembled with one all-gather and sampled rows of every expert,
              including the rows on both sides of every shard and tile boundary, compared with the CPU oracle
  e2e         the host-buffer entry point: inputs from pinned host memory, output back to it, every step

Other workloads can be run alone (single GPU): the secondary ones and moe_small.

`--impl reference` times the reference's own CPU golden (compiled from the reference tree into
oracle/_ref, else the oracle's plain-C restatement) on the host cores, on a bounded row sample per step.
"""
import argparse
import datetime
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MOE = dict(experts=64, k=7168, n=4096, tokens=16384, top_k=8, zipf_s=1.1, seed=20240)
# same law, 1/8 of the experts and rows: small enough for multi-pass profiler captures, still larger than L2
MOE_SMALL = dict(experts=8, k=7168, n=4096, tokens=2048, top_k=8, zipf_s=1.1, seed=20240)
DENSE = {
    "prefill": (4096, 4096, 4096),
    "decode_a": (16, 14336, 4096),
    "decode_b": (16, 4096, 14336),
}
SECONDARY = ["decode_a", "decode_b", "prefill", "w4a8", "w4a8_per_tensor", "mxfp8", "mxfp4", "mx_swiglu", "mx_routing",
             "quant_int8", "quant_mx"]
INT8_PER_BF16 = 2.0  # kind::i8 issues at twice the bf16 rate on the same tensor cores
L2_BYTES = 126e6


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p["bf16_tflops"]),
                    bf16_tflops_sustained=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


def zipf_group_sizes(total_rows, groups, seed, s):
    rng = np.random.default_rng(seed)
    p = np.arange(1, groups + 1, dtype=np.float64) ** (-s)
    p /= p.sum()
    return rng.multinomial(total_rows, p).astype(np.int64)


def moe_workload_string(cfg):
    return (f"moe_grouped_slice_m_w8a8: {cfg['experts']} experts, K={cfg['k']}, N={cfg['n']}, {cfg['tokens']} tokens x "
            f"top-{cfg['top_k']} = {cfg['tokens'] * cfg['top_k']} rows, Zipf({cfg['zipf_s']}) expert loads, "
            "B row-major [G,K,N], bf16 out")


def moe_config(cfg, placement, world):
    """The `config` object of the MoE line; both arms (ours, reference) print exactly this."""
    from catlass_b200 import sharding
    rows_total = cfg["tokens"] * cfg["top_k"]
    sizes = zipf_group_sizes(rows_total, cfg["experts"], cfg["seed"], cfg["zipf_s"])
    loads = [s.rows for s in sharding.plan(sizes, world, mode=placement)]
    return {
        "workload": moe_workload_string(cfg),
        "placement": placement, "rows_per_rank": loads,
        "l2": f"inputs exceed L2 ({(rows_total * (cfg['k'] + 2 * cfg['n']) + cfg['experts'] * cfg['k'] * cfg['n']) / 1e9:.2f} GB per pass)",
        "weights": "resident in HBM across steps",
    }


class ClockSampler:
    """Polls nvidia-smi for one GPU's clocks and throttle reasons for as long as the process runs; every timed
    region asks for the samples that fell inside its own wall-clock window."""
    QUERY = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, gpu_index, interval_ms=20):
        self.samples = []  # (unix time, sm MHz, max MHz, watts, [reasons])
        self.lock = threading.Lock()
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(gpu_index), f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", str(interval_ms)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 8:
                continue
            try:
                t = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                row = (t, float(f[1]), float(f[2]), float(f[3]) if f[3].replace(".", "", 1).isdigit() else None,
                       [n for n, v in zip(self.NAMES, f[4:8]) if v.lower().startswith("active")])
            except ValueError:
                continue
            with self.lock:
                self.samples.append(row)

    def wait_first_sample(self, timeout=10.0):
        t0 = time.time()
        while self.proc is not None and time.time() - t0 < timeout:
            with self.lock:
                if self.samples:
                    return
            time.sleep(0.02)

    def window(self, t0, t1):
        """Summary of the samples taken between two time.time() stamps."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["nvidia-smi unavailable"]}
        with self.lock:
            rows = [r for r in self.samples if t0 <= r[0] <= t1]
            near = None
            if not rows:
                # a region shorter than the polling interval (8 GPUs: 20 steps last 7 ms): the samples right
                # before and after it stand in, and the record says so
                near = 0.03
                rows = [r for r in self.samples if t0 - near <= r[0] <= t1 + near]
        if near is not None and not any(r[0] > t1 for r in rows):
            time.sleep(0.06)  # the poll after the region may not have been read yet
            with self.lock:
                rows = [r for r in self.samples if t0 - near <= r[0] <= t1 + near]
        sm = [r[1] for r in rows]
        reasons = sorted({x for r in rows for x in r[4]})
        watts = [r[3] for r in rows if r[3] is not None]
        out = {"sm_mhz": float(np.median(sm)) if sm else None, "sm_mhz_min": min(sm) if sm else None,
               "sm_max_mhz": max(r[2] for r in rows) if rows else None, "power_w_max": max(watts) if watts else None,
               "samples": len(rows), "reasons": reasons}
        if near is not None:
            out["note"] = (f"the {1e3 * (t1 - t0):.1f} ms region fell between two polls: samples within "
                           f"{int(1e3 * near)} ms of it")
        return out

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()


def dist_setup(n_gpus):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(0)
    if world != n_gpus:
        raise SystemExit(f"--gpus {n_gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    return rank, world, local


def barrier(world):
    import torch
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(value, world):
    import torch
    if world == 1:
        return value
    import torch.distributed as dist
    t = torch.tensor([value], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def time_steps(fn, steps, warmup, world):
    """W warm-up steps, then exactly K steps between CUDA events on the launching stream.
    Returns (max over ranks of the elapsed ms, this rank's elapsed ms, library launches in the timed region,
    (wall-clock start, end) of the timed region)."""
    import torch
    from catlass_b200 import capi
    for _ in range(warmup):
        fn()
    barrier(world)
    launches0 = capi.launch_count()
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    start.record()
    for _ in range(steps):
        fn()
    stop.record()
    torch.cuda.synchronize()
    t1 = time.time()
    ms = start.elapsed_time(stop)
    launches = capi.launch_count() - launches0
    barrier(world)
    return max_over_ranks(ms, world), ms, launches, (t0, t1)


def check_device_status():
    from catlass_b200 import capi
    st, code = capi.device_status()
    if st != 0:
        raise SystemExit(f"device status {st} code {code:#x}")


def graph_region(launch, variants, min_seconds, sampler):
    """Times `launch(i)` (i cycling over `variants` buffer sets) replayed from a CUDA graph: first a short burst
    region, then back-to-back replays for at least `min_seconds` with the clock samples of that region.
    Kernels of ten microseconds cannot be timed through a Python launch loop (the host is slower than the GPU);
    a graph of a few hundred launches keeps the GPU fed.  Returns a dict with ms per launch for both regions."""
    import torch
    from catlass_b200 import capi
    for i in range(max(3, variants)):
        launch(i)
    torch.cuda.synchronize()
    # size the graph to roughly 5 ms of GPU time
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(variants):
        launch(i)
    e1.record()
    torch.cuda.synchronize()
    rough_ms = max(e0.elapsed_time(e1) / variants, 1e-3)
    per_graph = int(min(400, max(variants, 5.0 / rough_ms)))
    per_graph = (per_graph + variants - 1) // variants * variants
    graph = torch.cuda.CUDAGraph()
    launches0 = capi.launch_count()
    try:
        with torch.cuda.graph(graph):
            for i in range(per_graph):
                launch(i % variants)
        use_graph = True
    except Exception as exc:  # capture refused: fall back to a plain loop and say so
        use_graph = False
        graph_error = str(exc).splitlines()[0][:120]
        torch.cuda.synchronize()
    launches_per_graph = capi.launch_count() - launches0 if use_graph else None

    def replay():
        if use_graph:
            graph.replay()
        else:
            for i in range(per_graph):
                launch(i % variants)

    replay()
    torch.cuda.synchronize()
    time.sleep(0.3)  # let the clocks return to idle: the next region starts from burst clocks
    e0.record()
    replay()
    e1.record()
    torch.cuda.synchronize()
    burst_ms = e0.elapsed_time(e1) / per_graph
    replays = max(2, int(np.ceil(min_seconds * 1e3 / (burst_ms * per_graph) * 1.15)))
    t0 = time.time()
    e0.record()
    for _ in range(replays):
        replay()
    e1.record()
    torch.cuda.synchronize()
    t1 = time.time()
    sustained_ms = e0.elapsed_time(e1) / (per_graph * replays)
    out = {"ms": sustained_ms, "burst_ms": burst_ms, "launches_timed": per_graph * replays,
           "kernels_per_step": (launches_per_graph // per_graph) if use_graph else None,
           "region_s": (e0.elapsed_time(e1)) / 1e3, "clocks": sampler.window(t0, t1) if sampler else None,
           "cuda_graph": use_graph}
    if not use_graph:
        out["cuda_graph_error"] = graph_error
    return out


# ------------------------------------------------------------------------------------------ CPU baseline

def cpu_reference_rate(n, k, seconds_target, b_row_major=True):
    """Times the reference's CPU golden for the grouped path on all host cores: every thread runs the
    golden on its own rows of one expert.  Returns (TOPS, cores, kind, sample description, seconds)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as O
    kind = "reference" if O.ref() is not None else "port"
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    rng = np.random.default_rng(7)
    b = rng.integers(-127, 128, size=k * n, dtype=np.int8)
    scale = rng.uniform(1e-3, 1e-2, n).astype(np.float32)

    def run(rows_per_thread):
        a = rng.integers(-127, 128, size=(cores, rows_per_thread * k), dtype=np.int8)
        pt = rng.uniform(1e-3, 1e-2, (cores, rows_per_thread)).astype(np.float32)
        gl = np.array([rows_per_thread], np.int64)
        lb = O.ROW_MAJOR if b_row_major else O.COL_MAJOR

        def work(i):
            if kind == "reference":
                O.ref_grouped_quant_matmul(a[i], b, gl, scale, pt[i], rows_per_thread, n, k, lb)
            else:
                O.grouped_quant_matmul(a[i], b, gl, scale, pt[i], rows_per_thread, n, k, lb)
        threads = [threading.Thread(target=work, args=(i,)) for i in range(cores)]
        t0 = time.perf_counter()
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        return time.perf_counter() - t0

    probe_rows = 2
    t_probe = run(probe_rows)
    rows = int(max(probe_rows, min(512, probe_rows * seconds_target / max(t_probe, 1e-6))))
    secs = run(rows)
    ops = 2.0 * cores * rows * n * k
    sample = (f"{cores} threads x {rows} rows of one expert (N={n}, K={k}, "
              f"{'row' if b_row_major else 'column'}-major B), golden called once per thread")
    return ops / secs / 1e12, cores, kind, sample, secs


# ------------------------------------------------------------------------------------------ MoE workload

def build_moe_rank(rank, world, mode, cfg):
    """ONE global seeded problem (the same on every rank), cut by sharding.plan; returns this rank's device
    buffers, and what rank 0 needs to check the assembled output."""
    import torch
    from catlass_b200 import sharding
    rows_total = cfg["tokens"] * cfg["top_k"]
    sizes = zipf_group_sizes(rows_total, cfg["experts"], cfg["seed"], cfg["zipf_s"])
    shards = sharding.plan(sizes, world, mode=mode)
    mine = shards[rank]
    n, k, experts = cfg["n"], cfg["k"], cfg["experts"]
    dev = torch.device("cuda")
    gen = torch.Generator(device="cuda")
    gen.manual_seed(cfg["seed"])
    a_all = torch.randint(-127, 128, (rows_total, k), dtype=torch.int8, device=dev, generator=gen)
    b_all = torch.randint(-127, 128, (experts, k, n), dtype=torch.int8, device=dev, generator=gen)
    scale_all = torch.empty((experts, n), device=dev).uniform_(1e-3, 1e-2, generator=gen)
    pt_all = torch.empty(rows_total, device=dev).uniform_(1e-3, 1e-2, generator=gen)

    groups = mine.local_groups()
    gl = np.cumsum([r for _, r in groups]).astype(np.int64)
    m = int(gl[-1]) if len(gl) else 0
    # this rank's rows of the global problem, in its local order (pieces sorted by expert, row)
    ranges = sharding.global_row_ranges(sizes, mine)
    row_index = np.concatenate([np.arange(b, b + r) for b, r in ranges]) if ranges else np.zeros(0, np.int64)
    if world == 1:
        a, b, scale, pt = a_all, b_all, scale_all, pt_all   # one shard: the global buffers are the rank's own
    else:
        idx = torch.from_numpy(row_index).to(dev)
        a = a_all.index_select(0, idx) if m else a_all[:1].clone()
        pt = pt_all.index_select(0, idx) if m else pt_all[:1].clone()
        eidx = torch.tensor([e for e, _ in groups] or [0], device=dev)
        b = b_all.index_select(0, eidx)
        scale = scale_all.index_select(0, eidx)
    d = torch.empty((max(m, 1), n), dtype=torch.bfloat16, device=dev)
    gl_dev = torch.from_numpy(gl if len(gl) else np.zeros(1, np.int64)).to(dev)

    check = None
    if rank == 0:
        check = sample_for_check(sizes, shards, a_all, b_all, scale_all, pt_all, n, cfg["seed"])
    if world > 1:
        del a_all, b_all, scale_all, pt_all
        torch.cuda.empty_cache()
    return dict(a=a, b=b, scale=scale, pt=pt, d=d, gl=gl_dev, m=m, n=n, k=k, groups=len(groups),
                rows_total=rows_total, loads=[s.rows for s in shards], sizes=sizes, shards=shards,
                row_index=row_index, check=check)


def sample_for_check(sizes, shards, a_all, b_all, scale_all, pt_all, n, seed):
    """Rows and columns of the global problem that the oracle recomputes: per expert its first, last and one random
    row, the rows on both sides of every shard boundary, of its first 256-row tile boundary and of the start of
    its last (partial) row tile; a fixed spread of columns including tile edges."""
    import torch
    rng = np.random.default_rng(seed + 1)
    starts = np.concatenate([[0], np.cumsum(sizes)[:-1]])
    rows_of = {}
    for e, size in enumerate(sizes):
        size = int(size)
        if size == 0:
            continue
        local = {0, size - 1, int(rng.integers(0, size))}
        if size > 256:
            local |= {255, 256}
        tail = (size - 1) // 256 * 256
        local |= {tail, max(tail - 1, 0), min(tail + 31, size - 1), min(tail + 32, size - 1)}
        rows_of[e] = local
    for sh in shards:
        for p in sh.pieces:
            if p.row_begin > 0:
                rows_of[p.expert] |= {p.row_begin - 1, p.row_begin}
    cols = sorted(set([0, 1, 127, 128, 255, 256, 257, n - 257, n - 256, n - 1]) |
                  set(int(c) for c in rng.integers(0, n, 118)))
    cols_t = torch.tensor(cols, device=a_all.device)
    items = []
    for e, local in rows_of.items():
        loc = np.array(sorted(local))
        g_rows = torch.from_numpy(loc + starts[e]).to(a_all.device)
        items.append(dict(expert=e, global_rows=(loc + starts[e]),
                          a=a_all.index_select(0, g_rows).cpu().numpy(),
                          b=b_all[e].index_select(1, cols_t).contiguous().cpu().numpy(),
                          scale=scale_all[e].index_select(0, cols_t).cpu().numpy(),
                          pt=pt_all.index_select(0, g_rows).cpu().numpy()))
    return dict(cols=cols, items=items)


def verify_moe(w, rank, world):
    """Assembles the ranks' outputs with ONE all-gather (padded to the largest shard) and compares the sampled
    rows with the CPU oracle on rank 0.  Outside every timed region."""
    import torch
    n = w["n"]
    if world > 1:
        import torch.distributed as dist
        max_rows = max(max(w["loads"]), 1)
        padded = torch.zeros((max_rows, n), dtype=torch.bfloat16, device="cuda")
        if w["m"]:
            padded[:w["m"]].copy_(w["d"][:w["m"]])
        gathered = torch.empty((world, max_rows, n), dtype=torch.bfloat16, device="cuda")
        dist.all_gather_into_tensor(gathered, padded)
    else:
        gathered = w["d"][None]
    if rank != 0:
        return None
    from catlass_b200 import sharding
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as O
    # where every global row sits: (rank, local row)
    where_rank = np.empty(w["rows_total"], np.int32)
    where_row = np.empty(w["rows_total"], np.int64)
    for sh in w["shards"]:
        local = 0
        for begin, rows in sharding.global_row_ranges(w["sizes"], sh):
            where_rank[begin:begin + rows] = sh.rank
            where_row[begin:begin + rows] = np.arange(local, local + rows)
            local += rows
    cols = w["check"]["cols"]
    cols_t = torch.tensor(cols, device="cuda")
    checked = bad = rows_checked = 0
    results = [None] * len(w["check"]["items"])

    def work(i, it):
        want = O.quant_matmul(it["a"], it["b"], it["scale"], it["pt"], len(it["global_rows"]), len(cols), w["k"],
                              O.ROW_MAJOR, O.ROW_MAJOR)
        results[i] = O.bf16_bits(want)

    threads = [threading.Thread(target=work, args=(i, it)) for i, it in enumerate(w["check"]["items"])]
    for chunk in range(0, len(threads), 16):
        for t in threads[chunk:chunk + 16]:
            t.start()
        for t in threads[chunk:chunk + 16]:
            t.join()
    for it, want_bits in zip(w["check"]["items"], results):
        g_rows = it["global_rows"]
        r = torch.from_numpy(where_rank[g_rows].astype(np.int64)).cuda()
        lr = torch.from_numpy(where_row[g_rows]).cuda()
        got = gathered[r, lr].index_select(1, cols_t).view(torch.int16).cpu().numpy().view(np.uint16)
        bad += int((got != want_bits).sum())
        checked += got.size
        rows_checked += len(g_rows)
    return {"rows_checked": rows_checked, "outputs_checked": checked, "mismatches": bad,
            "columns_per_row": len(cols), "assembled_with": "one NCCL all_gather" if world > 1 else "single shard",
            "oracle": "CPU oracle (pinned to the reference golden), bf16 bits compared"}


def run_moe(args, rank, world, local, sampler):
    import torch
    from catlass_b200 import capi, kernel_facts, sharding
    cfg = MOE_SMALL if args.workload == "moe_small" else MOE
    w = build_moe_rank(rank, world, args.placement, cfg)
    m, n, k, g = w["m"], w["n"], w["k"], w["groups"]

    def step():
        if m > 0:
            capi.grouped_quant_matmul(w["a"], w["b"], w["gl"], w["scale"], w["pt"], w["d"], m, n, k, g,
                                      layout_b=capi.ROW_MAJOR)

    ms, ms_local, launches_timed, win = time_steps(step, args.steps, args.warmup, world)
    clocks = sampler.window(*win) if sampler else None
    check_device_status()
    verify = verify_moe(w, rank, world)

    total_ops = 2.0 * w["rows_total"] * n * k
    ms_step = ms / args.steps
    tops = total_ops / (ms_step * 1e-3) / 1e12
    # dominant kernel: this rank's launch (rank 0 reports its own kernel's roofline)
    rank_ops = 2.0 * m * n * k
    peaks = measured_peaks()
    peak_tops = peaks["bf16_tflops"] * INT8_PER_BF16
    # one step is one launch of the grouped kernel on each rank: this rank's average launch duration over
    # the timed region is its elapsed time / steps
    kernel_ms = ms_local / args.steps
    achieved = rank_ops / (kernel_ms * 1e-3) / 1e12 if m > 0 else 0.0

    # sustained: the same launch for >= 2 s; the 1 kW power cap then holds the SM clock well below its maximum
    time.sleep(0.2)
    sus_steps = max(args.steps, int(np.ceil(args.sustained_seconds * 1e3 / max(ms_step, 1e-3))))
    sus_ms, sus_local, _, sus_win = time_steps(step, sus_steps, 0, world)
    sus_clocks = sampler.window(*sus_win) if sampler else None
    sus_tops = total_ops / (sus_ms / sus_steps * 1e-3) / 1e12
    sus_achieved = rank_ops / (sus_local / sus_steps * 1e-3) / 1e12 if m > 0 else 0.0
    sustained_peak = peaks["bf16_tflops_sustained"] * INT8_PER_BF16

    # tile accounting of this rank's launch: issued MMA work over the work the rows need
    issued_over_needed = w["shards"][rank].cost * sharding.ROW_TILE / max(m, 1)

    # ---- end to end: host buffers in, host buffer out, through the same C-ABI call
    a_h = torch.empty_like(w["a"], device="cpu").pin_memory()
    a_h.copy_(w["a"])
    pt_h = torch.empty_like(w["pt"], device="cpu").pin_memory()
    pt_h.copy_(w["pt"])
    gl_h = torch.empty_like(w["gl"], device="cpu").pin_memory()
    gl_h.copy_(w["gl"])
    d_h = torch.empty_like(w["d"], device="cpu").pin_memory()
    ws = None
    if m > 0:
        ws = torch.empty(capi.grouped_quant_matmul_host_workspace_size(m, n, k, g, args.e2e_chunks),
                         dtype=torch.uint8, device="cuda")

    def e2e_step():
        if m > 0:
            capi.grouped_quant_matmul_host(a_h, gl_h, pt_h, d_h, w["b"], w["scale"], m, n, k, g, ws,
                                           layout_b=capi.ROW_MAJOR, chunks=args.e2e_chunks)

    e2e_steps = max(1, min(args.steps, 10))
    e2e_ms = time_steps(e2e_step, e2e_steps, 1, world)[0] / e2e_steps
    e2e_tops = total_ops / (e2e_ms * 1e-3) / 1e12
    h2d = a_h.numel() * a_h.element_size() + pt_h.numel() * 4 + gl_h.numel() * 8
    d2h = d_h.numel() * d_h.element_size()
    check_device_status()

    result = {
        "metric": "w8a8_grouped_gemm_tops", "value": tops, "unit": "TOPS", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": moe_config(cfg, args.placement, world),
        "roofline": {
            "bound": "tensor", "achieved": achieved, "peak": peak_tops, "unit": "TFLOP/s",
            "frac": achieved / peak_tops if peak_tops else None,
            # DRAM bytes per launch: profiler capture of the 1/8-size case scaled by the rows of this launch
            "traffic": kernel_facts.traffic("w8a8_pair_kernel/moe_small", m / 16384.0) if cfg is MOE else None,
            "kernel": "w8a8_pair_kernel<row-major B>: 256x256 tiles on CTA pairs (rank 0 launch)", "kernel_ms": kernel_ms,
            "peak_source": f"2 x {peaks['source']} cuBLAS bf16 burst ({peaks['bf16_tflops']} TF/s); "
                           "int8 ops = 2*rows*N*K; nominal dense int8 is 4500",
            "frac_of_nominal_int8": achieved / 4500.0,
            "regime": f"burst: {args.steps} launches, {ms:.0f} ms",
            "issued_over_needed_mma_rows": issued_over_needed,
        },
        "sustained": {
            "value": sus_tops, "unit": "TOPS", "steps": sus_steps, "ms_per_step": sus_ms / sus_steps,
            "region_s": sus_ms / 1e3, "achieved_rank0": sus_achieved,
            "frac_of_2x_sustained_bf16": sus_achieved / sustained_peak if sustained_peak else None,
            "frac_of_nominal_int8": sus_achieved / 4500.0, "clocks": sus_clocks,
            "ms_x_sm_mhz": (sus_ms / sus_steps) * sus_clocks["sm_mhz"] if sus_clocks and sus_clocks.get("sm_mhz") else None,
        },
        "e2e": {"value": e2e_tops, "unit": "TOPS", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                "ms_per_step": e2e_ms, "steps": e2e_steps,
                "note": "cb200_grouped_quant_matmul_slice_m_host: activations, per-token scales and group list "
                        "come from pinned host memory and the bf16 output returns to it every step, in row chunks "
                        "whose copy-in, compute and copy-out overlap; expert weights stay resident"},
        "gpu_launches": int(launches_timed),
        "clocks": clocks,
        "verify": verify,
    }
    if clocks and clocks.get("sm_mhz"):
        result["ms_x_sm_mhz"] = ms_step * clocks["sm_mhz"]
    del a_h, d_h, ws
    return result, w


# ------------------------------------------------------------------------------------------ other workloads

def run_dense(name, sampler, seconds):
    import torch
    from catlass_b200 import capi, kernel_facts
    m, n, k = DENSE[name]
    dev = torch.device("cuda")
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1234)
    a = torch.randint(-127, 128, (m, k), dtype=torch.int8, device=dev, generator=gen)
    b = torch.randint(-127, 128, (n, k), dtype=torch.int8, device=dev, generator=gen)  # column-major B
    scale = torch.empty(n, device=dev).uniform_(1e-3, 1e-2, generator=gen)
    pt = torch.empty(m, device=dev).uniform_(1e-3, 1e-2, generator=gen)
    d = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    decode = m <= 128
    # decode shapes are HBM-bound: rotate over enough copies of the weights that a pass never finds its
    # copy in L2 (copies x bytes(B) > 2 x L2), instead of flushing with writes that would leave dirty lines
    copies = int(np.ceil(2 * L2_BYTES / (n * k))) + 1 if decode else 1
    bs = [b] + [b.clone() for _ in range(copies - 1)]

    def launch(i):
        # B is a fixed weight reused across calls (parameters): declared static, so the few-token kernel may
        # stream it while the previous launch drains
        capi.quant_matmul(a, bs[i % copies], scale, pt, d, m, n, k, layout_b=capi.COLUMN_MAJOR, static_weights=True)

    r = graph_region(launch, copies, seconds, sampler)
    check_device_status()
    ops = 2.0 * m * n * k
    nbytes = m * k + k * n + 4 * (m + n) + 2 * m * n
    peaks = measured_peaks()
    ms = r["ms"]
    if decode:
        value, unit, peak, bound = nbytes / (ms * 1e-3) / 1e9, "GB/s", peaks["hbm_gbs"], "hbm"
        burst = nbytes / (r["burst_ms"] * 1e-3) / 1e9
        metric = "w8a8_decode_gemm_hbm_gbs"
        traffic = kernel_facts.traffic("w8a8_smallm_kernel/decode_a") if name == "decode_a" else None
    else:
        value, unit, peak, bound = ops / (ms * 1e-3) / 1e12, "TOPS", peaks["bf16_tflops_sustained"] * INT8_PER_BF16, "tensor"
        burst = ops / (r["burst_ms"] * 1e-3) / 1e12
        metric = "w8a8_dense_gemm_tops"
        traffic = None
    return {
        "name": name, "metric": metric, "value": value, "unit": unit, "ms_per_step": ms,
        "burst_value": burst, "burst_ms_per_step": r["burst_ms"],
        "regime": f"sustained: {r['launches_timed']} launches back to back, {r['region_s']:.2f} s",
        "config": {"workload": f"{name}: W8A8 dequant GEMM M={m} N={n} K={k}, column-major B (static weights), bf16 out",
                   "l2": (f"weights rotate over {copies} copies ({copies * n * k / 1e6:.0f} MB > 2 x L2): every pass reads HBM"
                          if decode else "operands (50 MB) stay in L2: steady state of a reused weight")},
        "roofline": {"bound": bound, "achieved": value, "peak": peak, "unit": "GB/s" if decode else "TFLOP/s",
                     "frac": value / peak, "traffic": traffic,
                     "peak_source": (f"{peaks['source']} HBM copy rate" if decode else
                                     f"2 x {peaks['source']} cuBLAS bf16 sustained ({peaks['bf16_tflops_sustained']} TF/s)"),
                     "burst_frac": burst / (peak if decode else peaks["bf16_tflops"] * INT8_PER_BF16),
                     "algorithmic_bytes": nbytes, "ops": ops,
                     "frac_of_8TBs": value / 8000.0 if decode else None,
                     "frac_of_nominal_int8": None if decode else value / 4500.0},
        "gpu_launches": r["launches_timed"], "cuda_graph": r["cuda_graph"], "clocks": r["clocks"],
    }


def run_w4a8(sampler, seconds, split_k=False, per_tensor=False):
    """M=128, N=8192, K=8192, int4 weights packed along K, HBM-bound.  Scale groups of 128 (the headline W4A8 configuration), or
    one group over the whole K range: the scaling of the reference's own W4A8 example (one rounding of the int32 sum)."""
    import torch
    from catlass_b200 import capi, kernel_facts
    m, n, k = 128, 8192, 8192
    gs = k if per_tensor else 128
    name = "w4a8_per_tensor" if per_tensor else "w4a8"
    dev = torch.device("cuda")
    gen = torch.Generator(device="cuda")
    gen.manual_seed(4321)
    a = torch.randint(-127, 128, (m, k), dtype=torch.int8, device=dev, generator=gen)
    copies = int(np.ceil(2 * L2_BYTES / (n * k // 2))) + 1
    ws = [torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=dev, generator=gen) for _ in range(copies)]
    sw = torch.empty((k // gs, n), device=dev).uniform_(1e-3, 1e-2, generator=gen)
    sa = torch.empty(m, device=dev).uniform_(1e-3, 1e-2, generator=gen)
    d = torch.empty((m, n), dtype=torch.bfloat16, device=dev)

    def launch(i):
        capi.w4a8_matmul(a, ws[i % copies], sw, sa, d, m, n, k, gs, split_k=split_k, static_weights=True)

    r = graph_region(launch, copies, seconds, sampler)
    check_device_status()
    nbytes = m * k + k * n // 2 + 4 * (k // gs) * n + 4 * m + 2 * m * n
    peaks = measured_peaks()
    value = nbytes / (r["ms"] * 1e-3) / 1e9
    burst = nbytes / (r["burst_ms"] * 1e-3) / 1e9
    return {
        "name": name, "metric": "w4a8_gemm_hbm_gbs", "value": value, "unit": "GB/s", "ms_per_step": r["ms"],
        "burst_value": burst, "burst_ms_per_step": r["burst_ms"],
        "regime": f"sustained: {r['launches_timed']} launches back to back, {r['region_s']:.2f} s",
        "config": {"workload": f"{name}: M={m} N={n} K={k} group {gs}, int4 weights packed along K (static weights), bf16 out",
                   "summation": "K split over a CTA cluster, fp32 partial sums reassociated (CB200_W4A8_SPLIT_K)"
                                if split_k else "sequential over the scale groups (default: bit-exact)",
                   "l2": f"weights rotate over {copies} copies: every pass reads HBM"},
        "roofline": {"bound": "hbm", "achieved": value, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": value / peaks["hbm_gbs"],
                     "traffic": None if per_tensor else kernel_facts.traffic("w4a8_gemm_kernel/w4a8"),
                     "peak_source": f"{peaks['source']} HBM copy rate", "burst_frac": burst / peaks["hbm_gbs"],
                     "algorithmic_bytes": nbytes, "frac_of_8TBs": value / 8000.0},
        "gpu_launches": r["launches_timed"], "cuda_graph": r["cuda_graph"], "clocks": r["clocks"],
    }


def run_quant_int8(sampler, seconds):
    """Per-token int8 quantisation of bf16 activations, 32768 x 7168 (a quarter of the MoE workload's routed rows):
    the step in front of the W8A8 matmuls, HBM-bound."""
    import torch
    from catlass_b200 import capi, kernel_facts
    rows, k = 32768, 7168
    dev = torch.device("cuda")
    gen = torch.Generator(device="cuda")
    gen.manual_seed(99)
    copies = 2  # 470 MB of input each: every pass reads HBM
    xs = [torch.randn((rows, k), dtype=torch.float32, device=dev, generator=gen).to(torch.bfloat16) for _ in range(copies)]
    q = torch.empty((rows, k), dtype=torch.int8, device=dev)
    sc = torch.empty((rows,), dtype=torch.float32, device=dev)

    def launch(i):
        capi.quantize_per_token_int8(xs[i % copies], q, sc, rows, k, x_type=capi.DTYPE_BF16)

    r = graph_region(launch, copies, seconds, sampler)
    check_device_status()
    nbytes = 2 * rows * k + rows * k + 4 * rows
    peaks = measured_peaks()
    value = nbytes / (r["ms"] * 1e-3) / 1e9
    burst = nbytes / (r["burst_ms"] * 1e-3) / 1e9
    return {
        "name": "quant_int8", "metric": "quantize_int8_hbm_gbs", "value": value, "unit": "GB/s", "ms_per_step": r["ms"],
        "burst_value": burst, "burst_ms_per_step": r["burst_ms"],
        "regime": f"sustained: {r['launches_timed']} launches back to back, {r['region_s']:.2f} s",
        "config": {"workload": f"quant_int8: bf16 [{rows}][{k}] -> int8 codes + fp32 per-token scales",
                   "l2": f"inputs rotate over {copies} copies of 470 MB: every pass reads HBM"},
        "roofline": {"bound": "hbm", "achieved": value, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": value / peaks["hbm_gbs"],
                     "traffic": kernel_facts.traffic("quant_int8_staged_kernel/quant_int8"),
                     "peak_source": f"{peaks['source']} HBM copy rate", "burst_frac": burst / peaks["hbm_gbs"],
                     "algorithmic_bytes": nbytes, "frac_of_8TBs": value / 8000.0},
        "gpu_launches": r["launches_timed"], "cuda_graph": r["cuda_graph"], "clocks": r["clocks"],
    }


def run_quant_mx(sampler, seconds):
    """MX quantisation (E4M3 codes + E8M0 scales) of bf16 activations, 32768 x 7168: the step in front of the MX
    matmuls, HBM-bound by its bytes, bound by its per-element arithmetic in practice."""
    import torch
    from catlass_b200 import capi, kernel_facts
    rows, k = 32768, 7168
    dev = torch.device("cuda")
    gen = torch.Generator(device="cuda")
    gen.manual_seed(98)
    copies = 2
    xs = [torch.randn((rows, k), dtype=torch.float32, device=dev, generator=gen).to(torch.bfloat16) for _ in range(copies)]
    q = torch.empty((rows, k), dtype=torch.uint8, device=dev)
    sf = torch.empty((rows, k // 32), dtype=torch.uint8, device=dev)

    def launch(i):
        capi.mx_quantize(xs[i % copies], q, sf, rows, k, capi.MX_E4M3, x_type=capi.DTYPE_BF16)

    r = graph_region(launch, copies, seconds, sampler)
    check_device_status()
    nbytes = 2 * rows * k + rows * k + rows * (k // 32)
    peaks = measured_peaks()
    value = nbytes / (r["ms"] * 1e-3) / 1e9
    burst = nbytes / (r["burst_ms"] * 1e-3) / 1e9
    return {
        "name": "quant_mx", "metric": "quantize_mx_hbm_gbs", "value": value, "unit": "GB/s", "ms_per_step": r["ms"],
        "burst_value": burst, "burst_ms_per_step": r["burst_ms"],
        "regime": f"sustained: {r['launches_timed']} launches back to back, {r['region_s']:.2f} s",
        "config": {"workload": f"quant_mx: bf16 [{rows}][{k}] -> E4M3 codes + E8M0 scales per 32 elements",
                   "l2": f"inputs rotate over {copies} copies of 470 MB: every pass reads HBM"},
        "roofline": {"bound": "hbm", "achieved": value, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": value / peaks["hbm_gbs"],
                     "traffic": kernel_facts.traffic("mx_quantize_staged_kernel/quant_mx"),
                     "peak_source": f"{peaks['source']} HBM copy rate", "burst_frac": burst / peaks["hbm_gbs"],
                     "algorithmic_bytes": nbytes, "frac_of_8TBs": value / 8000.0},
        "gpu_launches": r["launches_timed"], "cuda_graph": r["cuda_graph"], "clocks": r["clocks"],
    }


def run_mx(name, sampler, seconds):
    """MXFP8 / MXFP4 block-scaled matmul at M=N=K=8192 (random element codes and exponents: timing only)."""
    import torch
    from catlass_b200 import capi, kernel_facts
    fp4 = name == "mxfp4"
    m = n = k = 8192
    dev = torch.device("cuda")
    gen = torch.Generator(device="cuda")
    gen.manual_seed(88)
    row_bytes = k // 2 if fp4 else k
    # element bytes: any bit pattern is a finite E2M1 pair; for E4M3 clear the exponent's top bit so that no
    # byte is the NaN code 0x7F/0xFF
    a = torch.randint(0, 256, (m, row_bytes), dtype=torch.uint8, device=dev, generator=gen)
    b = torch.randint(0, 256, (n, row_bytes), dtype=torch.uint8, device=dev, generator=gen)
    if not fp4:
        a &= 0xBF
        b &= 0xBF
    sfa = torch.randint(120, 135, (m, k // 32), dtype=torch.uint8, device=dev, generator=gen)
    sfb = torch.randint(120, 135, (n, k // 32), dtype=torch.uint8, device=dev, generator=gen)
    d = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    fmt = capi.MX_E2M1 if fp4 else capi.MX_E4M3
    ws = torch.empty(capi.mx_matmul_workspace_size(m, n, k, fmt), dtype=torch.uint8, device=dev)

    def launch(i):
        capi.mx_matmul(a, b, sfa, sfb, d, m, n, k, fmt, ws)

    r = graph_region(launch, 1, seconds, sampler)
    check_device_status()
    flops = 2.0 * m * n * k
    peaks = measured_peaks()
    factor = 4.0 if fp4 else 2.0   # dense fp4 / fp8 rate relative to bf16 on the same tensor cores
    value = flops / (r["ms"] * 1e-3) / 1e12
    burst = flops / (r["burst_ms"] * 1e-3) / 1e12
    peak = peaks["bf16_tflops_sustained"] * factor
    return {
        "name": name, "metric": "mxfp4_gemm_tflops" if fp4 else "mxfp8_gemm_tflops", "value": value,
        "unit": "TFLOP/s", "ms_per_step": r["ms"], "burst_value": burst, "burst_ms_per_step": r["burst_ms"],
        "regime": f"sustained: {r['launches_timed']} steps back to back, {r['region_s']:.2f} s",
        "config": {"workload": f"{name}: M=N=K=8192 block-scaled (32-element E8M0 blocks), bf16 out, "
                               "step = scale re-tiling + matmul",
                   "l2": "operands exceed L2" if not fp4 else "operands 64 MB + 134 MB output per pass"},
        "roofline": {"bound": "tensor", "achieved": value, "peak": peak, "unit": "TFLOP/s", "frac": value / peak,
                     "traffic": kernel_facts.traffic("mx_pair_kernel/" + name),
                     "peak_source": f"{factor:.0f} x {peaks['source']} cuBLAS bf16 sustained "
                                    f"({peaks['bf16_tflops_sustained']} TF/s)",
                     "burst_frac": burst / (peaks["bf16_tflops"] * factor),
                     "frac_of_nominal": value / (2250.0 * factor)},
        "gpu_launches": r["launches_timed"], "kernels_per_step": r["kernels_per_step"], "cuda_graph": r["cuda_graph"],
        "clocks": r["clocks"],
    }


def run_mx_swiglu(sampler, seconds):
    """Grouped MXFP8 matmul with the SwiGLU + MX quantisation epilogue fused in: the first GEMM of an MoE expert MLP
    (8 experts x 2048 rows, K=7168, gate|up width 4096), E4M3 + E8M0 out.  Random codes and exponents: timing only."""
    import torch
    from catlass_b200 import capi
    g, rows, n, k = 8, 2048, 4096, 7168
    m = g * rows
    dev = torch.device("cuda")
    gen = torch.Generator(device="cuda")
    gen.manual_seed(65)
    a = torch.randint(0, 256, (m, k), dtype=torch.uint8, device=dev, generator=gen) & 0xBF
    b = torch.randint(0, 256, (g, n, k), dtype=torch.uint8, device=dev, generator=gen) & 0xBF
    sfa = torch.randint(120, 130, (m, k // 32), dtype=torch.uint8, device=dev, generator=gen)
    sfb = torch.randint(120, 130, (g, n, k // 32), dtype=torch.uint8, device=dev, generator=gen)
    gl = torch.full((g,), rows, dtype=torch.int64, device=dev)
    q = torch.empty((m, n // 2), dtype=torch.uint8, device=dev)
    qs = torch.empty((m, n // 64), dtype=torch.uint8, device=dev)
    ws = torch.empty(capi.mx_grouped_swiglu_quant_workspace_size(m, n, k, g), dtype=torch.uint8, device=dev)

    def launch(i):
        capi.mx_grouped_swiglu_quant(a, b, gl, sfa, sfb, q, qs, m, n, k, g, ws)

    r = graph_region(launch, 1, seconds, sampler)
    check_device_status()
    flops = 2.0 * m * n * k
    peaks = measured_peaks()
    value = flops / (r["ms"] * 1e-3) / 1e12
    burst = flops / (r["burst_ms"] * 1e-3) / 1e12
    peak = peaks["bf16_tflops_sustained"] * 2.0
    return {
        "name": "mx_swiglu", "metric": "mxfp8_grouped_swiglu_quant_tflops", "value": value, "unit": "TFLOP/s",
        "ms_per_step": r["ms"], "burst_value": burst, "burst_ms_per_step": r["burst_ms"],
        "regime": f"sustained: {r['launches_timed']} steps back to back, {r['region_s']:.2f} s",
        "config": {"workload": f"mx_swiglu: grouped slice-M MXFP8, {g} experts x {rows} rows, K={k}, N={n} "
                               "(act | gate), SwiGLU + MX quantisation in the epilogue, E4M3 + E8M0 out; "
                               "step = group planning + scale re-tiling + matmul",
                   "l2": "operands exceed L2 (A 117 MB, B 235 MB)"},
        "roofline": {"bound": "tensor", "achieved": value, "peak": peak, "unit": "TFLOP/s", "frac": value / peak,
                     "traffic": None,
                     "peak_source": f"2 x {peaks['source']} cuBLAS bf16 sustained ({peaks['bf16_tflops_sustained']} TF/s)",
                     "burst_frac": burst / (peaks["bf16_tflops"] * 2.0), "frac_of_nominal": value / 4500.0},
        "gpu_launches": r["launches_timed"], "kernels_per_step": r["kernels_per_step"], "cuda_graph": r["cuda_graph"],
        "clocks": r["clocks"],
    }


def run_mx_routing(sampler, seconds):
    """Grouped MXFP8 matmul with the finalize-routing epilogue fused in: the second GEMM of an MoE expert MLP
    (2048 tokens x top-8 = 16384 routed rows over 8 experts, K=2048, N=7168), every row weighted and added into its
    token's fp32 output row.  Random codes and exponents: timing only."""
    import torch
    from catlass_b200 import capi
    g, rows, n, k, batch = 8, 2048, 7168, 2048, 2048
    m = g * rows
    dev = torch.device("cuda")
    gen = torch.Generator(device="cuda")
    gen.manual_seed(71)
    a = torch.randint(0, 256, (m, k), dtype=torch.uint8, device=dev, generator=gen) & 0xBF
    b = torch.randint(0, 256, (g, n, k), dtype=torch.uint8, device=dev, generator=gen) & 0xBF
    sfa = torch.randint(120, 130, (m, k // 32), dtype=torch.uint8, device=dev, generator=gen)
    sfb = torch.randint(120, 130, (g, n, k // 32), dtype=torch.uint8, device=dev, generator=gen)
    gl = torch.full((g,), rows, dtype=torch.int64, device=dev)
    logit = torch.rand(m, device=dev, generator=gen)
    row_index = torch.randperm(m, device=dev, generator=gen) % batch     # every token meets top-8 rows
    bias = torch.randn((g, n), device=dev, generator=gen).to(torch.bfloat16)
    out = torch.empty((batch, n), dtype=torch.float32, device=dev)
    ws = torch.empty(capi.mx_grouped_finalize_routing_workspace_size(m, n, k, g, batch), dtype=torch.uint8, device=dev)

    def launch(i):
        capi.mx_grouped_finalize_routing(a, b, gl, sfa, sfb, logit, row_index, out, m, n, k, g, batch, ws, bias=bias)

    r = graph_region(launch, 1, seconds, sampler)
    check_device_status()
    flops = 2.0 * m * n * k
    peaks = measured_peaks()
    value = flops / (r["ms"] * 1e-3) / 1e12
    burst = flops / (r["burst_ms"] * 1e-3) / 1e12
    peak = peaks["bf16_tflops_sustained"] * 2.0
    return {
        "name": "mx_routing", "metric": "mxfp8_grouped_finalize_routing_tflops", "value": value, "unit": "TFLOP/s",
        "ms_per_step": r["ms"], "burst_value": burst, "burst_ms_per_step": r["burst_ms"],
        "regime": f"sustained: {r['launches_timed']} steps back to back, {r['region_s']:.2f} s",
        "config": {"workload": f"mx_routing: grouped slice-M MXFP8, {g} experts x {rows} rows, K={k}, N={n}, rows "
                               f"weighted and added into {batch} fp32 token rows (vector atomics in the epilogue), "
                               "bf16 bias; step = output init + group planning + scale re-tiling + matmul",
                   "l2": "B 117 MB streams; the 59 MB output stays in L2"},
        "roofline": {"bound": "tensor", "achieved": value, "peak": peak, "unit": "TFLOP/s", "frac": value / peak,
                     "traffic": None,
                     "peak_source": f"2 x {peaks['source']} cuBLAS bf16 sustained ({peaks['bf16_tflops_sustained']} TF/s)",
                     "burst_frac": burst / (peaks["bf16_tflops"] * 2.0), "frac_of_nominal": value / 4500.0},
        "gpu_launches": r["launches_timed"], "kernels_per_step": r["kernels_per_step"], "cuda_graph": r["cuda_graph"],
        "clocks": r["clocks"],
    }


def run_secondary(name, sampler, seconds, args):
    if name == "mx_swiglu":
        return run_mx_swiglu(sampler, seconds)
    if name == "mx_routing":
        return run_mx_routing(sampler, seconds)
    if name in DENSE:
        return run_dense(name, sampler, seconds)
    if name == "quant_int8":
        return run_quant_int8(sampler, seconds)
    if name == "quant_mx":
        return run_quant_mx(sampler, seconds)
    if name in ("w4a8", "w4a8_per_tensor"):
        return run_w4a8(sampler, seconds, split_k=bool(args.w4a8_split_k), per_tensor=name == "w4a8_per_tensor")
    return run_mx(name, sampler, seconds)


def standalone_line(entry, args):
    """A secondary workload run on its own (--workload NAME) as a full bench line."""
    line = {"metric": entry["metric"], "value": entry["value"], "unit": entry["unit"], "n_gpus": 1,
            "steps": entry["gpu_launches"], "warmup": args.warmup, "ms_per_step": entry["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": {"w4a8": "int4xint8->int32->f32", "w4a8_per_tensor": "int4xint8->int32->f32", "quant_int8": "bf16->int8", "quant_mx": "bf16->e4m3xe8m0", "mxfp8": "e4m3xe8m0", "mxfp4": "e2m1xe8m0"}.get(entry["name"], "int8"),
            "data": "synthetic"}
    line.update({k: v for k, v in entry.items() if k not in ("name", "metric", "value", "unit", "ms_per_step")})
    return line


def run_reference(args):
    """The reference arm: the reference's CPU golden on the host cores, bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return None
    cfg = MOE
    per_step = max(1.0, min(args.cpu_seconds, 60.0 / max(args.steps + args.warmup, 1)))
    vals, secs_all = [], []
    sample = kind = None
    cores = 1
    for i in range(args.warmup + args.steps):
        v, cores, kind, sample, secs = cpu_reference_rate(cfg["n"], cfg["k"], per_step)
        if i >= args.warmup:
            vals.append(v)
            secs_all.append(secs)
    value = float(np.mean(vals))
    config = moe_config(cfg, args.placement, args.gpus)
    config["measured_on"] = "the reference's CPU golden, a bounded row sample of this workload per step"
    return {
        "impl": "reference", "metric": "w8a8_grouped_gemm_tops", "value": value, "unit": "TOPS",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": float(np.mean(secs_all)) * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": config,
        "cpu_baseline": {"value": value, "unit": "TOPS", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="moe", choices=["moe", "moe_small"] + SECONDARY)
    ap.add_argument("--placement", default="split", choices=["split", "whole"])
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="moe workload: skip the other workloads of the metric")
    ap.add_argument("--sustained-seconds", type=float, default=2.0)
    ap.add_argument("--secondary-seconds", type=float, default=1.6)
    ap.add_argument("--e2e-chunks", type=int, default=0, help="row chunks of the host-buffer pipeline (0 = default)")
    ap.add_argument("--w4a8-split-k", action="store_true",
                    help="w4a8 workload: time the opt-in split-K mode instead of the bit-exact default")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    if args.impl == "reference":
        res = run_reference(args)
        if res is not None:
            print(json.dumps(res), flush=True)
        return

    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    from catlass_b200 import capi
    capi.load()  # fails loudly when the CUDA library is missing
    rank, world, local = dist_setup(args.gpus)
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.wait_first_sample()
    try:
        if args.workload in ("moe", "moe_small"):
            res, w = run_moe(args, rank, world, local, sampler)
            if rank == 0 and world == 1:
                n, k = w["n"], w["k"]
                del w
                torch.cuda.empty_cache()
                if args.workload == "moe" and not args.no_secondary:
                    res["secondary"] = [run_secondary(name, sampler, args.secondary_seconds, args) for name in SECONDARY]
                if not args.no_cpu_baseline:
                    v, cores, kind, sample, secs = cpu_reference_rate(n, k, args.cpu_seconds)
                    res["cpu_baseline"] = {"value": v, "unit": "TOPS", "cores": cores, "kind": kind, "sample": sample,
                                           "seconds": secs}
        else:
            if world != 1:
                raise SystemExit("this workload is single-GPU")
            res = standalone_line(run_secondary(args.workload, sampler, max(args.secondary_seconds, 0.01), args), args)
    finally:
        if sampler:
            sampler.stop()
    if rank == 0:
        print(json.dumps(res), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
