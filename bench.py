#!/usr/bin/env python
"""Benchmark of the quantized-matmul path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload: the MoE grouped slice-M W8A8 matmul (64 experts, K=7168, N=4096, 131072 routed rows,
Zipf(1.1) expert loads), expert/row-sharded over the N ranks with no collective on the data path.
One step = one pass over all routed rows.  Prints ONE JSON line on rank 0.

Other workloads (single GPU): prefill (4096^3), decode_a (16x14336x4096), decode_b (16x4096x14336).

`--impl reference` times the reference's own CPU golden (compiled from the reference tree into
oracle/_ref, else the oracle's plain-C restatement) on the host cores, on a bounded row sample per step.
"""
import argparse
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
# same law, 1/8 of the experts and rows: small enough for multi-pass ncu captures, still larger than L2
MOE_SMALL = dict(experts=8, k=7168, n=4096, tokens=2048, top_k=8, zipf_s=1.1, seed=20240)
DENSE = {
    "prefill": (4096, 4096, 4096),
    "decode_a": (16, 14336, 4096),
    "decode_b": (16, 4096, 14336),
}
INT8_PER_BF16 = 2.0  # kind::i8 issues at twice the bf16 rate on the same tensor cores


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


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(gpu_index), f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for name, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


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
    Returns (max over ranks of the elapsed ms, this rank's elapsed ms, library launches in the timed region)."""
    import torch
    from catlass_b200 import capi
    for _ in range(warmup):
        fn()
    barrier(world)
    launches0 = capi.launch_count()
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop)
    launches = capi.launch_count() - launches0
    barrier(world)
    return max_over_ranks(ms, world), ms, launches


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


# ------------------------------------------------------------------------------------------ workloads

def build_moe_rank(rank, world, mode, cfg):
    """Device buffers of this rank's shard of the MoE workload."""
    import torch
    from catlass_b200 import sharding
    rows_total = cfg["tokens"] * cfg["top_k"]
    sizes = zipf_group_sizes(rows_total, cfg["experts"], cfg["seed"], cfg["zipf_s"])
    shards = sharding.plan(sizes, world, mode=mode)
    mine = shards[rank]
    groups = mine.local_groups()
    gl = np.cumsum([r for _, r in groups]).astype(np.int64)
    m = int(gl[-1]) if len(gl) else 0
    n, k = cfg["n"], cfg["k"]
    gen = torch.Generator(device="cuda")
    gen.manual_seed(cfg["seed"] + 1000 * rank)
    dev = torch.device("cuda")
    a = torch.randint(-127, 128, (max(m, 1), k), dtype=torch.int8, device=dev, generator=gen)
    b = torch.randint(-127, 128, (max(len(groups), 1), k, n), dtype=torch.int8, device=dev, generator=gen)
    scale = torch.empty((max(len(groups), 1), n), device=dev).uniform_(1e-3, 1e-2, generator=gen)
    pt = torch.empty(max(m, 1), device=dev).uniform_(1e-3, 1e-2, generator=gen)
    d = torch.empty((max(m, 1), n), dtype=torch.bfloat16, device=dev)
    gl_dev = torch.from_numpy(gl if len(gl) else np.zeros(1, np.int64)).to(dev)
    loads = [s.rows for s in shards]
    return dict(a=a, b=b, scale=scale, pt=pt, d=d, gl=gl_dev, m=m, n=n, k=k, groups=len(groups),
                rows_total=rows_total, loads=loads, sizes=sizes)


def run_moe(args, rank, world, local):
    import torch
    from catlass_b200 import capi
    cfg = MOE_SMALL if args.workload == "moe_small" else MOE
    w = build_moe_rank(rank, world, args.placement, cfg)
    m, n, k, g = w["m"], w["n"], w["k"], w["groups"]

    def step():
        if m > 0:
            capi.grouped_quant_matmul(w["a"], w["b"], w["gl"], w["scale"], w["pt"], w["d"], m, n, k, g,
                                      layout_b=capi.ROW_MAJOR)

    sampler = ClockSampler(local) if rank == 0 else None
    ms, ms_local, launches_timed = time_steps(step, args.steps, args.warmup, world)
    clocks = sampler.stop() if sampler else None
    st, code = capi.device_status()
    if st != 0:
        raise SystemExit(f"device status {st} code {code:#x}")

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

    # ---- end to end: host buffers in, host buffer out, through the same C-ABI call
    a_h = torch.empty_like(w["a"], device="cpu").pin_memory()
    a_h.copy_(w["a"])
    pt_h = torch.empty_like(w["pt"], device="cpu").pin_memory()
    pt_h.copy_(w["pt"])
    gl_h = torch.empty_like(w["gl"], device="cpu").pin_memory()
    gl_h.copy_(w["gl"])
    d_h = torch.empty_like(w["d"], device="cpu").pin_memory()

    # the library's host-buffer entry: rows are cut into chunks, copy-in / compute / copy-out overlap on
    # separate streams, the device staging buffers live in the workspace
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

    result = {
        "metric": "w8a8_grouped_gemm_tops", "value": tops, "unit": "TOPS", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {
            "workload": f"moe_grouped_slice_m_w8a8: {cfg['experts']} experts, K={k}, N={n}, {cfg['tokens']} tokens x "
                        f"top-{cfg['top_k']} = {w['rows_total']} rows, Zipf({cfg['zipf_s']}) expert loads, "
                        "B row-major [G,K,N], bf16 out",
            "placement": args.placement, "rows_per_rank": w["loads"],
            "l2": f"inputs exceed L2 ({(w['rows_total'] * (k + 2 * n) + cfg['experts'] * k * n) / 1e9:.2f} GB per pass)",
            "weights": "resident in HBM across steps",
        },
        "roofline": {
            "bound": "tensor", "achieved": achieved, "peak": peak_tops, "unit": "TFLOP/s",
            "frac": achieved / peak_tops if peak_tops else None,
            # DRAM bytes per launch: ncu capture of the 1/8-size `moe_small` case (540.2 MB, see profiles/),
            # scaled by the rows this launch processes (traffic is proportional to rows and experts)
            "traffic": 540.2e6 * m / 16384.0 if cfg is MOE else None,
            "kernel": "w8a8_pair_kernel<row-major B>: 256x256 tiles on CTA pairs (rank 0 launch)", "kernel_ms": kernel_ms,
            "peak_source": f"2 x {peaks['source']} cuBLAS bf16 burst ({peaks['bf16_tflops']} TF/s); "
                           "int8 ops = 2*rows*N*K; nominal dense int8 is 4500",
            "frac_of_nominal_int8": achieved / 4500.0,
        },
        "e2e": {"value": e2e_tops, "unit": "TOPS", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                "ms_per_step": e2e_ms, "steps": e2e_steps,
                "note": "cb200_grouped_quant_matmul_slice_m_host: activations, per-token scales and group list "
                        "come from pinned host memory and the bf16 output returns to it every step, in row chunks "
                        "whose copy-in, compute and copy-out overlap; expert weights stay resident"},
        "gpu_launches": int(launches_timed),
        "clocks": clocks,
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        v, cores, kind, sample, secs = cpu_reference_rate(n, k, args.cpu_seconds)
        result["cpu_baseline"] = {"value": v, "unit": "TOPS", "cores": cores, "kind": kind, "sample": sample,
                                  "seconds": secs}
    return result


def run_dense(args, rank, world, local):
    import torch
    from catlass_b200 import capi
    m, n, k = DENSE[args.workload]
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
    copies = 1
    if decode:
        copies = int(np.ceil(2 * 126e6 / (n * k))) + 1
    bs = [b] + [b.clone() for _ in range(copies - 1)]
    it = [0]

    def step():
        capi.quant_matmul(a, bs[it[0] % copies], scale, pt, d, m, n, k, layout_b=capi.COLUMN_MAJOR)
        it[0] += 1

    for _ in range(max(args.warmup, copies)):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    launches0 = capi.launch_count()
    # keep the GPU busy while the host enqueues the K timed launches: otherwise the events would time the
    # host's launch path (tens of microseconds in Python) instead of kernels that last ten
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda._sleep(int(2.0e6 * args.steps) + 10_000_000)
    s0.record()
    for _ in range(args.steps):
        step()
    s1.record()
    torch.cuda.synchronize()
    times = [s0.elapsed_time(s1) / args.steps]
    launches = capi.launch_count() - launches0
    clocks = sampler.stop()
    st, code = capi.device_status()
    if st != 0:
        raise SystemExit(f"device status {st} code {code:#x}")
    ms = float(np.mean(times))
    ops = 2.0 * m * n * k
    nbytes = m * k + k * n + 4 * (m + n) + 2 * m * n
    peaks = measured_peaks()
    if decode:
        achieved, peak, unit, bound = nbytes / (ms * 1e-3) / 1e9, peaks["hbm_gbs"], "GB/s", "hbm"
        metric, value, vunit = "w8a8_decode_gemm_hbm_gbs", achieved, "GB/s"
    else:
        achieved, peak, unit, bound = ops / (ms * 1e-3) / 1e12, peaks["bf16_tflops"] * INT8_PER_BF16, "TFLOP/s", "tensor"
        metric, value, vunit = "w8a8_dense_gemm_tops", achieved, "TOPS"
    return {
        "metric": metric, "value": value, "unit": vunit, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
        "data": "synthetic",
        "config": {"workload": f"{args.workload}: W8A8 dequant GEMM M={m} N={n} K={k}, column-major B, bf16 out",
                   "l2": (f"weights rotate over {copies} copies ({copies * n * k / 1e6:.0f} MB > 2 x L2): every pass reads HBM"
                          if decode else "inputs fit L2; steady state")},
        "roofline": {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
                     "traffic": None, "peak_source": peaks["source"], "algorithmic_bytes": nbytes, "ops": ops,
                     "frac_of_8TBs": achieved / 8000.0 if decode else None},
        "gpu_launches": int(launches), "clocks": clocks,
    }


def run_w4a8(args, rank, world, local):
    """M=128, N=8192, K=8192, group 128: int4 weights packed along K, HBM-bound."""
    import torch
    from catlass_b200 import capi
    m, n, k, gs = 128, 8192, 8192, 128
    dev = torch.device("cuda")
    gen = torch.Generator(device="cuda")
    gen.manual_seed(4321)
    a = torch.randint(-127, 128, (m, k), dtype=torch.int8, device=dev, generator=gen)
    copies = int(np.ceil(2 * 126e6 / (n * k // 2))) + 1
    ws = [torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=dev, generator=gen) for _ in range(copies)]
    sw = torch.empty((k // gs, n), device=dev).uniform_(1e-3, 1e-2, generator=gen)
    sa = torch.empty(m, device=dev).uniform_(1e-3, 1e-2, generator=gen)
    d = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    it = [0]

    split_k = bool(getattr(args, "w4a8_split_k", False))

    def step():
        capi.w4a8_matmul(a, ws[it[0] % copies], sw, sa, d, m, n, k, gs, split_k=split_k)
        it[0] += 1

    for _ in range(max(args.warmup, copies)):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    launches0 = capi.launch_count()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda._sleep(int(2.0e6 * args.steps) + 10_000_000)
    s0.record()
    for _ in range(args.steps):
        step()
    s1.record()
    torch.cuda.synchronize()
    ms = s0.elapsed_time(s1) / args.steps
    launches = capi.launch_count() - launches0
    clocks = sampler.stop()
    st, code = capi.device_status()
    if st != 0:
        raise SystemExit(f"device status {st} code {code:#x}")
    nbytes = m * k + k * n // 2 + 4 * (k // gs) * n + 4 * m + 2 * m * n
    peaks = measured_peaks()
    achieved = nbytes / (ms * 1e-3) / 1e9
    return {
        "metric": "w4a8_gemm_hbm_gbs", "value": achieved, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int4xint8->int32->f32", "data": "synthetic",
        "config": {"workload": f"w4a8: M={m} N={n} K={k} group {gs}, int4 weights packed along K, bf16 out",
                   "summation": "K split over a CTA cluster, fp32 partial sums reassociated (CB200_W4A8_SPLIT_K)"
                                if split_k else "sequential over the scale groups (default: bit-exact)",
                   "l2": f"weights rotate over {copies} copies: every pass reads HBM"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm_gbs"], "traffic": None, "peak_source": peaks["source"],
                     "algorithmic_bytes": nbytes, "frac_of_8TBs": achieved / 8000.0},
        "gpu_launches": int(launches), "clocks": clocks,
    }


def run_mx(args, rank, world, local):
    """MXFP8 / MXFP4 block-scaled matmul at M=N=K=8192 (random element codes and exponents: timing only)."""
    import torch
    from catlass_b200 import capi
    fp4 = args.workload == "mxfp4"
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

    def step():
        capi.mx_matmul(a, b, sfa, sfb, d, m, n, k, fmt, ws)

    sampler = ClockSampler(local)
    ms, _, launches = time_steps(step, args.steps, args.warmup, 1)
    clocks = sampler.stop()
    st, code = capi.device_status()
    if st != 0:
        raise SystemExit(f"device status {st} code {code:#x}")
    ms /= args.steps
    flops = 2.0 * m * n * k
    peaks = measured_peaks()
    factor = 4.0 if fp4 else 2.0   # dense fp4 / fp8 rate relative to bf16 on the same tensor cores
    achieved = flops / (ms * 1e-3) / 1e12
    peak = peaks["bf16_tflops"] * factor
    return {
        "metric": "mxfp4_gemm_tflops" if fp4 else "mxfp8_gemm_tflops", "value": achieved, "unit": "TFLOP/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "e2m1xe8m0" if fp4 else "e4m3xe8m0", "data": "synthetic",
        "config": {"workload": f"{args.workload}: M=N=K=8192 block-scaled (32-element E8M0 blocks), bf16 out, "
                               "step = scale re-tiling (2 launches) + matmul",
                   "l2": "operands exceed L2" if not fp4 else "operands 64 MB + 134 MB output per pass"},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                     "traffic": None, "peak_source": f"{factor:.0f} x {peaks['source']} cuBLAS bf16 burst"},
        "gpu_launches": int(launches), "clocks": clocks,
    }


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
    return {
        "impl": "reference", "metric": "w8a8_grouped_gemm_tops", "value": value, "unit": "TOPS",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": float(np.mean(secs_all)) * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {
            "workload": f"moe_grouped_slice_m_w8a8: {cfg['experts']} experts, K={cfg['k']}, N={cfg['n']}, "
                        f"{cfg['tokens']} tokens x top-{cfg['top_k']} = {cfg['tokens'] * cfg['top_k']} rows, "
                        f"Zipf({cfg['zipf_s']}) expert loads, B row-major [G,K,N], bf16 out",
            "measured_on": "the reference's CPU golden, a bounded row sample of this workload per step",
        },
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
    ap.add_argument("--workload", default="moe", choices=["moe", "moe_small", "w4a8", "mxfp8", "mxfp4"] + sorted(DENSE))
    ap.add_argument("--placement", default="split", choices=["split", "whole"])
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
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
    if args.workload in ("moe", "moe_small"):
        res = run_moe(args, rank, world, local)
    elif args.workload == "w4a8":
        res = run_w4a8(args, rank, world, local)
    elif args.workload in ("mxfp8", "mxfp4"):
        res = run_mx(args, rank, world, local)
    else:
        if world != 1:
            raise SystemExit("dense workloads are single-GPU")
        res = run_dense(args, rank, world, local)
    if rank == 0:
        print(json.dumps(res), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
