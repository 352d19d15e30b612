#!/usr/bin/env python
"""Benchmark of the contraction hot path: descriptor -> plan -> prepare -> timed launches.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg5|cfg2|cfg3|cfg4|cfg1]
                    [--scaling strong|weak] [--split external|contracted] [--split-mode M] [--impl reference]

A step is one contraction launch.  The default workload is the large TF32 contraction (all six
extents 128, 8.8 TFLOP), cut over the N ranks along the external mode `a` (strong scaling: rank r
owns a[r*128/N, (r+1)*128/N) of A and of C, no collective on the data path).  With N > 1 the script
is started by torch.distributed.run, one rank per GPU.  Rank 0 prints one JSON line; besides the
headline workload it carries one sub-record each for the other performance configurations
(`configs`: the TF32 3-D contraction, the FP64 6-D contraction cut along `a`, the bandwidth-bound
TF32 5-D contraction), every one with its own CUDA-event timing, roofline, end-to-end figure and
parity verdict.

`--impl reference` times the reference's own CPU contraction (its OpenMP verification loop,
compiled from its sources into oracle/_ref; the repository's CPU restatement when that file is
absent or the mode pattern is none of the reference's cases) on the host cores, on a bounded slab
of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# workload -> modes, extents, scalar (0 Float32/TF32, 1 FP64), seed, input range, the mode cut under
# weak and under strong scaling, roofline bound, and the slab (mode, extent) the CPU baseline is timed on
WORKLOADS = {
    "cfg1": dict(C="abcd", A="aebf", B="fdec", ext=dict(a=24, b=24, c=24, d=24, e=16, f=16), st=1, seed=0, lo=-1.0, hi=1.0,
                 weak="d", strong="d", bound="tensor", cpu=("d", 24)),
    "cfg2": dict(C="abc", A="adc", B="db", ext=dict(a=256, c=256, b=1024, d=1024), st=0, seed=1, lo=-1.0, hi=1.0,
                 weak="c", strong="c", bound="tensor", cpu=("c", 64)),
    "cfg3": dict(C="abcijk", A="aeij", B="bcek", ext=dict(a=48, b=48, c=48, e=48, i=24, j=24, k=24), st=1, seed=2, lo=-0.5, hi=0.5,
                 weak="k", strong="a", bound="tensor", cpu=("k", 8)),
    "cfg4": dict(C="abcde", A="efba", B="cfd", ext=dict(a=48, b=48, c=48, d=48, e=48, f=8), st=0, seed=3, lo=-1.0, hi=1.0,
                 weak="d", strong="d", bound="hbm", cpu=("d", 48)),
    "cfg5": dict(C="abcd", A="aebf", B="cfde", ext=dict(a=128, b=128, c=128, d=128, e=128, f=128), st=0, seed=4, lo=-1.0, hi=1.0,
                 weak="d", strong="a", bound="tensor", cpu=("d", 1)),
}
# DRAM bytes per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum) as captured with ncu
# on one GPU and summarised in the named file under profiles/; not measured by this run.
NCU_TRAFFIC = {
    "cfg5": (22.12e9, "profiles/umma_tf32_kernel_cfg5_full_dram.md"),
    "cfg2": (507.6e6, "profiles/umma_tf32_kernel_cfg2.md"),
    "cfg4": (964.4e6, "profiles/umma_tf32_kernel_cfg4.md"),
    "cfg3": (6 * (1980.4e6 + 53.7e6), "profiles/dmma_tma_kernel_cfg3.md (k=4 capture scaled by the tile count)"),
}
REF_CASE = {"cfg1": 21, "cfg2": 18}   # reference loop nests with the same mode pattern (tccg_verify.cpp:660-689, :567-592)
SUB_RECORDS = [("cfg2", "weak", 50), ("cfg3", "strong", 20), ("cfg4", "weak", 50)]   # (workload, scaling at N > 1, timed steps)
PARITY_SAMPLES = 100_000


def describe(name, ext=None):
    w = WORKLOADS[name]
    e = ",".join(f"{k}={v}" for k, v in sorted((ext or w["ext"]).items()))
    return (f"{name}: C[{','.join(w['C'])}]=sum A[{','.join(w['A'])}]*B[{','.join(w['B'])}] {e} "
            f"{'FP64' if w['st'] else 'TF32'} column-major")


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


REASON_BITS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}


def summarise_clock_samples(samples, windows):
    """samples: (time, gpu index, sm MHz, max sm MHz, power W, reasons bit mask) tuples read from NVML while the
    benchmark runs; windows: {name: (t0, t1)} host-clock brackets of the timed regions.  Returns the `clocks`
    object: the median SM clock under load (inside the headline timed region; the upper half of everything seen if that
    region holds no sample), the throttle reasons seen at all and
    those seen inside the headline timed region, and per window its sample count, median clock and reasons."""
    def reasons_of(rows):
        out = set()
        for r in rows:
            for bit, name in REASON_BITS.items():
                if r[5] & bit:
                    out.add(name)
        return sorted(out)

    def busy_median(rows):
        sm = sorted(r[2] for r in rows)
        busy = sm[len(sm) // 2:]
        return statistics.median(busy) if busy else None

    out = {"sm_mhz": busy_median(samples), "sm_max_mhz": max((r[3] for r in samples), default=None),
           "reasons": reasons_of(samples), "samples": len(samples), "power_w_max": max((r[4] for r in samples), default=None)}
    per = {}
    for name, (t0, t1) in windows.items():
        rows = [r for r in samples if t0 <= r[0] <= t1]
        per[name] = {"samples": len(rows), "sm_mhz": statistics.median(r[2] for r in rows) if rows else None,
                     "reasons": reasons_of(rows), "seconds": t1 - t0}
    head = per.get("headline", {"samples": 0, "reasons": [], "sm_mhz": None})
    # "under load" is the headline timed region where it holds samples: an idle GPU (during the CPU legs of the run)
    # shows the maximum clock, a power-capped one under load a lower one
    if head["samples"]:
        out["sm_mhz"] = head["sm_mhz"]
    out["samples_in_timed_region"] = head["samples"]
    out["reasons_in_timed_region"] = head["reasons"]
    out["sm_mhz_in_timed_region"] = head["sm_mhz"]
    out["windows"] = per
    return out


class ClockSampler:
    """Reads SM clock, power and throttle reasons of the job's GPUs from NVML every few milliseconds in a
    thread (read-only queries), so that even a timed region of some tens of milliseconds holds samples."""

    def __init__(self, gpu_indices, period_s=0.004):
        self.gpus, self.period = list(gpu_indices), period_s
        self.samples, self.windows = [], {}
        self._stop = threading.Event()
        self._thread = None
        self.error = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = [int(x) for x in visible.split(",")] if visible and all(x.strip().isdigit() for x in visible.split(",")) else None
            handles = [(g, pynvml.nvmlDeviceGetHandleByIndex(phys[g] if phys and g < len(phys) else g)) for g in self.gpus]
            smax = {g: float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)) for g, h in handles}
            get_reasons = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
        except Exception as e:   # no NVML in this process: the record says so
            self.error = f"NVML unavailable: {e}"
            return

        def loop():
            while not self._stop.is_set():
                for g, h in handles:
                    try:
                        self.samples.append((time.time(), g, float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)), smax[g],
                                             pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0, int(get_reasons(h))))
                    except Exception:
                        pass
                self._stop.wait(self.period)

        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()

    def window(self, name, t0, t1):
        self.windows[name] = (t0, t1)

    def reasons_between(self, t0, t1):
        """Throttle reasons NVML reported between two host times (the samples taken so far)."""
        out = set()
        for r in list(self.samples):
            if t0 <= r[0] <= t1:
                out.update(name for bit, name in REASON_BITS.items() if r[5] & bit)
        return sorted(out)

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2.0)
        if self.error:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [self.error], "samples": 0, "samples_in_timed_region": 0,
                    "reasons_in_timed_region": []}
        return summarise_clock_samples(list(self.samples), self.windows)


def cpu_baseline(name: str):
    """The reference's CPU contraction on a slab of the workload. Returns (dict, tflops)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from oracle_lib import Contraction, Oracle, RefVerifier
    w = WORKLOADS[name]
    ext = dict(w["ext"])
    smode, sext = w["cpu"]
    full = ext[smode]
    ext[smode] = min(sext, full)
    c = Contraction(w["C"], w["A"], w["B"], ext, w["st"])
    oracle = Oracle()
    # all the cores this process may run on, whatever OMP_NUM_THREADS the launcher exported
    # (torch.distributed.run sets it to 1 for several ranks)
    oracle.set_num_threads(len(os.sched_getaffinity(0)))
    A, B = oracle.inputs(c, w["seed"], w["lo"], w["hi"])
    sample = f"{name} with {smode}={ext[smode]} of {full} (a {ext[smode]}/{full} slab of the outputs, all other modes full)"
    use_ref = RefVerifier.available() and name in REF_CASE
    if use_ref:
        ref = RefVerifier()
        out = np.zeros(c.size(c.modeC), dtype=c.dtype)
        sys.stdout.flush()
        saved = os.dup(1)
        devnull = os.open(os.devnull, os.O_WRONLY)
        os.dup2(devnull, 1)                      # the reference prints its comparison report to stdout
        try:
            t0 = time.perf_counter()
            ref.verify(REF_CASE[name], c, out, A, B)
            dt = time.perf_counter() - t0
        finally:
            os.dup2(saved, 1)
            os.close(devnull)
            os.close(saved)
        kind = "reference"
        sample += "; timed through the reference's verify_tccg_case, comparator pass included"
    else:
        t0 = time.perf_counter()
        oracle.contract(c, A, B)
        dt = time.perf_counter() - t0
        kind = "port"
    tflops = c.flops() / dt / 1e12
    return {"value": tflops, "unit": "TFLOP/s", "cores": oracle.num_threads(), "kind": kind, "sample": sample,
            "seconds": dt}, tflops


def run_reference(args, name):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals = []
    info = None
    for _ in range(max(1, min(args.warmup, 1))):
        cpu_baseline(name)
    for _ in range(max(1, min(args.steps, 3))):
        info, v = cpu_baseline(name)
        vals.append(v)
    v = statistics.mean(vals)
    info["value"] = v
    line = {"impl": "reference", "metric": "contraction throughput", "value": v, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": len(vals), "warmup": 1, "ms_per_step": info["seconds"] * 1e3, "higher_is_better": True, "scaling": args.scaling,
            "vs_baseline": None, "dtype": "f64",
            "data": "synthetic", "config": {"workload": describe(name)}, "cpu_baseline": info,
            "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


class Job:
    """Process-wide state of one benchmark run: rank layout, the distributed helpers, the clock sampler."""

    def __init__(self, torch, dist, rank, world):
        self.torch, self.dist, self.rank, self.world = torch, dist, rank, world
        self.sampler = None

    def sync_all(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
            self.torch.cuda.synchronize()

    def reduce(self, value, op):
        t = self.torch.tensor([value], device="cuda", dtype=self.torch.float64)
        if self.world > 1:
            self.dist.all_reduce(t, op=getattr(self.dist.ReduceOp, op))
        return float(t.item())


def parity_verdict(job, local_eq, A, B, out, kernel, seed):
    """Correctness evidence outside the timed region, on this rank's own slice: PARITY_SAMPLES sampled
    outputs against the CPU oracle (the checker, never the thing measured).  FP64 and plain FP32: the
    reference criterion (benchmarks/tccg/tccg_verify.cpp:1620-1701) must hold on every sample.  TF32
    tensor-core results get two verdicts: the count and fraction of samples outside the reference criterion
    against the double oracle (format error of a single TF32 pass on signed inputs), and the worst
    |out - TF32-operand oracle| / sum|a b| (accumulation error only: what a kernel bug would break)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from oracle_lib import F32, F64, Contraction, Oracle
    c = Contraction(local_eq.modeC, local_eq.modeA, local_eq.modeB, dict(local_eq.extent), int(local_eq.scalar_type))
    oracle = Oracle()
    oracle.set_num_threads(max(1, len(os.sched_getaffinity(0)) // job.world))
    n = min(max(PARITY_SAMPLES // job.world, 20_000), out.size)     # PARITY_SAMPLES over the whole job, 20 000 per rank at least
    idx = np.sort(np.random.default_rng(seed + 17 * job.rank).integers(0, out.size, size=n)) if n < out.size else np.arange(out.size)
    got = out[idx].astype(np.float64)
    finite = bool(np.isfinite(got).all())
    v = {"samples_per_rank": int(n), "criterion": "reference comparator: FP64 abs 1e-11 / rel 1e-9, Float32 abs 2e-3 / rel 5e-2"}
    if c.scalar_type == F64:
        diff, nonfinite = oracle.compare(oracle.contract_sampled(c, A, B, idx), got, F64)
        worst = None
    else:
        diff, nonfinite = oracle.compare(oracle.contract_sampled(c, A, B, idx, rounding=0), got, F32)
        tensor = kernel == "umma_tf32"
        ref = oracle.contract_sampled(c, A, B, idx, rounding=1 if tensor else 0)
        scale = oracle.contract_sampled(c, np.abs(A), np.abs(B), idx, rounding=1)
        worst = float((np.abs(got - ref) / (scale + 1e-30)).max())
    diff_all = job.reduce(float(diff), "SUM")
    bad_all = job.reduce(float(nonfinite) + (0.0 if finite else 1.0), "SUM")
    n_all = job.reduce(float(n), "SUM")
    v.update({"samples": int(n_all), "outside_reference_criterion": int(diff_all), "fraction_outside": diff_all / max(n_all, 1.0),
              "non_finite": int(bad_all), "ranks_checked": job.world})
    if worst is not None:
        w_all = job.reduce(worst, "MAX")
        v["worst_error_over_sum_abs_products"] = w_all
        v["against"] = ("TF32-operand oracle (operands truncated as the tensor core does, double accumulation)"
                        if kernel == "umma_tf32" else "double oracle")
        v["pass"] = bool(bad_all == 0 and w_all < 2e-5 and (diff_all == 0 if kernel != "umma_tf32" else diff_all <= 0.005 * n_all))
    else:
        v["pass"] = bool(diff_all == 0 and bad_all == 0)
    return v


def contracted_parity(job, full_eq, A, B, mine, first, kernel, seed):
    """Parity of a contracted-mode split: this rank's range of the SUMMED C (elements first .. first+len(mine) of the
    whole tensor) against the oracle on the whole contraction, on sampled elements; same two verdicts as parity_verdict."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from oracle_lib import F32, Contraction, Oracle
    c = Contraction(full_eq.modeC, full_eq.modeA, full_eq.modeB, dict(full_eq.extent), int(full_eq.scalar_type))
    oracle = Oracle()
    oracle.set_num_threads(max(1, len(os.sched_getaffinity(0)) // job.world))
    n = min(max(PARITY_SAMPLES // job.world, 20_000), mine.size)
    local = np.sort(np.random.default_rng(seed + 31 * job.rank).integers(0, mine.size, size=n))
    idx = local + first
    got = mine[local].astype(np.float64)
    diff, nonfinite = oracle.compare(oracle.contract_sampled(c, A, B, idx, rounding=0), got, F32)
    ref = oracle.contract_sampled(c, A, B, idx, rounding=1 if kernel == "umma_tf32" else 0)
    scale = oracle.contract_sampled(c, np.abs(A), np.abs(B), idx, rounding=1)
    worst = job.reduce(float((np.abs(got - ref) / (scale + 1e-30)).max()), "MAX")
    diff_all, bad_all, n_all = job.reduce(float(diff), "SUM"), job.reduce(float(nonfinite), "SUM"), job.reduce(float(n), "SUM")
    return {"samples": int(n_all), "outside_reference_criterion": int(diff_all), "fraction_outside": diff_all / max(n_all, 1.0),
            "non_finite": int(bad_all), "worst_error_over_sum_abs_products": worst, "ranks_checked": job.world,
            "pass": bool(bad_all == 0 and worst < 2e-5 and diff_all <= 0.005 * n_all)}


def run_workload(job, args, name, scaling, split, split_mode, steps, warmup, tag, peaks, tf32_peak, e2e_steps, with_cpu):
    """One workload: shard, plan, prepare, warm up, time `steps` launches with CUDA events, then (untimed)
    single-launch spread, the end-to-end leg through the host-buffer entry point, the parity verdict and the
    CPU baseline.  Returns the record (rank 0) or None."""
    torch, dist = job.torch, job.dist
    import tcont_b200 as tc
    from tcont_b200 import api, sharding
    w = WORKLOADS[name]
    rank, world = job.rank, job.world
    ext = dict(w["ext"])
    changed = []
    for ov in (args.extent if tag == "headline" else []):
        m, v = ov.split("=")
        if m not in ext:
            raise SystemExit(f"--extent: workload {name} has no mode '{m}'")
        ext[m] = int(v)
        changed.append(ov)
    mC, mA, mB, st = w["C"], w["A"], w["B"], w["st"]
    sel = {"model": 0, "cogent": 1, "ttgt": 2}[args.backend]
    full_eq = tc.TCEquation(mC, mA, mB, dict(ext), "-", tc.ScalarType(st), tc.BackendSelection(sel))
    if split.startswith("contracted") and world == 1:
        split, split_mode = "external", None     # one GPU: nothing to sum across
    contracted = split.startswith("contracted")
    fused = contracted and split == "contracted"
    if contracted:
        scaling = "strong"
        shard_mode = split_mode or next(m for m in mA if m not in mC)
        local_eq, sl = sharding.shard_contracted(full_eq, shard_mode, world, rank)
        global_eq = full_eq
    elif scaling == "strong":
        shard_mode = split_mode or w["strong"]
        local_eq, sl = sharding.shard_equation(full_eq, shard_mode, world, rank)
        global_eq = full_eq
    else:
        shard_mode = split_mode or w["weak"]
        local_eq, sl = full_eq, None
        global_eq = sharding.grow_equation(local_eq, shard_mode, world)
    # Inputs: the global tensors come from one seeded stream (A at offset 0, B behind it).  Under strong
    # scaling every rank generates the global operand that carries the cut mode and keeps its slice;
    # under weak scaling the cut mode is the slowest one of its carrier, so a rank's slice is a contiguous
    # range of the stream and is generated directly.
    nA, nB = local_eq.size(mA), local_eq.size(mB)
    gA = global_eq.size(mA)
    a_cut, b_cut = shard_mode in mA, shard_mode in mB

    whole = {}

    def operand(modes, n_local, n_global, cut, base):
        if not cut or world == 1:
            return tc.fill_uniform(n_local, local_eq.scalar_type, w["seed"], base, w["lo"], w["hi"])
        if scaling == "strong":
            full = tc.fill_uniform(n_global, local_eq.scalar_type, w["seed"], base, w["lo"], w["hi"])
            if contracted:
                whole[modes] = full      # the parity check of a contracted split needs the global operands
            return sharding.take_slice(full, modes, global_eq.extent, shard_mode, sl)
        return tc.fill_uniform(n_local, local_eq.scalar_type, w["seed"], base + rank * n_local, w["lo"], w["hi"])

    A = operand(mA, nA, gA, a_cut, 0)
    B = operand(mB, nB, global_eq.size(mB), b_cut, gA)
    plan = tc.plan(local_eq)
    desc = plan.describe()
    nC = local_eq.size(mC)
    elt = 8 if st else 4
    if fused:
        # Contracted-mode split, fused: the kernel stores every partial tile straight into the owner's staging
        # slots over NVLink (peer stores; the staging areas are exchanged as CUDA IPC handles), a one-element
        # all-reduce on the same stream is the barrier among the ranks, then every owner adds its slots up.
        dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
        reduced = torch.empty(nC // world, dtype=dA.dtype, device="cuda")
        run = api.prepare_on_device(plan, dA.data_ptr(), dB.data_ptr(), reduced.data_ptr(), keep=(dA, dB, reduced))
        run.set_stream(torch.cuda.current_stream().cuda_stream)
        run.ksplit_enable(world, rank)
        handles = [None] * world
        dist.all_gather_object(handles, run.ksplit_export())
        for r in range(world):
            if r != rank:
                run.ksplit_import(r, handles[r])
        flag = torch.zeros(1, device="cuda")
    elif contracted:
        # the same split with the library collective: a full-size partial C per rank, then ncclReduceScatter
        # (partial C and its output live in torch tensors; the engine works on them in place on torch's
        # current stream, so the NCCL call is ordered behind the kernel)
        dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
        partial = torch.empty(nC, dtype=dA.dtype, device="cuda")
        reduced = torch.empty(nC // world, dtype=dA.dtype, device="cuda")
        run = api.prepare_on_device(plan, dA.data_ptr(), dB.data_ptr(), partial.data_ptr(), keep=(dA, dB, partial))
        run.set_stream(torch.cuda.current_stream().cuda_stream)
    else:
        run = tc.prepare(plan, A, B)

    def step():
        tc.launch(run)
        if fused:
            dist.all_reduce(flag)
            run.ksplit_reduce()
        elif contracted:
            dist.reduce_scatter_tensor(reduced, partial)

    for _ in range(warmup):
        step()
    job.sync_all()
    t_host0 = time.time()
    if contracted:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        launches = steps * (1 + int(desc["transpose_a"] is not None) + int(desc["transpose_b"] is not None) + int(fused))
    else:
        ms, launches = run.time_launches(steps)
    t_host1 = time.time()
    job.sync_all()
    capped = False
    if job.sampler is not None:
        job.sampler.window(tag, t_host0, t_host1)
        capped = "sw_power_cap" in job.sampler.reasons_between(t_host0, t_host1)
    ms_total = job.reduce(ms, "MAX")
    extra_steps = 0
    if tag == "headline" and ms_total < 300.0:
        # The same step repeated, untimed, until about 0.3 s of this load have been sampled: shows the clock the
        # chip settles at under the workload (the count comes from the all-reduced time: equal on every rank).
        extra_steps = min(100_000, int(300.0 / max(ms_total / steps, 1e-3)) + 1)
        t2 = time.time()
        for _ in range(extra_steps):
            step()
        job.sync_all()
        if job.sampler is not None:
            job.sampler.window("untimed_repeats", t2, time.time())
    if run.device_status() != 0:
        raise SystemExit("a kernel reported a timed-out wait; the numbers are invalid")
    ms_step = ms_total / steps
    flops_local = plan.flops
    value = world * flops_local / (ms_step * 1e-3) / 1e12

    # spread of single launches (the reference's per-iteration harness reports min and stddev,
    # benchmarks/test/tccg/bench_tccg_iter.cpp:218-233); outside the timed region
    launch_stats = None
    if not contracted:
        one = [run.time_launches(1)[0] for _ in range(min(20, max(steps, 1)))]
        mean = sum(one) / len(one)
        launch_stats = {"n": len(one), "min_ms": min(one), "mean_ms": mean,
                        "std_ms": (sum((x - mean) ** 2 for x in one) / len(one)) ** 0.5}

    # end to end through the host-buffer entry point: pinned host A, B -> device, launch, C -> pinned host
    hA = torch.from_numpy(A).pin_memory()
    hB = torch.from_numpy(B).pin_memory()
    hC = torch.empty(nC, dtype=hA.dtype).pin_memory()
    split_check = None
    if contracted:
        # the summed result of the split, this rank's range of C, against the oracle on the WHOLE contraction
        torch.cuda.synchronize()
        if not args.no_parity:
            split_check = contracted_parity(job, full_eq, whole.get(mA, A), whole.get(mB, B), reduced.cpu().numpy(), rank * (nC // world),
                                            desc["kernel"], w["seed"])
        del run
        run = tc.prepare(plan, A, B)   # the end-to-end leg measures the host-buffer entry point of one rank's share
    run.contract_host_ptr(hA.data_ptr(), hB.data_ptr(), hC.data_ptr())
    job.sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    h2d = d2h = 0
    for _ in range(e2e_steps):
        h2d, d2h = run.contract_host_ptr(hA.data_ptr(), hB.data_ptr(), hC.data_ptr())
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = job.reduce(e0.elapsed_time(e1) / e2e_steps, "MAX")
    e2e_value = world * flops_local / (e2e_ms * 1e-3) / 1e12
    out = hC.numpy()
    parity = parity_verdict(job, local_eq, A, B, out, desc["kernel"], w["seed"]) if not args.no_parity else None
    del run, hA, hB, hC
    torch.cuda.empty_cache()
    if rank != 0:
        return None

    alg_bytes = (nA + nB + nC) * elt
    extra = {}
    if w["bound"] == "tensor":
        achieved = flops_local / (ms_step * 1e-3) / 1e12
        unit = "TFLOP/s"
        if st == 0:
            # TF32 dense rate is half the bf16 rate of the same tensor cores, so the driver-measured cuBLAS bf16
            # figures, halved, are the denominators: the sustained one for a timed region that ran on the power cap
            # (NVML reported sw_power_cap inside it: seconds of back-to-back tensor work), the burst one otherwise.
            # Both fractions are printed whichever `frac` uses, and beside them the fraction of this process's own
            # tcgen05 microbenchmark (resident zero operands, no loads: an upper bound no kernel that moves data reaches).
            peak = peaks["bf16_tflops_sustained" if capped else "bf16_tflops"] / 2.0
            source = peaks["source"] + (" sustained (sw_power_cap seen in the timed region)" if capped else " burst") + " bf16 dense / 2 (TF32 rate)"
            extra["frac_of_burst_bf16_half"] = achieved / (peaks["bf16_tflops"] / 2.0)
            extra["frac_of_sustained_bf16_half"] = achieved / (peaks["bf16_tflops_sustained"] / 2.0)
            if tf32_peak:
                extra["tcgen05_tf32_peak_microbenchmark"] = tf32_peak
                extra["frac_of_tcgen05_microbenchmark"] = achieved / tf32_peak
        else:
            # the peaks file has no FP64 entry: measured here, mma.sync m8n8k4 on every SM at once
            peak = max(api.measure_peak("fp64_dmma"), api.measure_peak("fp64_dfma"))
            source = "FP64 microbenchmark run by this process (max of mma.sync m8n8k4 and DFMA)"
            extra["hbm_write_floor_ms"] = nC * elt / (peaks["hbm_gbs"] * 1e9) * 1e3
        bound_used = "tensor"
    else:
        bound_used, peak, unit = "hbm", peaks["hbm_gbs"], "GB/s"
        achieved = alg_bytes / (ms_step * 1e-3) / 1e9
        source = peaks["source"] + " copy bandwidth"
    traffic, traffic_src = NCU_TRAFFIC.get(name, (None, None)) if (world == 1 and not changed) else (None, None)
    roofline = {"bound": bound_used, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
                "traffic": traffic, "traffic_source": traffic_src, "kernel": desc["kernel"], "peak_source": source,
                "algorithmic_bytes_per_launch": alg_bytes, "flops_per_launch": flops_local, **extra}
    rec = {"value": value, "unit": "TFLOP/s", "steps": steps, "warmup": warmup, "ms_per_step": ms_step, "scaling": scaling,
           "dtype": "f64" if st else "tf32",
           "config": {"workload": describe(name, ext) + (" (changed: " + ",".join(changed) + ")" if changed else ""),
                      "global": {shard_mode: int(global_eq.extent[shard_mode])}, "local": {shard_mode: int(local_eq.extent[shard_mode])},
                      "sharded_mode": shard_mode, "split": split, "backend": desc["backend"], "kernel": desc["kernel"],
                      "l2": "inputs and output exceed the 126 MB L2" if alg_bytes > 126e6 else "working set fits L2; launches back to back",
                      "timing": "CUDA events on the launching stream, max over ranks"},
           "gpu_launches": int(launches), "launch_stats": launch_stats,
           "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                   "ms_per_step": e2e_ms, "steps": e2e_steps},
           "roofline": roofline, "parity": parity}
    if extra_steps:
        rec["untimed_repeats_for_the_clock_record"] = extra_steps
    if contracted:
        rec["config"]["collective"] = {
            "op": ("none: partial tiles stored straight into the owner's slots over NVLink by the contraction kernel (peer stores), "
                   "one-element all-reduce as the barrier, owners add their slots; all inside the timed region") if fused
            else "ncclReduceScatter sum over NVLink, after every launch, inside the timed region",
            "nvlink_bytes_sent_per_gpu_per_step": int((world - 1) / world * nC * elt)}
        rec["parity_of_the_summed_result"] = split_check
    if with_cpu:
        rec["cpu_baseline"], _ = cpu_baseline(name)
    return rec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="cfg5", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--backend", default="model", choices=["model", "cogent", "ttgt"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the sampled parity verdicts (profiling runs)")
    ap.add_argument("--no-configs", action="store_true", help="headline workload only, no sub-records for the other configurations")
    ap.add_argument("--e2e-steps", type=lambda v: max(1, int(v)), default=3, help="passes through the host-buffer entry point (at least 1)")
    ap.add_argument("--extent", action="append", default=[], metavar="MODE=N",
                    help="override one extent of the workload (repeatable), e.g. --workload cfg5 --extent e=16 for a "
                         "case small enough to profile; the JSON line then names the changed extents")
    ap.add_argument("--scaling", default="strong", choices=["weak", "strong"],
                    help="strong (default): the named configuration is cut into N slices; weak: every rank runs the named "
                         "configuration and the global problem grows with N")
    ap.add_argument("--split", default="external", choices=["external", "contracted", "contracted-nccl"],
                    help="contracted: cut a contracted mode; every rank's kernel stores its partial tiles straight into the "
                         "owners' memory over NVLink and the owners add them up (strong scaling only); contracted-nccl: the "
                         "same split with a full-size partial C per rank and ncclReduceScatter, for comparison")
    ap.add_argument("--split-mode", default=None, help="mode letter to cut (default: `a` for the sharded configurations, else the "
                                                       "slowest external mode; for --split contracted the first contracted mode of A)")
    args = ap.parse_args()
    name = args.workload
    if args.impl == "reference":
        run_reference(args, name)
        return

    import torch
    import torch.distributed as dist

    from tcont_b200 import api

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU path (use --impl reference for the CPU baseline)")
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    job = Job(torch, dist, rank, world)
    peaks = measured_peaks()
    warmup = max(args.warmup, 3)
    # tcgen05 TF32 microbenchmark on this process's GPU (resident operands, no loads), before anything is timed
    tf32_peak = api.measure_peak("tf32") if rank == 0 else None
    if rank == 0:
        job.sampler = ClockSampler(range(world))
        job.sampler.start()
    with_cpu = world == 1 and not args.no_cpu_baseline and not args.extent
    head = run_workload(job, args, name, args.scaling, args.split, args.split_mode, args.steps, warmup, "headline", peaks, tf32_peak,
                        args.e2e_steps, with_cpu)
    subs = {}
    if not args.no_configs and not args.extent and args.split == "external":
        for sub, sub_scaling, sub_steps in SUB_RECORDS:
            if sub == name:
                continue
            rec = run_workload(job, args, sub, sub_scaling if world > 1 else "strong", "external", None, sub_steps, warmup, sub, peaks,
                               tf32_peak, 2, with_cpu)
            if rec is not None:
                subs[sub] = rec
    if rank == 0:
        clocks = job.sampler.stop()
        line = {"metric": "contraction throughput", "value": head["value"], "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
                "warmup": warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": head["scaling"],
                "vs_baseline": None, "dtype": head["dtype"], "data": "synthetic", "config": head["config"], "clocks": clocks,
                "gpu_launches": head["gpu_launches"], "launch_stats": head["launch_stats"], "e2e": head["e2e"],
                "roofline": head["roofline"], "parity": head["parity"]}
        if "cpu_baseline" in head:
            line["cpu_baseline"] = head["cpu_baseline"]
        if "parity_of_the_summed_result" in head:
            line["parity_of_the_summed_result"] = head["parity_of_the_summed_result"]
        if subs:
            line["configs"] = subs
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
