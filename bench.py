#!/usr/bin/env python
"""Benchmark of the contraction hot path: descriptor -> plan -> prepare -> timed launches.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2|cfg3|cfg4|cfg5|cfg1] [--impl reference]

A step is one contraction launch.  With N > 1 (started by torch.distributed.run, one rank per
GPU) the contraction is cut along an external output mode: every rank owns a slice, no
collective is on the data path, and the global problem grows with N (weak scaling).  Rank 0
prints one JSON line.

`--impl reference` times the reference's own CPU contraction (its OpenMP verification loop,
compiled from its sources into oracle/_ref; the repository's CPU restatement when that file is
absent) on the host cores, on a bounded slab of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# workload -> (modeC, modeA, modeB, extents, scalar, seed, lo, hi, shard mode, roofline bound, cpu-sample mode, cpu-sample extent)
WORKLOADS = {
    "cfg1": ("abcd", "aebf", "fdec", dict(a=24, b=24, c=24, d=24, e=16, f=16), 1, 0, -1.0, 1.0, "d", "tensor", "d", 24),
    "cfg2": ("abc", "adc", "db", dict(a=256, c=256, b=1024, d=1024), 0, 1, -1.0, 1.0, "c", "tensor", "c", 64),
    "cfg3": ("abcijk", "aeij", "bcek", dict(a=48, b=48, c=48, e=48, i=24, j=24, k=24), 1, 2, -0.5, 0.5, "k", "tensor", "k", 1),
    "cfg4": ("abcde", "efba", "cfd", dict(a=48, b=48, c=48, d=48, e=48, f=8), 0, 3, -1.0, 1.0, "d", "hbm", "d", 24),
    "cfg5": ("abcd", "aebf", "cfde", dict(a=128, b=128, c=128, d=128, e=128, f=128), 0, 4, -1.0, 1.0, "d", "tensor", "d", 1),
}
# DRAM bytes per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum) from the ncu
# captures summarised under profiles/; None where no capture of that workload exists.
NCU_TRAFFIC = {"cfg2": 501.7e6, "cfg4": 964.4e6, "cfg3": 6 * (1980.4e6 + 53.7e6)}  # cfg3: k=4 capture scaled by the tile count
REF_CASE = {"cfg1": 21, "cfg2": 18}   # reference loop nests with the same mode pattern (tccg_verify.cpp:660-689, :567-592)


def describe(name):
    mC, mA, mB, ext, st, *_ = WORKLOADS[name]
    e = ",".join(f"{k}={v}" for k, v in sorted(ext.items()))
    return f"{name}: C[{','.join(mC)}]=sum A[{','.join(mA)}]*B[{','.join(mB)}] {e} {'FP64' if st else 'TF32'} column-major"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def summarise_clock_samples(lines, gpu_indices, t_mark=None):
    """nvidia-smi CSV lines (timestamp, index, clocks.sm, clocks.max.sm, power, active mask, four reasons) -> the
    `clocks` object.  Samples stamped up to `t_mark` (seconds since the epoch, local time) belong to the timed region;
    their throttle reasons are also reported on their own."""
    import datetime
    sm, smax, reasons, reasons_timed, n_timed = [], [], set(), set(), 0
    names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    for line in lines:
        f = [x.strip() for x in line.split(",")]
        if len(f) < 10 or not f[1].isdigit() or int(f[1]) not in gpu_indices:
            continue
        try:
            sm.append(float(f[2]))
            smax.append(float(f[3]))
        except ValueError:
            continue
        timed = False
        if t_mark is not None:
            try:
                timed = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp() <= t_mark
            except ValueError:
                timed = False
        n_timed += int(timed)
        for n, v in zip(names, f[6:10]):
            if v.lower().startswith("active"):
                reasons.add(n)
                if timed:
                    reasons_timed.add(n)
    # samples under load only: the upper half of what was seen
    sm.sort()
    busy = sm[len(sm) // 2:] if sm else []
    return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(smax) if smax else None,
            "reasons": sorted(reasons), "samples": len(sm), "samples_in_timed_region": n_timed,
            "reasons_in_timed_region": sorted(reasons_timed)}


class ClockSampler:
    """nvidia-smi clock/throttle samples taken while the timed region runs."""

    FIELDS = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc, self.path, self.t_mark = None, None, None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def mark(self):
        """The timed region ends here; later samples see untimed repeats of the same load."""
        self.t_mark = time.time()

    def stop(self, gpu_indices):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        self.proc.wait()
        with open(self.path) as f:
            out = summarise_clock_samples(f.readlines(), gpu_indices, self.t_mark)
        os.unlink(self.path)
        return out


def cpu_baseline(name: str, max_seconds: float = 60.0):
    """The reference's CPU contraction on a slab of the workload. Returns (dict, tflops)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from oracle_lib import Contraction, Oracle, RefVerifier
    mC, mA, mB, ext, st, seed, lo, hi, _, _, smode, sext = WORKLOADS[name]
    ext = dict(ext)
    full = ext[smode]
    ext[smode] = min(sext, full)
    c = Contraction(mC, mA, mB, ext, st)
    oracle = Oracle()
    # all the cores this process may run on, whatever OMP_NUM_THREADS the launcher exported
    # (torch.distributed.run sets it to 1 for several ranks)
    oracle.set_num_threads(len(os.sched_getaffinity(0)))
    A, B = oracle.inputs(c, seed, lo, hi)
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
    mC, mA, mB, ext, st, *_ = WORKLOADS[name]
    line = {"impl": "reference", "metric": "contraction throughput", "value": v, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": len(vals), "warmup": 1, "ms_per_step": info["seconds"] * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f64",
            "data": "synthetic", "config": {"workload": describe(name)}, "cpu_baseline": info,
            "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--backend", default="model", choices=["model", "cogent", "ttgt"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--e2e-steps", type=lambda v: max(1, int(v)), default=5, help="passes through the host-buffer entry point (at least 1)")
    ap.add_argument("--extent", action="append", default=[], metavar="MODE=N",
                    help="override one extent of the workload (repeatable), e.g. --workload cfg3 --extent k=4 for a "
                         "case small enough to profile; the JSON line then names the changed extents")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="weak: the global problem grows with N (default); strong: the named configuration is cut into N slices")
    ap.add_argument("--split", default="external", choices=["external", "contracted"],
                    help="contracted: cut a contracted mode; every rank produces a full-size partial C and an NCCL "
                         "reduce-scatter over NVLink adds them (strong scaling only)")
    ap.add_argument("--split-mode", default=None, help="mode letter to cut (default: the workload's slowest external mode; "
                                                       "for --split contracted the first contracted mode of A)")
    args = ap.parse_args()
    name = args.workload
    if args.impl == "reference":
        run_reference(args, name)
        return

    import torch
    import torch.distributed as dist

    import tcont_b200 as tc
    from tcont_b200 import api, sharding

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU path (use --impl reference for the CPU baseline)")
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    mC, mA, mB, ext, st, seed, lo, hi, shard_mode, bound, _, _ = WORKLOADS[name]
    ext = dict(ext)
    for ov in args.extent:
        m, v = ov.split("=")
        if m not in ext:
            raise SystemExit(f"--extent: workload {name} has no mode '{m}'")
        ext[m] = int(v)
    sel = {"model": 0, "cogent": 1, "ttgt": 2}[args.backend]
    full_eq = tc.TCEquation(mC, mA, mB, dict(ext), "-", tc.ScalarType(st), tc.BackendSelection(sel))
    contracted = args.split == "contracted"
    if contracted:
        args.scaling = "strong"
        shard_mode = args.split_mode or next(m for m in mA if m not in mC)
        local_eq, _ = sharding.shard_contracted(full_eq, shard_mode, world, rank)
        global_eq = full_eq
    elif args.scaling == "strong":
        shard_mode = args.split_mode or shard_mode
        local_eq, _ = sharding.shard_equation(full_eq, shard_mode, world, rank)
        global_eq = full_eq
    else:
        shard_mode = args.split_mode or shard_mode
        local_eq = full_eq
        global_eq = sharding.grow_equation(local_eq, shard_mode, world)
    # every rank generates its own slice of the global inputs: a sharded operand at the rank's
    # offset of the stream, a shared operand identically everywhere
    nA, nB = local_eq.size(mA), local_eq.size(mB)
    a_sharded, b_sharded = shard_mode in mA, shard_mode in mB
    A = tc.fill_uniform(nA, local_eq.scalar_type, seed, rank * nA if a_sharded else 0, lo, hi)
    offB = world * nA if a_sharded else nA
    B = tc.fill_uniform(nB, local_eq.scalar_type, seed, offB + (rank * nB if b_sharded else 0), lo, hi)
    plan = tc.plan(local_eq)
    desc = plan.describe()
    nC = local_eq.size(mC)
    if contracted:
        # partial C and the reduce-scatter output live in torch tensors; the engine works on them in
        # place on torch's current stream, so the NCCL call is ordered behind the kernel
        dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
        partial = torch.empty(nC, dtype=dA.dtype, device="cuda")
        reduced = torch.empty(nC // world, dtype=dA.dtype, device="cuda")
        run = api.prepare_on_device(plan, dA.data_ptr(), dB.data_ptr(), partial.data_ptr(), keep=(dA, dB, partial))
        run.set_stream(torch.cuda.current_stream().cuda_stream)
    else:
        run = tc.prepare(plan, A, B)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def step():
        tc.launch(run)
        if contracted and world > 1:
            dist.reduce_scatter_tensor(reduced, partial)

    for _ in range(max(args.warmup, 3)):
        step()
    sampler = ClockSampler()
    if rank == 0:
        sampler.start()
    sync_all()
    if contracted:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        ms, launches = e0.elapsed_time(e1), args.steps * (1 + int(desc["transpose_a"] is not None) + int(desc["transpose_b"] is not None))
    else:
        ms, launches = run.time_launches(args.steps)
    sync_all()
    sampler.mark()
    # nvidia-smi samples every 100 ms; a timed region of a few milliseconds would leave one sample or none.
    # The same step is then repeated, untimed, until the sampler has seen about 0.6 s of this load.
    t = torch.tensor([ms], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())
    extra_steps = 0
    if ms_total < 600.0:   # (the count comes from the all-reduced time, so every rank repeats equally often)
        extra_steps = min(200_000, int(600.0 / max(ms_total / args.steps, 1e-3)) + 1)
        for _ in range(extra_steps):
            step()
        sync_all()
    clocks = sampler.stop(set(range(world))) if rank == 0 else None
    if clocks is not None:
        clocks["window"] = "timed region" + (f" + {extra_steps} untimed repeats of the same step" if extra_steps else "")
    if run.device_status() != 0:
        raise SystemExit("a kernel reported a timed-out wait; the numbers are invalid")
    ms_step = ms_total / args.steps
    flops_local = plan.flops
    value = world * flops_local / (ms_step * 1e-3) / 1e12
    if contracted:
        nccl_bytes = (world - 1) / world * nC * (8 if st else 4)   # leaves each GPU in the reduce-scatter

    # spread of single launches (the reference's per-iteration harness reports min and stddev,
    # benchmarks/test/tccg/bench_tccg_iter.cpp:218-233); outside the timed region
    launch_stats = None
    if not contracted:
        one = [run.time_launches(1)[0] for _ in range(min(20, max(args.steps, 1)))]
        mean = sum(one) / len(one)
        launch_stats = {"n": len(one), "min_ms": min(one), "mean_ms": mean,
                        "std_ms": (sum((x - mean) ** 2 for x in one) / len(one)) ** 0.5}

    # end to end through the host-buffer entry point: pinned host A, B -> device, launch, C -> pinned host
    hA = torch.from_numpy(A).pin_memory()
    hB = torch.from_numpy(B).pin_memory()
    hC = torch.empty(local_eq.size(mC), dtype=hA.dtype).pin_memory()
    if contracted:
        run = tc.prepare(plan, A, B)   # the end-to-end leg measures the host-buffer entry point of one rank's share
    run.contract_host_ptr(hA.data_ptr(), hB.data_ptr(), hC.data_ptr())
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    h2d = d2h = 0
    for _ in range(args.e2e_steps):
        h2d, d2h = run.contract_host_ptr(hA.data_ptr(), hB.data_ptr(), hC.data_ptr())
    e1.record()
    torch.cuda.synchronize()
    te = torch.tensor([e0.elapsed_time(e1) / args.e2e_steps], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_ms = float(te.item())
    e2e_value = world * flops_local / (e2e_ms * 1e-3) / 1e12
    checksum = float(hC[:: max(1, hC.numel() // 4096)].double().abs().sum())

    if rank == 0:
        peaks = measured_peaks()
        elt = 8 if st else 4
        alg_bytes = (nA + nB + local_eq.size(mC)) * elt
        extra = {}
        if bound == "tensor":
            achieved = flops_local / (ms_step * 1e-3) / 1e12
            unit = "TFLOP/s"
            if st == 0:
                # TF32 dense rate is half the bf16 rate of the same tensor cores.  A timed region that
                # ran into the power cap (seconds of back-to-back tensor work, cfg5) is held against the
                # sustained figure, a short one against the burst figure.
                # (only samples stamped inside the timed region decide; the untimed repeats that follow a short region
                # for the clock record's sake may reach the cap although the timed launches did not)
                capped = bool(clocks and "sw_power_cap" in (clocks.get("reasons_in_timed_region") or []))
                peak = peaks["bf16_tflops_sustained" if capped else "bf16_tflops"] / 2.0
                source = peaks["source"] + (" sustained" if capped else " burst") + " bf16 dense / 2 (TF32 rate)"
                extra["tcgen05_tf32_peak_microbenchmark"] = 1113.9  # tcontb_measure_peak(0) on this pool's B200, resident operands
            else:
                # the peaks file has no FP64 entry: measured here, mma.sync m8n8k4 on every SM at once
                peak = max(api.measure_peak("fp64_dmma"), api.measure_peak("fp64_dfma"))
                source = "FP64 microbenchmark run by this process (max of mma.sync m8n8k4 and DFMA)"
                extra["hbm_write_floor_ms"] = local_eq.size(mC) * elt / (peaks["hbm_gbs"] * 1e9) * 1e3
            bound_used = "tensor"
        else:
            bound_used, peak, unit = "hbm", peaks["hbm_gbs"], "GB/s"
            achieved = alg_bytes / (ms_step * 1e-3) / 1e9
            source = peaks["source"] + " copy bandwidth"
        roofline = {"bound": bound_used, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
                    "traffic": NCU_TRAFFIC.get(name), "kernel": desc["kernel"], "peak_source": source,
                    "algorithmic_bytes_per_launch": alg_bytes, "flops_per_launch": flops_local, **extra}
        line = {"metric": "contraction throughput", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": args.scaling,
                "vs_baseline": None, "dtype": "f64" if st else "tf32", "data": "synthetic",
                "config": {"workload": describe(name) + (" with " + ",".join(args.extent) if args.extent else ""), "global": {shard_mode: int(global_eq.extent[shard_mode])},
                           "sharded_mode": shard_mode, "split": args.split, "backend": desc["backend"], "kernel": desc["kernel"],
                           "l2": "inputs and output exceed the 126 MB L2" if alg_bytes > 126e6 else "working set fits L2",
                           "timing": "CUDA events on the launching stream, max over ranks"},
                "clocks": clocks, "gpu_launches": int(launches), "launch_stats": launch_stats,
                "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                        "ms_per_step": e2e_ms, "checksum": checksum},
                "roofline": roofline}
        if contracted:
            line["config"]["collective"] = {"op": "ncclReduceScatter sum over NVLink, after every launch, inside the timed region",
                                            "bytes_sent_per_gpu_per_step": int(nccl_bytes)}
        if world == 1 and not args.no_cpu_baseline and not args.extent:
            info, _ = cpu_baseline(name)
            line["cpu_baseline"] = info
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
