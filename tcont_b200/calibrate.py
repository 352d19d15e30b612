"""Fills the planner's cost table from measurements on the current GPU and writes it as a "key value"
file named after the device, beside the library, where the engine looks for it:

    python -m tcont_b200.calibrate            # writes tcont_b200/tcont_cost_table.<device name>.txt
    python -m tcont_b200.calibrate -o FILE    # any other place; use it with TCONT_COST_TABLE=FILE

Lines whose key starts with `info_` are measurements for the record (rates of the helper kernels); the
planner ignores them.

The reference decides between its two backends with a LightGBM model trained offline on A100
runs (final_model/*.json, src/backend_model_selector.cpp:365-403); the trainer is not part of its
tree.  Here the decision is an explicit time estimate per route, and these are its constants:
copy bandwidth, the rate of each contraction kernel on a large well-shaped problem, the launch
overhead, and the penalty for TMA boxes whose rows lie far apart in memory.
"""
from __future__ import annotations

import argparse
import os


def _rate(tc, api, torch, modes, extent, scalar, iters=10, env=None):
    old = {}
    for k, v in (env or {}).items():
        old[k] = os.environ.get(k)
        os.environ[k] = v
    try:
        eq = tc.TCEquation(*modes, dict(extent), "-", scalar, tc.BackendSelection.COGENT)
        plan = tc.plan(eq)
        dt = torch.float64 if scalar == tc.ScalarType.Float64 else torch.float32
        a = torch.rand(eq.size(eq.modeA), device="cuda", dtype=dt) - 0.5
        b = torch.rand(eq.size(eq.modeB), device="cuda", dtype=dt) - 0.5
        c = torch.empty(eq.size(eq.modeC), device="cuda", dtype=dt)
        run = api.prepare_on_device(plan, a.data_ptr(), b.data_ptr(), c.data_ptr(), keep=(a, b, c))
        tc.warmup(run, 3)
        ms, _ = run.time_launches(iters)
        return plan.flops / (ms / iters * 1e-3) / 1e12, plan.describe()["kernel"]
    finally:
        for k, v in old.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v


def calibrate() -> dict:
    import torch

    import tcont_b200 as tc
    from tcont_b200 import api

    F32, F64 = tc.ScalarType.Float32, tc.ScalarType.Float64
    table = {}
    # copy bandwidth through the permutation kernel with an identity permutation (read + write)
    n = 1 << 28
    src = torch.empty(n, device="cuda", dtype=torch.float32)
    dst = torch.empty_like(src)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    stream = torch.cuda.current_stream().cuda_stream
    for _ in range(3):
        api.transpose(src.data_ptr(), dst.data_ptr(), [n // 1024, 1024], [0, 1], 4, stream)
    e0.record()
    for _ in range(10):
        api.transpose(src.data_ptr(), dst.data_ptr(), [n // 1024, 1024], [0, 1], 4, stream)
    e1.record()
    torch.cuda.synchronize()
    table["hbm_gbs"] = 2 * n * 4 * 10 / (e0.elapsed_time(e1) * 1e-3) / 1e9
    del src, dst
    gemm = (("ab", "ka", "kb"), dict(a=8192, b=8192, k=4096))
    table["umma_tf32_tflops"], k = _rate(tc, api, torch, *gemm, F32)
    assert k == "umma_tf32", k
    table["simt_f32_tflops"], _ = _rate(tc, api, torch, ("ab", "ka", "kb"), dict(a=4096, b=4096, k=1024), F32, env={"TCONT_KERNEL": "simt"})
    gemm64 = (("ab", "ak", "kb"), dict(a=4096, b=4096, k=2048))
    table["dmma_f64_tflops"], k = _rate(tc, api, torch, *gemm64, F64)
    assert k == "dmma_f64_tma", k
    table["dmma_f64_gather_tflops"], k = _rate(tc, api, torch, *gemm64, F64, env={"TCONT_KERNEL": "gather"})
    assert k == "dmma_f64", k
    # one operand whose stride-1 mode leads neither its rows nor the contracted modes: 8-byte gathers
    table["dmma_f64_gather8_tflops"], k = _rate(tc, api, torch, ("abc", "akc", "kb"), dict(a=2, b=2048, c=2048, k=2048), F64,
                                                env={"TCONT_KERNEL": "gather"})
    assert k == "dmma_f64", k
    table["dmma_f64_gather_narrow_tflops"], k = _rate(tc, api, torch, ("abc", "dca", "bd"), dict(a=312, b=24, c=296, d=312), F64,
                                                      env={"TCONT_KERNEL": "gather"})
    assert k == "dmma_f64", k
    table["simt_f64_tflops"], _ = _rate(tc, api, torch, ("ab", "ak", "bk"), dict(a=4096, b=4096, k=1024), F64, env={"TCONT_KERNEL": "simt"})
    # scattered stores of the TMA-fed kernels: two contractions of the same size with a short contracted
    # extent, one whose tile rows run along C's stride-1 mode and one whose rows do not (every element of C
    # stored on its own); the time of the second per element of C
    # (a = 30: no multiple of 8, so the FP64 kernel cannot store across slabs and the rows really are scattered)
    ext6 = dict(a=30, b=16, c=16, d=24, e=16, f=16, g=24)
    size_c = 30 * 16 * 16 * 24 * 16 * 16
    flops6 = 2.0 * size_c * 24
    for key, scalar in (("scatter_store_ps", F64), ("scatter_store_f32_ps", F32)):
        # (FP64: the planner itself would send the second one to the CUDA cores, which is what this figure is for)
        env = {"TCONT_KERNEL": "tma"} if scalar == F64 else None
        _, k1 = _rate(tc, api, torch, ("abcdef", "degb", "gfac"), ext6, scalar, env=env)
        t_scat, k2 = _rate(tc, api, torch, ("abcdef", "dega", "gfbc"), ext6, scalar, env=env)
        if k1 == k2 and k1 in ("dmma_f64_tma", "umma_tf32"):
            table[key] = flops6 / (t_scat * 1e12) / size_c * 1e12
        else:
            print(f"# {key}: not measured (kernels {k1} / {k2}); the compiled-in figure stays")
    # far-row penalty: the same 4-D contraction with A where the large configuration has it (the k rows of a TMA box
    # 8 MB apart, every one in another 2 MB page: half of the bytes a CTA of a pair stages) and with A already in the
    # layout the transpose-assisted route gives it (rows 512 bytes apart): rate_far = rate_near * (1 - p / 2)
    # (f = 64: the contracted mode that is cut into chunks must be long enough for the kernel form the large
    # configuration runs on, CTA pairs with a k chunk of 64; on the one-CTA form with chunks of 32 the two layouts
    # differ by 3 to 8 %, on pairs by a quarter)
    ext = dict(a=128, b=128, c=128, d=128, e=128, f=64)
    far, _ = _rate(tc, api, torch, ("abcd", "aebf", "cfde"), ext, F32, iters=3)
    near, _ = _rate(tc, api, torch, ("abcd", "afeb", "cfde"), ext, F32, iters=3)
    table["far_row_penalty"] = max(0.0, min(1.0, 2.0 * (1.0 - far / max(near, 1e-9))))
    # what one more kernel costs in a chain of back-to-back launches: a contraction too small to matter, launched in
    # a loop inside the library (a loop in Python would measure the interpreter)
    eq = tc.TCEquation("ab", "ak", "kb", dict(a=16, b=16, k=16), "-", F32, tc.BackendSelection.COGENT)
    plan = tc.plan(eq)
    ta = torch.zeros(256, device="cuda", dtype=torch.float32)
    tb = torch.zeros(256, device="cuda", dtype=torch.float32)
    tcc = torch.zeros(256, device="cuda", dtype=torch.float32)
    run = api.prepare_on_device(plan, ta.data_ptr(), tb.data_ptr(), tcc.data_ptr(), keep=(ta, tb, tcc))
    tc.warmup(run, 20)
    ms, _ = run.time_launches(2000)
    table["launch_us"] = ms / 2000 * 1e3

    # ---- for the record: rates of the helper kernels (CUDA events; read + write bytes over time) ----
    def permute_gbs(extent, perm, dtype, iters=10):
        n = 1
        for e in extent:
            n *= e
        x = torch.empty(n, device="cuda", dtype=dtype)
        y = torch.empty_like(x)
        for _ in range(3):
            api.transpose(x.data_ptr(), y.data_ptr(), extent, perm, x.element_size(), stream)
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(iters):
            api.transpose(x.data_ptr(), y.data_ptr(), extent, perm, x.element_size(), stream)
        a1.record()
        torch.cuda.synchronize()
        return 2 * n * x.element_size() * iters / (a0.elapsed_time(a1) * 1e-3) / 1e9

    # the input transpose of the large 4-D TF32 configuration: A[a,e,b,f] -> [a,f,e,b], rows of 128 floats kept
    table["info_permute_rows_f32_gbs"] = permute_gbs([128, 128, 128, 128], [0, 3, 1, 2], torch.float32)
    table["info_permute_rows_f64_gbs"] = permute_gbs([48, 48, 576, 16], [0, 2, 1, 3], torch.float64)
    # a plain matrix transpose through the shared-memory tile
    table["info_permute_tiled_f32_gbs"] = permute_gbs([8192, 8192], [1, 0], torch.float32)
    table["info_permute_tiled_f64_gbs"] = permute_gbs([4096, 8192], [1, 0], torch.float64)
    # split-K (contraction into four partial tensors + the kernel that adds them up), both precisions
    lk = (("ab", "acd", "dbc"), dict(a=1024, b=1024, c=128, d=128))
    table["info_splitk4_tf32_tflops"], _ = _rate(tc, api, torch, *lk, F32, env={"TCONT_SPLITK": "4"})
    table["info_splitk4_f64_tflops"], _ = _rate(tc, api, torch, *lk, F64, env={"TCONT_SPLITK": "4"})
    return table


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("-o", "--output", default=None)
    args = ap.parse_args()
    import torch
    name = torch.cuda.get_device_name().replace(" ", "_").replace("/", "_")
    out = args.output or os.path.join(os.path.dirname(os.path.abspath(__file__)), f"tcont_cost_table.{name}.txt")
    os.environ["TCONT_COST_TABLE"] = os.devnull     # measure with the compiled-in defaults, not with an older table
    table = calibrate()
    with open(out, "w") as f:
        for k, v in table.items():
            f.write(f"{k} {v:.6g}\n")
            print(f"{k} {v:.6g}")
    print(f"wrote {out}" + ("" if args.output is None else f"; use it with TCONT_COST_TABLE={out}"))


if __name__ == "__main__":
    main()
