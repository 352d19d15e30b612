"""How good is the planner's choice between its two routes?  (Run on a GPU box; not a pytest module.)

    python tests/regret_sweep.py [--precision fp64|tf32|both] [--start 1] [--end 48] > regret.md
    python tests/regret_sweep.py --verified > verified.md     # `--backend model --verify`, cases 12 and 20-30 left out

For every case of the reference's table the reference's own unchanged driver (oracle/_ref/bench_tccg, see
tests/test_reference_harness_gpu.py) is run three times: `--backend cogent` (direct kernel), `--backend ttgt`
(input transposes + direct kernel) and `--backend model` (the cost table decides).  The table lists the three
times, the route the model took, whether that was the faster one, and the regret (time of the model's choice
over the time of the better route).  The reference reports the same two figures for its LightGBM selector
(final_model/lgbm_small_i120_depth3_leaf15_lr005_l2_1_export.json: accuracy 0.958 and a maximum regret of
1.088 on its 48 cases).  No `--verify`: correctness of these cases is what the tests check.
"""
import argparse
import os
import re
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BENCH = os.path.join(ROOT, "oracle", "_ref", "bench_tccg")
LINE = re.compile(r"^TCCG_RESULT equation=(\d+) precision=(\w+) backend=(\w+) operations=(\d+) time_ms=([0-9.]+) gflops=([0-9.]+) validation=(\w+)$")


def run(equation, precision, backend, verify=False):
    env = dict(os.environ)
    env["TCONT_SEED"] = "7"
    cmd = [BENCH, "-b", str(equation), f"--{precision}", "--backend", backend] + (["--verify"] if verify else [])
    done = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=1800)
    for line in (done.stdout + done.stderr).splitlines():
        m = LINE.match(line.strip())
        if m and done.returncode == 0:
            return (m.group(3), float(m.group(5)), float(m.group(6))) + ((m.group(7),) if verify else ())
    return (None, None, None) + ((None,) if verify else ())


def verified_sweep(args):
    """`--backend model --verify` on every case but those whose CPU loop nest takes minutes (12, 20-30)."""
    slow = {12} | set(range(20, 31))
    for precision in (["fp64", "tf32"] if args.precision == "both" else [args.precision]):
        print(f"\n## {precision}, --backend model --verify\n")
        print("| case | backend | ms | GFLOP/s | validation |")
        print("|---|---|---|---|---|")
        passed = failed = 0
        for eq in range(args.start, args.end + 1):
            if eq in slow:
                continue
            took, ms, gf, val = run(eq, precision, "model", verify=True)
            if took is None:
                print(f"| {eq} | error | | | |")
                failed += 1
                continue
            passed += int(val == "PASS")
            failed += int(val != "PASS")
            print(f"| {eq} | {took} | {ms:.4f} | {gf:.0f} | {val} |")
            sys.stdout.flush()
        print(f"\n{precision}: {passed} passed, {failed} failed (the reference's own loop nest and comparator).")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--precision", default="both", choices=["fp64", "tf32", "both"])
    ap.add_argument("--start", type=int, default=1)
    ap.add_argument("--end", type=int, default=48)
    ap.add_argument("--verified", action="store_true", help="run `--backend model --verify` instead of the three-way timing")
    args = ap.parse_args()
    if not os.path.exists(BENCH):
        raise SystemExit("oracle/_ref/bench_tccg is missing (make -C oracle, where the reference tree is available)")
    if args.verified:
        verified_sweep(args)
        return
    for precision in (["fp64", "tf32"] if args.precision == "both" else [args.precision]):
        print(f"\n## {precision}\n")
        print("| case | direct ms | ttgt ms | model ms | model GFLOP/s | model took | faster | right | regret |")
        print("|---|---|---|---|---|---|---|---|---|")
        right = total = 0
        worst = 1.0
        for eq in range(args.start, args.end + 1):
            _, t_direct, _ = run(eq, precision, "cogent")
            took_t, t_ttgt, _ = run(eq, precision, "ttgt")
            took, t_model, gf_model = run(eq, precision, "model")
            if None in (t_direct, t_ttgt, t_model):
                print(f"| {eq} | error | | | | | | | |")
                continue
            # `--backend ttgt` on a case that needs no transpose runs the direct kernel and reports it as such
            same_route = abs(t_direct - t_ttgt) <= 0.03 * min(t_direct, t_ttgt)
            faster = "either" if same_route else ("cogent" if t_direct < t_ttgt else "ttgt")
            best = min(t_direct, t_ttgt)
            chosen = t_direct if took == "cogent" else t_ttgt
            ok = faster == "either" or took == faster
            regret = max(1.0, chosen / best)
            total += 1
            right += int(ok)
            worst = max(worst, regret)
            print(f"| {eq} | {t_direct:.4f} | {t_ttgt:.4f} | {t_model:.4f} | {gf_model:.0f} | {took} | {faster} | {'yes' if ok else 'no'} | {regret:.3f} |")
            sys.stdout.flush()
        if total:
            print(f"\n{precision}: the model took the faster route (or the routes tie within 3 %) in {right} of {total} cases "
                  f"(accuracy {right / total:.3f}); maximum regret {worst:.3f}.")


if __name__ == "__main__":
    main()
