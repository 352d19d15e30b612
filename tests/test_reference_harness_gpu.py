"""GPU: the reference's own benchmark drivers, unchanged, on this engine.

oracle/_ref/bench_tccg and oracle/_ref/bench_tccg_iter are the reference's bench_tccg.cpp and
bench_tccg_iter.cpp (plus its case table and verifier), compiled from where the reference tree lies
against the reference's own include/tcont.hpp and linked with this repository's libtcont.so
(oracle/Makefile).  The tests run them as the reference's batch runner does
(benchmarks/tccg/run_tccg_benchmarks.py:59-112: `bench_tccg -b N --fp64 --backend B --verify` as a
subprocess, exit code 0, one stdout line matching its RESULT_PATTERN, :11-15) and require
validation=PASS, i.e. zero differing elements under the reference's own OpenMP loop nest and
comparator.  The batch runner itself is a file of the reference tree and does not travel to the GPU
box; its per-case protocol is restated here line for line.  Skipped where oracle/_ref was not built.
"""
import os
import re
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BENCH = os.path.join(ROOT, "oracle", "_ref", "bench_tccg")
BENCH_ITER = os.path.join(ROOT, "oracle", "_ref", "bench_tccg_iter")

# The batch runner's pattern (run_tccg_benchmarks.py:11-15), restated.
RESULT_PATTERN = re.compile(
    r"^TCCG_RESULT equation=(?P<equation>\d+) precision=(?P<precision>\w+) "
    r"backend=(?P<backend>\w+) "
    r"operations=(?P<operations>\d+) time_ms=(?P<time_ms>[0-9.]+) "
    r"gflops=(?P<gflops>[0-9.]+) validation=(?P<validation>\w+)$")

needs_harness = pytest.mark.skipif(not os.path.exists(BENCH), reason="oracle/_ref/bench_tccg was not built (no reference tree at build time)")


def run_case(equation: int, precision: str, backend: str, verify: bool = True, env=None, timeout=900):
    """What run_tccg_benchmarks.py:59-112 does for one row."""
    cmd = [BENCH, "-b", str(equation), f"--{precision}", "--backend", backend]
    if verify:
        cmd.append("--verify")
    e = dict(os.environ)
    e["TCONT_SEED"] = "7"
    e.update(env or {})
    done = subprocess.run(cmd, capture_output=True, text=True, env=e, timeout=timeout)
    output = done.stdout + done.stderr
    assert done.returncode == 0, f"exit code {done.returncode}:\n{output[-2000:]}"
    rows = [m for m in (RESULT_PATTERN.match(line.strip()) for line in output.splitlines()) if m]
    assert len(rows) == 1, f"no single TCCG_RESULT line:\n{output[-2000:]}"
    return rows[0], output


# One case per family of the reference's table (benchmarks/tccg/tccg_cases.cpp): tensor x matrix with a
# permuted 3-D output (1) and a 5-D one that needs a transposed input (3), matrix x 4-D tensor (9), two
# contracted modes into a 2-D output (13, split-K), 3-D outputs (15, 19), one contracted mode into a 6-D
# output (31).
FAMILY_CASES = [1, 3, 9, 13, 15, 19, 31]


@needs_harness
@pytest.mark.parametrize("precision", ["fp64", "tf32"])
@pytest.mark.parametrize("equation", FAMILY_CASES)
def test_bench_tccg_case_passes_the_reference_verifier(equation, precision):
    m, output = run_case(equation, precision, "model")
    assert int(m["equation"]) == equation and m["precision"] == precision
    assert m["backend"] in ("cogent", "ttgt")
    assert m["validation"] == "PASS", output[-2000:]
    assert float(m["time_ms"]) > 0 and float(m["gflops"]) > 0 and int(m["operations"]) > 0


@needs_harness
@pytest.mark.parametrize("backend", ["cogent", "ttgt"])
def test_bench_tccg_backend_names_select_the_route(backend):
    """`--backend cogent` keeps the direct kernel, `--backend ttgt` the transpose-assisted route; the line
    reports the name the harness printed for the reference's backends."""
    m, output = run_case(3, "fp64", backend)
    assert m["backend"] == backend and m["validation"] == "PASS", output[-2000:]


@needs_harness
def test_bench_tccg_4d_family_case_21_verified():
    """Case 21 (all extents 72, two contracted modes: the family of the small FP64 configuration) with the
    verifier on; its CPU loop nest is 1.4e11 multiply-adds, hence the long time limit."""
    m, output = run_case(21, "fp64", "model", timeout=1500)
    assert m["validation"] == "PASS", output[-2000:]


@needs_harness
@pytest.mark.skipif(not os.path.exists(BENCH_ITER), reason="oracle/_ref/bench_tccg_iter was not built")
def test_bench_tccg_iter_reports_stage_times():
    """The per-iteration harness (benchmarks/test/tccg/bench_tccg_iter.cpp:171-204, 218-233) on a case the
    planner sends through input transposes, with TCONT_STAGE_TIMES=1: TconT::stage_times must be available and
    its transposes + contraction must add up to the total."""
    e = dict(os.environ)
    e.update({"TCONT_SEED": "7", "TCONT_STAGE_TIMES": "1"})
    done = subprocess.run([BENCH_ITER, "-b", "3", "--fp64", "--backend", "ttgt"], capture_output=True, text=True, env=e, timeout=600)
    output = done.stdout + done.stderr
    assert done.returncode == 0, output[-3000:]
    nums = {}
    for key in ("transpose_a_ms", "transpose_b_ms", "gemm_ms", "transpose_c_ms", "total_ms"):
        found = re.findall(rf"{key}[^0-9\-]*([0-9]+\.[0-9]+(?:e-?[0-9]+)?)", output)
        if found:
            nums[key] = float(found[-1])
    assert "total_ms" in nums and nums["total_ms"] > 0, f"no stage times in the output:\n{output[-3000:]}"
    parts = nums.get("transpose_a_ms", 0.0) + nums.get("transpose_b_ms", 0.0) + nums.get("gemm_ms", 0.0) + nums.get("transpose_c_ms", 0.0)
    assert parts > 0 and abs(parts - nums["total_ms"]) <= 0.05 * nums["total_ms"] + 1e-3, nums


def test_stage_times_through_the_binding(engine, oracle, monkeypatch):
    """TCONT_STAGE_TIMES=1 through the C ABI: available, every stage non-negative, the parts add up, and a route
    without transposes reports zeros for them."""
    from cases import to_equation
    from oracle_lib import F64, Contraction
    monkeypatch.setenv("TCONT_STAGE_TIMES", "1")
    c = Contraction("abcde", "efba", "cfd", dict(a=12, b=8, c=16, d=6, e=8, f=8), F64)
    A, B = oracle.inputs(c, 2, -1.0, 1.0)
    for sel, transposed in ((2, True), (1, False)):
        p = engine.plan(to_equation(engine, c, sel))
        r = engine.prepare(p, A, B)
        engine.launch(r)
        engine.copy_output_to_host(r)
        t = engine.stage_times(r)
        assert t["available"] is True and t["total_ms"] > 0 and t["gemm_ms"] > 0 and t["transpose_c_ms"] == 0.0
        assert abs(t["transpose_a_ms"] + t["transpose_b_ms"] + t["gemm_ms"] - t["total_ms"]) <= 1e-3 + 0.02 * t["total_ms"]
        assert (t["transpose_a_ms"] + t["transpose_b_ms"] > 0) == transposed
