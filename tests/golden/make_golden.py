"""Generates tests/golden/oracle_golden.json.

The reference holds no golden vectors for the contraction path (its verification inputs are
time-seeded), so the fixtures are made here, where the reference tree is mounted: for each of
the 49 mode patterns of benchmarks/tccg/tccg_cases.cpp (FP64 and Float32 tables), at small and
deliberately ragged extents, seeded inputs go through the CPU restatement (oracle/) and the
result is handed to the reference's own loop nest + comparator for that case
(verify_tccg_case, benchmarks/tccg/tccg_verify.cpp:1805-1840, compiled into oracle/_ref).  A
fixture is written only if the reference reports zero differences; it stores the descriptor, the
seed, and a digest of the output (sum, sum of magnitudes, 16 sampled elements).

The five benchmark configurations are added at reduced extents; the first two share the mode
patterns of cases 21 and 18 and are verified the same way, the others match no reference case
and are marked "ref_case": null.

Case 0 of the reference table is skipped: it is a placeholder whose loop nest
(tccg_verify.cpp:18-44) reads the left operand as [k,m] while its descriptor
(tccg_cases.cpp:5-9) declares A[m,k]; the reference's own batch runner starts at case 1
(run_tccg_benchmarks.py:37-41).

Run from the repository root, in a container that has the reference tree:
    python tests/golden/make_golden.py
"""
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from oracle_lib import F32, F64, Contraction, Oracle, RefVerifier  # noqa: E402

SMALL = [6, 5, 7, 4, 9, 3, 8]  # ragged on purpose: no multiple of a tile size


def digest(out: np.ndarray):
    rng = np.random.default_rng(out.size)
    idx = np.sort(rng.choice(out.size, size=min(16, out.size), replace=False))
    return {"sum": float(out.sum()), "abssum": float(np.abs(out).sum()),
            "sample_index": [int(i) for i in idx], "sample_value": [float(out[i]) for i in idx]}


def entry(name, c, seed, lo, hi, ref_case, out):
    return {"name": name, "modeC": c.modeC, "modeA": c.modeA, "modeB": c.modeB, "extent": c.extent,
            "scalar_type": c.scalar_type, "seed": seed, "lo": lo, "hi": hi, "ref_case": ref_case, **digest(out)}


def main():
    oracle, ref = Oracle(), RefVerifier()
    fixtures = []
    for fp32 in (False, True):
        for i in range(1, ref.count()):  # case 0 is the reference's dummy entry, see below
            full = ref.case(i, fp32)
            modes = sorted(full.extent)
            c = Contraction(full.modeC, full.modeA, full.modeB,
                            {m: SMALL[(j + i) % len(SMALL)] for j, m in enumerate(modes)}, full.scalar_type)
            seed = 1000 + i
            A, B = oracle.inputs(c, seed, -1.0, 1.0)
            out = oracle.contract(c, A, B)
            ok, diff, total = ref.verify(i, c, out.astype(c.dtype), A, B)
            if not ok:
                raise SystemExit(f"case {i} fp32={fp32}: oracle disagrees with the reference ({diff}/{total})")
            fixtures.append(entry(f"tccg{i:02d}_{'f32' if fp32 else 'f64'}", c, seed, -1.0, 1.0, i, out))

    configs = [
        ("cfg1_full", Contraction("abcd", "aebf", "fdec", dict(a=24, b=24, c=24, d=24, e=16, f=16), F64), 0, -1.0, 1.0, 21),
        ("cfg2_small", Contraction("abc", "adc", "db", dict(a=64, b=48, c=8, d=40), F32), 1, -1.0, 1.0, 18),
        ("cfg3_small", Contraction("abcijk", "aeij", "bcek", dict(a=12, b=6, c=6, e=12, i=4, j=4, k=4), F64), 2, -0.5, 0.5, None),
        ("cfg4_small", Contraction("abcde", "efba", "cfd", dict(a=12, b=6, c=12, d=6, e=12, f=8), F32), 3, -1.0, 1.0, None),
        ("cfg5_small", Contraction("abcd", "aebf", "cfde", dict(a=32, b=4, c=32, d=4, e=8, f=8), F32), 4, -1.0, 1.0, None),
    ]
    for name, c, seed, lo, hi, ref_case in configs:
        A, B = oracle.inputs(c, seed, lo, hi)
        out = oracle.contract(c, A, B)
        if ref_case is not None:
            ok, diff, total = ref.verify(ref_case, c, out.astype(c.dtype), A, B)
            if not ok:
                raise SystemExit(f"{name}: oracle disagrees with the reference ({diff}/{total})")
        fixtures.append(entry(name, c, seed, lo, hi, ref_case, out))

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle_golden.json")
    with open(path, "w") as f:
        json.dump({"generator": "tests/golden/make_golden.py", "fixtures": fixtures}, f, indent=1)
    print(f"wrote {len(fixtures)} fixtures to {path}")


if __name__ == "__main__":
    main()
