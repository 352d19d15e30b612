"""Contraction descriptors shared by the tests: the golden fixtures and the benchmark configurations."""
import json
import os

from oracle_lib import F32, F64, Contraction

HERE = os.path.dirname(os.path.abspath(__file__))


def golden_fixtures():
    with open(os.path.join(HERE, "golden", "oracle_golden.json")) as f:
        return json.load(f)["fixtures"]


def fixture_contraction(fx) -> Contraction:
    return Contraction(fx["modeC"], fx["modeA"], fx["modeB"], {k: int(v) for k, v in fx["extent"].items()}, fx["scalar_type"])


# The five benchmark configurations at full size: (descriptor, seed, lo, hi)
CONFIGS = {
    "cfg1": (Contraction("abcd", "aebf", "fdec", dict(a=24, b=24, c=24, d=24, e=16, f=16), F64), 0, -1.0, 1.0),
    "cfg2": (Contraction("abc", "adc", "db", dict(a=256, c=256, b=1024, d=1024), F32), 1, -1.0, 1.0),
    "cfg3": (Contraction("abcijk", "aeij", "bcek", dict(a=48, b=48, c=48, e=48, i=24, j=24, k=24), F64), 2, -0.5, 0.5),
    "cfg4": (Contraction("abcde", "efba", "cfd", dict(a=48, b=48, c=48, d=48, e=48, f=8), F32), 3, -1.0, 1.0),
    "cfg5": (Contraction("abcd", "aebf", "cfde", dict(a=128, b=128, c=128, d=128, e=128, f=128), F32), 4, -1.0, 1.0),
}


def to_equation(engine, c: Contraction, selection=0):
    return engine.TCEquation(c.modeC, c.modeA, c.modeB, dict(c.extent), "-", engine.ScalarType(c.scalar_type),
                             engine.BackendSelection(selection))


SMALL_EXTENTS = (1, 2, 3, 4, 5, 7, 8, 12, 16, 24, 32, 33, 40, 64, 72, 96, 128)
LARGE_EXTENTS = (4, 6, 8, 12, 16, 24, 32, 40, 64, 72, 96, 128, 160, 200)


def random_contraction(rng, scalar_type, max_out=200_000, max_macs=30_000_000, pool=SMALL_EXTENTS) -> Contraction:
    """A random well-formed contraction: 1-3 modes per group, ragged extents, random memory orders."""
    letters = list("abcdefghi")
    while True:
        nM, nN, nK = (int(rng.integers(1, 4)) for _ in range(3))
        names = letters[: nM + nN + nK]
        ext = {n: int(rng.choice(pool)) for n in names}
        M, N, K = names[:nM], names[nM:nM + nN], names[nM + nN:]
        out = 1
        for n in M + N:
            out *= ext[n]
        macs = out
        for n in K:
            macs *= ext[n]
        if out <= max_out and macs <= max_macs:
            break
    order = lambda modes: "".join(rng.permutation(modes))  # noqa: E731
    return Contraction(order(M + N), order(M + K), order(N + K), ext, scalar_type)
