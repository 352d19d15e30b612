"""GPU (needs 2 or more devices): several GPUs behind ONE run object, the form the reference's
unchanged single-process harness drives (TCONT_NUM_GPUS / TCONT_SPLIT in the environment).  The
contraction is cut along an external mode, so every output element is computed by exactly one GPU.
A shard is planned as a contraction of its own, so it may run another kernel or other k ranges
than the full problem does: results must agree within the reference's tolerance, and be
bit-identical when split-K is off and both plans run the same kernel."""
import numpy as np
import pytest

from cases import to_equation
from oracle_lib import F32, F64, Contraction

pytestmark = pytest.mark.gpu


def _ngpus():
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


needs_two = pytest.mark.skipif(_ngpus() < 2, reason="needs two GPUs")

CASES = [
    (Contraction("abcd", "aebf", "fdec", dict(a=24, b=24, c=24, d=24, e=16, f=16), F64), None),      # cut d: slowest mode of C, in B
    (Contraction("abcd", "aebf", "fdec", dict(a=24, b=24, c=24, d=24, e=16, f=16), F64), "ext:a"),   # cut C's stride-1 mode, in A
    (Contraction("abc", "adc", "db", dict(a=128, c=6, b=96, d=64), F32), None),                      # tcgen05 kernel per shard
    (Contraction("abcde", "efba", "cfd", dict(a=12, b=8, c=16, d=6, e=8, f=8), F32), "ext:b"),       # transposes + tcgen05 per shard
]


@needs_two
@pytest.mark.parametrize("c,split", CASES, ids=lambda v: v if isinstance(v, str) else None)
def test_two_gpus_equal_one(engine, oracle, monkeypatch, c, split):
    A, B = oracle.inputs(c, 3, -1.0, 1.0)
    eq = to_equation(engine, c)
    single = engine.prepare(engine.plan(eq), A, B)
    engine.launch(single)
    want = engine.copy_output_to_host(single)

    monkeypatch.setenv("TCONT_NUM_GPUS", "2")
    if split:
        monkeypatch.setenv("TCONT_SPLIT", split)
    multi = engine.prepare(engine.plan(eq), A, B)
    engine.warmup(multi, 2)
    engine.zero_output(multi)
    assert not engine.copy_output_to_host(multi).any()
    ms, launches = multi.time_launches(3)
    got = engine.copy_output_to_host(multi)
    assert multi.device_status() == 0 and ms > 0 and launches >= 6
    np.testing.assert_array_equal(engine.input_left_host_data(multi), A)    # the global inputs, as the harness's verifier needs
    np.testing.assert_array_equal(engine.input_right_host_data(multi), B)
    assert oracle.compare(want, got, c.scalar_type) == (0, 0)
    if c.scalar_type == F64:
        assert oracle.compare(oracle.contract(c, A, B), got, F64) == (0, 0)


@needs_two
def test_unsplittable_falls_back_and_bad_split_is_rejected(engine, oracle, monkeypatch):
    c = Contraction("ab", "ak", "kb", dict(a=7, b=5, k=4), F64)    # no external extent divides by 2
    A, B = oracle.inputs(c, 1)
    monkeypatch.setenv("TCONT_NUM_GPUS", "2")
    r = engine.prepare(engine.plan(to_equation(engine, c)), A, B)
    engine.launch(r)
    diff, _ = oracle.compare(oracle.contract(c, A, B), engine.copy_output_to_host(r), F64)
    assert diff == 0
    monkeypatch.setenv("TCONT_SPLIT", "ext:k")                     # a contracted mode cannot be cut without a reduction
    with pytest.raises(ValueError):
        engine.prepare(engine.plan(to_equation(engine, c)), A, B)
