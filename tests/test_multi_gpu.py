"""GPU: several shards behind ONE run object, the form the reference's unchanged single-process harness
drives (TCONT_NUM_GPUS / TCONT_SPLIT in the environment).  Cut along an external mode every output element
is computed by exactly one shard; cut along a contracted mode (TCONT_SPLIT=k:<mode>) every shard stores its
partial tiles straight into the owner's staging slots and the owners add them up.  A shard is planned as a
contraction of its own, so it may run another kernel or other k ranges than the full problem does: results
must agree within the reference's tolerance.

On a box with two or more GPUs the shards live on different devices.  On a box with one GPU the same tests
run with TCONT_SHARDS_ON_ONE_DEVICE=1: every shard on that device, which exercises the slicing, the owner
routing, the joins and the gather (the kernels then run one after the other; none waits for another)."""
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


needs_two = pytest.mark.skipif(_ngpus() < 1, reason="needs a GPU")


@pytest.fixture(autouse=True)
def _one_device_when_alone(monkeypatch):
    if _ngpus() < 2:
        monkeypatch.setenv("TCONT_SHARDS_ON_ONE_DEVICE", "1")

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


KSPLIT_CASES = [
    # (descriptor, contracted mode to cut, shards): C's slowest mode lies in the operand without C's stride-1 mode
    (Contraction("abcd", "aebf", "cfde", dict(a=128, b=4, c=128, d=8, e=16, f=32), F32), "e", 2),
    (Contraction("abcd", "aebf", "cfde", dict(a=128, b=4, c=128, d=8, e=16, f=32), F32), "e", 4),
    (Contraction("abcd", "aebf", "cfde", dict(a=64, b=6, c=96, d=8, e=8, f=24), F32), "f", 2),       # ragged slabs, the other contracted mode
    (Contraction("abc", "adc", "db", dict(a=256, c=6, b=512, d=256), F32), "d", 4),                  # C's slowest mode c lies in A: roles as the planner sets them
]


@needs_two
@pytest.mark.parametrize("c,mode,shards", KSPLIT_CASES, ids=lambda v: v if isinstance(v, (str, int)) else None)
def test_contracted_split_behind_one_run(engine, oracle, monkeypatch, c, mode, shards):
    """TCONT_SPLIT=k:<mode>: partial tiles stored into the owners' slots, summed by the owners, gathered."""
    if _ngpus() >= 2 and _ngpus() < shards:
        pytest.skip("fewer GPUs than shards")
    A, B = oracle.inputs(c, 8, -1.0, 1.0)
    eq = to_equation(engine, c)
    monkeypatch.setenv("TCONT_SPLITK", "1")
    monkeypatch.setenv("TCONT_NUM_GPUS", str(shards))
    monkeypatch.setenv("TCONT_SPLIT", f"k:{mode}")
    try:
        multi = engine.prepare(engine.plan(eq), A, B)
    except NotImplementedError as e:
        assert c.modeC[-1] in c.modeA and "slowest mode" in str(e)      # the documented limit: C's slowest mode in the row operand
        return
    assert c.modeC[-1] not in c.modeA
    for _ in range(3):   # the two sets of slots alternate; the third launch reuses the first set
        engine.zero_output(multi)
        engine.launch(multi)
    got = engine.copy_output_to_host(multi)
    assert multi.device_status() == 0
    exact = oracle.contract(c, A, B, rounding=0)
    trunc = oracle.contract(c, A, B, rounding=1)
    scale = oracle.contract(c, np.abs(A), np.abs(B), rounding=1)
    worst = float((np.abs(got.astype(np.float64) - trunc) / (scale + 1e-30)).max())
    assert worst < 2e-5, worst
    diff, nonfinite = oracle.compare(exact, got, F32)
    assert nonfinite == 0 and diff <= 0.005 * got.size + 4


@needs_two
def test_contracted_split_rejects_what_it_cannot_route(engine, oracle, monkeypatch):
    monkeypatch.setenv("TCONT_NUM_GPUS", "2")
    c = Contraction("abcd", "aebf", "cfde", dict(a=128, b=4, c=128, d=8, e=16, f=32), F32)
    A, B = oracle.inputs(c, 8, -1.0, 1.0)
    monkeypatch.setenv("TCONT_SPLIT", "k:a")                       # not a contracted mode
    with pytest.raises(ValueError):
        engine.prepare(engine.plan(to_equation(engine, c)), A, B)
    c64 = Contraction("abcd", "aebf", "cfde", dict(a=24, b=4, c=24, d=8, e=16, f=8), F64)
    A, B = oracle.inputs(c64, 8, -1.0, 1.0)
    monkeypatch.setenv("TCONT_SPLIT", "k:e")                       # FP64: no tcgen05 kernel to route tiles
    with pytest.raises(NotImplementedError):
        engine.prepare(engine.plan(to_equation(engine, c64)), A, B)


@needs_two
def test_contracted_split_between_runs_of_one_process(engine, oracle, monkeypatch):
    """The per-rank form (tcontb_run_ksplit_enable / attach / reduce) with two ranks as two runs of this process on
    one device; the IPC handle a rank in another process would import is exported as well."""
    import torch
    from tcont_b200 import api, sharding
    monkeypatch.setenv("TCONT_SPLITK", "1")
    c = Contraction("abcd", "aebf", "cfde", dict(a=128, b=4, c=128, d=8, e=16, f=32), F32)
    A, B = oracle.inputs(c, 9, -1.0, 1.0)
    eq = to_equation(engine, c)
    world = 2
    runs, outs = [], []
    for r in range(world):
        local, sl = sharding.shard_contracted(eq, "e", world, r)
        a_loc = sharding.take_slice(A, eq.modeA, eq.extent, "e", sl)
        b_loc = sharding.take_slice(B, eq.modeB, eq.extent, "e", sl)
        dA, dB = torch.from_numpy(a_loc).cuda(), torch.from_numpy(b_loc).cuda()
        dC = torch.full((c.size(c.modeC) // world,), float("nan"), dtype=torch.float32, device="cuda")
        run = api.prepare_on_device(engine.plan(local), dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), keep=(dA, dB, dC))
        run.ksplit_enable(world, r)
        assert run.ksplit_range_elements() == c.size(c.modeC) // world and len(run.ksplit_export()) == 64
        runs.append(run)
        outs.append(dC)
    runs[0].ksplit_attach(1, runs[1])
    runs[1].ksplit_attach(0, runs[0])
    for _ in range(2):
        for run in runs:
            engine.launch(run)
        torch.cuda.synchronize()              # the barrier among the ranks
        for run in runs:
            run.ksplit_reduce()
        torch.cuda.synchronize()
    got = torch.cat(outs).cpu().numpy()
    trunc = oracle.contract(c, A, B, rounding=1)
    scale = oracle.contract(c, np.abs(A), np.abs(B), rounding=1)
    assert float((np.abs(got.astype(np.float64) - trunc) / (scale + 1e-30)).max()) < 2e-5
    assert all(r.device_status() == 0 for r in runs)


@needs_two
def test_contracted_split_on_cta_pairs(engine, oracle, monkeypatch):
    """The same routing with the kernel in its CTA-pair form (256-wide tile columns, both CTAs of a pair store to the owner)."""
    if 2 <= _ngpus() < 2:
        pytest.skip("fewer GPUs than shards")
    c = Contraction("abcd", "aebf", "cfde", dict(a=128, b=8, c=128, d=40, e=8, f=128), F32)
    A, B = oracle.inputs(c, 10, -1.0, 1.0)
    monkeypatch.setenv("TCONT_SPLITK", "1")
    monkeypatch.setenv("TCONT_UMMA_PAIR", "1")
    monkeypatch.setenv("TCONT_NUM_GPUS", "2")
    monkeypatch.setenv("TCONT_SPLIT", "k:f")
    multi = engine.prepare(engine.plan(to_equation(engine, c)), A, B)
    for _ in range(2):
        engine.launch(multi)
    got = engine.copy_output_to_host(multi)
    assert multi.device_status() == 0
    trunc = oracle.contract(c, A, B, rounding=1)
    scale = oracle.contract(c, np.abs(A), np.abs(B), rounding=1)
    assert float((np.abs(got.astype(np.float64) - trunc) / (scale + 1e-30)).max()) < 2e-5
