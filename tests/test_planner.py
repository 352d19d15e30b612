"""CPU-only: the host-side planner behind TconT::plan, driven through the C ABI."""
import pytest

from cases import CONFIGS, fixture_contraction, golden_fixtures, to_equation
from oracle_lib import Contraction


def describe(engine, c, selection=0):
    return engine.plan(to_equation(engine, c, selection)).describe()


def test_mode_groups_and_fusion(engine):
    d = describe(engine, CONFIGS["cfg3"][0])
    assert d["A"] == ["a:48", "e:48", "ij:576"] and d["B"] == ["bc:2304", "e:48", "k:24"]
    assert d["M"] == ["a:48", "ij:576"] and d["N"] == ["bc:2304", "k:24"] and d["K"] == ["e:48"]
    assert (d["Mtot"], d["Ntot"], d["Ktot"]) == (27648, 55296, 48)
    # cfg5's (a,b) are neighbours in C but split by e in A: nothing may fuse
    d5 = describe(engine, CONFIGS["cfg5"][0])
    assert d5["C"] == ["a:128", "b:128", "c:128", "d:128"]


def test_roles_follow_position_not_names(engine):
    # C's stride-1 mode lives in the right operand: roles are exchanged (the reference keys this
    # on the letter 'a', backends/cogent/plan/tc_gen_inner_group.py:450)
    eq = engine.TCEquation("xyz", "kz", "ykx", dict(x=8, y=4, z=6, k=5))
    d = engine.plan(eq).describe()
    assert d["swapped"] is True and d["M"][0].startswith("x") and d["K"] == ["k:5"]
    eq2 = engine.TCEquation("xyz", "ykx", "kz", dict(x=8, y=4, z=6, k=5))
    assert engine.plan(eq2).describe()["swapped"] is False


def test_backend_selection_and_names(engine):
    c = CONFIGS["cfg1"][0]
    assert engine.plan(to_equation(engine, c, 1)).backend == engine.Backend.COGENT
    p = engine.plan(to_equation(engine, c, 2))
    assert p.backend == engine.Backend.TTGT_CUTT
    d = p.describe()
    # role A = A[a,e,b,f] -> [a,b | f,e] (lead = ab, K in B's order); B[f,d,e,c] is K-major on f and
    # is used where it lies; C never needs a transpose
    assert d["transpose_a"] == [0, 2, 3, 1] and d["transpose_b"] is None
    assert d["A"] == ["ab:576", "f:16", "e:16"] and d["B"] == ["f:16", "d:24", "e:16", "c:24"]


def test_configs_pick_the_intended_kernels(engine):
    d2 = describe(engine, CONFIGS["cfg2"][0])
    assert d2["backend"] == "direct" and d2["kernel"] == "umma_tf32"
    u = d2["umma"]
    # CTA pairs on 256 x 256 tiles with a k chunk of 64: three stages of 64 KB per CTA, one copy per operand and stage
    assert (u["a_major"], u["b_major"], u["BN"], u["BK"], u["k_iters"], u["pair"], u["stages"]) == ("MN", "K", 256, 64, 16, True, 3)
    assert (u["a_slabs_per_copy"], u["b_slab_w"], u["b_slabs"]) == (4, 128, 2)
    assert u["tiles_m"] * u["tiles_n"] == 2048 and u["coalesced_store"] and u["smem_bytes"] <= 227 * 1024
    d4 = describe(engine, CONFIGS["cfg4"][0])
    assert d4["backend"] == "ttgt" and d4["kernel"] == "umma_tf32" and d4["umma"]["BK"] == 8
    assert d4["transpose_a"] == [3, 2, 1, 0] and d4["A"] == ["ab:2304", "f:8", "e:48"] and d4["umma"]["pair"] is False
    # cfg5: A's contracted rows lie 8 MB apart; the cost table sends A through one transpose to
    # [a | f,e | b] so that every TMA box is one contiguous piece, and keeps B where it lies
    d5 = describe(engine, CONFIGS["cfg5"][0])
    assert d5["backend"] == "ttgt" and d5["transpose_a"] == [0, 3, 1, 2] and d5["transpose_b"] is None
    assert d5["kernel"] == "umma_tf32" and d5["umma"]["k_iters"] == 256 and d5["umma"]["kc"] == "f"
    assert d5["umma"]["pair"] is True and d5["umma"]["BK"] == 64 and d5["umma"]["b_slabs_per_copy"] == 4
    d3 = describe(engine, CONFIGS["cfg3"][0])   # TMA-fed FP64 kernel: one 128-byte row of 16 doubles per box row
    assert d3["backend"] == "direct" and d3["kernel"] == "dmma_f64_tma"
    assert (d3["umma"]["BN"], d3["umma"]["BK"], d3["umma"]["stages"], d3["umma"]["k_iters"]) == (64, 16, 8, 3)
    assert d3["umma"]["coalesced_store"] and d3["umma"]["smem_bytes"] <= 227 * 1024


def test_fp64_kernel_choice_follows_the_cost_table(engine, monkeypatch):
    F64 = 1
    # A's stride-1 mode is not C's: where C's stride-1 mode lies behind the contracted mode in A and its extent is a
    # multiple of 8, a tile takes 8 of its indices x 16 elements of A's stride-1 mode and stores across slabs
    c31 = Contraction("abcdef", "dega", "gfbc", dict(a=24, b=16, c=16, d=24, e=16, f=16, g=24), F64)
    d = describe(engine, c31)
    assert d["backend"] == "direct" and d["kernel"] == "dmma_f64_tma" and d["umma"]["store_across_slabs"]
    assert d["umma"]["a_slabs_per_copy"] == 8 and not d["umma"]["coalesced_store"]
    c1 = Contraction("abc", "bda", "dc", dict(a=312, b=312, c=24, d=312), F64)
    d = describe(engine, c1)
    assert d["backend"] == "direct" and d["kernel"] == "dmma_f64_tma" and d["umma"]["store_across_slabs"]
    # ... where it cannot (extent 30 is no multiple of 8), rows along A's stride-1 mode would be stored element by
    # element, and one transpose of A is cheaper
    c31r = Contraction("abcdef", "dega", "gfbc", dict(a=30, b=16, c=16, d=24, e=16, f=16, g=24), F64)
    d = describe(engine, c31r)
    assert d["backend"] == "ttgt" and d["kernel"] == "dmma_f64_tma" and d["umma"]["coalesced_store"] and not d["umma"]["store_across_slabs"]
    # operands that are K-major on different contracted modes cannot be described to TMA where they lie
    c28 = Contraction("abcd", "eafb", "fdec", dict(a=72, b=72, c=72, d=72, e=72, f=72), F64)
    d = describe(engine, c28)
    assert d["backend"] == "ttgt" and d["kernel"] == "dmma_f64_tma"
    monkeypatch.setenv("TCONT_KERNEL", "gather")
    assert describe(engine, c28, 1)["kernel"] == "dmma_f64"
    monkeypatch.setenv("TCONT_KERNEL", "simt")
    assert describe(engine, c28, 1)["kernel"] == "simt"
    monkeypatch.delenv("TCONT_KERNEL")
    # tiny problems stay on the CUDA-core tiles
    assert describe(engine, CONFIGS["cfg1"][0])["kernel"] in ("simt", "dmma_f64_tma")


def test_fp64_row_widths_and_split_k(engine, monkeypatch):
    F64 = 1
    # extents of 72: slabs of 8 doubles (9 x 8) instead of 16 (5 x 16, 11 % padding) for the MN-major A,
    # 8 rows per slab for the K-major B
    d = describe(engine, Contraction("abcd", "aebf", "fdec", dict(a=72, b=72, c=72, d=72, e=72, f=72), F64), 1)
    u = d["umma"]
    assert d["kernel"] == "dmma_f64_tma" and (u["a_major"], u["b_major"], u["a_slab_w"], u["b_slab_w"]) == ("MN", "K", 8, 8)
    assert u["tiles_m"] == 41 and u["tiles_n"] == 81 and u["BK"] == 16        # ceil(5184 / 128), 5184 / 64
    # a contracted extent of 24: k chunks of 8 (64-byte rows for the K-major operand) instead of 2 x 16
    d = describe(engine, Contraction("abcdef", "degc", "gfab", dict(a=24, b=16, c=16, d=24, e=16, f=16, g=24), F64), 1)
    assert d["kernel"] == "dmma_f64_tma" and d["umma"]["BK"] == 8 and d["umma"]["k_iters"] == 3
    # narrow N: 128 x 32 tiles
    d = describe(engine, Contraction("abc", "dca", "bd", dict(a=312, b=24, c=296, d=312), F64), 1)
    assert d["kernel"] == "dmma_f64_tma" and d["umma"]["BN"] == 32
    # few tiles and a long contracted extent: split-K into a count of work units that fills whole waves
    # (296 units per wave for the FP64 kernel with its two consumer groups, 148 for tcgen05)
    for st, wave in ((F64, 296), (0, 148)):
        d = describe(engine, Contraction("ab", "acd", "dbc", dict(a=312, b=296, c=296, d=312), st), 1)
        u = d["umma"]
        units = u["tiles_m"] * u["tiles_n"] * u["k_splits"]
        assert u["k_splits"] > 1 and units / (-(-units // wave) * wave) >= 0.9, u
    # a little over one wave of tiles (162 on 148 SMs) is cut as well
    d = describe(engine, Contraction("abc", "adec", "ebd", dict(a=72, b=72, c=72, d=72, e=72), 0), 1)
    assert d["umma"]["tiles_m"] * d["umma"]["tiles_n"] == 162 and d["umma"]["k_splits"] >= 3
    monkeypatch.setenv("TCONT_SPLITK", "1")
    assert describe(engine, Contraction("ab", "acd", "dbc", dict(a=312, b=296, c=296, d=312), F64), 1)["umma"]["k_splits"] == 1


def test_every_reference_pattern_plans(engine):
    for fx in golden_fixtures():
        c = fixture_contraction(fx)
        for sel in (0, 1, 2):
            d = describe(engine, c, sel)
            assert d["Mtot"] * d["Ntot"] == c.size(c.modeC)
            assert d["Mtot"] * d["Ktot"] == c.size(c.modeB if d["swapped"] else c.modeA)


def test_plan_is_deterministic(engine):
    c = CONFIGS["cfg4"][0]
    assert describe(engine, c) == describe(engine, c)


def test_error_conventions(engine):
    E = engine.TCEquation
    with pytest.raises(ValueError, match="Missing extent for mode: d"):     # std::invalid_argument, src/tcont.cpp:44
        engine.plan(E("abc", "adc", "db", dict(a=2, b=2, c=2)))
    with pytest.raises(ValueError):
        engine.plan(E("ab", "ak", "kb", dict(a=2, b=0, k=2)))
    with pytest.raises(NotImplementedError, match="batch"):
        engine.plan(E("abn", "akn", "kbn", dict(a=2, b=2, k=2, n=2)))
    with pytest.raises(NotImplementedError):
        engine.plan(E("ab", "akx", "kb", dict(a=2, b=2, k=2, x=2)))
    with pytest.raises(ValueError):
        engine.launch(None)
    with pytest.raises(ValueError, match="ExecutionPlan is empty"):
        engine.prepare(None)


def test_flop_count_is_the_reference_formula(engine):
    c = CONFIGS["cfg2"][0]
    p = engine.plan(to_equation(engine, c))
    assert p.flops == pytest.approx(2.0 * 65536 * 1024 * 1024)
    assert engine.compute_gflops(p.equation, 1.0) == pytest.approx(p.flops / 1e6)
    assert engine.compute_gflops(p.equation, 0.0) == 0.0


def test_random_descriptors_plan_consistently(engine):
    """300 random descriptors (1-3 modes per group, ragged extents, random orders, both precisions, every backend
    selection): the planner accepts each one and its GEMM view multiplies out to the descriptor's extents."""
    import numpy as np

    from cases import random_contraction
    rng = np.random.default_rng(2024)
    for i in range(300):
        c = random_contraction(rng, int(rng.integers(0, 2)))
        sel = int(rng.integers(0, 3))
        d = engine.plan(to_equation(engine, c, sel)).describe()
        assert d["Mtot"] * d["Ntot"] == c.size(c.modeC), (i, c)
        assert d["Mtot"] * d["Ktot"] in (c.size(c.modeA), c.size(c.modeB)), (i, c)
        assert d["backend"] in ("direct", "ttgt") and d["kernel"] in ("simt", "umma_tf32", "dmma_f64", "dmma_f64_tma")
        if sel == 1:
            assert d["backend"] == "direct" and d["transpose_a"] is None and d["transpose_b"] is None
        u = d["umma"]
        if d["kernel"] in ("umma_tf32", "dmma_f64_tma"):
            assert u["eligible"] and u["smem_bytes"] <= 227 * 1024
            assert u["tiles_m"] * u["BM"] >= d["Mtot"] and u["tiles_n"] * u["BN"] >= d["Ntot"]
            assert u["k_iters"] * u["BK"] >= d["Ktot"] and 1 <= u["k_splits"] <= u["k_iters"]


def test_planning_is_reentrant(engine):
    """plan() from eight threads at once (ctypes releases the GIL) gives what a single thread gets, and an error raised
    in one thread does not leak into another's tcontb_last_error (it is thread-local)."""
    import threading

    import numpy as np

    from cases import random_contraction
    rng = np.random.default_rng(5)
    eqs = [to_equation(engine, random_contraction(rng, i % 2), i % 3) for i in range(40)]
    want = [engine.plan(e).describe() for e in eqs]
    bad = engine.TCEquation("ab", "ak", "kb", dict(a=4, b=4))   # extent of k missing
    failures = []

    def worker(tid):
        try:
            for rep in range(5):
                for i, e in enumerate(eqs):
                    if (i + tid) % 7 == 0:
                        with pytest.raises(ValueError, match="k"):
                            engine.plan(bad)
                    if engine.plan(e).describe() != want[i]:
                        failures.append((tid, rep, i))
        except Exception as ex:  # noqa: BLE001
            failures.append((tid, repr(ex)))

    threads = [threading.Thread(target=worker, args=(t,)) for t in range(8)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not failures, failures[:3]


def test_sub_tensor_views_take_their_strides_from_the_parent(engine):
    """tcontb_plan_create_strided: modes fuse only where the view leaves no gap between them; a view whose strides
    are not multiples of 16 bytes cannot be staged by TMA; parents must cover their views."""
    c = CONFIGS["cfg3"][0]
    eq = to_equation(engine, c)
    dense = engine.plan(eq).describe()
    assert dense["views"] is False and dense["A"] == ["a:48", "e:48", "ij:576"]
    # A is a view with a gap after i (parent 26 wide in i): i and j no longer fuse anywhere; b and c still do
    d = engine.plan_views(eq, None, [48, 48, 26, 24], None).describe()
    assert d["views"] is True and d["A"] == ["a:48", "e:48", "i:24", "j:24"] and d["B"][0] == "bc:2304"
    assert d["C"] == ["a:48", "bc:2304", "i:24", "j:24", "k:24"]
    assert d["kernel"] == "dmma_f64_tma"                      # strides stay multiples of 16 bytes
    # a parent that is one element wider in the stride-1 mode: 8-byte-aligned rows only, so no TMA
    d = engine.plan_views(eq, None, [49, 48, 24, 24], None).describe()
    assert d["kernel"] in ("dmma_f64", "simt") and "16 bytes" in d["umma"]["why_not"]
    # C as a view: no split-K (there is no workspace laid out like C)
    lk = Contraction("ab", "acd", "dbc", dict(a=312, b=296, c=296, d=312), 1)
    assert engine.plan(to_equation(engine, lk, 1)).describe()["umma"]["k_splits"] > 1
    assert engine.plan_views(to_equation(engine, lk, 1), [320, 296], None, None).describe()["umma"]["k_splits"] == 1
    with pytest.raises(ValueError):
        engine.plan_views(eq, None, [40, 48, 24, 24], None)   # parent smaller than the view


def test_tcgen05_kernel_forms(engine, monkeypatch):
    """Which form of the tcgen05 kernel a plan asks for: CTA pairs with stages of 64 k and one producer warp for
    large problems; one CTA per tile with two producer warps (and an even number of stages) otherwise; k chunks of
    24 where 32 would pad an MN-major contracted mode by a quarter."""
    from oracle_lib import F32
    pair = describe(engine, CONFIGS["cfg2"][0])["umma"]
    assert pair["pair"] is True and pair["BK"] == 64 and pair["producers"] == 1 and pair["stages"] == 3
    # the 72-extent 4-D family (reference case 22): both operands MN-major, chunked mode of extent 72
    c22 = Contraction("abcd", "aecf", "bfde", dict(a=72, b=72, c=72, d=72, e=72, f=72), F32)
    one = describe(engine, c22, 1)["umma"]
    assert one["pair"] is False and one["producers"] == 2 and one["stages"] % 2 == 0 and one["BK"] == 24
    monkeypatch.setenv("TCONT_UMMA_NO_BK24", "1")
    assert describe(engine, c22, 1)["umma"]["BK"] == 32
    monkeypatch.delenv("TCONT_UMMA_NO_BK24")
    # one k iteration per tile (the low-K configuration after its transposes): a second producer has nothing to do
    low_k = describe(engine, CONFIGS["cfg4"][0])["umma"]
    assert low_k["pair"] is False and low_k["producers"] == 1
    monkeypatch.setenv("TCONT_UMMA_PRODUCERS", "1")
    assert describe(engine, c22, 1)["umma"]["producers"] == 1
