"""CPU-only: the oracle against the committed golden fixtures and the reference's own verifier."""
import numpy as np
import pytest

from cases import fixture_contraction, golden_fixtures
from oracle_lib import F32, F64, Contraction, RefVerifier

FIXTURES = golden_fixtures()


@pytest.mark.parametrize("fx", FIXTURES, ids=[f["name"] for f in FIXTURES])
def test_oracle_matches_golden(oracle, fx):
    c = fixture_contraction(fx)
    A, B = oracle.inputs(c, fx["seed"], fx["lo"], fx["hi"])
    out = oracle.contract(c, A, B)
    idx = np.array(fx["sample_index"])
    np.testing.assert_allclose(out[idx], np.array(fx["sample_value"]), rtol=1e-13, atol=1e-15)
    assert out.sum() == pytest.approx(fx["sum"], rel=1e-12, abs=1e-12)
    assert np.abs(out).sum() == pytest.approx(fx["abssum"], rel=1e-12)


@pytest.mark.skipif(not RefVerifier.available(), reason="oracle/_ref was not built (no reference tree at build time)")
@pytest.mark.parametrize("fx", [f for f in FIXTURES if f["ref_case"] is not None][::7], ids=lambda f: f["name"])
def test_oracle_passes_reference_verifier(oracle, fx, capfd):
    ref = RefVerifier()
    c = fixture_contraction(fx)
    A, B = oracle.inputs(c, fx["seed"], fx["lo"], fx["hi"])
    out = oracle.contract(c, A, B)
    ok, diff, total = ref.verify(fx["ref_case"], c, out.astype(c.dtype), A, B)
    assert ok and diff == 0 and total == out.size
    bad = out.copy()
    bad[0] += 1.0
    ok, diff, _ = ref.verify(fx["ref_case"], c, bad.astype(c.dtype), A, B)
    assert not ok and diff == 1


def test_oracle_equals_einsum(oracle):
    c = Contraction("abcd", "aebf", "fdec", dict(a=6, b=5, c=4, d=3, e=7, f=2), F64)
    A, B = oracle.inputs(c, 9)
    out = oracle.contract(c, A, B)
    An = A.reshape(2, 5, 7, 6).transpose(3, 2, 1, 0)   # numpy sees the reversed mode order
    Bn = B.reshape(4, 7, 3, 2).transpose(3, 2, 1, 0)
    want = np.einsum("aebf,fdec->abcd", An, Bn).transpose(3, 2, 1, 0).ravel()
    np.testing.assert_allclose(out, want, rtol=1e-13, atol=1e-14)


def test_comparator_semantics(oracle):
    # tccg_verify.cpp:1655-1683: non-finite counts as a difference; tol = max(abs, rel*max(|h|,|d|))
    ref = np.array([1.0, 0.0, 100.0, 1.0])
    out = np.array([1.0 + 5e-10, 5e-12, 100.0 + 5e-8, np.nan])
    diff, nonfinite = oracle.compare(ref, out, F64)
    assert (diff, nonfinite) == (1, 1)
    diff, _ = oracle.compare(ref[:3], ref[:3] + np.array([2e-9, 2e-11, 2e-7]), F64)
    assert diff == 3
    assert oracle.tolerance(F32) == (2e-3, 5e-2)
    assert oracle.tolerance(F64) == (1e-11, 1e-9)


def test_tf32_operand_rounding_modes(oracle):
    c = Contraction("ab", "ak", "kb", dict(a=1, b=1, k=1), F32)
    x = np.array([1.0 + 2.0 ** -11 + 2.0 ** -12], dtype=np.float32)  # bits below the TF32 mantissa
    one = np.array([1.0], dtype=np.float32)
    exact = oracle.contract(c, x, one, rounding=0)[0]
    trunc = oracle.contract(c, x, one, rounding=1)[0]
    rna = oracle.contract(c, x, one, rounding=2)[0]
    assert exact == float(x[0]) and trunc == 1.0 and rna == 1.0 + 2.0 ** -10


def test_sampled_equals_full(oracle):
    c = Contraction("abc", "adc", "db", dict(a=8, b=6, c=5, d=7), F32)
    A, B = oracle.inputs(c, 3)
    full = oracle.contract(c, A, B, rounding=1)
    idx = np.array([0, 5, 17, 239, 100], dtype=np.int64)
    np.testing.assert_array_equal(oracle.contract_sampled(c, A, B, idx, rounding=1), full[idx])


def test_fill_is_counter_based(oracle):
    a = oracle.fill(100, F64, 7, 0, -1.0, 1.0)
    b = oracle.fill(60, F64, 7, 40, -1.0, 1.0)
    np.testing.assert_array_equal(a[40:], b)
    assert a.min() >= -1.0 and a.max() < 1.0 and abs(a.mean()) < 0.3
    assert not np.array_equal(a, oracle.fill(100, F64, 8, 0, -1.0, 1.0))


def test_rejects_inexpressible(oracle):
    with pytest.raises(ValueError):
        oracle.contract(Contraction("ab", "ab", "ab", dict(a=2, b=2), F64), np.zeros(4), np.zeros(4))
