"""GPU: sub-tensor views (tcontb_plan_create_strided).  Every tensor may be a view into a larger column-major parent:
strides come from the parent's extents, the data pointer is the view's first element.  The views are cut out of parents
on the host, the contraction of the dense copies by the oracle is the expected result, and what lies outside the view of
C in its parent must stay untouched."""
import numpy as np
import pytest

from cases import to_equation
from oracle_lib import F32, F64, Contraction

pytestmark = pytest.mark.gpu


def _view(rng, modes, extent, pads, dtype, lo_offsets):
    """A parent tensor (numpy order: slowest mode first), the view's offsets and the flat element offset of its start."""
    shape_view = [extent[m] for m in modes]
    parent = [extent[m] + pads.get(m, 0) for m in modes]
    full = rng.uniform(-1.0, 1.0, size=parent[::-1]).astype(dtype)
    start = [lo_offsets.get(m, 0) for m in modes]
    index = tuple(slice(s, s + e) for s, e in zip(start[::-1], shape_view[::-1]))
    flat_start, stride = 0, 1
    for s, p in zip(start, parent):
        flat_start += s * stride
        stride *= p
    return full, index, parent, flat_start


CASES = [
    # (descriptor, per-tensor {mode: extra parent extent}, per-tensor {mode: offset of the view}, backend selection)
    ("tf32_tma", Contraction("abc", "adc", "db", dict(a=128, c=5, b=96, d=64), F32),
     dict(A=dict(a=32, d=8, c=2), B=dict(d=32, b=4), C=dict(a=64, b=3, c=1)), dict(A=dict(a=16, d=3, c=1), B=dict(d=8, b=2), C=dict(a=32, b=1)), 0),
    ("tf32_ttgt", Contraction("abcde", "efba", "cfd", dict(a=12, b=8, c=16, d=6, e=8, f=8), F32),
     dict(A=dict(e=8, b=2), B=dict(c=16, d=1), C=dict(a=4, e=3)), dict(A=dict(e=4, b=1), B=dict(c=8), C=dict(a=4, e=1)), 2),
    ("fp64_tma", Contraction("abcd", "aebf", "cfde", dict(a=64, b=6, c=48, d=5, e=16, f=4), F64),
     dict(A=dict(a=16, e=2, f=1), B=dict(c=16, d=2), C=dict(a=32, c=2, d=1)), dict(A=dict(a=8, e=1), B=dict(c=8, d=1), C=dict(a=16, c=2)), 1),
    ("fp64_simt_unaligned_rows", Contraction("abc", "adc", "db", dict(a=13, c=5, b=11, d=7), F64),
     dict(A=dict(a=3, d=1), B=dict(d=2), C=dict(a=5, b=1)), dict(A=dict(a=2), B=dict(d=2), C=dict(a=2, b=1)), 0),
    ("fp64_fusable_but_gapped", Contraction("abcijk", "aeij", "bcek", dict(a=48, b=6, c=4, e=16, i=4, j=3, k=5), F64),
     dict(A=dict(i=2), B=dict(b=1), C=dict(b=1, i=1)), dict(A=dict(i=1), B=dict(), C=dict(i=1)), 1),
]


@pytest.mark.parametrize("name,c,pads,offs,sel", CASES, ids=[x[0] for x in CASES])
def test_views_match_dense_copies(engine, oracle, monkeypatch, name, c, pads, offs, sel):
    import torch
    from tcont_b200 import api
    if name == "fp64_tma":
        monkeypatch.setenv("TCONT_KERNEL", "tma")   # (the cost table would send a problem this small to the CUDA cores)
    rng = np.random.default_rng(12)
    dt = c.dtype
    pa, ia, parA, offA = _view(rng, c.modeA, c.extent, pads["A"], dt, offs["A"])
    pb, ib, parB, offB = _view(rng, c.modeB, c.extent, pads["B"], dt, offs["B"])
    pc, ic, parC, offC = _view(rng, c.modeC, c.extent, pads["C"], dt, offs["C"])
    elt = np.dtype(dt).itemsize
    if name != "fp64_simt_unaligned_rows":
        assert offA * elt % 16 == 0 and offB * elt % 16 == 0 and offC * elt % 16 == 0
    dA, dB, dC = torch.from_numpy(pa.ravel()).cuda(), torch.from_numpy(pb.ravel()).cuda(), torch.from_numpy(pc.ravel()).cuda()
    eq = to_equation(engine, c, sel)
    plan = engine.plan_views(eq, parC, parA, parB)
    desc = plan.describe()
    assert desc["views"] is True
    assert desc["kernel"] == {"tf32_tma": "umma_tf32", "tf32_ttgt": "umma_tf32", "fp64_tma": "dmma_f64_tma"}.get(name, desc["kernel"])
    if name == "fp64_fusable_but_gapped":
        # i and j would fuse in dense tensors; the view of A leaves a gap after i, b and c fuse nowhere because B's parent is wider in b
        assert all(":" in m and not m.startswith("ij") for m in desc["A"]) and not any(m.startswith("bc") for m in desc["B"])
    try:
        run = api.prepare_on_device(plan, dA.data_ptr() + offA * elt, dB.data_ptr() + offB * elt, dC.data_ptr() + offC * elt, keep=(dA, dB, dC))
    except ValueError as e:
        assert name == "fp64_simt_unaligned_rows" and "16-byte aligned" in str(e)   # documented: view pointers must be 16-byte aligned
        return
    engine.launch(run)
    engine.launch(run)
    torch.cuda.synchronize()
    assert run.device_status() == 0
    got_parent = dC.cpu().numpy().reshape(pc.shape)
    A, B = np.ascontiguousarray(pa[ia]).ravel(), np.ascontiguousarray(pb[ib]).ravel()
    got = np.ascontiguousarray(got_parent[ic]).ravel()
    if c.scalar_type == F64:
        assert oracle.compare(oracle.contract(c, A, B), got, F64) == (0, 0)
    else:
        tensor = desc["kernel"] == "umma_tf32"
        ref = oracle.contract(c, A, B, rounding=1 if tensor else 0)
        scale = oracle.contract(c, np.abs(A), np.abs(B), rounding=1)
        assert float((np.abs(got.astype(np.float64) - ref) / (scale + 1e-30)).max()) < 2e-5
    # nothing outside the view of C was written
    mask = np.ones(pc.shape, dtype=bool)
    mask[ic] = False
    np.testing.assert_array_equal(got_parent[mask], pc[mask])
    # what views cannot do says so
    with pytest.raises(NotImplementedError):
        engine.copy_output_to_host(run)
    with pytest.raises(NotImplementedError):
        engine.prepare(plan, A, B)


def test_view_errors(engine):
    eq = engine.TCEquation("abc", "adc", "db", dict(a=8, b=8, c=8, d=8))
    with pytest.raises(ValueError):
        engine.plan_views(eq, [8, 8, 4], None, None)        # a parent smaller than its view
    with pytest.raises(ValueError):
        engine.plan_views(eq, [8, 8], None, None)           # not one extent per mode
    d = engine.plan_views(eq, None, [16, 8, 8], None).describe()
    assert d["views"] is True
