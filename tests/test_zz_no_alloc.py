"""GPU: the allocation-free entry point (tcontb_contract_no_alloc) against the regular run objects.

That entry point exists for callers that cannot let the library allocate device memory (their
own pool holds the whole GPU, or they cannot take cudaMalloc's synchronisation); it keeps its
scratch in an array built into the library.  The file is named so that pytest collects it last.
Both entry points are called through the C ABI on the same device buffers; FP64 results must be
bit-identical (same kernel, same tables), FP32 results are held to the reference tolerance because
the regular path may use TF32 tensor cores.  Each case runs twice in a row, and a small case
follows a large one, so stale scratch contents would show.
"""
import numpy as np
import pytest

from oracle_lib import F32, F64, Contraction

pytestmark = pytest.mark.gpu

CASES = [
    Contraction("abcd", "aebf", "fdec", dict(a=24, b=24, c=24, d=24, e=16, f=16), F64),
    Contraction("abc", "bda", "dc", dict(a=13, b=7, c=5, d=9), F64),
    Contraction("abcde", "efba", "cfd", dict(a=12, b=6, c=12, d=6, e=12, f=8), F32),
    Contraction("abc", "db", "adc", dict(a=20, c=6, b=14, d=10), F64),       # C's stride-1 mode in the right operand
]


def _both(engine, oracle, c):
    import torch
    from tcont_b200 import api
    lo, hi = (0.0, 1.0) if c.scalar_type == F32 else (-1.0, 1.0)
    A, B = oracle.inputs(c, 21, lo, hi)
    dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    n = c.size(c.modeC)
    c_regular = torch.zeros(n, dtype=dA.dtype, device="cuda")
    c_noalloc = torch.full((n,), float("nan"), dtype=dA.dtype, device="cuda")
    eq = engine.TCEquation(c.modeC, c.modeA, c.modeB, dict(c.extent), "-", engine.ScalarType(c.scalar_type),
                           engine.BackendSelection.COGENT)
    run = api.prepare_on_device(engine.plan(eq), dA.data_ptr(), dB.data_ptr(), c_regular.data_ptr(), keep=(dA, dB, c_regular))
    engine.launch(run)
    stream = torch.cuda.current_stream().cuda_stream
    outs = []
    for call in range(2):   # two calls in a row through the allocation-free entry point
        c_noalloc.fill_(float("nan"))
        torch.cuda.synchronize()
        # free device memory as the driver counts it (cudaMemGetInfo): sees any allocation, whoever makes it,
        # not only those of torch's caching allocator
        free_before, _ = torch.cuda.mem_get_info()
        api.contract_no_alloc(eq, dA.data_ptr(), dB.data_ptr(), c_noalloc.data_ptr(), stream)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        if call == 1:   # (the first call on a device may load the kernels' module)
            assert free_after == free_before, f"device memory changed by {free_before - free_after} bytes across the call"
        outs.append(c_noalloc.cpu().numpy().copy())
    return c_regular.cpu().numpy(), outs, (A, B)


@pytest.mark.parametrize("c", CASES, ids=lambda c: f"{c.modeC}-{c.modeA}-{c.modeB}-{'f64' if c.scalar_type else 'f32'}")
def test_no_alloc_matches_regular_entry_point(engine, oracle, c):
    regular, outs, (A, B) = _both(engine, oracle, c)
    for got in outs:
        # the regular entry point may run another kernel (tensor path, split-K): same tolerance as against the oracle
        diff, nonfinite = oracle.compare(regular, got, c.scalar_type)
        assert (diff, nonfinite) == (0, 0)
        diff, nonfinite = oracle.compare(oracle.contract(c, A, B), got, c.scalar_type)
        assert (diff, nonfinite) == (0, 0)


def test_no_alloc_size_limit_is_exact(engine, oracle):
    """2*(M+N+K) = 524288 entries is the last size that fits the built-in scratch: accepted and correct;
    one row more is rejected before any device work."""
    import torch
    from tcont_b200 import api
    c = Contraction("ab", "ak", "kb", dict(a=262000, b=136, k=8), F64)
    assert 2 * (262000 + 136 + 8) == 524288
    A, B = oracle.inputs(c, 4, -1.0, 1.0)
    dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    dC = torch.full((c.size(c.modeC),), float("nan"), dtype=torch.float64, device="cuda")
    eq = engine.TCEquation(c.modeC, c.modeA, c.modeB, dict(c.extent))
    api.contract_no_alloc(eq, dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    diff, nonfinite = oracle.compare(oracle.contract(c, A, B), dC.cpu().numpy(), F64)
    assert (diff, nonfinite) == (0, 0)
    over = engine.TCEquation("ab", "ak", "kb", dict(a=262001, b=136, k=8))
    with pytest.raises(NotImplementedError, match="too large for the allocation-free entry point"):
        api.contract_no_alloc(over, dA.data_ptr(), dB.data_ptr(), dC.data_ptr())


def test_no_alloc_rejects_oversized_contractions(engine):
    import torch
    from tcont_b200 import api
    big = engine.TCEquation("ab", "ak", "kb", dict(a=300000, b=8, k=8))
    x = torch.zeros(8, device="cuda", dtype=torch.float64)
    with pytest.raises(NotImplementedError, match="too large for the allocation-free entry point"):
        api.contract_no_alloc(big, x.data_ptr(), x.data_ptr(), x.data_ptr())
    with pytest.raises(ValueError):
        api.contract_no_alloc(engine.TCEquation("ab", "ak", "kb", dict(a=4, b=4)), x.data_ptr(), x.data_ptr(), x.data_ptr())
