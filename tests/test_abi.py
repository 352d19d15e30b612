"""CPU-only: the C-ABI library loads, exports what include/tcontb.h declares, and refuses to
compute without a GPU (no CPU fallback)."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "tcontb.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tcontb_[a-z_0-9]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(engine):
    lib = ctypes.CDLL(engine.library_path())
    names = declared_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/tcontb.h but not exported"


def test_cpp_surface_library_exports_tcont_namespace(engine):
    path = os.path.join(os.path.dirname(engine.library_path()), "libtcont.so")
    assert os.path.exists(path)
    lib = ctypes.CDLL(path)
    # the symbols the reference harness imports (mangled), e.g. TconT::plan(TconT::TCEquation const&)
    for sym in ["_ZN5TconT4planERKNS_10TCEquationE", "_ZN5TconT7prepareERKNS_13ExecutionPlanE",
                "_ZN5TconT6launchERKNS_12ExecutionRunE", "_ZN5TconT6warmupERKNS_12ExecutionRunEi",
                "_ZN5TconT11zero_outputERKNS_12ExecutionRunE", "_ZN5TconT11stage_timesERKNS_12ExecutionRunE",
                "_ZN5TconT20input_left_host_dataERKNS_12ExecutionRunE", "_ZN5TconT21input_right_host_dataERKNS_12ExecutionRunE",
                "_ZN5TconT19copy_output_to_hostERKNS_12ExecutionRunEPvm", "_ZN5TconT14compute_gflopsERKNS_10TCEquationEf",
                "_ZN5TconT10check_cudaE9cudaErrorPKc"]:
        assert hasattr(lib, sym), sym


def test_fill_matches_oracle_stream(engine, oracle):
    for st, dt in ((0, np.float32), (1, np.float64)):
        a = engine.fill_uniform(1000, engine.ScalarType(st), 42, 17, -0.5, 0.5)
        b = oracle.fill(1000, st, 42, 17, -0.5, 0.5)
        assert a.dtype == dt
        np.testing.assert_array_equal(a, b)


def test_no_cpu_fallback(engine):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    p = engine.plan(engine.TCEquation("ab", "ak", "kb", dict(a=4, b=4, k=4)))
    with pytest.raises(engine.TcontError, match="no usable CUDA device"):
        engine.prepare(p)


def test_status_codes_map_like_the_cpp_surface(engine):
    """TCONTB_INVALID_ARGUMENT -> std::invalid_argument (ValueError here), TCONTB_RUNTIME_ERROR -> std::runtime_error
    (TcontError here: what a raised device status word turns a result call into), TCONTB_UNSUPPORTED -> its own
    exception here, std::runtime_error in the C++ surface (tcont_shim.cpp: everything but invalid_argument)."""
    from tcont_b200 import api
    api._check(0)
    with pytest.raises(ValueError):
        api._check(1)
    with pytest.raises(api.TcontError):
        api._check(2)
    with pytest.raises(NotImplementedError):
        api._check(3)
