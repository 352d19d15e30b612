"""tcont_b200 -- B200-native tensor-contraction engine behind TconT's plan/prepare/launch surface.

The product is the pair of shared libraries built from csrc/ (the C ABI of include/tcontb.h and
the C++ surface of include/tcont.hpp).  This package is the thin Python binding used by the tests
and the benchmark; it mirrors the reference's names (TCEquation, plan, prepare, launch, warmup,
zero_output, copy_output_to_host, compute_gflops).
"""
import importlib

from . import sharding  # noqa: F401

# Names of .api, resolved on first use: importing the package must not need the shared library,
# because `python -m tcont_b200.build` (which creates it) imports the package first.  Anything that
# computes goes through .api, whose import fails loudly when libtcontb.so is missing.
_API_NAMES = (
    "Backend", "BackendSelection", "ExecutionPlan", "ExecutionRun", "ScalarType", "TCEquation", "TcontError",
    "compute_gflops", "copy_output_to_host", "fill_uniform", "input_left_host_data", "input_right_host_data",
    "launch", "library_path", "plan", "plan_views", "prepare", "stage_times", "transpose", "warmup", "zero_output",
)


def __getattr__(name):
    if name == "api":
        return importlib.import_module(".api", __name__)
    if name in _API_NAMES:
        return getattr(importlib.import_module(".api", __name__), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def __dir__():
    return sorted(list(globals()) + list(_API_NAMES))
