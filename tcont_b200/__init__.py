"""tcont_b200 -- B200-native tensor-contraction engine behind TconT's plan/prepare/launch surface.

The product is the pair of shared libraries built from csrc/ (the C ABI of include/tcontb.h and
the C++ surface of include/tcont.hpp).  This package is the thin Python binding used by the tests
and the benchmark; it mirrors the reference's names (TCEquation, plan, prepare, launch, warmup,
zero_output, copy_output_to_host, compute_gflops).
"""
from . import sharding  # noqa: F401
from .api import (  # noqa: F401
    Backend,
    BackendSelection,
    ExecutionPlan,
    ExecutionRun,
    ScalarType,
    TCEquation,
    TcontError,
    compute_gflops,
    copy_output_to_host,
    fill_uniform,
    input_left_host_data,
    input_right_host_data,
    launch,
    library_path,
    plan,
    prepare,
    stage_times,
    transpose,
    warmup,
    zero_output,
)
