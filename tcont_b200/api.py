"""ctypes binding of libtcontb.so, shaped like the reference's C++ surface (include/tcont.hpp).

There is no fallback of any kind: if the shared library is missing the import fails, and every
compute call raises when no B200-class device is present.
"""
from __future__ import annotations

import ctypes as C
import json
import os
from dataclasses import dataclass, field
from enum import IntEnum

import numpy as np

_PKG = os.path.dirname(os.path.abspath(__file__))


def library_path() -> str:
    return os.path.join(_PKG, "libtcontb.so")


if not os.path.exists(library_path()):
    raise ImportError(
        f"{library_path()} is missing: build it with `python -m tcont_b200.build` (needs nvcc). "
        "The engine is CUDA-only; there is no Python or CPU implementation to fall back to.")

_lib = C.CDLL(library_path())


class ScalarType(IntEnum):  # TconT::ScalarType (tcont.hpp:12-15)
    Float32 = 0
    Float64 = 1


class BackendSelection(IntEnum):  # TconT::BackendSelection (tcont.hpp:44-48)
    MODEL = 0
    COGENT = 1
    TTGT_CUTT = 2


class Backend(IntEnum):  # TconT::Backend (tcont.hpp:39-42)
    COGENT = 0
    TTGT_CUTT = 1


def backend_name(b: Backend) -> str:
    return "cogent" if b == Backend.COGENT else "ttgt"


class TcontError(RuntimeError):
    pass


class _Desc(C.Structure):
    _fields_ = [("nC", C.c_int), ("nA", C.c_int), ("nB", C.c_int),
                ("modeC", C.c_char_p), ("modeA", C.c_char_p), ("modeB", C.c_char_p),
                ("op", C.c_char), ("scalar_type", C.c_int), ("n_ext", C.c_int),
                ("ext_mode", C.c_char_p), ("ext_val", C.POINTER(C.c_int64)), ("backend_selection", C.c_int)]


_lib.tcontb_last_error.restype = C.c_char_p
_lib.tcontb_plan_create.argtypes = [C.POINTER(_Desc), C.POINTER(C.c_void_p)]
_lib.tcontb_plan_create_strided.argtypes = [C.POINTER(_Desc), C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.POINTER(C.c_int64),
                                            C.POINTER(C.c_void_p)]
_lib.tcontb_plan_destroy.argtypes = [C.c_void_p]
_lib.tcontb_plan_backend.argtypes = [C.c_void_p]
_lib.tcontb_plan_describe.argtypes = [C.c_void_p, C.c_char_p, C.c_size_t]
_lib.tcontb_plan_flops.argtypes = [C.c_void_p]
_lib.tcontb_plan_flops.restype = C.c_double
_lib.tcontb_run_create.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
_lib.tcontb_run_create_with_inputs.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p)]
_lib.tcontb_run_create_on_device.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p)]
_lib.tcontb_run_destroy.argtypes = [C.c_void_p]
_lib.tcontb_run_set_stream.argtypes = [C.c_void_p, C.c_void_p]
_lib.tcontb_run_upload_inputs.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
_lib.tcontb_run_set_scalars.argtypes = [C.c_void_p, C.c_double, C.c_double]
_lib.tcontb_run_launch.argtypes = [C.c_void_p]
_lib.tcontb_run_warmup.argtypes = [C.c_void_p, C.c_int]
_lib.tcontb_run_zero_output.argtypes = [C.c_void_p]
_lib.tcontb_run_stage_times.argtypes = [C.c_void_p, C.POINTER(C.c_float)]
_lib.tcontb_run_host_input.argtypes = [C.c_void_p, C.c_int]
_lib.tcontb_run_host_input.restype = C.c_void_p
_lib.tcontb_run_copy_output.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
_lib.tcontb_run_time_launches.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_float), C.POINTER(C.c_int64)]
_lib.tcontb_run_contract_host.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_int64),
                                          C.POINTER(C.c_int64)]
_lib.tcontb_run_device_status.argtypes = [C.c_void_p, C.POINTER(C.c_int)]
_lib.tcontb_run_ksplit_enable.argtypes = [C.c_void_p, C.c_int, C.c_int]
_lib.tcontb_run_ksplit_export.argtypes = [C.c_void_p, C.c_char_p, C.c_size_t]
_lib.tcontb_run_ksplit_import.argtypes = [C.c_void_p, C.c_int, C.c_char_p, C.c_size_t]
_lib.tcontb_run_ksplit_attach.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
_lib.tcontb_run_ksplit_reduce.argtypes = [C.c_void_p]
_lib.tcontb_run_ksplit_range_elements.argtypes = [C.c_void_p]
_lib.tcontb_run_ksplit_range_elements.restype = C.c_int64
_lib.tcontb_fill_uniform.argtypes = [C.c_void_p, C.c_int, C.c_int64, C.c_uint64, C.c_uint64, C.c_double, C.c_double]
_lib.tcontb_transpose.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.POINTER(C.c_int64), C.POINTER(C.c_int), C.c_int,
                                  C.c_void_p]


_lib.tcontb_contract_no_alloc.argtypes = [C.POINTER(_Desc), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
_lib.tcontb_no_alloc_last_error.restype = C.c_char_p


def _check(status: int):
    if status == 0:
        return
    msg = (_lib.tcontb_last_error() or b"").decode()
    if status == 1:
        raise ValueError(msg)          # std::invalid_argument in the C++ surface
    if status == 3:
        raise NotImplementedError(msg)
    raise TcontError(msg)              # std::runtime_error


@dataclass
class TCEquation:
    """TconT::TCEquation (tcont.hpp:74-83): modes are strings of single-character names."""

    modeC: str
    modeA: str
    modeB: str
    extent: dict = field(default_factory=dict)
    op: str = "-"
    scalar_type: ScalarType = ScalarType.Float64
    backend_selection: BackendSelection = BackendSelection.MODEL

    def size(self, modes: str) -> int:
        n = 1
        for m in modes:
            if m not in self.extent:
                raise ValueError(f"Missing extent for mode: {m}")
            n *= int(self.extent[m])
        return n

    @property
    def dtype(self):
        return np.float64 if self.scalar_type == ScalarType.Float64 else np.float32


class ExecutionPlan:
    def __init__(self, handle, equation: TCEquation):
        self._h = handle
        self.equation = equation
        self.backend = Backend(_lib.tcontb_plan_backend(handle))

    def describe(self) -> dict:
        buf = C.create_string_buffer(8192)
        _check(_lib.tcontb_plan_describe(self._h, buf, len(buf)))
        return json.loads(buf.value.decode())

    @property
    def flops(self) -> float:
        return float(_lib.tcontb_plan_flops(self._h))

    def __del__(self):
        if getattr(self, "_h", None) and _lib is not None:   # (module globals are gone at interpreter exit)
            _lib.tcontb_plan_destroy(self._h)
            self._h = None


class ExecutionRun:
    def __init__(self, handle, plan_: ExecutionPlan, keep=()):
        self._h = handle
        self.plan = plan_
        self.equation = plan_.equation
        self.backend = plan_.backend
        self._keep = keep  # device tensors that must outlive the run

    def set_stream(self, cuda_stream: int):
        _check(_lib.tcontb_run_set_stream(self._h, C.c_void_p(cuda_stream)))

    def set_scalars(self, alpha: float = 1.0, beta: float = 0.0):
        """Later launches compute C = alpha * (A*B) + beta * C; (1, 0) is the reference's overwrite."""
        _check(_lib.tcontb_run_set_scalars(self._h, float(alpha), float(beta)))

    def time_launches(self, iterations: int):
        ms, n = C.c_float(), C.c_int64()
        _check(_lib.tcontb_run_time_launches(self._h, iterations, C.byref(ms), C.byref(n)))
        return ms.value, n.value

    def contract_host(self, a: np.ndarray, b: np.ndarray, c: np.ndarray):
        """Upload a and b, launch, download into c (host buffers). Returns (h2d, d2h) bytes."""
        hi, ho = C.c_int64(), C.c_int64()
        _check(_lib.tcontb_run_contract_host(self._h, a.ctypes.data, b.ctypes.data, c.ctypes.data, C.byref(hi), C.byref(ho)))
        return hi.value, ho.value

    def contract_host_ptr(self, a_ptr: int, b_ptr: int, c_ptr: int):
        hi, ho = C.c_int64(), C.c_int64()
        _check(_lib.tcontb_run_contract_host(self._h, a_ptr, b_ptr, c_ptr, C.byref(hi), C.byref(ho)))
        return hi.value, ho.value

    # ---- contracted-mode split over the GPUs of one box (include/tcontb.h) ----
    def ksplit_enable(self, ranks: int, rank: int):
        _check(_lib.tcontb_run_ksplit_enable(self._h, int(ranks), int(rank)))

    def ksplit_export(self) -> bytes:
        buf = C.create_string_buffer(64)
        _check(_lib.tcontb_run_ksplit_export(self._h, buf, 64))
        return buf.raw

    def ksplit_import(self, peer_rank: int, handle: bytes):
        _check(_lib.tcontb_run_ksplit_import(self._h, int(peer_rank), handle, len(handle)))

    def ksplit_attach(self, peer_rank: int, peer: "ExecutionRun"):
        _check(_lib.tcontb_run_ksplit_attach(self._h, int(peer_rank), peer._h))

    def ksplit_reduce(self):
        _check(_lib.tcontb_run_ksplit_reduce(self._h))

    def ksplit_range_elements(self) -> int:
        return int(_lib.tcontb_run_ksplit_range_elements(self._h))

    def device_status(self) -> int:
        s = C.c_int()
        _check(_lib.tcontb_run_device_status(self._h, C.byref(s)))
        return s.value

    def __del__(self):
        if getattr(self, "_h", None) and _lib is not None:
            _lib.tcontb_run_destroy(self._h)
            self._h = None


def plan(desc: TCEquation) -> ExecutionPlan:
    """TconT::plan (src/tcont.cpp:58-88)."""
    modes = "".join(sorted(desc.extent))
    vals = (C.c_int64 * max(1, len(modes)))(*[int(desc.extent[m]) for m in modes])
    d = _Desc(len(desc.modeC), len(desc.modeA), len(desc.modeB), desc.modeC.encode(), desc.modeA.encode(),
              desc.modeB.encode(), desc.op.encode()[:1] or b"?", int(desc.scalar_type), len(modes), modes.encode(), vals,
              int(desc.backend_selection))
    h = C.c_void_p()
    _check(_lib.tcontb_plan_create(C.byref(d), C.byref(h)))
    return ExecutionPlan(h, desc)


def plan_views(desc: TCEquation, parent_c=None, parent_a=None, parent_b=None) -> ExecutionPlan:
    """tcontb_plan_create_strided: the tensors are sub-tensor views of larger column-major tensors; parent_x lists
    the extents of tensor x's modes in its parent (None = dense).  Run it with prepare_on_device on pointers at the
    views' first elements."""
    modes = "".join(sorted(desc.extent))
    vals = (C.c_int64 * max(1, len(modes)))(*[int(desc.extent[m]) for m in modes])
    d = _Desc(len(desc.modeC), len(desc.modeA), len(desc.modeB), desc.modeC.encode(), desc.modeA.encode(),
              desc.modeB.encode(), desc.op.encode()[:1] or b"?", int(desc.scalar_type), len(modes), modes.encode(), vals,
              int(desc.backend_selection))

    def arr(p, n):
        if p is None:
            return None
        if len(p) != n:
            raise ValueError("parent extents must be given for every mode of the tensor")
        return (C.c_int64 * n)(*[int(x) for x in p])

    h = C.c_void_p()
    _check(_lib.tcontb_plan_create_strided(C.byref(d), arr(parent_c, len(desc.modeC)), arr(parent_a, len(desc.modeA)),
                                           arr(parent_b, len(desc.modeB)), C.byref(h)))
    return ExecutionPlan(h, desc)


def prepare(plan_: ExecutionPlan, a: np.ndarray | None = None, b: np.ndarray | None = None) -> ExecutionRun:
    """TconT::prepare (src/tcont.cpp:90-100). With a and b (host arrays in memory order) the run
    uses them instead of generating inputs."""
    if plan_ is None or not plan_._h:
        raise ValueError("ExecutionPlan is empty")
    h = C.c_void_p()
    if a is None and b is None:
        _check(_lib.tcontb_run_create(plan_._h, C.byref(h)))
        return ExecutionRun(h, plan_)
    eq = plan_.equation
    a = np.ascontiguousarray(a, dtype=eq.dtype).ravel()
    b = np.ascontiguousarray(b, dtype=eq.dtype).ravel()
    if a.size != eq.size(eq.modeA) or b.size != eq.size(eq.modeB):
        raise ValueError("input sizes do not match the descriptor")
    _check(_lib.tcontb_run_create_with_inputs(plan_._h, a.ctypes.data, b.ctypes.data, C.byref(h)))
    return ExecutionRun(h, plan_)


def prepare_on_device(plan_: ExecutionPlan, a_ptr: int, b_ptr: int, c_ptr: int, keep=()) -> ExecutionRun:
    """Run over caller-owned device buffers (raw device pointers)."""
    h = C.c_void_p()
    _check(_lib.tcontb_run_create_on_device(plan_._h, C.c_void_p(a_ptr), C.c_void_p(b_ptr), C.c_void_p(c_ptr), C.byref(h)))
    return ExecutionRun(h, plan_, keep)


def launch(run: ExecutionRun):
    if run is None or not run._h:
        raise ValueError("ExecutionRun is empty")
    _check(_lib.tcontb_run_launch(run._h))


def warmup(run: ExecutionRun, iterations: int):
    if run is None or not run._h:
        raise ValueError("ExecutionRun is empty")
    if iterations > 0:
        _check(_lib.tcontb_run_warmup(run._h, iterations))


def zero_output(run: ExecutionRun):
    _check(_lib.tcontb_run_zero_output(run._h))


def stage_times(run: ExecutionRun) -> dict:
    out = (C.c_float * 6)()
    _check(_lib.tcontb_run_stage_times(run._h, out))
    keys = ["available", "total_ms", "transpose_a_ms", "transpose_b_ms", "gemm_ms", "transpose_c_ms"]
    d = dict(zip(keys, [float(x) for x in out]))
    d["available"] = bool(d["available"])
    return d


def _host_input(run: ExecutionRun, which: int) -> np.ndarray:
    eq = run.equation
    n = eq.size(eq.modeA if which == 0 else eq.modeB)
    ptr = _lib.tcontb_run_host_input(run._h, which)
    if not ptr:
        raise ValueError("this run keeps no host inputs")
    ctype = C.c_double if eq.scalar_type == ScalarType.Float64 else C.c_float
    return np.ctypeslib.as_array(C.cast(ptr, C.POINTER(ctype)), shape=(n,)).copy()


def input_left_host_data(run: ExecutionRun) -> np.ndarray:
    return _host_input(run, 0)


def input_right_host_data(run: ExecutionRun) -> np.ndarray:
    return _host_input(run, 1)


def copy_output_to_host(run: ExecutionRun, destination: np.ndarray | None = None) -> np.ndarray:
    eq = run.equation
    if destination is None:
        destination = np.empty(eq.size(eq.modeC), dtype=eq.dtype)
    _check(_lib.tcontb_run_copy_output(run._h, destination.ctypes.data, destination.nbytes))
    return destination


def compute_gflops(equation: TCEquation, avg_ms: float) -> float:
    """TconT::compute_gflops (src/tcont.cpp:33-56): 2*sqrt(|A||B||C|) / (ms * 1e6)."""
    if avg_ms <= 0.0:
        return 0.0
    ops = 2.0 * float(np.sqrt(float(equation.size(equation.modeA)) * equation.size(equation.modeB) * equation.size(equation.modeC)))
    return ops / (avg_ms * 1.0e6)


def fill_uniform(n: int, scalar_type: ScalarType, seed: int, offset: int = 0, lo: float = 0.0, hi: float = 1.0) -> np.ndarray:
    out = np.empty(n, dtype=np.float64 if scalar_type == ScalarType.Float64 else np.float32)
    _check(_lib.tcontb_fill_uniform(out.ctypes.data, int(scalar_type), n, seed, offset, lo, hi))
    return out


def transpose(src_ptr: int, dst_ptr: int, src_extent, perm, elem_bytes: int, cuda_stream: int = 0):
    """Device-side permutation: dst mode i = src mode perm[i] (raw device pointers)."""
    r = len(src_extent)
    ext = (C.c_int64 * r)(*[int(x) for x in src_extent])
    pm = (C.c_int * r)(*[int(x) for x in perm])
    _check(_lib.tcontb_transpose(C.c_void_p(src_ptr), C.c_void_p(dst_ptr), r, ext, pm, elem_bytes, C.c_void_p(cuda_stream)))


def contract_no_alloc(desc: TCEquation, a_ptr: int, b_ptr: int, c_ptr: int, cuda_stream: int = 0):
    """tcontb_contract_no_alloc: one contraction on caller-owned device buffers without any device
    allocation (for callers whose memory pool owns the whole GPU, or that cannot take cudaMalloc's
    synchronisation). Limited to 2*(M+N+K) <= 524288; calls share one built-in scratch array, so
    keep them on one stream."""
    modes = "".join(sorted(desc.extent))
    vals = (C.c_int64 * max(1, len(modes)))(*[int(desc.extent[m]) for m in modes])
    d = _Desc(len(desc.modeC), len(desc.modeA), len(desc.modeB), desc.modeC.encode(), desc.modeA.encode(),
              desc.modeB.encode(), desc.op.encode()[:1] or b"?", int(desc.scalar_type), len(modes), modes.encode(), vals,
              int(desc.backend_selection))
    st = _lib.tcontb_contract_no_alloc(C.byref(d), C.c_void_p(a_ptr), C.c_void_p(b_ptr), C.c_void_p(c_ptr),
                                       C.c_void_p(cuda_stream))
    if st:
        msg = (_lib.tcontb_no_alloc_last_error() or b"").decode()
        if st == 1:
            raise ValueError(msg)
        if st == 3:
            raise NotImplementedError(msg)
        raise TcontError(msg)


_lib.tcontb_measure_peak.argtypes = [C.c_int, C.POINTER(C.c_double)]
_lib.tcontb_peak_last_error.restype = C.c_char_p


def measure_peak(which: str) -> float:
    """Arithmetic peak of the current device in TFLOP/s: 'tf32' (tcgen05), 'fp64_dfma', 'fp64_dmma'."""
    v = C.c_double()
    st = _lib.tcontb_measure_peak({"tf32": 0, "fp64_dfma": 1, "fp64_dmma": 2}[which], C.byref(v))
    if st:
        raise TcontError((_lib.tcontb_peak_last_error() or b"").decode())
    return v.value
