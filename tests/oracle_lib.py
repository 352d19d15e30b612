"""ctypes access to the CPU checkers under oracle/ (test infrastructure, never the product path).

`Oracle` wraps oracle/_build/liboracle.so (the CPU restatement of the reference loops,
benchmarks/tccg/tccg_verify.cpp) and builds it with the system gcc when it is missing.
`RefVerifier` wraps oracle/_ref/libtccg_ref.so, the reference's own verifier compiled from its
own sources; it exists only where that tree was available at build time.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass, field

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
ORACLE_SO = os.path.join(ORACLE_DIR, "_build", "liboracle.so")
REF_SO = os.path.join(ORACLE_DIR, "_ref", "libtccg_ref.so")

F32, F64 = 0, 1


@dataclass
class Contraction:
    """A contraction descriptor in the reference's vocabulary (include/tcont.hpp:74-83)."""

    modeC: str
    modeA: str
    modeB: str
    extent: dict = field(default_factory=dict)
    scalar_type: int = F64

    def size(self, modes: str) -> int:
        n = 1
        for m in modes:
            n *= int(self.extent[m])
        return n

    @property
    def dtype(self):
        return np.float64 if self.scalar_type == F64 else np.float32

    def flops(self) -> float:
        # 2 * sqrt(|A| |B| |C|): the reference's operation count (src/tcont.cpp:51-55)
        return 2.0 * float(np.sqrt(float(self.size(self.modeA)) * self.size(self.modeB) * self.size(self.modeC)))


class _Desc(C.Structure):
    _fields_ = [("nC", C.c_int), ("nA", C.c_int), ("nB", C.c_int),
                ("modeC", C.c_char_p), ("modeA", C.c_char_p), ("modeB", C.c_char_p),
                ("n_ext", C.c_int), ("ext_mode", C.c_char_p), ("ext_val", C.POINTER(C.c_int64))]


class _CmpResult(C.Structure):
    _fields_ = [("differences", C.c_int64), ("total", C.c_int64), ("same", C.c_int64),
                ("non_finite", C.c_int64), ("passed", C.c_int)]


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


class Oracle:
    def __init__(self):
        if not os.path.exists(ORACLE_SO):
            subprocess.run(["make", "-C", ORACLE_DIR, "_build/liboracle.so"], check=True, capture_output=True)
        self.lib = C.CDLL(ORACLE_SO)
        L = self.lib
        L.oracle_contract.argtypes = [C.POINTER(_Desc), C.c_void_p, C.c_void_p, C.c_void_p]
        L.oracle_contract_f32.argtypes = [C.POINTER(_Desc), C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
        L.oracle_contract_sampled.argtypes = [C.POINTER(_Desc), C.c_int, C.c_void_p, C.c_void_p, C.c_int64,
                                              C.c_void_p, C.c_void_p, C.c_int]
        L.oracle_tolerance.argtypes = [C.c_int, C.POINTER(C.c_double), C.POINTER(C.c_double)]
        L.oracle_compare.argtypes = [C.c_int64, C.c_void_p, C.c_void_p, C.c_double, C.c_double, C.POINTER(_CmpResult)]
        L.oracle_fill_uniform.argtypes = [C.c_void_p, C.c_int, C.c_int64, C.c_uint64, C.c_uint64, C.c_double, C.c_double]
        L.oracle_num_threads.restype = C.c_int

    @staticmethod
    def _desc(c: Contraction):
        modes = "".join(sorted(c.extent))
        vals = (C.c_int64 * len(modes))(*[int(c.extent[m]) for m in modes])
        d = _Desc(len(c.modeC), len(c.modeA), len(c.modeB), c.modeC.encode(), c.modeA.encode(), c.modeB.encode(),
                  len(modes), modes.encode(), vals)
        d._keep = vals
        return d

    def num_threads(self) -> int:
        return int(self.lib.oracle_num_threads())

    def set_num_threads(self, n: int):
        """Team size of later OpenMP regions entered from this thread (the reference verifier shares the
        same OpenMP runtime, so this also governs RefVerifier.verify)."""
        self.lib.oracle_set_num_threads.argtypes = [C.c_int]
        self.lib.oracle_set_num_threads(int(n))

    def fill(self, n: int, scalar_type: int, seed: int, offset: int, lo: float, hi: float) -> np.ndarray:
        out = np.empty(n, dtype=np.float64 if scalar_type == F64 else np.float32)
        self.lib.oracle_fill_uniform(_ptr(out), scalar_type, n, seed, offset, lo, hi)
        return out

    def inputs(self, c: Contraction, seed: int, lo: float = -1.0, hi: float = 1.0):
        """A then B from one seeded stream: A at offset 0, B at offset |A|."""
        nA, nB = c.size(c.modeA), c.size(c.modeB)
        return self.fill(nA, c.scalar_type, seed, 0, lo, hi), self.fill(nB, c.scalar_type, seed, nA, lo, hi)

    def contract(self, c: Contraction, A: np.ndarray, B: np.ndarray, rounding: int = 0) -> np.ndarray:
        out = np.empty(c.size(c.modeC), dtype=np.float64)
        d = self._desc(c)
        if c.scalar_type == F64:
            rc = self.lib.oracle_contract(C.byref(d), _ptr(A), _ptr(B), _ptr(out))
        else:
            rc = self.lib.oracle_contract_f32(C.byref(d), _ptr(A), _ptr(B), _ptr(out), rounding)
        if rc:
            raise ValueError(f"oracle rejected the descriptor (code {rc})")
        return out

    def contract_sampled(self, c: Contraction, A, B, index: np.ndarray, rounding: int = 0) -> np.ndarray:
        index = np.ascontiguousarray(index, dtype=np.int64)
        out = np.empty(index.size, dtype=np.float64)
        d = self._desc(c)
        rc = self.lib.oracle_contract_sampled(C.byref(d), c.scalar_type, _ptr(A), _ptr(B), index.size,
                                              _ptr(index), _ptr(out), rounding)
        if rc:
            raise ValueError(f"oracle rejected the descriptor (code {rc})")
        return out

    def tolerance(self, scalar_type: int):
        a, r = C.c_double(), C.c_double()
        self.lib.oracle_tolerance(scalar_type, C.byref(a), C.byref(r))
        return a.value, r.value

    def compare(self, ref: np.ndarray, out: np.ndarray, scalar_type: int):
        """The reference criterion (tccg_verify.cpp:1620-1687). Returns (differences, non_finite)."""
        ref = np.ascontiguousarray(ref, dtype=np.float64)
        out = np.ascontiguousarray(out, dtype=np.float64)
        assert ref.size == out.size
        a, r = self.tolerance(scalar_type)
        res = _CmpResult()
        self.lib.oracle_compare(ref.size, _ptr(ref), _ptr(out), a, r, C.byref(res))
        return int(res.differences), int(res.non_finite)


class _RefResult(C.Structure):
    _fields_ = [("passed", C.c_int), ("differences", C.c_int), ("total_size", C.c_int), ("same", C.c_int),
                ("non_finite", C.c_int)]


class RefVerifier:
    """The reference's verify_tccg_case + case table, when oracle/_ref was built."""

    @staticmethod
    def available() -> bool:
        return os.path.exists(REF_SO)

    def __init__(self):
        self.lib = C.CDLL(REF_SO)

    def case(self, index: int, fp32: bool = False) -> Contraction:
        mc, ma, mb, em = (C.create_string_buffer(16) for _ in range(4))
        ev = (C.c_int64 * 16)()
        nC, nA, nB, ne = C.c_int(), C.c_int(), C.c_int(), C.c_int()
        op = C.c_char()
        st = self.lib.ref_case_get(index, int(fp32), mc, C.byref(nC), ma, C.byref(nA), mb, C.byref(nB), em, ev,
                                   C.byref(ne), C.byref(op))
        if st < 0:
            raise IndexError(index)
        ext = {em.raw[i:i + 1].decode(): int(ev[i]) for i in range(ne.value)}
        return Contraction(mc.raw[:nC.value].decode(), ma.raw[:nA.value].decode(), mb.raw[:nB.value].decode(), ext, st)

    def count(self) -> int:
        return int(self.lib.ref_case_count())

    def verify(self, case_index: int, c: Contraction, out: np.ndarray, A: np.ndarray, B: np.ndarray):
        modes = "".join(sorted(c.extent))
        vals = (C.c_int64 * len(modes))(*[int(c.extent[m]) for m in modes])
        r = _RefResult()
        out = np.ascontiguousarray(out, dtype=c.dtype)
        rc = self.lib.ref_verify_case(case_index, c.scalar_type, c.modeC.encode(), len(c.modeC), c.modeA.encode(),
                                      len(c.modeA), c.modeB.encode(), len(c.modeB), modes.encode(), vals, len(modes),
                                      _ptr(out), _ptr(A), _ptr(B), C.byref(r))
        if rc:
            raise RuntimeError("reference verifier threw")
        return bool(r.passed), int(r.differences), int(r.total_size)
