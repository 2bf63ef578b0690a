"""ctypes front end of the plain-C oracle and, when built, of the reference's own CPU routine.

TEST INFRASTRUCTURE ONLY.  Importers: tests/, the smoke check and the cpu_baseline / reference legs
of bench.py.  The product package (cute_mma_b200) must never import this module.

All matrices are numpy arrays: fp16 data as ``np.float16`` (C-contiguous), layouts as documented
in oracle/oft_oracle.c (A [m,k], R [G*b,k], B [n,k], C [m,n], all row-major).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "liboft_oracle.so")
_REF = os.path.join(_HERE, "_ref", "libref_cpu_oft.so")

_u16p = ctypes.POINTER(ctypes.c_uint16)


def build(with_reference: bool = True) -> None:
    """Compile the C restatement (gcc) and, if the reference tree is present, oracle/_ref."""
    subprocess.run(["make", "-C", _HERE, "liboft_oracle.so"], check=True, stdout=subprocess.DEVNULL)
    if with_reference:
        subprocess.run([os.path.join(_HERE, "build_ref.sh")], check=True, stdout=subprocess.DEVNULL)


_lib = None
_ref = None


def _load():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB):
            build(with_reference=False)
        _lib = ctypes.CDLL(_LIB)
        _lib.oft_oracle_cpu_oft_tn.restype = ctypes.c_int
        _lib.oft_oracle_f64.restype = ctypes.c_int
        _lib.gemm_oracle_f64_sampled.restype = ctypes.c_int
        _lib.oft_oracle_check_result.restype = ctypes.c_uint64
        _lib.oft_oracle_num_threads.restype = ctypes.c_int
    return _lib


def have_reference() -> bool:
    return os.path.exists(_REF)


def num_threads() -> int:
    return int(_load().oft_oracle_num_threads())


def _h(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a)
    assert a.dtype == np.float16, a.dtype
    return a


def _p16(a: np.ndarray):
    return a.ctypes.data_as(_u16p)


def cpu_oft_tn(A, R, B, m, group_size, n_groups, k, reconn_sz, threads: int = 1) -> np.ndarray:
    """Restatement of cpu_oft_tn (cpu_oft.hpp:22-116).  Returns C [m, n] fp16."""
    A, R, B = _h(A), _h(R), _h(B)
    n = group_size * n_groups
    assert A.size == m * k and R.size == n_groups * reconn_sz * k and B.size == n * k
    C = np.empty((m, n), dtype=np.float16)
    rc = _load().oft_oracle_cpu_oft_tn(_p16(A), _p16(R), _p16(B), _p16(C), m, group_size, n_groups, k,
                                       reconn_sz, int(threads))
    if rc != 0:
        raise ValueError(f"oft_oracle_cpu_oft_tn rejected its arguments (code {rc})")
    return C


def ref_cpu_oft_tn(A, R, B, m, group_size, n_groups, k, reconn_sz) -> np.ndarray:
    """The reference's own cpu_oft_tn, compiled from its header (oracle/_ref).  Single-threaded."""
    global _ref
    if _ref is None:
        if not have_reference():
            raise FileNotFoundError("oracle/_ref/libref_cpu_oft.so not built (oracle/build_ref.sh)")
        _ref = ctypes.CDLL(_REF)
        _ref.ref_cpu_oft_tn.restype = ctypes.c_int
    A, R, B = _h(A), _h(R), _h(B)
    n = group_size * n_groups
    C = np.empty((m, n), dtype=np.float16)
    _ref.ref_cpu_oft_tn(_p16(A), _p16(R), _p16(B), _p16(C), m, group_size, n_groups, k, reconn_sz)
    return C


def oft_f64(A, R, B, m, group_size, n_groups, k, reconn_sz, round_xr: bool = True, threads: int = 0) -> np.ndarray:
    """fp64-accumulate analysis variant (no per-K-block rounding of C).  Returns float64 [m, n]."""
    A, R, B = _h(A), _h(R), _h(B)
    n = group_size * n_groups
    C = np.empty((m, n), dtype=np.float64)
    rc = _load().oft_oracle_f64(_p16(A), _p16(R), _p16(B), C.ctypes.data_as(ctypes.POINTER(ctypes.c_double)),
                                m, group_size, n_groups, k, reconn_sz, int(round_xr), threads or num_threads())
    if rc != 0:
        raise ValueError(f"oft_oracle_f64 rejected its arguments (code {rc})")
    return C


def gemm_f64_sampled(transA: str, transB: str, m, n, k, A, ldA, B, ldB, rows, cols, tf32_mode: int = 0,
                     threads: int = 0) -> np.ndarray:
    """fp64 truth of gemm_sm80_tc.cu:557-568 on sampled rows x cols.  Returns float64 [len(rows), len(cols)]."""
    A = np.ascontiguousarray(A)
    B = np.ascontiguousarray(B)
    assert A.dtype == B.dtype and A.dtype in (np.float16, np.float32)
    dtype = 0 if A.dtype == np.float16 else 1
    rows = np.ascontiguousarray(rows, dtype=np.int32)
    cols = np.ascontiguousarray(cols, dtype=np.int32)
    out = np.empty((len(cols), len(rows)), dtype=np.float64)  # column-major sample
    ip = ctypes.POINTER(ctypes.c_int)
    rc = _load().gemm_oracle_f64_sampled(ctypes.c_char(transA.encode()), ctypes.c_char(transB.encode()), m, n, k,
                                         A.ctypes.data_as(ctypes.c_void_p), ldA, B.ctypes.data_as(ctypes.c_void_p), ldB,
                                         rows.ctypes.data_as(ip), len(rows), cols.ctypes.data_as(ip), len(cols),
                                         out.ctypes.data_as(ctypes.POINTER(ctypes.c_double)), dtype, tf32_mode,
                                         threads or num_threads())
    if rc != 0:
        raise ValueError(f"gemm_oracle_f64_sampled rejected its arguments (code {rc})")
    return out.T.copy()


def check_result(result, ref, threshold: float = 5e-3):
    """check_result of cute_oft_pc.cu:31-77 -> (error_count, max_relative_error)."""
    result, ref = _h(result), _h(ref)
    mx = ctypes.c_float(0)
    with np.errstate(all="ignore"):
        cnt = _load().oft_oracle_check_result(_p16(result), _p16(ref), ctypes.c_uint64(result.size),
                                              ctypes.c_float(threshold), ctypes.byref(mx))
    return int(cnt), float(mx.value)
