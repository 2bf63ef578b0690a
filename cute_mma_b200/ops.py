"""Host-side mirror of the reference operator surface over the C ABI (ctypes).

Names and argument order follow the reference launchers:
  oft_tn(m, n, k, A, ldA, B, ldB, R, ldR, C, ldC, stream)        cute_oft_coop_pc.hpp:17-23
  gemm_tn / gemm_nt(m, n, k, A, ldA, B, ldB, C, ldC, stream)     gemm_sm80_tc.cu:163-168 / 95-100
  gemm(transA, transB, m, n, k, ...)                             gemm_sm80_tc.cu:393-398
with the reference's compile-time KernelParams (group_size, reconn_sz) as keyword arguments.
Matrix arguments are device pointers: anything with ``data_ptr()`` (a torch tensor) or an int.
Where the reference throws std::runtime_error from GEMM_CHECK_CUDA (common.hpp:8-14), these raise
``Error`` carrying the library's status code and message.  There is no CPU fallback: if the CUDA
library is missing, importing works but the first call raises.
"""
from __future__ import annotations

import ctypes
import json
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
_LIB_ENV = "CUTE_MMA_B200_LIB"

OK, EINVAL, EUNSUPPORTED, ECUDA, EDEVICE = 0, 1, 2, 3, 4

# every symbol include/cute_mma_b200.h declares
SYMBOLS = (
    "b200_oft_tn_f16", "b200_oft_tn_f16_two_pass", "b200_rotate_f16", "b200_oft_plan", "b200_oft_tn_f16_host", "b200_oft_tn_f16_static", "b200_transform_weight_f16", "b200_oft_tn_f16_a_rw", "b200_gemm_tn_f16", "b200_gemm_nt_f16", "b200_gemm_tn_tf32",
    "b200_gemm_nt_tf32", "b200_gemm", "b200_gemm_tn_f16_acc2", "b200_lora_tn_f16", "b200_gemm_rowmajor", "b200_peer_copy_async", "b200_shard_range", "b200_tile_coord", "b200_device_status", "b200_selftest_wait_timeout", "b200_wait_profile", "b200_kernel_info",
    "b200_last_error", "b200_shutdown", "b200_static_status", "b200_set_option", "b200_get_option", "b200_gemm_ex", "b200_oft_tn_f16_sharded", "b200_oft_tn_f16_gather",
)


class Error(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"cute_mma_b200 status {code}: {message}")
        self.code = code
        self.message = message


_lib = None


def library_path() -> str:
    return os.environ.get(_LIB_ENV) or os.path.join(_PKG, "libcute_mma_b200.so")


def load_library(path: str | None = None):
    """Loads the CUDA library (built by ``python -m cute_mma_b200.build``).  Fails loudly if absent."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    p = path or library_path()
    if not os.path.exists(p):
        raise FileNotFoundError(f"{p} not found: build it with `python -m cute_mma_b200.build` (no CPU fallback exists)")
    lib = ctypes.CDLL(p)
    i, vp, c = ctypes.c_int, ctypes.c_void_p, ctypes.c_char
    lib.b200_oft_tn_f16.argtypes = [i, i, i, i, i, vp, i, vp, i, vp, i, vp, i, vp]
    lib.b200_oft_tn_f16_static.argtypes = [i, i, i, i, i, vp, i, vp, i, vp, i, vp, i, vp]
    lib.b200_oft_tn_f16_two_pass.argtypes = [i, i, i, i, i, vp, i, vp, i, vp, i, vp, i, vp]
    lib.b200_rotate_f16.argtypes = [i, i, i, vp, i, vp, i, vp, i, vp]
    lib.b200_oft_plan.argtypes = [i, i, i, i, i, ctypes.POINTER(i), ctypes.POINTER(i)]
    lib.b200_oft_tn_f16_a_rw.argtypes = [i, i, i, i, i, vp, i, vp, i, vp, i, vp, i, vp]
    lib.b200_transform_weight_f16.argtypes = [i, i, i, i, vp, i, vp, i, vp, i, vp]
    lib.b200_oft_tn_f16_host.argtypes = [i, i, i, i, i, vp, i, vp, i, vp, i, vp, i]
    for name in ("b200_gemm_tn_f16", "b200_gemm_nt_f16", "b200_gemm_tn_tf32", "b200_gemm_nt_tf32"):
        getattr(lib, name).argtypes = [i, i, i, vp, i, vp, i, vp, i, vp]
    lib.b200_gemm.argtypes = [c, c, i, i, i, i, vp, i, vp, i, vp, i, vp]
    pp = ctypes.POINTER(ctypes.c_void_p)
    lib.b200_oft_tn_f16_sharded.argtypes = [i, i, i, i, i, i, ctypes.POINTER(i), pp, i, pp, i, pp, i, pp, i, pp]
    lib.b200_oft_tn_f16_gather.argtypes = [i, i, i, i, i, vp, i, vp, i, vp, i, i, pp, i, vp]
    lib.b200_gemm_ex.argtypes = [c, c, i, i, i, i, i, ctypes.c_float, vp, i, vp, i, ctypes.c_float, vp, i, vp]
    lib.b200_gemm_tn_f16_acc2.argtypes = [i, i, i, vp, i, vp, i, i, vp, i, vp, i, vp, i, vp]
    lib.b200_lora_tn_f16.argtypes = [i, i, i, i, vp, i, vp, i, vp, i, vp, i, vp, i, vp]
    lib.b200_gemm_rowmajor.argtypes = [c, c, i, i, i, i, vp, i, vp, i, vp, i, vp]
    lib.b200_peer_copy_async.argtypes = [vp, i, vp, i, ctypes.c_size_t, vp]
    lib.b200_shard_range.argtypes = [i, i, i, i, ctypes.POINTER(i), ctypes.POINTER(i)]
    lib.b200_tile_coord.argtypes = [ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.POINTER(ctypes.c_uint), ctypes.POINTER(ctypes.c_uint)]
    lib.b200_device_status.argtypes = [ctypes.POINTER(ctypes.c_int)]
    lib.b200_selftest_wait_timeout.argtypes = [ctypes.c_uint, ctypes.POINTER(ctypes.c_int)]
    lib.b200_wait_profile.argtypes = [ctypes.POINTER(ctypes.c_ulonglong), i]
    lib.b200_static_status.argtypes = [ctypes.POINTER(ctypes.c_int)]
    lib.b200_set_option.argtypes = [ctypes.c_char_p, i]
    lib.b200_get_option.argtypes = [ctypes.c_char_p, ctypes.POINTER(i)]
    lib.b200_kernel_info.restype = ctypes.c_char_p
    lib.b200_last_error.restype = ctypes.c_char_p
    for name in SYMBOLS:
        if name not in ("b200_kernel_info", "b200_last_error"):
            getattr(lib, name).restype = ctypes.c_int
    if path is None:
        _lib = lib
    return lib


def _ptr(x) -> int:
    if x is None:
        return 0
    if hasattr(x, "data_ptr"):
        return int(x.data_ptr())
    if hasattr(x, "ctypes"):  # numpy array: host memory, only valid for the *_host entry point
        return int(x.ctypes.data)
    return int(x)


def _stream(s) -> int:
    if s is None:
        return 0
    if hasattr(s, "cuda_stream"):
        return int(s.cuda_stream)
    return int(s)


def _check(lib, rc: int) -> None:
    if rc != OK:
        raise Error(rc, lib.b200_last_error().decode())


def oft_tn(m, n, k, A, ldA, B, ldB, R, ldR, C, ldC, stream=None, *, group_size=None, reconn_sz=8, lib=None) -> None:
    """C[m,n] = (A[m,k] . R) . B^T on the current CUDA device, asynchronous on ``stream``.
    group_size defaults to n (one block-diagonal R for all of N)."""
    lib = lib or load_library()
    gs = n if group_size is None else group_size
    _check(lib, lib.b200_oft_tn_f16(m, n, k, gs, reconn_sz, _ptr(A), ldA, _ptr(B), ldB, _ptr(R), ldR, _ptr(C), ldC, _stream(stream)))


def oft_tn_two_pass(m, n, k, A, ldA, B, ldB, R, ldR, C, ldC, stream=None, *, group_size=None, reconn_sz=8, lib=None) -> None:
    """oft_tn as a rotation pass (X.R written once to device scratch) followed by the plain GEMM, the route
    oft_tn takes by itself when a group spans many N tiles (see b200_oft_tn_f16_two_pass in the header)."""
    lib = lib or load_library()
    gs = n if group_size is None else group_size
    _check(lib, lib.b200_oft_tn_f16_two_pass(m, n, k, gs, reconn_sz, _ptr(A), ldA, _ptr(B), ldB, _ptr(R), ldR, _ptr(C), ldC, _stream(stream)))


def rotate(m, k, A, ldA, R, ldR, XR, ldX, stream=None, *, reconn_sz=8, lib=None) -> None:
    """XR[m,k] = half(A . blockdiag(R^T)) for one N-group's R: the first pass of the two-pass route."""
    lib = lib or load_library()
    _check(lib, lib.b200_rotate_f16(m, k, reconn_sz, _ptr(A), ldA, _ptr(R), ldR, _ptr(XR), ldX, _stream(stream)))


ROUTES = {1: "fused_tmem", 2: "two_pass", 3: "fused_ring", 4: "fused_ring_split"}


def oft_plan(m, n, k, *, group_size=None, reconn_sz=8, lib=None) -> dict:
    """{'path': 'fused_tmem' | 'two_pass' | 'fused_ring' | 'fused_ring_split', 'kernel_launches': launches of the
    library's kernels per oft_tn call}: fused_tmem keeps X.R in tensor memory per N tile, fused_ring shares one X.R
    per row block among the N tiles of a group through an L2-resident ring (fused_ring_split: with the rotation on
    SM pairs of its own), two_pass writes X.R to memory first."""
    lib = lib or load_library()
    path, launches = ctypes.c_int(0), ctypes.c_int(0)
    _check(lib, lib.b200_oft_plan(m, n, k, n if group_size is None else group_size, reconn_sz, ctypes.byref(path), ctypes.byref(launches)))
    return {"path": ROUTES[path.value], "kernel_launches": launches.value}


def set_option(name: str, value: int, lib=None) -> None:
    """Process-wide override of a launch heuristic (see b200_set_option in the header)."""
    lib = lib or load_library()
    _check(lib, lib.b200_set_option(name.encode(), int(value)))


def get_option(name: str, lib=None) -> int:
    lib = lib or load_library()
    v = ctypes.c_int(0)
    _check(lib, lib.b200_get_option(name.encode(), ctypes.byref(v)))
    return v.value


class option:
    """``with ops.option("oft_route", 1): ...`` sets an option for the block and restores the old value."""

    def __init__(self, name: str, value: int, lib=None):
        self.name, self.value, self.lib = name, value, lib

    def __enter__(self):
        self.old = get_option(self.name, self.lib)
        set_option(self.name, self.value, self.lib)
        return self

    def __exit__(self, *exc):
        set_option(self.name, self.old, self.lib)
        return False


def static_status(lib=None, raise_on_error: bool = True):
    """The status record of oft_tn_static's scratch array (b200_static_status): synchronises, reads, clears."""
    lib = lib or load_library()
    out = (ctypes.c_int * 4)()
    rc = lib.b200_static_status(out)
    if rc != OK and raise_on_error:
        raise Error(rc, lib.b200_last_error().decode())
    return list(out)


def oft_tn_static(m, n, k, A, ldA, B, ldB, R, ldR, C, ldC, stream=None, *, group_size=None, reconn_sz=8, lib=None) -> None:
    """oft_tn for callers that must not allocate device memory: the kernel's scratch is a fixed array
    inside the library (see b200_oft_tn_f16_static in the header for the sharing rules)."""
    lib = lib or load_library()
    gs = n if group_size is None else group_size
    _check(lib, lib.b200_oft_tn_f16_static(m, n, k, gs, reconn_sz, _ptr(A), ldA, _ptr(B), ldB, _ptr(R), ldR, _ptr(C), ldC, _stream(stream)))


def oft_tn_sharded(m, n, k, devices, A, ldA, B_slabs, ldB, R_slabs, ldR, C_slabs, ldC, streams=None, *, group_size=None, reconn_sz=8, lib=None) -> None:
    """One call for all GPUs of this process: slab r of shard_range(n, group_size, len(devices), r) runs on devices[r]
    (see b200_oft_tn_f16_sharded).  A, B_slabs, R_slabs, C_slabs: one device pointer per entry of ``devices``."""
    lib = lib or load_library()
    w = len(devices)
    arr = lambda xs: (ctypes.c_void_p * w)(*[_ptr(x) for x in xs])
    st = None if streams is None else (ctypes.c_void_p * w)(*[_stream(s_) for s_ in streams])
    gs = n if group_size is None else group_size
    _check(lib, lib.b200_oft_tn_f16_sharded(m, n, k, gs, reconn_sz, w, (ctypes.c_int * w)(*devices), arr(A), ldA, arr(B_slabs), ldB,
                                            arr(R_slabs), ldR, arr(C_slabs), ldC, st))


def oft_tn_gather(m, n, k, A, ldA, B, ldB, R, ldR, C_dsts, ldC, stream=None, *, group_size=None, reconn_sz=8, lib=None) -> None:
    """oft_tn whose result goes to every buffer of ``C_dsts`` (same ldC), e.g. this rank's columns of Y on every GPU of
    the node (see b200_oft_tn_f16_gather)."""
    lib = lib or load_library()
    w = len(C_dsts)
    gs = n if group_size is None else group_size
    _check(lib, lib.b200_oft_tn_f16_gather(m, n, k, gs, reconn_sz, _ptr(A), ldA, _ptr(B), ldB, _ptr(R), ldR, w,
                                           (ctypes.c_void_p * w)(*[_ptr(x) for x in C_dsts]), ldC, _stream(stream)))


def transform_weight(n, k, B, ldB, R, ldR, Bt, ldBt, stream=None, *, group_size=None, reconn_sz=8, lib=None) -> None:
    """Bt = weight with the rotation folded in (the A_RW order): see b200_transform_weight_f16."""
    lib = lib or load_library()
    gs = n if group_size is None else group_size
    _check(lib, lib.b200_transform_weight_f16(n, k, gs, reconn_sz, _ptr(B), ldB, _ptr(R), ldR, _ptr(Bt), ldBt, _stream(stream)))


def oft_tn_a_rw(m, n, k, A, ldA, B, ldB, R, ldR, C, ldC, stream=None, *, group_size=None, reconn_sz=8, lib=None) -> None:
    """Same product as oft_tn computed as X . (R . W): weight transform, then one plain GEMM."""
    lib = lib or load_library()
    gs = n if group_size is None else group_size
    _check(lib, lib.b200_oft_tn_f16_a_rw(m, n, k, gs, reconn_sz, _ptr(A), ldA, _ptr(B), ldB, _ptr(R), ldR, _ptr(C), ldC, _stream(stream)))


def oft_tn_host(m, n, k, A, ldA, B, ldB, R, ldR, C, ldC, *, group_size=None, reconn_sz=8, lib=None) -> None:
    """Same product on HOST buffers (numpy arrays or host addresses); synchronous."""
    lib = lib or load_library()
    gs = n if group_size is None else group_size
    _check(lib, lib.b200_oft_tn_f16_host(m, n, k, gs, reconn_sz, _ptr(A), ldA, _ptr(B), ldB, _ptr(R), ldR, _ptr(C), ldC))


def _gemm(fn_name, m, n, k, A, ldA, B, ldB, C, ldC, stream, lib):
    lib = lib or load_library()
    _check(lib, getattr(lib, fn_name)(m, n, k, _ptr(A), ldA, _ptr(B), ldB, _ptr(C), ldC, _stream(stream)))


def gemm_tn(m, n, k, A, ldA, B, ldB, C, ldC, stream=None, *, dtype="half", lib=None) -> None:
    """C(i,j) = sum_l A[i*ldA+l] B[j*ldB+l], C column-major.  dtype 'half' or 'float' (TF32)."""
    _gemm("b200_gemm_tn_f16" if dtype == "half" else "b200_gemm_tn_tf32", m, n, k, A, ldA, B, ldB, C, ldC, stream, lib)


def gemm_nt(m, n, k, A, ldA, B, ldB, C, ldC, stream=None, *, dtype="half", lib=None) -> None:
    """C(i,j) = sum_l A[i+l*ldA] B[j+l*ldB], C column-major."""
    _gemm("b200_gemm_nt_f16" if dtype == "half" else "b200_gemm_nt_tf32", m, n, k, A, ldA, B, ldB, C, ldC, stream, lib)


def gemm(transA, transB, m, n, k, A, ldA, B, ldB, C, ldC, stream=None, *, dtype="half", lib=None) -> None:
    lib = lib or load_library()
    _check(lib, lib.b200_gemm(transA.encode(), transB.encode(), 0 if dtype == "half" else 1, m, n, k, _ptr(A), ldA,
                              _ptr(B), ldB, _ptr(C), ldC, _stream(stream)))


F16, F32, TF32 = 0, 1, 2


def gemm_ex(transA, transB, m, n, k, alpha, A, ldA, B, ldB, beta, C, ldC, stream=None, *, in_type=F16, out_type=F16, lib=None) -> None:
    """C (column-major) = alpha * A.B^T + beta * C, half or float result from half operands, float from float (TF32)."""
    lib = lib or load_library()
    _check(lib, lib.b200_gemm_ex(transA.encode(), transB.encode(), in_type, out_type, m, n, k, float(alpha), _ptr(A), ldA, _ptr(B), ldB,
                                 float(beta), _ptr(C), ldC, _stream(stream)))


def gemm_tn_acc2(m, n, k, A, ldA, B, ldB, k2, A2, ldA2, B2, ldB2, C, ldC, stream=None, *, lib=None) -> None:
    """C (column-major m x n) = A . B^T + A2 . B2^T, fp16, one pass."""
    lib = lib or load_library()
    _check(lib, lib.b200_gemm_tn_f16_acc2(m, n, k, _ptr(A), ldA, _ptr(B), ldB, k2, _ptr(A2), ldA2, _ptr(B2), ldB2, _ptr(C), ldC, _stream(stream)))


def lora_tn(m, n, k, r, X, ldX, W, ldW, L1, ldL1, L2, ldL2, C, ldC, stream=None, *, lib=None) -> None:
    """C[m][n] = X . W^T + (X . L1^T) . L2^T (row-major C), the LoRA-equivalent of oft_tn."""
    lib = lib or load_library()
    _check(lib, lib.b200_lora_tn_f16(m, n, k, r, _ptr(X), ldX, _ptr(W), ldW, _ptr(L1), ldL1, _ptr(L2), ldL2, _ptr(C), ldC, _stream(stream)))


def gemm_rowmajor(transA, transB, m, n, k, A, ldA, B, ldB, C, ldC, stream=None, *, dtype="half", lib=None) -> None:
    """gemm with C row-major [m][ldC]."""
    lib = lib or load_library()
    _check(lib, lib.b200_gemm_rowmajor(transA.encode(), transB.encode(), 0 if dtype == "half" else 1, m, n, k, _ptr(A), ldA,
                                       _ptr(B), ldB, _ptr(C), ldC, _stream(stream)))


def peer_copy_async(dst, dst_device: int, src, src_device: int, nbytes: int, stream=None, lib=None) -> None:
    """Copy-engine transfer between two GPUs (dst may be IPC-mapped memory of another process)."""
    lib = lib or load_library()
    _check(lib, lib.b200_peer_copy_async(_ptr(dst), dst_device, _ptr(src), src_device, nbytes, _stream(stream)))


def shard_range(n: int, group_size: int, world: int, rank: int, lib=None):
    """[n_begin, n_end) of the N columns owned by ``rank`` (whole groups / whole 256-column tiles)."""
    lib = lib or load_library()
    a, b = ctypes.c_int(0), ctypes.c_int(0)
    _check(lib, lib.b200_shard_range(n, group_size, world, rank, ctypes.byref(a), ctypes.byref(b)))
    return a.value, b.value


def tile_coord(tiles_m: int, tiles_n: int, idx: int, lib=None):
    lib = lib or load_library()
    tm, tn = ctypes.c_uint(0), ctypes.c_uint(0)
    _check(lib, lib.b200_tile_coord(tiles_m, tiles_n, idx, ctypes.byref(tm), ctypes.byref(tn)))
    return tm.value, tn.value


def device_status(lib=None, raise_on_error: bool = True):
    """Synchronises the device and returns the kernels' status record [code, cta, site, parity]."""
    lib = lib or load_library()
    out = (ctypes.c_int * 4)()
    rc = lib.b200_device_status(out)
    if rc != OK and raise_on_error:
        raise Error(rc, lib.b200_last_error().decode())
    return list(out)


def selftest_wait_timeout(limit_us: int = 1000, lib=None):
    """Runs the bounded-wait self-test; returns the status record the timed-out wait wrote."""
    lib = lib or load_library()
    out = (ctypes.c_int * 4)()
    _check(lib, lib.b200_selftest_wait_timeout(limit_us, out))
    return list(out)


def wait_profile(lib=None):
    """{site: (cycles waited, waits)} from a library built with -DB200_PROFILE_WAITS."""
    lib = lib or load_library()
    out = (ctypes.c_ulonglong * 128)()
    _check(lib, lib.b200_wait_profile(out, 128))
    return {s: (out[s], out[64 + s]) for s in range(64) if out[64 + s]}


def kernel_info(lib=None) -> dict:
    lib = lib or load_library()
    return json.loads(lib.b200_kernel_info().decode())
