"""Helpers shared by the parity tests (not collected by pytest)."""
import numpy as np

from cute_mma_b200 import inputs

OFT_TOL = 1e-2  # |y - y_ref| <= OFT_TOL * (|y_ref| + 1): fp16 in, fp32 accumulate (the stated tolerance)
TF32_TOL = 5e-3  # relative, with the magnitude floor documented in tf32_ok


TRUTH_TOL = 2e-3  # kernel vs exact arithmetic: only the fp16 rounding of XR and of the output remain


def oft_ok(y, y_ref, tol=OFT_TOL, truth=None):
    """Counts elements with |y - y_ref| > tol * (|y_ref| + 1) and returns (count, worst normalised error).

    cpu_oft_tn re-rounds C to fp16 after every K block (cpu_oft.hpp:13-17), so the oracle itself
    drifts from exact arithmetic: with U(-1,1) operands and K/b >= 16 the drift alone exceeds the
    stated tolerance on a fraction of a percent of the elements (a running sum that passes through
    |C| ~ 30 collects roundings of 2^-6 and may end near zero).  When ``truth`` (fp64 accumulation of
    the same fp16-rounded XR) is given, that measured self-drift |y_ref - truth| is added to the
    bound, so the test asks the kernel to be inside the stated tolerance of the oracle up to the
    oracle's own rounding noise, no more."""
    y = np.asarray(y, dtype=np.float64)
    r = np.asarray(y_ref, dtype=np.float64)
    err = np.abs(y - r)
    bound = tol * (np.abs(r) + 1.0)
    if truth is not None:
        bound = bound + np.abs(r - np.asarray(truth, dtype=np.float64))
    bad = err > bound
    return int(bad.sum()), float((err / (np.abs(r) + 1.0)).max())


def truth_ok(y, truth, tol=TRUTH_TOL):
    y = np.asarray(y, dtype=np.float64)
    t = np.asarray(truth, dtype=np.float64)
    nerr = np.abs(y - t) / (np.abs(t) + 1.0)
    return int((nerr > tol).sum()), float(nerr.max())


def tf32_ok(c, ref, a_rows, b_cols, k, tol=TF32_TOL):
    """|c - ref| <= tol * max(|ref|, floor) with floor = ||a_row|| * ||b_col|| / sqrt(K): the typical
    magnitude of a K-term dot product of these vectors.  N(0,1) operands give outputs arbitrarily
    close to zero, where a purely relative test is meaningless (the reference sidesteps this with
    positive inputs, gemm_sm80_tc.cu:499)."""
    c = np.asarray(c, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    floor = np.outer(np.linalg.norm(a_rows, axis=1), np.linalg.norm(b_cols, axis=1)) / np.sqrt(k)
    scale = np.maximum(np.abs(ref), floor)
    rel = np.abs(c - ref) / scale
    return int((rel > tol).sum()), float(rel.max())


def make_oft_case(m, n, k, b, group_size=None, seed=0, kind="qr", xdist="uniform", wsigma=None):
    """Returns (A[m,k], Rstore[G*b,k], B[n,k]) fp16 numpy arrays."""
    gs = n if group_size is None else group_size
    G = n // gs
    if xdist == "uniform":
        A = inputs.uniform_pm1((m, k), seed)
    elif xdist == "u01":
        A = inputs.uniform_01((m, k), seed)
    elif xdist == "01":
        A = inputs.zero_one((m, k), seed)
    else:
        A = inputs.normal((m, k), seed, 1.0)
    if xdist == "u01":
        B = inputs.uniform_01((n, k), seed + 1)
    elif xdist == "01":
        B = inputs.zero_one((n, k), seed + 1)
    elif wsigma is not None:
        B = inputs.normal((n, k), seed + 1, wsigma)
    else:
        B = inputs.uniform_pm1((n, k), seed + 1)
    if kind == "qr":
        blocks = inputs.blocks_qr(G, k // b, b, seed + 2)
    elif kind == "cayley":
        blocks = inputs.blocks_cayley(G, k // b, b, seed + 2)
    elif kind == "perm":
        blocks = inputs.blocks_permutation(G, k // b, b, seed + 2)
    else:
        blocks = inputs.blocks_structured(G, k // b, b)
    return A, inputs.pack_r(blocks), B
