"""CPU: the plain-C oracle against the reference's golden vectors, the reference build (when present)
and the algebraic pins the reference's own checks rely on."""
import os

import numpy as np
import pytest

from _util import make_oft_case
from cute_mma_b200 import inputs
from oracle import oracle

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "oft_ref_vectors.npz")


def golden_cases():
    z = np.load(GOLDEN)
    names = sorted({k.split("__")[0] for k in z.files})
    return z, names


def test_oracle_reproduces_reference_golden_vectors():
    z, names = golden_cases()
    assert len(names) >= 6
    for name in names:
        m, gs, G, k, b = (int(x) for x in z[f"{name}__dims"])
        A, R, B, C = (z[f"{name}__{key}"].view(np.float16) for key in "ARBC")
        got = oracle.cpu_oft_tn(A, R, B, m, gs, G, k, b, threads=1)
        assert np.array_equal(got.view(np.uint16), C.view(np.uint16)), name
        got_mt = oracle.cpu_oft_tn(A, R, B, m, gs, G, k, b, threads=4)
        assert np.array_equal(got_mt.view(np.uint16), C.view(np.uint16)), name + " (threads)"


@pytest.mark.skipif(not oracle.have_reference(), reason="oracle/_ref not built (needs the reference tree)")
@pytest.mark.parametrize("m,gs,G,k,b", [(33, 48, 1, 96, 32), (16, 32, 2, 64, 8), (7, 64, 2, 256, 64), (3, 40, 1, 256, 128), (64, 256, 1, 512, 16)])
def test_oracle_is_bit_identical_to_reference_build(m, gs, G, k, b):
    A, R, B = make_oft_case(m, gs * G, k, b, gs, seed=m + k)
    ref = oracle.ref_cpu_oft_tn(A, R, B, m, gs, G, k, b)
    got = oracle.cpu_oft_tn(A, R, B, m, gs, G, k, b, threads=3)
    assert np.array_equal(got.view(np.uint16), ref.view(np.uint16))


def test_row_and_column_sampling_is_exact():
    """The sampled parity tests rely on this: an output element depends only on its row of A, on R and
    on its column of B (single group)."""
    m, n, k, b = 40, 96, 128, 32
    A, R, B = make_oft_case(m, n, k, b, seed=3)
    full = oracle.cpu_oft_tn(A, R, B, m, n, 1, k, b)
    rows, cols = np.array([0, 5, 39]), np.array([1, 2, 64, 95])
    part = oracle.cpu_oft_tn(A[rows], R, B[cols], len(rows), len(cols), 1, k, b)
    assert np.array_equal(part.view(np.uint16), full[np.ix_(rows, cols)].view(np.uint16))


def test_stored_r_is_the_transpose_of_the_rotation():
    """Y = (X . R_math) . W with stored block = R_math^T (cpu_oft.hpp:9-20,101-108)."""
    m, n, k, b = 8, 16, 64, 16
    A, _, B = make_oft_case(m, n, k, b, seed=5)
    blocks = inputs.blocks_qr(1, k // b, b, 9)
    R = inputs.pack_r(blocks)
    R16 = inputs.unpack_r(R, b)  # the fp16-rounded rotation actually stored
    X = A.astype(np.float64)
    XR = np.concatenate([X[:, j * b:(j + 1) * b] @ R16[0, j] for j in range(k // b)], axis=1)
    Y = XR @ B.astype(np.float64).T
    got = oracle.oft_f64(A, R, B, m, n, 1, k, b, round_xr=False)
    assert np.allclose(got, Y, rtol=0, atol=1e-9)
    # the transposed convention gives a different answer (the blocks are not symmetric)
    XRt = np.concatenate([X[:, j * b:(j + 1) * b] @ R16[0, j].T for j in range(k // b)], axis=1)
    assert not np.allclose(XRt @ B.astype(np.float64).T, Y, atol=1e-3)


def test_structured_block_known_answer_both_conventions():
    """Known-answer block (idea of playgrounds/bd_construct.cu:117-159): R_math = I + e0 1^T."""
    m, n, k, b = 6, 8, 32, 8
    A, R, B = make_oft_case(m, n, k, b, seed=7, kind="structured", xdist="01")
    Xp = A.astype(np.float64).reshape(m, k // b, b).copy()
    Xp += Xp[:, :, :1]                       # (x R)[q] = x[q] + x[0]
    expect = Xp.reshape(m, k) @ B.astype(np.float64).T
    got = oracle.cpu_oft_tn(A, R, B, m, n, 1, k, b).astype(np.float64)
    assert np.array_equal(got, expect)
    # with the opposite storage convention (bd_construct.cu:28 uses CUBLAS_OP_T) column 0 collects the block sum
    Rt = inputs.pack_r(inputs.blocks_structured(1, k // b, b).transpose(0, 1, 3, 2))
    Xq = A.astype(np.float64).reshape(m, k // b, b).copy()
    Xq[:, :, 0] += Xq.sum(axis=2)
    got_t = oracle.cpu_oft_tn(A, Rt, B, m, n, 1, k, b).astype(np.float64)
    assert np.array_equal(got_t, Xq.reshape(m, k) @ B.astype(np.float64).T)


def test_arw_equals_a_rw_algebra():
    """(X.R).W == X.(R.W): the cross-check of cute_oft_pc.cu:300-332, in fp64 on the CPU."""
    m, n, k, b = 10, 24, 96, 32
    A, R, B = make_oft_case(m, n, k, b, seed=11)
    R16 = inputs.unpack_r(R, b)
    W = B.astype(np.float64).T
    RW = np.concatenate([R16[0, j] @ W[j * b:(j + 1) * b] for j in range(k // b)], axis=0)
    assert np.allclose(oracle.oft_f64(A, R, B, m, n, 1, k, b, round_xr=False), A.astype(np.float64) @ RW, atol=1e-9)


def test_permutation_blocks_make_xr_exact():
    m, n, k, b = 9, 16, 64, 16
    A, R, B = make_oft_case(m, n, k, b, seed=13, kind="perm", xdist="u01")
    a = oracle.oft_f64(A, R, B, m, n, 1, k, b, round_xr=True)
    c = oracle.oft_f64(A, R, B, m, n, 1, k, b, round_xr=False)
    assert np.array_equal(a, c)
    errors, worst = oracle.check_result(oracle.cpu_oft_tn(A, R, B, m, n, 1, k, b), a.astype(np.float16))
    assert errors == 0 and worst < 5e-3


def test_check_result_counts_like_the_reference():
    ref = np.array([1.0, 2.0, 4.0, 0.0], dtype=np.float16)
    res = np.array([1.0, 2.02, 4.0, 0.0], dtype=np.float16)
    errors, worst = oracle.check_result(res, ref, 5e-3)
    assert errors == 1 and 9e-3 < worst < 1.1e-2  # 0/0 is NaN: compares false, not counted (cute_oft_pc.cu:52-60)


def test_oracle_rejects_bad_shapes():
    A = np.zeros((2, 10), np.float16)
    with pytest.raises(ValueError):
        oracle.cpu_oft_tn(A, np.zeros((4, 10), np.float16), np.zeros((4, 10), np.float16), 2, 4, 1, 10, 4)


def test_gemm_truth_follows_reference_indexing():
    """gemm_sm80_tc.cu:557-568: TN reads A[i*ldA+l], B[l+j*ldB]; NT reads A[i+l*ldA], B[l*ldB+j]."""
    rng = np.random.default_rng(0)
    m, n, k = 5, 7, 9
    A = rng.standard_normal((m, k)).astype(np.float32)
    B = rng.standard_normal((n, k)).astype(np.float32)
    want = A.astype(np.float64) @ B.astype(np.float64).T
    rows, cols = np.arange(m), np.arange(n)
    assert np.allclose(oracle.gemm_f64_sampled("T", "N", m, n, k, A, k, B, k, rows, cols), want)
    assert np.allclose(oracle.gemm_f64_sampled("N", "T", m, n, k, A.T.copy(), m, B.T.copy(), n, rows, cols), want)
    h = oracle.gemm_f64_sampled("T", "N", m, n, k, A.astype(np.float16), k, B.astype(np.float16), k, rows[:2], cols[:3])
    assert np.allclose(h, A.astype(np.float16).astype(np.float64)[:2] @ B.astype(np.float16).astype(np.float64)[:3].T)
    t = oracle.gemm_f64_sampled("T", "N", m, n, k, A, k, B, k, rows, cols, tf32_mode=1)
    trunc = lambda x: (x.view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32).astype(np.float64)
    assert np.allclose(t, trunc(A) @ trunc(B).T)
