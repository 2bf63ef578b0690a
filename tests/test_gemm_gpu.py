"""GPU parity of gemm_tn / gemm_nt (half and float/TF32) against the fp64 truth, through the C ABI."""
import numpy as np
import pytest

from _util import TF32_TOL, oft_ok, tf32_ok
from cute_mma_b200 import inputs, ops
from oracle import oracle

pytestmark = pytest.mark.gpu


def run_gemm(lib, cuda, layout, dtype, m, n, k, A, B, ldA, ldB, ldC):
    import torch

    tdt = torch.float16 if dtype == "half" else torch.float32
    dA = torch.from_numpy(A).to(cuda)
    dB = torch.from_numpy(B).to(cuda)
    dC = torch.full((n + 1, ldC), -7.0, dtype=tdt, device=cuda)  # column-major: n columns of ldC elements
    fn = ops.gemm_tn if layout == "TN" else ops.gemm_nt
    fn(m, n, k, dA, ldA, dB, ldB, dC, ldC, dtype=dtype, lib=lib)
    assert ops.device_status(lib)[0] == 0
    out = dC.cpu().numpy()
    assert np.all(out[n, :] == -7.0), "column past the end of C was written"
    if ldC > m:
        assert np.all(out[:n, m:] == -7.0), "padding rows of C were written"
    return out[:n, :m].T.copy()  # -> [m, n]


def make_operands(layout, dtype, m, n, k, seed, ldA=None, ldB=None, dist="uniform"):
    npdt = np.float16 if dtype == "half" else np.float32
    gen = (lambda shape, s: inputs.uniform_pm1(shape, s, npdt)) if dist == "uniform" else (lambda shape, s: inputs.normal(shape, s, 1.0, npdt))
    if layout == "TN":   # A [m][ldA>=k], B [n][ldB>=k]
        ldA, ldB = ldA or k, ldB or k
        A = np.zeros((m, ldA), npdt); A[:, :k] = gen((m, k), seed)
        B = np.zeros((n, ldB), npdt); B[:, :k] = gen((n, k), seed + 1)
        a_rows, b_cols = A[:, :k], B[:, :k]
    else:                # A [k][ldA>=m], B [k][ldB>=n]
        ldA, ldB = ldA or m, ldB or n
        A = np.zeros((k, ldA), npdt); A[:, :m] = gen((k, m), seed)
        B = np.zeros((k, ldB), npdt); B[:, :n] = gen((k, n), seed + 1)
        a_rows, b_cols = A[:, :m].T, B[:, :n].T
    return A, B, ldA, ldB, a_rows, b_cols


def truth(layout, m, n, k, A, ldA, B, ldB, rows, cols, tf32_mode=0):
    ta, tb = ("T", "N") if layout == "TN" else ("N", "T")
    return oracle.gemm_f64_sampled(ta, tb, m, n, k, A, ldA, B, ldB, rows, cols, tf32_mode=tf32_mode)


SHAPES = [(128, 256, 64), (128, 256, 512), (384, 512, 256), (200, 328, 136), (72, 40, 64), (640, 1280, 1024)]


@pytest.mark.parametrize("layout", ["TN", "NT"])
@pytest.mark.parametrize("m,n,k", SHAPES)
def test_gemm_half_matches_fp64_truth(lib, cuda, layout, m, n, k):
    A, B, ldA, ldB, _, _ = make_operands(layout, "half", m, n, k, seed=1)
    got = run_gemm(lib, cuda, layout, "half", m, n, k, A, B, ldA, ldB, ldC=m)
    ref = truth(layout, m, n, k, A, ldA, B, ldB, np.arange(m), np.arange(n))
    bad, worst = oft_ok(got, ref)  # fp16 in / fp32 accumulate / fp16 out: |c-ref| <= 1e-2 (|ref|+1)
    assert bad == 0, (bad, worst)
    # fp32 accumulation leaves only the final fp16 rounding: much tighter than the stated bound
    assert worst < 2e-3, worst


@pytest.mark.parametrize("layout", ["TN", "NT"])
@pytest.mark.parametrize("m,n,k", SHAPES)
def test_gemm_float_tf32_matches_fp64_truth(lib, cuda, layout, m, n, k):
    A, B, ldA, ldB, a_rows, b_cols = make_operands(layout, "float", m, n, k, seed=2, dist="normal")
    got = run_gemm(lib, cuda, layout, "float", m, n, k, A, B, ldA, ldB, ldC=m)
    ref = truth(layout, m, n, k, A, ldA, B, ldB, np.arange(m), np.arange(n))
    bad, worst = tf32_ok(got, ref, a_rows, b_cols, k)
    assert bad == 0, (bad, worst)
    # against operands truncated to TF32 the result must be far closer (fp32 accumulation only)
    ref_t = truth(layout, m, n, k, A, ldA, B, ldB, np.arange(m), np.arange(n), tf32_mode=1)
    bad_t, worst_t = tf32_ok(got, ref_t, a_rows, b_cols, k, tol=2e-4)
    assert bad_t == 0, (bad_t, worst_t)


@pytest.mark.parametrize("layout,dtype", [("TN", "half"), ("NT", "half"), ("TN", "float"), ("NT", "float")])
def test_gemm_padded_leading_dimensions(lib, cuda, layout, dtype):
    m, n, k = 200, 328, 136
    pad = 8 if dtype == "half" else 4
    base = (k, k) if layout == "TN" else (m, n)
    A, B, ldA, ldB, a_rows, b_cols = make_operands(layout, dtype, m, n, k, seed=3, ldA=base[0] + pad, ldB=base[1] + 2 * pad)
    got = run_gemm(lib, cuda, layout, dtype, m, n, k, A, B, ldA, ldB, ldC=m + 5)
    ref = truth(layout, m, n, k, A, ldA, B, ldB, np.arange(m), np.arange(n))
    if dtype == "half":
        bad, worst = oft_ok(got, ref)
    else:
        bad, worst = tf32_ok(got, ref, a_rows, b_cols, k)
    assert bad == 0, (bad, worst)


def test_gemm_dispatcher_and_errors(lib, cuda):
    import torch

    m, n, k = 128, 256, 64
    A, B, ldA, ldB, _, _ = make_operands("TN", "half", m, n, k, seed=4)
    dA, dB = torch.from_numpy(A).to(cuda), torch.from_numpy(B).to(cuda)
    c1 = torch.empty((n, m), dtype=torch.float16, device=cuda)
    c2 = torch.empty((n, m), dtype=torch.float16, device=cuda)
    ops.gemm("T", "N", m, n, k, dA, ldA, dB, ldB, c1, m, lib=lib)
    ops.gemm("t", "n", m, n, k, dA, ldA, dB, ldB, c2, m, lib=lib)
    ops.gemm_tn(m, n, k, dA, ldA, dB, ldB, c2, m, lib=lib)
    assert ops.device_status(lib)[0] == 0
    assert torch.equal(c1, c2)
    with pytest.raises(ops.Error) as e:
        ops.gemm("N", "N", m, n, k, dA, ldA, dB, ldB, c1, m, lib=lib)
    assert e.value.code == ops.EUNSUPPORTED
    with pytest.raises(ops.Error) as e:  # misaligned base pointer
        ops.gemm_tn(m, n, k, dA.data_ptr() + 2, ldA, dB, ldB, c1, m, lib=lib)
    assert e.value.code == ops.EINVAL


@pytest.mark.parametrize("layout,dtype", [("TN", "half"), ("NT", "half"), ("TN", "float"), ("NT", "float")])
def test_gemm_rowmajor_is_the_transpose_of_colmajor(lib, cuda, layout, dtype):
    """b200_gemm_rowmajor writes C[i][j] where b200_gemm writes C[i + j*ldC]: same numbers, bit for bit
    (the same MMAs accumulate each element in the same K order), padding of C untouched."""
    import torch

    m, n, k = 200, 328, 96
    A, B, ldA, ldB, _, _ = make_operands(layout, dtype, m, n, k, seed=6)
    tdt = torch.float16 if dtype == "half" else torch.float32
    dA, dB = torch.from_numpy(A).to(cuda), torch.from_numpy(B).to(cuda)
    c_col = torch.empty((n, m), dtype=tdt, device=cuda)
    c_row = torch.full((m, n + 8), -7.0, dtype=tdt, device=cuda)
    ta, tb = ("T", "N") if layout == "TN" else ("N", "T")
    ops.gemm(ta, tb, m, n, k, dA, ldA, dB, ldB, c_col, m, dtype=dtype, lib=lib)
    ops.gemm_rowmajor(ta, tb, m, n, k, dA, ldA, dB, ldB, c_row, n + 8, dtype=dtype, lib=lib)
    assert ops.device_status(lib)[0] == 0
    assert torch.equal(c_row[:, :n], c_col.t())
    assert bool((c_row[:, n:] == -7.0).all())
    with pytest.raises(ops.Error) as e:
        ops.gemm_rowmajor(ta, tb, m, n, k, dA, ldA, dB, ldB, c_row, n - 8, dtype=dtype, lib=lib)
    assert e.value.code == ops.EINVAL


@pytest.mark.parametrize("layout", ["TN", "NT"])
@pytest.mark.parametrize("in_type,out_type,alpha,beta", [(0, 0, 1.0, 0.0), (0, 0, 0.5, 0.0), (0, 0, -1.25, 0.75), (0, 1, 1.0, 0.0), (0, 1, 2.0, -0.5),
                                                         (2, 1, 1.0, 0.0), (2, 1, 0.25, 1.0)])
def test_gemm_ex_scaled_and_float_output(lib, cuda, layout, in_type, out_type, alpha, beta):
    """b200_gemm_ex: C = alpha * A.B^T + beta * C with half or float C from half operands and float C from float (TF32)
    operands, against fp64 arithmetic on the same inputs; (1, 0) must return the bits of the plain entry point."""
    import torch

    m, n, k = 328, 264, 200 if layout == "TN" else 264
    dtype = "half" if in_type == 0 else "float"
    A, B, ldA, ldB, a_rows, b_cols = make_operands(layout, dtype, m, n, k, seed=5, dist="uniform" if in_type == 0 else "normal")
    out_dt = torch.float16 if out_type == 0 else torch.float32
    c0 = (np.random.default_rng(6).standard_normal((n, m)) * 4).astype(np.float16 if out_type == 0 else np.float32)  # column-major C: n columns of m
    dA, dB = torch.from_numpy(A).to(cuda), torch.from_numpy(B).to(cuda)
    dC = torch.from_numpy(c0).to(cuda).to(out_dt).contiguous()
    ta, tb = ("T", "N") if layout == "TN" else ("N", "T")
    ops.gemm_ex(ta, tb, m, n, k, alpha, dA, ldA, dB, ldB, beta, dC, m, in_type=in_type, out_type=out_type, lib=lib)
    assert ops.device_status(lib)[0] == 0
    got = dC.cpu().numpy().T.astype(np.float64)
    prod = truth(layout, m, n, k, A, ldA, B, ldB, np.arange(m), np.arange(n))
    want = alpha * prod + beta * c0.T.astype(np.float64)
    if in_type == 2:
        floor = abs(alpha) * np.outer(np.linalg.norm(a_rows, axis=1), np.linalg.norm(b_cols, axis=1)) / np.sqrt(k) + abs(beta) * np.abs(c0.T)
        assert np.all(np.abs(got - want) <= TF32_TOL * np.maximum(np.abs(want), floor))
    else:
        tol = 1e-2 if out_type == 0 else 2e-4  # float result: only the fp32 summation order separates it from fp64
        assert np.all(np.abs(got - want) <= tol * (np.abs(want) + abs(beta) * np.abs(c0.T.astype(np.float64)) + 1.0)), float(np.abs(got - want).max())
    if (alpha, beta) == (1.0, 0.0) and out_type == (0 if in_type == 0 else 1):
        plain = run_gemm(lib, cuda, layout, dtype, m, n, k, A, B, ldA, ldB, ldC=m)
        assert np.array_equal(plain.astype(np.float64), got)
    with pytest.raises(ops.Error) as e:
        ops.gemm_ex(ta, tb, m, n, k, 1.0, dA, ldA, dB, ldB, 0.0, dC, m, in_type=2, out_type=0, lib=lib)  # float operands, half result
    assert e.value.code == ops.EUNSUPPORTED


@pytest.mark.parametrize("m,n,k,k2", [(200, 328, 192, 64), (384, 512, 136, 16), (128, 256, 64, 200), (256, 256, 0, 72)])
def test_gemm_second_operand_pair(lib, cuda, pair_build, m, n, k, k2):
    if not pair_build:
        pytest.skip("the second operand pair is a feature of the CTA-pair kernel")
    """C = A.B^T + A2.B2^T in one pass equals the fp64 sum of the two products within the fp16 GEMM tolerance,
    including a ragged last K step of either pair and k = 0."""
    import torch

    rng = np.random.default_rng(12)
    A, B = rng.uniform(-1, 1, (m, max(k, 8))).astype(np.float16), rng.uniform(-1, 1, (n, max(k, 8))).astype(np.float16)
    A2, B2 = rng.uniform(-1, 1, (m, k2)).astype(np.float16), rng.uniform(-1, 1, (n, k2)).astype(np.float16)
    dA, dB, dA2, dB2 = (torch.from_numpy(x).to(cuda) for x in (A, B, A2, B2))
    dC = torch.empty((n, m), dtype=torch.float16, device=cuda)
    ops.gemm_tn_acc2(m, n, k, dA, A.shape[1], dB, B.shape[1], k2, dA2, k2, dB2, k2, dC, m, lib=lib)
    assert ops.device_status(lib)[0] == 0
    ref = A[:, :k].astype(np.float64) @ B[:, :k].astype(np.float64).T + A2.astype(np.float64) @ B2.astype(np.float64).T
    got = dC.cpu().numpy().T
    bad, worst = oft_ok(got, ref)
    assert bad == 0, (bad, worst)
    assert np.all(np.abs(got.astype(np.float64) - ref) <= 2e-3 * (np.abs(ref) + 1))


@pytest.mark.parametrize("m,n,k,r", [(256, 512, 256, 16), (200, 328, 192, 64), (1024, 1024, 512, 8), (128, 256, 128, 0)])
def test_lora_matches_three_gemm_arithmetic(lib, cuda, pair_build, m, n, k, r):
    if not pair_build and r > 0:
        pytest.skip("the second operand pair is a feature of the CTA-pair kernel")
    """b200_lora_tn_f16 against the arithmetic of the reference's comparator (playgrounds/lora.cu:33-64) done in
    fp64, with the intermediate X.L1^T rounded to fp16 as there."""
    import torch

    rng = np.random.default_rng(13)
    X = rng.normal(0, 1, (m, k)).astype(np.float16)
    W = rng.normal(0, 0.05, (n, k)).astype(np.float16)
    L1 = rng.normal(0, 0.05, (max(r, 1), k)).astype(np.float16)
    L2 = rng.normal(0, 0.05, (n, max(r, 8))).astype(np.float16)  # ld a multiple of 8 elements
    dX, dW, dL1, dL2 = (torch.from_numpy(x).to(cuda) for x in (X, W, L1, L2))
    dC = torch.full((m + 1, n), -7.0, dtype=torch.float16, device=cuda)
    ops.lora_tn(m, n, k, r, dX, k, dW, k, dL1, k, dL2, L2.shape[1], dC, n, lib=lib)
    assert ops.device_status(lib)[0] == 0
    T = (X.astype(np.float64) @ L1[:r].astype(np.float64).T).astype(np.float16).astype(np.float64) if r else np.zeros((m, 0))
    ref = X.astype(np.float64) @ W.astype(np.float64).T + T @ L2[:, :r].astype(np.float64).T
    out = dC.cpu().numpy()
    assert np.all(out[m] == np.float16(-7.0))
    got = out[:m].astype(np.float64)
    assert np.all(np.abs(got - ref) <= 2e-3 * (np.abs(ref) + 1)), float(np.abs(got - ref).max())


def test_phase_locked_gemms_on_two_streams(lib, cuda, pair_build):
    """Two GEMMs large enough for the cross-CTA phase lock (operand beyond three times L2), launched on two streams
    without a synchronisation between them: each launch has its own round counters and is started cooperatively,
    so both finish, report no timed-out wait and return the bits of a launch that ran alone."""
    import torch

    if not pair_build:
        pytest.skip("the phase lock is a feature of the CTA-pair kernels")
    m, n, k = 512, 26624, 8192   # B: 26624 x 8192 fp16 = 416 MB
    g = torch.Generator(device=cuda).manual_seed(77)
    dA = (torch.rand((m, k), generator=g, device=cuda) * 2 - 1).to(torch.float16)
    dB = (torch.rand((n, k), generator=g, device=cuda) * 2 - 1).to(torch.float16)
    alone = torch.empty((n, m), dtype=torch.float16, device=cuda)
    ops.gemm_tn(m, n, k, dA, k, dB, k, alone, m, lib=lib)
    torch.cuda.synchronize()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    c1, c2 = torch.empty_like(alone), torch.empty_like(alone)
    for _ in range(3):
        ops.gemm_tn(m, n, k, dA, k, dB, k, c1, m, s1.cuda_stream, lib=lib)
        ops.gemm_tn(m, n, k, dA, k, dB, k, c2, m, s2.cuda_stream, lib=lib)
    torch.cuda.synchronize()
    assert ops.device_status(lib)[0] == 0
    assert torch.equal(c1, alone) and torch.equal(c2, alone)


def _sampled(lib, cuda, layout, dtype, m, n, k, seed, dist):
    import torch

    g = torch.Generator(device=cuda).manual_seed(seed)
    tdt = torch.float16 if dtype == "half" else torch.float32
    shapeA, shapeB = ((m, k), (n, k)) if layout == "TN" else ((k, m), (k, n))
    if dist == "uniform":
        dA = (torch.rand(shapeA, generator=g, device=cuda) * 2 - 1).to(tdt)
        dB = (torch.rand(shapeB, generator=g, device=cuda) * 2 - 1).to(tdt)
    else:
        dA = torch.randn(shapeA, generator=g, device=cuda).to(tdt)
        dB = torch.randn(shapeB, generator=g, device=cuda).to(tdt)
    dC = torch.empty((n, m), dtype=tdt, device=cuda)
    fn = ops.gemm_tn if layout == "TN" else ops.gemm_nt
    fn(m, n, k, dA, shapeA[1], dB, shapeB[1], dC, m, dtype=dtype, lib=lib)
    assert ops.device_status(lib)[0] == 0
    rng = np.random.default_rng(seed)
    rows = np.unique(np.concatenate([[0, 127, 128, m - 1], rng.integers(0, m, 60)]))
    cols = np.unique(np.concatenate([[0, 255, 256, n - 1], rng.integers(0, n, 60)]))
    A, B = dA.cpu().numpy(), dB.cpu().numpy()
    ref = truth(layout, m, n, k, A, shapeA[1], B, shapeB[1], rows, cols)
    got = dC.cpu().numpy().T[np.ix_(rows, cols)]
    if dtype == "half":
        bad, worst = oft_ok(got, ref)
    else:
        a_rows = A[rows] if layout == "TN" else A[:, rows].T
        b_cols = B[cols] if layout == "TN" else B[:, cols].T
        bad, worst = tf32_ok(got, ref, a_rows, b_cols, k)
    assert bad == 0, (bad, worst)
    # size-independent property: a second launch is bitwise identical
    dC2 = torch.empty_like(dC)
    fn(m, n, k, dA, shapeA[1], dB, shapeB[1], dC2, m, dtype=dtype, lib=lib)
    assert ops.device_status(lib)[0] == 0
    assert torch.equal(dC, dC2)


def test_gemm_half_tn_8192_sampled(lib, cuda):
    """gemm_half TN, M=N=K=8192, U(-1,1): full size on the GPU, fp64 truth on sampled rows x columns."""
    _sampled(lib, cuda, "TN", "half", 8192, 8192, 8192, 21, "uniform")


def test_gemm_float_nt_4096_sampled(lib, cuda):
    """gemm_float NT on TF32 tensor cores, M=N=K=4096, N(0,1)."""
    _sampled(lib, cuda, "NT", "float", 4096, 4096, 4096, 22, "normal")
