"""GPU parity of the OFT product (every route of the library) against the CPU oracle, through the C ABI."""
import numpy as np
import pytest

from _util import make_oft_case, oft_ok, truth_ok
from cute_mma_b200 import ops
from oracle import oracle

pytestmark = pytest.mark.gpu


def run_oft(lib, cuda, A, R, B, m, n, k, b, group_size=None, ldA=None, ldB=None, ldR=None, ldC=None, canary=True, fn=None, route=None):
    """Uploads the operands (optionally with padded leading dimensions), runs b200_oft_tn_f16 and
    returns C[m,n] as numpy.  The padding of C is filled with a canary and must come back untouched.
    ``route`` forces one of the library's routes (option "oft_route") for this call."""
    import torch

    if route is not None:
        with ops.option("oft_route", route, lib):
            return run_oft(lib, cuda, A, R, B, m, n, k, b, group_size, ldA, ldB, ldR, ldC, canary, fn)

    ldA, ldB, ldR, ldC = ldA or k, ldB or k, ldR or k, ldC or n

    def up(x, ld):
        rows = x.shape[0]
        buf = torch.full((rows, ld), float("nan"), dtype=torch.float16, device=cuda)
        buf[:, : x.shape[1]] = torch.from_numpy(x).to(cuda)
        return buf

    dA, dB, dR = up(A, ldA), up(B, ldB), up(R, ldR)
    dC = torch.full((m + 1, ldC), -7.0, dtype=torch.float16, device=cuda)  # one canary row + canary columns
    (fn or ops.oft_tn)(m, n, k, dA, ldA, dB, ldB, dR, ldR, dC, ldC, group_size=group_size, reconn_sz=b, lib=lib)
    st = ops.device_status(lib)
    assert st[0] == 0, st
    out = dC.cpu().numpy()
    if canary:
        assert np.all(out[m, :] == np.float16(-7.0)), "row past the end of C was written"
        if ldC > n:
            assert np.all(out[:m, n:] == np.float16(-7.0)), "padding columns of C were written"
    return out[:m, :n].copy()


def oracle_full(A, R, B, m, n, k, b, group_size=None):
    gs = n if group_size is None else group_size
    return oracle.cpu_oft_tn(A, R, B, m, gs, n // gs, k, b, threads=oracle.num_threads())


CASES = [
    # m, n, k, b, group_size
    (128, 256, 64, 64, None),      # one tile, one unit
    (128, 256, 256, 64, None),     # one tile, several units
    (384, 512, 512, 64, None),     # several tiles per CTA order
    (384, 512, 512, 32, None),
    (384, 512, 512, 16, None),
    (256, 512, 512, 128, None),
    (512, 1024, 1024, 32, None),   # the CPU-oracle configuration: 32 blocks of 32x32
    (200, 328, 192, 64, None),     # ragged M and N
    (136, 264, 96, 32, None),      # K not a multiple of the 64-wide stage
    (72, 40, 128, 16, None),       # smaller than one tile
    (256, 512, 256, 32, 256),      # two N-groups, each with its own R
    (128, 768, 128, 16, 256),      # three groups
    (256, 512, 256, 8, None),      # 8 x 8 blocks (the reference's default edge): expanded to 16 x 16 pairs
    (200, 328, 264, 8, None),      # odd number of 8-wide blocks (K = 33 * 8), ragged M and N
    (256, 512, 128, 8, 256),       # 8 x 8 blocks, two N-groups
    (256, 512, 256, 64, 128),      # groups smaller than the N tile: two per tile
    (384, 512, 512, 32, 64),       # four per tile
    (200, 320, 192, 16, 32),       # eight per tile, ragged M, last tile holds two of its eight groups
    (256, 256, 128, 8, 64),        # 8 x 8 blocks, four groups per tile
    (512, 768, 512, 64, 64),       # R tiles of four groups travel with every stage of X
]


@pytest.mark.parametrize("m,n,k,b,gs", CASES)
def test_oft_matches_oracle(lib, cuda, pair_build, m, n, k, b, gs):
    if gs is not None and gs < 256 and not pair_build:
        pytest.skip("groups smaller than the N tile need the CTA-pair build")
    A, R, B = make_oft_case(m, n, k, b, gs, seed=0, kind="qr")
    ref = oracle_full(A, R, B, m, n, k, b, gs)
    got = run_oft(lib, cuda, A, R, B, m, n, k, b, gs)
    truth = oracle.oft_f64(A, R, B, m, n if gs is None else gs, 1 if gs is None else n // gs, k, b, round_xr=True)
    bad, worst = oft_ok(got, ref, truth=truth)
    assert bad == 0, f"{bad} elements outside 1e-2*(|ref|+1) + oracle drift; worst normalised error {worst:.3e}"
    bad_t, worst_t = truth_ok(got, truth)
    assert bad_t == 0, f"{bad_t} elements further than 2e-3*(|y|+1) from exact arithmetic; worst {worst_t:.3e}"
    if k // b <= 4:  # few re-roundings in the oracle: the stated tolerance holds without any allowance
        assert oft_ok(got, ref)[0] == 0


@pytest.mark.parametrize("route", [1, 2, 3])
def test_oft_cpu_oracle_configuration_tolerance_accounting(lib, cuda, pair_build, route):
    """The CPU-oracle configuration (M 512, K 1024, N 1024, 32 blocks of 32 x 32, U(-1,1) operands) against the stated
    tolerance |y - y_ref| <= 1e-2 (|y_ref| + 1) with NO allowance, counted: cpu_oft_tn re-rounds C to fp16 after each of
    its 32 K blocks (cpu_oft.hpp:13-17), so even the exact result (fp64 accumulation of the same fp16 X.R) misses the
    bound on some elements.  The kernel must miss it on no more elements than exact arithmetic rounded to fp16 does
    (up to a handful of borderline elements that the fp32 summation order flips), and on less than 0.2 % of them;
    the counts are printed (pytest -s) and recorded in the design notes."""
    if route == 3 and not pair_build:
        pytest.skip("the shared-X.R kernel exists in the CTA-pair build only")
    m, n, k, b = 512, 1024, 1024, 32
    A, R, B = make_oft_case(m, n, k, b, seed=0, kind="qr")
    ref = oracle_full(A, R, B, m, n, k, b)
    truth = oracle.oft_f64(A, R, B, m, n, 1, k, b, round_xr=True)
    got = run_oft(lib, cuda, A, R, B, m, n, k, b, route=route)
    outside_kernel, worst_kernel = oft_ok(got, ref)
    outside_truth, worst_truth = oft_ok(truth.astype(np.float16), ref)
    print(f"route {route}: outside 1e-2(|y_ref|+1): kernel {outside_kernel} (worst {worst_kernel:.3e}), "
          f"exact arithmetic rounded to fp16 {outside_truth} (worst {worst_truth:.3e}), of {m * n} elements")
    assert outside_truth > 0, "the oracle no longer drifts out of its own tolerance: drop the allowance in oft_ok"
    assert outside_kernel <= 1.02 * outside_truth + 2
    assert outside_kernel / (m * n) <= 2e-3
    assert truth_ok(got, truth)[0] == 0


TWO_PASS_CASES = [
    (128, 256, 64, 64, None),
    (384, 512, 512, 64, None),
    (384, 512, 512, 32, None),
    (384, 512, 512, 16, None),
    (256, 512, 512, 128, None),
    (200, 328, 192, 64, None),     # ragged M and N
    (136, 264, 96, 32, None),      # K not a multiple of the 64-wide unit
    (200, 328, 264, 8, None),      # 8 x 8 blocks, odd number of them
    (72, 40, 128, 16, None),       # smaller than one tile
    (128, 768, 128, 16, 256),      # three groups: the passes repeat per group on the one X.R buffer
    (256, 512, 256, 128, 256),
]


@pytest.mark.parametrize("m,n,k,b,gs", TWO_PASS_CASES)
def test_oft_two_pass_matches_oracle_and_fused(lib, cuda, m, n, k, b, gs):
    """Rotation pass + plain GEMM: same tolerances against the oracle as the fused kernel, and the two
    routes agree with each other to fp32-summation-order noise (both round X.R to fp16 once)."""
    A, R, B = make_oft_case(m, n, k, b, gs, seed=21, kind="qr")
    ref = oracle_full(A, R, B, m, n, k, b, gs)
    got = run_oft(lib, cuda, A, R, B, m, n, k, b, gs, fn=ops.oft_tn_two_pass)
    truth = oracle.oft_f64(A, R, B, m, n if gs is None else gs, 1 if gs is None else n // gs, k, b, round_xr=True)
    bad, worst = oft_ok(got, ref, truth=truth)
    assert bad == 0, (bad, worst)
    bad_t, worst_t = truth_ok(got, truth)
    assert bad_t == 0, (bad_t, worst_t)
    if k // b <= 4:
        assert oft_ok(got, ref)[0] == 0
    fused = run_oft(lib, cuda, A, R, B, m, n, k, b, gs, route=1)
    d = np.abs(got.astype(np.float64) - fused.astype(np.float64))
    assert np.all(d <= 2.0 ** -10 * (np.abs(fused.astype(np.float64)) + 1.0)), float(d.max())


RING_CASES = [
    # m, n, k, b, group_size: the route in which one X.R per row block serves all N tiles of a group
    (128, 256, 64, 64, None),      # one tile, one rotation unit
    (384, 512, 512, 64, None),     # two row blocks x two N tiles
    (384, 512, 512, 32, None),
    (384, 512, 512, 16, None),
    (256, 512, 512, 128, None),    # a rotation unit spans two stages
    (512, 1024, 1024, 32, None),   # the CPU-oracle configuration
    (200, 328, 192, 64, None),     # ragged M and N
    (136, 264, 96, 32, None),      # K not a multiple of the 64-wide stage
    (200, 328, 264, 8, None),      # 8 x 8 blocks, odd number of them
    (72, 40, 128, 16, None),       # smaller than one tile
    (128, 768, 128, 16, 256),      # three groups: one launch per group
    (256, 1024, 256, 128, 512),    # two groups of two N tiles
    (2304, 5120, 256, 64, None),   # 180 tiles: several tiles per SM pair, more rotation units than pairs
]


@pytest.mark.parametrize("m,n,k,b,gs", RING_CASES)
def test_oft_ring_route_matches_oracle_and_two_pass(lib, cuda, pair_build, m, n, k, b, gs):
    """oft3_kernel (route 3): the oracle tolerances of the other routes, and the bits of the rotation pass +
    GEMM (same X.R rounded once to fp16, same order of the fp32 sums over K)."""
    if not pair_build:
        pytest.skip("the shared-X.R kernel exists in the CTA-pair build only")
    A, R, B = make_oft_case(m, n, k, b, gs, seed=23, kind="qr")
    got = run_oft(lib, cuda, A, R, B, m, n, k, b, gs, route=3)
    with ops.option("gemm_split", 0, lib):  # small problems: the plain GEMM would otherwise sum K in up to four pieces
        two = run_oft(lib, cuda, A, R, B, m, n, k, b, gs, route=2)
    diff = float(np.abs(got.astype(np.float64) - two.astype(np.float64)).max())
    assert np.array_equal(got.view(np.uint16), two.view(np.uint16)), f"max difference {diff}"
    if m * n * k <= 1 << 30:
        ref = oracle_full(A, R, B, m, n, k, b, gs)
        truth = oracle.oft_f64(A, R, B, m, n if gs is None else gs, 1 if gs is None else n // gs, k, b, round_xr=True)
        bad, worst = oft_ok(got, ref, truth=truth)
        assert bad == 0, (bad, worst)
        bad_t, worst_t = truth_ok(got, truth)
        assert bad_t == 0, (bad_t, worst_t)
        if k // b <= 4:
            assert oft_ok(got, ref)[0] == 0


def test_oft_ring_route_reuses_its_slots_and_phase_locks(lib, cuda, pair_build):
    """More row blocks (41) than the ring holds (16): slots are rewritten two bands later, after every tile that
    read them has finished.  Run with and without the cross-CTA phase lock, with padded leading dimensions and
    canaries around C, twice (the counters are per launch), against the rotation pass + GEMM."""
    if not pair_build:
        pytest.skip("the shared-X.R kernel exists in the CTA-pair build only")
    m, n, k, b = 256 * 40 + 72, 768, 320, 64
    A, R, B = make_oft_case(m, n, k, b, seed=27, kind="qr")
    with ops.option("gemm_split", 0, lib):
        two = run_oft(lib, cuda, A, R, B, m, n, k, b, route=2)
    for sync in (0, 1, 1):
        with ops.option("tile_sync", sync, lib):
            got = run_oft(lib, cuda, A, R, B, m, n, k, b, ldA=k + 8, ldB=k + 16, ldR=k + 24, ldC=n + 8, route=3)
        assert np.array_equal(got.view(np.uint16), two.view(np.uint16))
    with ops.option("raster", 2, lib):  # bands of 2 row blocks, a ring of 4: twenty reuses per slot
        got = run_oft(lib, cuda, A, R, B, m, n, k, b, route=3)
    assert np.array_equal(got.view(np.uint16), two.view(np.uint16))
    rows = np.array([0, 255, 256, 4095, 4096, 4097, m - 1])
    ref = oracle.cpu_oft_tn(A[rows], R, B, len(rows), n, 1, k, b, threads=oracle.num_threads())
    assert oft_ok(got[rows], ref)[0] == 0


@pytest.mark.parametrize("m,n,k,b,gs", RING_CASES)
def test_oft_split_ring_route_small_cases(lib, cuda, pair_build, m, n, k, b, gs):
    """oft4_kernel (route 4) on problems whose row blocks all fit the ring: every SM pair rotates, then every pair
    multiplies.  Same bits as the rotation pass + GEMM."""
    if not pair_build:
        pytest.skip("the shared-X.R kernels exist in the CTA-pair build only")
    A, R, B = make_oft_case(m, n, k, b, gs, seed=29, kind="qr")
    got = run_oft(lib, cuda, A, R, B, m, n, k, b, gs, route=4)
    with ops.option("gemm_split", 0, lib):
        two = run_oft(lib, cuda, A, R, B, m, n, k, b, gs, route=2)
    assert np.array_equal(got.view(np.uint16), two.view(np.uint16))


SPLIT_CASES = [
    # m, n, k, b, raster, ring_bands, rot_pairs: more row blocks than the ring holds, so some pairs only rotate
    (4096, 2048, 1024, 64, 2, 2, 1),
    (4096, 2048, 1024, 64, 2, 2, 5),
    (4096, 1024, 1024, 128, 2, 2, -1),
    (4096, 2048, 512, 32, 2, 2, 2),
    (4096, 2048, 512, 16, 2, 2, 3),
    (4001, 2304, 1088, 64, 2, 2, -1),   # ragged M, 17 blocks of 64
    (4001, 2304, 1152, 128, 3, 2, 2),   # a ragged last band
    (256 * 40 + 72, 768, 320, 64, 4, 2, 30),  # far more rotation pairs than needed
]


@pytest.mark.parametrize("m,n,k,b,raster,bands,rot_pairs", SPLIT_CASES)
def test_oft_split_ring_route_rotation_pairs_and_slot_reuse(lib, cuda, pair_build, m, n, k, b, raster, bands, rot_pairs):
    """oft4_kernel with rotation pairs at work: the first bands are rotated by all pairs, the rest by the rotation
    pairs, which rewrite a ring slot only after every tile that read it has finished.  Padded leading dimensions,
    canaries around C, three launches (the counters are per launch), with and without the phase lock; against the
    rotation pass + GEMM bit for bit and sampled rows against the oracle."""
    if not pair_build:
        pytest.skip("the shared-X.R kernels exist in the CTA-pair build only")
    A, R, B = make_oft_case(m, n, k, b, seed=33, kind="qr")
    with ops.option("gemm_split", 0, lib):
        two = run_oft(lib, cuda, A, R, B, m, n, k, b, route=2)
    with ops.option("raster", raster, lib), ops.option("ring_bands", bands, lib), ops.option("rot_pairs", rot_pairs, lib):
        for sync in (0, 1, 1):
            with ops.option("tile_sync", sync, lib):
                got = run_oft(lib, cuda, A, R, B, m, n, k, b, ldA=k + 8, ldB=k + 16, ldR=k + 24, ldC=n + 8, route=4)
            assert np.array_equal(got.view(np.uint16), two.view(np.uint16))
    rows = np.array([0, 255, 256, 2047, 2048, m - 1])
    ref = oracle.cpu_oft_tn(A[rows], R, B, len(rows), n, 1, k, b, threads=oracle.num_threads())
    truth = oracle.oft_f64(A[rows], R, B, len(rows), n, 1, k, b, round_xr=True)
    bad, worst = oft_ok(got[rows], ref, truth=truth)
    assert bad == 0, (bad, worst)
    assert truth_ok(got[rows], truth)[0] == 0


def test_oft_two_pass_padded_and_bit_exact_cases(lib, cuda):
    m, n, k, b = 200, 328, 192, 64
    A, R, B = make_oft_case(m, n, k, b, seed=3)
    ref = oracle_full(A, R, B, m, n, k, b)
    got = run_oft(lib, cuda, A, R, B, m, n, k, b, ldA=k + 8, ldB=k + 16, ldR=k + 24, ldC=n + 8, fn=ops.oft_tn_two_pass)
    assert oft_ok(got, ref)[0] == 0
    # 0/1 inputs with permutation blocks: every partial sum is an exactly representable integer
    m, n, k, b = 256, 512, 256, 32
    A, R, B = make_oft_case(m, n, k, b, seed=9, kind="perm", xdist="01")
    ref = oracle_full(A, R, B, m, n, k, b)
    got = run_oft(lib, cuda, A, R, B, m, n, k, b, fn=ops.oft_tn_two_pass)
    assert np.array_equal(got.view(np.uint16), ref.view(np.uint16))


def test_oft_path_choice_is_invisible(lib, cuda, pair_build):
    """A shape the library sends down the shared-X.R route (one group over many N tiles, b = 128) gives the
    same answer, to summation-order noise, as the kernel that keeps X.R in tensor memory (route 1) and as the
    two passes (route 2)."""
    m, n, k, b = 1024, 8192, 1024, 128
    A, R, B = make_oft_case(m, n, k, b, seed=31, kind="qr", xdist="normal", wsigma=0.02)
    if pair_build:
        assert ops.oft_plan(m, n, k, reconn_sz=b, lib=lib)["path"] == "fused_ring"
    auto = run_oft(lib, cuda, A, R, B, m, n, k, b)
    fused = run_oft(lib, cuda, A, R, B, m, n, k, b, route=1)
    two = run_oft(lib, cuda, A, R, B, m, n, k, b, route=2)
    d = np.abs(auto.astype(np.float64) - fused.astype(np.float64))
    assert np.all(d <= 2.0 ** -10 * (np.abs(fused.astype(np.float64)) + 1.0)), float(d.max())
    d = np.abs(auto.astype(np.float64) - two.astype(np.float64))
    assert np.all(d <= 2.0 ** -10 * (np.abs(two.astype(np.float64)) + 1.0)), float(d.max())
    truth = oracle.oft_f64(A, R, B, m, n, 1, k, b, round_xr=True)
    assert truth_ok(auto, truth)[0] == 0


@pytest.mark.parametrize("m,k,b,ldx", [(200, 192, 64, 192), (136, 96, 32, 104), (384, 512, 128, 512), (72, 264, 8, 264), (1000, 320, 16, 328)])
def test_rotate_matches_blockwise_product(lib, cuda, m, k, b, ldx):
    """b200_rotate_f16 alone: XR[:, kb*b:(kb+1)*b] = half(A[:, kb*b:(kb+1)*b] . Rstore_kb^T) with fp32 accumulation
    (summation order free: one fp16 ulp allowed), ragged M and K edges clipped, padding of XR untouched."""
    import torch

    A, R, _ = make_oft_case(m, 8, k, b, seed=17, kind="qr")
    dA, dR = torch.from_numpy(A).to(cuda), torch.from_numpy(R).to(cuda)
    dX = torch.full((m + 1, ldx), -7.0, dtype=torch.float16, device=cuda)
    ops.rotate(m, k, dA, k, dR, k, dX, ldx, reconn_sz=b, lib=lib)
    assert ops.device_status(lib)[0] == 0
    out = dX.cpu().numpy()
    assert np.all(out[m, :] == np.float16(-7.0)) and np.all(out[:m, k:] == np.float16(-7.0))
    ref = np.empty((m, k), dtype=np.float64)
    for kb in range(k // b):
        ref[:, kb * b:(kb + 1) * b] = A[:, kb * b:(kb + 1) * b].astype(np.float64) @ R[:, kb * b:(kb + 1) * b].astype(np.float64).T
    got = out[:m, :k].astype(np.float64)
    assert np.all(np.abs(got - ref) <= 2.0 ** -10 * (np.abs(ref) + 2.0 ** -4)), float(np.abs(got - ref).max())
    with pytest.raises(ops.Error) as e:  # rows of XR must start on 16-byte boundaries (tile stores)
        ops.rotate(m, k, dA, k, dR, k, dX, ldx + 1, reconn_sz=b, lib=lib)
    assert e.value.code == ops.EINVAL


def test_oft_group_size_limits(lib, cuda, pair_build):
    if not pair_build:
        pytest.skip("the single-CTA build refuses every group smaller than the N tile")
    """Groups that neither divide the N tile nor are a multiple of it, and 128 x 128 blocks with several groups
    per tile, are refused with a message instead of computed wrongly."""
    import torch
    z = torch.zeros(1 << 16, dtype=torch.float16, device="cuda")
    for n, gs, b in ((384, 96, 16), (512, 128, 128)):
        with pytest.raises(ops.Error) as e:
            ops.oft_tn(128, n, 128, z, 128, z, 128, z, 128, z, n, group_size=gs, reconn_sz=b, lib=lib)
        assert e.value.code == ops.EUNSUPPORTED and "group_size" in e.value.message


def test_oft_padded_leading_dimensions(lib, cuda):
    m, n, k, b = 200, 328, 192, 64
    A, R, B = make_oft_case(m, n, k, b, seed=3)
    ref = oracle_full(A, R, B, m, n, k, b)
    got = run_oft(lib, cuda, A, R, B, m, n, k, b, ldA=k + 8, ldB=k + 16, ldR=k + 24, ldC=n + 8)
    bad, worst = oft_ok(got, ref)
    assert bad == 0, (bad, worst)
    # ldC not a multiple of 8 elements: the epilogue must take its scalar path
    got2 = run_oft(lib, cuda, A, R, B, m, n, k, b, ldC=n + 3)
    assert np.array_equal(got.view(np.uint16), got2.view(np.uint16))


def test_oft_permutation_blocks_reference_check(lib, cuda):
    """The reference's own correctness protocol (cute_oft_pc.cu:195-236, 334-350): positive inputs,
    permutation blocks, count of elements above 5e-3 relative error must be zero."""
    m, n, k, b = 256, 512, 512, 32
    A, R, B = make_oft_case(m, n, k, b, seed=5, kind="perm", xdist="u01")
    ref = oracle_full(A, R, B, m, n, k, b)
    got = run_oft(lib, cuda, A, R, B, m, n, k, b)
    errors, worst = oracle.check_result(got, ref, 5e-3)
    assert errors == 0, (errors, worst)


def test_oft_zero_one_init_is_bit_exact(lib, cuda):
    """--01init (cute_oft_pc.cu:202-216): every partial sum is a small integer, exact in fp16 and
    fp32, so the kernel must agree with the oracle bit for bit (K <= 2048 keeps sums <= 2048)."""
    m, n, k, b = 256, 512, 256, 64
    A, R, B = make_oft_case(m, n, k, b, seed=7, kind="perm", xdist="01")
    ref = oracle_full(A, R, B, m, n, k, b)
    got = run_oft(lib, cuda, A, R, B, m, n, k, b)
    assert np.array_equal(got.view(np.uint16), ref.view(np.uint16))


def test_oft_structured_block_known_answer(lib, cuda):
    """Known-answer block (idea of playgrounds/bd_construct.cu:117-159): with R_math = I + e0 1^T,
    (x R)[q] = x[q] + x[0] per block, so Y = X' W with X' computed in closed form.  A transposed-R
    bug would instead add the block's row sum to column 0."""
    m, n, k, b = 128, 256, 128, 32
    A, R, B = make_oft_case(m, n, k, b, seed=9, kind="structured", xdist="01")
    Xp = A.astype(np.float64).reshape(m, k // b, b).copy()
    Xp += Xp[:, :, :1]
    expect = Xp.reshape(m, k) @ B.astype(np.float64).T
    got = run_oft(lib, cuda, A, R, B, m, n, k, b)
    assert np.array_equal(got.astype(np.float64), expect)  # integers below 2048: exact


def test_oft_is_deterministic(lib, cuda):
    m, n, k, b = 384, 512, 512, 64
    A, R, B = make_oft_case(m, n, k, b, seed=11)
    a = run_oft(lib, cuda, A, R, B, m, n, k, b)
    c = run_oft(lib, cuda, A, R, B, m, n, k, b)
    assert np.array_equal(a.view(np.uint16), c.view(np.uint16))


def test_oft_k_zero_and_empty(lib, cuda):
    import torch

    dC = torch.full((8, 16), 3.0, dtype=torch.float16, device=cuda)
    d = torch.zeros(16, dtype=torch.float16, device=cuda)
    ops.oft_tn(8, 16, 0, d, 8, d, 8, d, 8, dC, 16, reconn_sz=16, lib=lib)   # K = 0: C = 0 like cpu_oft_tn
    assert torch.all(dC == 0)
    ops.oft_tn(0, 16, 64, d, 64, d, 64, d, 64, dC, 16, reconn_sz=16, lib=lib)  # M = 0: nothing to do
    assert ops.device_status(lib)[0] == 0


def _sampled_parity(lib, cuda, m, n, k, b, kind, wsigma, n_rows, seed):
    """Full-size run on the GPU from device-generated operands; the oracle recomputes sampled rows
    (an output row depends only on its own row of X, all of R and all of W)."""
    import torch
    from cute_mma_b200 import inputs

    g = torch.Generator(device=cuda).manual_seed(seed)
    dA = torch.randn((m, k), generator=g, device=cuda, dtype=torch.float32).to(torch.float16)
    dB = (torch.randn((n, k), generator=g, device=cuda, dtype=torch.float32) * wsigma).to(torch.float16)
    blocks = inputs.blocks_cayley(1, k // b, b, seed) if kind == "cayley" else inputs.blocks_qr(1, k // b, b, seed)
    R = inputs.pack_r(blocks)
    dR = torch.from_numpy(R).to(cuda)
    dC = torch.empty((m, n), dtype=torch.float16, device=cuda)
    ops.oft_tn(m, n, k, dA, k, dB, k, dR, k, dC, n, reconn_sz=b, lib=lib)
    assert ops.device_status(lib)[0] == 0
    rows = np.unique(np.concatenate([[0, 127, 128, m - 1], np.random.default_rng(seed).integers(0, m, n_rows)]))
    idx = torch.from_numpy(rows).to(cuda)
    A_s = dA[idx].cpu().numpy()
    got = dC[idx].cpu().numpy()
    ref = oracle.cpu_oft_tn(A_s, R, dB.cpu().numpy(), len(rows), n, 1, k, b, threads=oracle.num_threads())
    bad, worst = oft_ok(got, ref)
    assert bad == 0, (bad, worst)
    truth = oracle.oft_f64(A_s, R, dB.cpu().numpy(), len(rows), n, 1, k, b, round_xr=True)
    bad_t, worst_t = truth_ok(got, truth)
    assert bad_t == 0, (bad_t, worst_t)
    # size-independent property over the whole output: linearity in X.  Scaling by 2 commutes with
    # every rounding except for fp16 subnormals (|XR| or |Y| below 2^-14), so all but a sliver of the
    # elements must match bit for bit and the rest within one fp16 ulp.
    dC2 = torch.empty_like(dC)
    dA2 = dA * 2
    ops.oft_tn(m, n, k, dA2, k, dB, k, dR, k, dC2, n, reconn_sz=b, lib=lib)
    assert ops.device_status(lib)[0] == 0
    twice = dC.float() * 2
    diff = (dC2.float() - twice).abs()
    assert bool((diff <= twice.abs() * 2.0 ** -10 + 2.0 ** -13).all())
    assert float((diff != 0).float().mean()) < 1e-3


def test_oft_reference_benchmark_point_sampled(lib, cuda):
    """The reference's own benchmark point (autotune/runner_oft.py:64): M = N = K = 8192, group 256 (32
    N-groups, each with its own R), 8 x 8 blocks; positive U[0,1) operands and permutation blocks as in
    its driver, on sampled rows.  With K/b = 1024 re-roundings of a sum that grows to ~2000 (fp16 ulp 1-2)
    cpu_oft_tn itself drifts from exact arithmetic by up to 2e-2 relative here, so the reference's
    relative-error count (cute_oft_pc.cu:31-77, 5e-3) is applied against the exact result (fp64
    accumulation of the same fp16 XR), and the oracle is compared with its own drift allowed for."""
    import torch
    from cute_mma_b200 import inputs

    m = n = k = 8192
    gs, b = 256, 8
    G = n // gs
    g = torch.Generator(device=cuda).manual_seed(8)
    dA = torch.rand((m, k), generator=g, device=cuda).to(torch.float16)
    dB = torch.rand((n, k), generator=g, device=cuda).to(torch.float16)
    R = inputs.pack_r(inputs.blocks_permutation(G, k // b, b, 8))
    dR = torch.from_numpy(R).to(cuda)
    dC = torch.empty((m, n), dtype=torch.float16, device=cuda)
    ops.oft_tn(m, n, k, dA, k, dB, k, dR, k, dC, n, group_size=gs, reconn_sz=b, lib=lib)
    assert ops.device_status(lib)[0] == 0
    rows = np.unique(np.concatenate([[0, 255, 256, m - 1], np.random.default_rng(8).integers(0, m, 12)]))
    idx = torch.from_numpy(rows).to(cuda)
    ref = oracle.cpu_oft_tn(dA[idx].cpu().numpy(), R, dB.cpu().numpy(), len(rows), gs, G, k, b, threads=oracle.num_threads())
    got = dC[idx].cpu().numpy()
    truth = oracle.oft_f64(dA[idx].cpu().numpy(), R, dB.cpu().numpy(), len(rows), gs, G, k, b, round_xr=True)
    errors, worst = oracle.check_result(got, truth.astype(np.float16), 5e-3)
    assert errors == 0, (errors, worst)
    bad, worst_n = oft_ok(got, ref, truth=truth)
    assert bad == 0, (bad, worst_n)


def test_oft_projection_shape_sampled(lib, cuda):
    """M=16384, K=N=4096, b=64, Cayley blocks, X~N(0,1), W~N(0,0.02): the headline configuration."""
    _sampled_parity(lib, cuda, 16384, 4096, 4096, 64, "cayley", 0.02, 40, seed=4)


def test_oft_large_slab_sampled(lib, cuda):
    """One GPU's slab of the N-sharded large configuration at 8 GPUs (N = 28672/8 = 3584), K = 8192,
    b = 128, QR blocks; M reduced to 8192 rows to keep the run short (rows are independent)."""
    _sampled_parity(lib, cuda, 8192, 3584, 8192, 128, "qr", 0.02, 12, seed=5)


def test_oft_large_full_size_sampled_and_routes_agree(lib, cuda, pair_build):
    """The large configuration whole on one GPU (M 65536, K 8192, N 28672, b 128, QR blocks): sampled rows
    against the oracle, linearity over the whole output, and the route the library picks here (one X.R per row
    block shared through the L2 ring, rotated by SM pairs of their own) must return the same bits as the rotation pass + GEMM."""
    import torch

    m, k, n, b = 65536, 8192, 28672, 128
    if pair_build:
        assert ops.oft_plan(m, n, k, reconn_sz=b, lib=lib)["path"] == "fused_ring_split"
        assert ops.oft_plan(16384, 4096, 4096, reconn_sz=64, lib=lib) == {"path": "fused_ring", "kernel_launches": 1}
    assert ops.oft_plan(8192, 8192, 8192, group_size=256, reconn_sz=8, lib=lib) == {"path": "fused_tmem", "kernel_launches": 2}
    _sampled_parity(lib, cuda, m, n, k, b, "qr", 0.02, 8, seed=6)
    g = torch.Generator(device=cuda).manual_seed(6)  # the operands _sampled_parity drew
    dA = torch.randn((m, k), generator=g, device=cuda, dtype=torch.float32).to(torch.float16)
    dB = (torch.randn((n, k), generator=g, device=cuda, dtype=torch.float32) * 0.02).to(torch.float16)
    from cute_mma_b200 import inputs
    dR = torch.from_numpy(inputs.pack_r(inputs.blocks_qr(1, k // b, b, 6))).to(cuda)
    c_auto = torch.empty((m, n), dtype=torch.float16, device=cuda)
    c_fused = torch.empty((m, n), dtype=torch.float16, device=cuda)
    ops.oft_tn(m, n, k, dA, k, dB, k, dR, k, c_auto, n, reconn_sz=b, lib=lib)
    with ops.option("oft_route", 2, lib):
        ops.oft_tn(m, n, k, dA, k, dB, k, dR, k, c_fused, n, reconn_sz=b, lib=lib)
    assert ops.device_status(lib)[0] == 0
    assert torch.equal(c_auto.view(torch.int16), c_fused.view(torch.int16))


@pytest.mark.parametrize("m,n,k,b,gs,pad", [(200, 328, 192, 64, None, 0), (5000, 512, 256, 32, None, 8), (4200, 512, 128, 8, 256, 0), (4300, 1024, 128, 16, None, 8)])
def test_host_buffer_entry_point_matches_device_path(lib, cuda, m, n, k, b, gs, pad):
    """b200_oft_tn_f16_host (pageable numpy buffers here; several row chunks when M exceeds 2048, the chunks'
    uploads, products and downloads on three streams, the first chunk piecewise over N when N is a multiple of 1024) returns the bits of the device entry point, with padded
    host leading dimensions and with the padding of C untouched."""
    A, R, B = make_oft_case(m, n, k, b, gs, seed=41)
    dev = run_oft(lib, cuda, A, R, B, m, n, k, b, gs)

    def padded(x):
        out = np.full((x.shape[0], x.shape[1] + pad), np.float16(3.0))
        out[:, : x.shape[1]] = x
        return np.ascontiguousarray(out.astype(np.float16))

    hA, hB, hR = padded(A), padded(B), padded(R)
    hC = np.full((m, n + pad), np.float16(-7.0), dtype=np.float16)
    ops.oft_tn_host(m, n, k, hA, k + pad, hB, k + pad, hR, k + pad, hC, n + pad, group_size=gs, reconn_sz=b, lib=lib)
    assert ops.device_status(lib)[0] == 0
    assert np.array_equal(hC[:, :n].view(np.uint16), dev.view(np.uint16))
    assert np.all(hC[:, n:] == np.float16(-7.0))
    if m <= 512:
        assert oft_ok(hC[:, :n], oracle_full(A, R, B, m, n, k, b, gs))[0] == 0


def test_bounded_wait_reports_and_recovers(lib, cuda):
    """A wait that runs out is reported through the status record and leaves the context usable
    (no trap, no fault): the self-test waits 2 ms on a barrier nothing sets."""
    rec = ops.selftest_wait_timeout(2000, lib=lib)
    assert rec[0] == 1 and rec[2] == 99
    assert ops.device_status(lib)[0] == 0          # record cleared
    m, n, k, b = 128, 256, 128, 64                 # and the next real launch works
    A, R, B = make_oft_case(m, n, k, b, seed=31)
    got = run_oft(lib, cuda, A, R, B, m, n, k, b)
    assert oft_ok(got, oracle_full(A, R, B, m, n, k, b))[0] == 0


@pytest.mark.parametrize("m,n,k,b,gs", [(384, 512, 512, 64, None), (200, 328, 192, 32, None), (256, 512, 256, 8, 256), (128, 256, 256, 128, None)])
def test_a_rw_order_matches_oracle(lib, cuda, m, n, k, b, gs):
    """Y = X.(R.W) (cublas_oft.hpp:58-65): the weight transform against its definition, and the product
    against the oracle (same tolerance as the fused order; only the place of the fp16 rounding differs)."""
    import torch

    A, R, B = make_oft_case(m, n, k, b, gs, seed=41)
    g_sz = n if gs is None else gs
    dA, dB, dR = (torch.from_numpy(x).to(cuda) for x in (A, B, R))
    dBt = torch.full((n, k), float("nan"), dtype=torch.float16, device=cuda)
    ops.transform_weight(n, k, dB, k, dR, k, dBt, k, group_size=gs, reconn_sz=b, lib=lib)
    torch.cuda.synchronize()
    Rb = R.astype(np.float64).reshape(n // g_sz, b, k // b, b)            # [g][q][kb][p]
    Bb = B.astype(np.float64).reshape(n // g_sz, g_sz, k // b, b)         # [g][j][kb][q]
    want = np.einsum("gqkp,gjkq->gjkp", Rb, Bb).reshape(n, k)
    got_t = dBt.cpu().numpy().astype(np.float64)
    assert np.abs(got_t - want).max() <= 2e-3 * (np.abs(want).max() + 1.0)
    dC = torch.full((m + 1, n), -7.0, dtype=torch.float16, device=cuda)
    ops.oft_tn_a_rw(m, n, k, dA, k, dB, k, dR, k, dC, n, group_size=gs, reconn_sz=b, lib=lib)
    assert ops.device_status(lib)[0] == 0
    out = dC.cpu().numpy()
    assert np.all(out[m] == np.float16(-7.0))
    ref = oracle_full(A, R, B, m, n, k, b, gs)
    truth = oracle.oft_f64(A, R, B, m, g_sz, n // g_sz, k, b, round_xr=False)
    assert oft_ok(out[:m], ref, truth=truth)[0] == 0
    # against exact arithmetic on the fp16-rounded transformed weight (this order's only intermediate rounding)
    exact = A.astype(np.float64) @ want.astype(np.float16).astype(np.float64).T
    assert truth_ok(out[:m], exact)[0] == 0


def test_route_choice_either_side_of_the_crossover(lib, cuda, pair_build):
    """b200_oft_plan on shapes either side of the measured crossover between the kernel that keeps X.R in tensor
    memory (few N tiles per group) and the kernel that shares one X.R per row block (8 tiles or more; 4 for 128 x 128
    blocks), and the option that overrides the choice."""
    if not pair_build:
        pytest.skip("the single-CTA build has one route")
    plan = lambda n, b, gs=None: ops.oft_plan(16384, n, 4096, group_size=gs, reconn_sz=b, lib=lib)["path"]
    assert plan(1792, 64) == "fused_tmem" and plan(2048, 64) == "fused_ring"
    assert plan(768, 128) == "fused_tmem" and plan(1024, 128) == "fused_ring"
    assert plan(4096, 8) == "fused_ring" and plan(1024, 16) == "fused_tmem"
    assert plan(8192, 64, 256) == "fused_tmem" and plan(8192, 64, 2048) == "fused_ring"   # the group's width counts, not N
    # very wide groups: two or three SM pairs that only rotate keep up, the others run the plain GEMM's loop
    wide = lambda n: ops.oft_plan(65536, n, 8192, reconn_sz=128, lib=lib)["path"]
    assert wide(28672) == "fused_ring_split" and wide(14336) == "fused_ring_split" and wide(7168) == "fused_ring" and wide(3584) == "fused_ring"
    assert ops.oft_plan(1024, 28672, 8192, reconn_sz=128, lib=lib)["path"] == "fused_ring"  # every row block fits the ring
    # ... and long tiles: K 1024 stays on the kernel in which every pair does both, K 2048 needs two pairs or fewer
    assert ops.oft_plan(32768, 28672, 1024, reconn_sz=64, lib=lib)["path"] == "fused_ring"
    assert ops.oft_plan(65536, 28672, 2048, reconn_sz=128, lib=lib)["path"] == "fused_ring_split"
    assert ops.oft_plan(262144, 12288, 2048, reconn_sz=64, lib=lib)["path"] == "fused_ring"
    assert ops.oft_plan(16384, 8192, 4096, group_size=2048, reconn_sz=64, lib=lib)["kernel_launches"] == 4  # one launch per group
    with ops.option("oft_route", 2, lib):
        assert plan(4096, 64) == "two_pass"
    with ops.option("oft_route", 1, lib):
        assert plan(4096, 64) == "fused_tmem"
    assert plan(4096, 64) == "fused_ring"
    with pytest.raises(ops.Error):
        ops.set_option("no_such_option", 1, lib)


@pytest.mark.parametrize("n,gs,b,world", [(1024, None, 32, 2), (2560, None, 64, 3), (1024, 256, 16, 2), (512, None, 64, 1)])
def test_sharded_entry_point_slabs_on_one_device(lib, cuda, n, gs, b, world):
    """b200_oft_tn_f16_sharded with every rank mapped to this GPU (its slabs then run one after the other): the
    slabs written side by side equal the unsharded product bit for bit."""
    import torch

    m, k = 384, 256
    A, R, B = make_oft_case(m, n, k, b, gs, seed=51)
    whole = run_oft(lib, cuda, A, R, B, m, n, k, b, gs, route=1)
    dA, dB, dR = (torch.from_numpy(x).to(cuda) for x in (A, B, R))
    dC = torch.full((m, n), -7.0, dtype=torch.float16, device=cuda)
    g_sz = n if gs is None else gs
    Bs, Rs, Cs = [], [], []
    for r in range(world):
        n0, n1 = ops.shard_range(n, g_sz, world, r, lib=lib)
        Bs.append(dB[n0:]); Cs.append(dC[:, n0:])
        Rs.append(dR[(n0 // g_sz) * b:] if gs is not None else dR)
    with ops.option("oft_route", 1, lib):
        ops.oft_tn_sharded(m, n, k, [0] * world, [dA] * world, k, Bs, k, Rs, k, Cs, n, group_size=gs, reconn_sz=b, lib=lib)
    assert ops.device_status(lib)[0] == 0
    assert np.array_equal(dC.cpu().numpy().view(np.uint16), whole.view(np.uint16))


def test_sharded_entry_point_on_two_devices(lib, cuda):
    """Two GPUs of this process, one call (skipped on a single-GPU box)."""
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    m, n, k, b = 512, 4096, 512, 64
    A, R, B = make_oft_case(m, n, k, b, seed=52, xdist="normal", wsigma=0.02)
    whole = run_oft(lib, cuda, A, R, B, m, n, k, b)
    parts = []
    As, Bs, Rs, Cs = [], [], [], []
    for r in range(2):
        dev = torch.device("cuda", r)
        n0, n1 = ops.shard_range(n, n, 2, r, lib=lib)
        As.append(torch.from_numpy(A).to(dev)); Bs.append(torch.from_numpy(B[n0:n1]).to(dev)); Rs.append(torch.from_numpy(R).to(dev))
        Cs.append(torch.empty((m, n1 - n0), dtype=torch.float16, device=dev))
    ops.oft_tn_sharded(m, n, k, [0, 1], As, k, Bs, k, Rs, k, Cs, n // 2, reconn_sz=b, lib=lib)
    for r in range(2):
        torch.cuda.synchronize(r)
    got = np.concatenate([c.cpu().numpy() for c in Cs], axis=1)
    torch.cuda.set_device(0)
    assert np.array_equal(got.view(np.uint16), whole.view(np.uint16))


@pytest.mark.parametrize("route", [3, 4])
def test_oft_ring_route_on_two_streams(lib, cuda, pair_build, route):
    """Two launches of a shared-X.R kernel (every pair does both jobs; rotation pairs of their own) queued on two streams with no synchronisation between them, repeatedly:
    each has its own ring and counters (stream-ordered from the library's pool) and is launched cooperatively, so
    both finish, no wait runs out, and both return the bits of a launch that ran alone."""
    import torch

    if not pair_build:
        pytest.skip("the shared-X.R kernel exists in the CTA-pair build only")
    m, n, k, b = 4608, 2304, 512, 64   # 18 row blocks (more than the ring of 16 holds) x 9 N tiles
    g = torch.Generator(device=cuda).manual_seed(78)
    dA = torch.randn((m, k), generator=g, device=cuda).to(torch.float16)
    dB = (torch.randn((n, k), generator=g, device=cuda) * 0.05).to(torch.float16)
    from cute_mma_b200 import inputs
    dR = torch.from_numpy(inputs.pack_r(inputs.blocks_qr(1, k // b, b, 78))).to(cuda)
    alone = torch.empty((m, n), dtype=torch.float16, device=cuda)
    with ops.option("oft_route", route, lib), ops.option("raster", 4, lib), ops.option("ring_bands", 2, lib):
        ops.oft_tn(m, n, k, dA, k, dB, k, dR, k, alone, n, reconn_sz=b, lib=lib)
        torch.cuda.synchronize()
        s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
        c1, c2 = torch.empty_like(alone), torch.empty_like(alone)
        for _ in range(4):
            ops.oft_tn(m, n, k, dA, k, dB, k, dR, k, c1, n, s1.cuda_stream, reconn_sz=b, lib=lib)
            ops.oft_tn(m, n, k, dA, k, dB, k, dR, k, c2, n, s2.cuda_stream, reconn_sz=b, lib=lib)
        torch.cuda.synchronize()
    assert ops.device_status(lib)[0] == 0
    assert torch.equal(c1, alone) and torch.equal(c2, alone)


@pytest.mark.parametrize("m,n,k,b,gs,pad", [(384, 2048, 256, 64, None, 8), (200, 2056, 192, 32, None, 8), (200, 2055, 192, 32, None, 3),
                                            (200, 2056, 192, 32, None, 9), (256, 512, 256, 64, None, 8), (256, 2048, 128, 128, 1024, 8),
                                            (2304, 5120, 256, 64, None, 8)])
def test_gather_entry_point_stores_every_destination(lib, cuda, pair_build, m, n, k, b, gs, pad):
    """b200_oft_tn_f16_gather with three destinations on this GPU (padded ldC, canaries): each holds the bits of the
    plain call, whether the shared-X.R kernel stores them from its epilogue (wide groups: whole 128-byte lines after
    a transpose in registers when ldC is even, ragged last column included; one row per lane when it is odd) or the
    library copies."""
    import torch

    A, R, B = make_oft_case(m, n, k, b, gs, seed=81)
    want = run_oft(lib, cuda, A, R, B, m, n, k, b, gs)
    dA, dB, dR = (torch.from_numpy(x).to(cuda) for x in (A, B, R))
    ldc = n + pad
    dsts = [torch.full((m + 1, ldc), -7.0, dtype=torch.float16, device=cuda) for _ in range(3)]
    ops.oft_tn_gather(m, n, k, dA, k, dB, k, dR, k, dsts, ldc, group_size=gs, reconn_sz=b, lib=lib)
    assert ops.device_status(lib)[0] == 0
    for d in dsts:
        out = d.cpu().numpy()
        assert np.array_equal(out[:m, :n].view(np.uint16), want.view(np.uint16))
        assert np.all(out[m] == np.float16(-7.0)) and np.all(out[:m, n:] == np.float16(-7.0))
    with pytest.raises(ops.Error):
        ops.oft_tn_gather(m, n, k, dA, k, dB, k, dR, k, dsts * 3, ldc, group_size=gs, reconn_sz=b, lib=lib)  # nine destinations
