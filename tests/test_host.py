"""CPU: host-side logic of the library - exported symbols, argument validation (which returns before
any CUDA call), tile order, shard arithmetic, input builders.  No compute call is made."""
import ctypes
import os
import re

import numpy as np
import pytest

from cute_mma_b200 import inputs, ops

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(lib):
    header = open(os.path.join(ROOT, "include", "cute_mma_b200.h")).read()
    declared = set(re.findall(r"\b(b200_\w+)\s*\(", header))
    assert declared == set(ops.SYMBOLS), declared ^ set(ops.SYMBOLS)
    for name in declared:
        assert hasattr(lib, name), name


def test_kernel_info_matches_config_headers(lib):
    info = ops.kernel_info(lib)
    cfg = open(os.path.join(ROOT, "cute_mma_b200", "configs", "default", "oft_config.hpp")).read()
    for key in ("bM", "bN", "bK", "bP1", "bP2"):
        want = int(re.search(rf"\b{key}\s*=\s*(\d+)", cfg).group(1))
        assert info["oft"][key] == want
    assert info["oft"]["b64"]["tmem_cols"] <= 512 and info["oft"]["b128"]["tmem_cols"] <= 512
    assert info["oft"]["b128"]["smem"] <= 232448
    ring = info["oft_ring"]   # the shared-X.R kernel: 5 stages of 32 KB, 2 of {X, R}, 16 KB staging, barriers, alignment slack
    for b, r_half in ((64, 4096), (128, 8192)):
        assert ring[f"b{b}"]["smem"] == 5 * 32768 + 2 * (16384 + r_half) + 16384 + (2 * 2 + 2 * 5 + 2 * ring[f"b{b}"]["rotation_bufs"] + 2) * 8 + 64 + 1024
        assert ring[f"b{b}"]["smem"] <= 232448 and 256 + ring[f"b{b}"]["rotation_bufs"] * max(b, 64) <= 512
    split = info["oft_ring_split"]  # product pairs: 6 stages of 32 KB, 2 accumulators; rotation pairs: {X, R} stages + 8 staging buffers of 4 KB
    assert split["stages_xr_w"] == 6 and split["accumulators"] == 2 and split["threads"] == 192
    for b, r_half in ((64, 4096), (128, 8192)):
        s1 = split[f"b{b}"]["stages_x_r"]
        data = max(6 * 32768, s1 * (16384 + r_half) + 8 * 4096)
        assert split[f"b{b}"]["smem"] == data + (2 * 6 + 2 * 2 + 2 * s1 + 2 * split["rotation_bufs"]) * 8 + 64 + 1024 <= 232448
        assert split["rotation_bufs"] * max(b, 64) <= 512 and s1 >= 2 * max(b, 64) // 64


def test_argument_validation_without_a_gpu(lib):
    """Shape errors are reported by status code before the library touches CUDA."""
    buf = (ctypes.c_uint16 * 64)()
    p = ctypes.addressof(buf)

    def oft(m, n, k, gs, b, A=p, B=p, R=p, C=p, ldA=None, ldC=None):
        return lib.b200_oft_tn_f16(m, n, k, gs, b, A, ldA or k, B, k, R, k, C, ldC or n, None)

    assert oft(-1, 8, 8, 8, 8) == ops.EINVAL
    assert oft(8, 8, 12, 8, 8) == ops.EINVAL and b"multiple of reconn_sz" in lib.b200_last_error()
    assert oft(8, 12, 16, 8, 8) == ops.EINVAL and b"group_size" in lib.b200_last_error()
    assert oft(8, 8, 16, 8, 0) == ops.EINVAL
    assert oft(8, 8, 16, 8, 8, C=None) == ops.EINVAL
    assert oft(8, 8, 16, 8, 8, ldC=4) == ops.EINVAL
    assert oft(0, 8, 16, 8, 8) == ops.OK and lib.b200_last_error() == b""   # empty problem: nothing to do
    assert lib.b200_gemm_tn_f16(8, 8, 8, p, 8, p, 8, p, 4, None) == ops.EINVAL  # ldC < m (column-major C)
    assert lib.b200_gemm(b"N", b"N", 0, 8, 8, 8, p, 8, p, 8, p, 8, None) == ops.EUNSUPPORTED
    with pytest.raises(ops.Error) as e:
        ops.gemm("T", "T", 8, 8, 8, p, 8, p, 8, p, 8, lib=lib)
    assert e.value.code == ops.EUNSUPPORTED and "('T','N')" in e.value.message


def test_new_entry_points_validate_before_any_cuda_call(lib):
    """b200_gemm_ex, b200_oft_tn_f16_sharded and the option calls reject bad arguments by status code without a GPU."""
    buf = (ctypes.c_uint16 * 64)()
    p = ctypes.addressof(buf)
    assert lib.b200_gemm_ex(b"N", b"N", 0, 0, 8, 8, 8, 1.0, p, 8, p, 8, 0.0, p, 8, None) == ops.EUNSUPPORTED   # only TN and NT exist
    assert lib.b200_gemm_ex(b"T", b"N", 2, 0, 8, 8, 8, 1.0, p, 8, p, 8, 0.0, p, 8, None) == ops.EUNSUPPORTED   # float operands, half result
    assert b"f16 -> f32" in lib.b200_last_error()
    assert lib.b200_gemm_ex(b"T", b"N", 0, 1, -1, 8, 8, 1.0, p, 8, p, 8, 0.0, p, 8, None) == ops.EINVAL
    devs = (ctypes.c_int * 1)(0)
    ptrs = (ctypes.c_void_p * 1)(p)
    assert lib.b200_oft_tn_f16_sharded(8, 16, 16, 16, 16, 0, devs, ptrs, 16, ptrs, 16, ptrs, 16, ptrs, 16, None) == ops.EINVAL  # world = 0
    assert lib.b200_oft_tn_f16_sharded(8, 16, 16, 5, 16, 1, devs, ptrs, 16, ptrs, 16, ptrs, 16, ptrs, 16, None) == ops.EINVAL  # n % group_size
    assert lib.b200_oft_tn_f16_sharded(8, 16, 16, 16, 16, 1, devs, None, 16, ptrs, 16, ptrs, 16, ptrs, 16, None) == ops.EINVAL
    with pytest.raises(ops.Error):
        ops.set_option("no_such_option", 1, lib)
    for name in ("oft_route", "raster", "tile_sync", "l2_hints", "gemm_tile_sync", "gemm_l2_hints", "gemm_split", "maps_3d", "ring_bands", "prefetch", "rot_pairs"):
        old = ops.get_option(name, lib)
        with ops.option(name, 3, lib):
            assert ops.get_option(name, lib) == 3
        assert ops.get_option(name, lib) == old


def test_rotation_shares_cover_every_unit_once():
    """The split of the rotation units among the SM pairs of the shared-X.R kernel (a contiguous share of every band per
    pair, bands in tile order), restated here: every (row block, unit) exactly once, shares differ by at most one
    unit per band, and a pair's units come in non-decreasing row-block order."""
    def shares(raster, tiles_m, upb, pairs):
        out = []
        for p in range(pairs):
            mine = []
            band = 0
            while band * raster < tiles_m:
                rows = min(raster, tiles_m - band * raster)
                u = rows * upb
                for j in range(p * u // pairs, (p + 1) * u // pairs):
                    mine.append((band * raster + j // upb, j % upb))
                band += 1
            out.append(mine)
        return out

    for raster, tiles_m, upb, pairs in ((4, 64, 64, 74), (8, 256, 64, 74), (8, 3, 5, 74), (2, 41, 5, 74), (4, 18, 8, 37), (1, 7, 129, 74)):
        sh = shares(raster, tiles_m, upb, pairs)
        flat = [u for mine in sh for u in mine]
        assert sorted(flat) == [(tm, ku) for tm in range(tiles_m) for ku in range(upb)]
        for mine in sh:
            assert [tm for tm, _ in mine] == sorted(tm for tm, _ in mine)
        full = tiles_m // raster
        counts = [len(m_) for m_ in sh]
        assert max(counts) - min(counts) <= full + (1 if tiles_m % raster else 0)


def test_missing_library_fails_loudly(tmp_path):
    with pytest.raises(FileNotFoundError):
        ops.load_library(str(tmp_path / "nope.so"))


# ---- tile order -------------------------------------------------------------------------------------


def z_curve_restated(grid, idx):
    """Independent restatement of z_curve (z_curve.hpp:4-49) for a 2-D grid."""

    def spf(n):
        if n == 1:
            return 1, 1
        for p in (2, 3, 5, 7):
            if n % p == 0:
                return n // p, p
        i = 11
        while i * i <= n:
            if n % i == 0:
                return n // i, i
            i += 1
        return 1, n

    sizes = [spf(g) for g in grid]
    coord, layer = [0, 0], [1, 1]
    while any(s[1] != 1 for s in sizes):
        ps = [s[1] for s in sizes]
        level = idx % (ps[0] * ps[1])
        idx //= ps[0] * ps[1]
        li = (level % ps[0], (level // ps[0]) % ps[1])
        for d in range(2):
            coord[d] += li[d] * layer[d]
            layer[d] *= ps[d]
        sizes = [spf(s[0]) for s in sizes]
    return tuple(coord)


@pytest.mark.parametrize("grid", [(12, 15), (128, 16), (1, 7), (7, 1), (13, 11), (512, 112), (6, 35), (1, 1), (121, 3)])
def test_tile_order_is_a_bijection_and_matches_z_curve(lib, grid):
    tm, tn = grid
    seen = set()
    for idx in range(tm * tn):
        c = ops.tile_coord(tm, tn, idx, lib=lib)
        assert c == z_curve_restated(grid, idx), (grid, idx)
        assert 0 <= c[0] < tm and 0 <= c[1] < tn
        seen.add(c)
    assert len(seen) == tm * tn
    with pytest.raises(ops.Error):
        ops.tile_coord(tm, tn, tm * tn, lib=lib)


def test_tile_order_is_morton_on_power_of_two_grids(lib):
    for idx in range(64):
        m = sum(((idx >> (2 * i)) & 1) << i for i in range(3))
        n = sum(((idx >> (2 * i + 1)) & 1) << i for i in range(3))
        assert ops.tile_coord(8, 8, idx, lib=lib) == (m, n)


# ---- shard arithmetic -----------------------------------------------------------------------------------


@pytest.mark.parametrize("n,gs,world", [(28672, 28672, 8), (28672, 28672, 4), (4096, 4096, 2), (1000, 1000, 4), (1024, 256, 3), (512, 64, 8), (256, 256, 4)])
def test_shard_ranges_partition_n(lib, n, gs, world):
    ranges = [ops.shard_range(n, gs, world, r, lib=lib) for r in range(world)]
    assert ranges[0][0] == 0 and ranges[-1][1] == n
    for (a0, a1), (b0, b1) in zip(ranges, ranges[1:]):
        assert a1 == b0 and a0 <= a1
    unit = gs if gs < n else 256
    for a0, a1 in ranges:
        assert a0 % unit == 0 or a0 == n
    sizes = [b - a for a, b in ranges]
    assert max(sizes) - min(sizes) <= unit


def test_large_configuration_splits_into_whole_tiles(lib):
    for world in (1, 2, 4, 8):
        for r in range(world):
            a, b = ops.shard_range(28672, 28672, world, r, lib=lib)
            assert (b - a) == 28672 // world and (b - a) % 256 == 0


# ---- input builders ---------------------------------------------------------------------------------------


@pytest.mark.parametrize("builder", [inputs.blocks_qr, inputs.blocks_cayley, inputs.blocks_permutation])
def test_blocks_are_orthogonal_and_seeded(builder):
    a = builder(2, 3, 16, 5)
    b = builder(2, 3, 16, 5)
    assert np.array_equal(a, b)
    for blk in a.reshape(-1, 16, 16):
        assert np.allclose(blk @ blk.T, np.eye(16), atol=1e-10)
    assert not np.array_equal(a, builder(2, 3, 16, 6))


def test_cayley_blocks_are_near_identity():
    blk = inputs.blocks_cayley(1, 1, 64, 0, sigma=0.01)[0, 0]
    assert np.abs(blk - np.eye(64)).max() < 0.2 and np.linalg.det(blk) > 0.99


def test_pack_r_transposes_each_block():
    blocks = np.arange(2 * 3 * 4 * 4, dtype=np.float64).reshape(2, 3, 4, 4)
    stored = inputs.pack_r(blocks, dtype=np.float64)
    assert stored.shape == (8, 12)
    for g in range(2):
        for kb in range(3):
            assert np.array_equal(stored[g * 4:(g + 1) * 4, kb * 4:(kb + 1) * 4], blocks[g, kb].T)
    assert np.array_equal(inputs.unpack_r(stored, 4), blocks)


def test_flop_accounting_matches_reference_formula():
    # cute_oft_pc.cu:362-367: base 2MNK, AR_W extra 2*G*M*K*b
    assert inputs.oft_flops(16384, 4096, 4096, 64) == 2 * 16384 * 4096 * 4096 + 2 * 16384 * 4096 * 64
    assert inputs.oft_flops(8, 8, 8, 2, n_groups=4) == 2 * 8 * 8 * 8 + 2 * 4 * 8 * 8 * 2
