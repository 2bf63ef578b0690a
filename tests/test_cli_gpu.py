"""GPU: the C++ benchmark drivers, which reach the kernels through the header-only shim of the reference's templates
(oft_tn<CurrKernelParams>, gemm<TO, TR>), run as the autotune runners run them: correctness mode must report no
errors and the reference's own regular expressions (autotune/runner_oft.py:32, autotune/runner.py:23) must find the
throughput figure in the lines they print."""
import os
import re
import subprocess

import pytest

from cute_mma_b200 import build
from cute_mma_b200.autotune import runner, runner_oft

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def bin_dir(lib):
    build.build_cli()
    return build.BIN_DIR


def _run(exe, *args):
    res = subprocess.run([exe, *args], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    return res.stdout


def test_cute_oft_pc_default_problem_class_and_contract(bin_dir):
    """The reference's default problem class (group 256, 8 x 8 blocks, cute_oft_coop_pc.hpp:4-15) on a small problem."""
    out = _run(os.path.join(bin_dir, "cute_oft_pc"), "--correctness", "-m", "512", "-n", "512", "-k", "512", "-w", "2", "-t", "5", "-rs", "7")
    assert "Number of groups: 2" in out and "Number of blocks: 64" in out
    assert re.search(r"error count: 0, max error: ", out), out
    assert re.search(r"TFLOPS/s \(AR_W\): \[\d+\.\d{2}\], \(AR_W_sparse\): \d+\.\d{2}, \(A_RW\): \d+\.\d{2}, Time: \d+\.\d{3} ms", out), out
    assert runner_oft.get_flops(out) > 0


@pytest.mark.parametrize("extra", [("--group_size", "0", "--reconn_sz", "64", "-m", "1024", "-n", "2048", "-k", "512"),   # the shared-X.R route
                                   ("--group_size", "0", "--reconn_sz", "32", "-m", "512", "-n", "512", "-k", "256", "--mode", "A_RW"),
                                   ("--01init", "-m", "256", "-n", "512", "-k", "256")])
def test_cute_oft_pc_other_problem_classes(bin_dir, extra):
    out = _run(os.path.join(bin_dir, "cute_oft_pc"), "--correctness", "-w", "1", "-t", "3", "-rs", "11", *extra)
    assert re.search(r"error count: 0, max error: ", out), out
    assert runner_oft.get_flops(out) > 0


@pytest.mark.parametrize("exe,trans", [("gemm_half_half", ("T", "N")), ("gemm_half_half", ("N", "T")), ("gemm_float_float", ("N", "T")),
                                       ("gemm_float_float", ("T", "N")), ("gemm_half_half", ("t", "n"))])
def test_gemm_drivers_correct_and_parsed(bin_dir, exe, trans):
    out = _run(os.path.join(bin_dir, exe), "--correctness", "-m", "768", "-n", "512", "-k", "1024", "--transA", trans[0], "--transB", trans[1], "-t", "5")
    assert f"C = A^{trans[0]} B^{trans[1]}" in out
    assert re.search(r"error count: 0, max error: ", out), out
    m = runner.NUMBER.search(out)
    assert m and float(m.group(0)[1:-1]) > 0, out


def test_route_sweep_times_every_route(capsys):
    """The route comparison tool on a small shape: every route runs, the library's choice is named, the table prints."""
    from cute_mma_b200.autotune import route_sweep

    rows = route_sweep.sweep((2048, 2048, 512, 64), [0, 1, 2, 3, 4], 2, 1.0)
    assert [r["route"] for r in rows] == [0, 1, 2, 3, 4]
    assert rows[0]["name"] == "fused_ring" and rows[0]["ratio_to_choice"] == 1.0
    assert all(r["ms"] > 0 and r["tflops"] > 0 for r in rows)
    assert route_sweep.main(["256x512x128x32", "--routes", "0,1", "--rounds", "1", "--ms", "0.5"]) == 0
    out = capsys.readouterr().out
    assert "route 0 (fused_tmem)" in out and "route 1 fused_tmem" in out
