"""CPU: autotune generator and runner plumbing (no GPU, no nvcc: executables are faked)."""
import asyncio
import json
import math
import os
import stat

from cute_mma_b200.autotune import gen_oft_autotune_config as gen
from cute_mma_b200.autotune import runner_oft


def test_generator_writes_complete_include_dirs(tmp_path):
    rows = gen.generate(str(tmp_path), b=64)
    assert len(rows) >= 20
    for r in rows:
        d = tmp_path / r["config"]
        text = (d / "oft_config.hpp").read_text()
        assert f"bN = {r['bN']};" in text and f"bP1 = {r['bP1']};" in text and f"bP2 = {r['bP2']};" in text and f"ctas = {r['ctas']};" in text
        assert (d / "gemm_config.hpp").exists()
        assert r["smem"] <= gen.SMEM_LIMIT
    assert (tmp_path / "config_csvs" / "param.csv").read_text().startswith("config,ctas,bN,bP1,bP2,smem")
    # the larger R tile of b = 128 rules out more candidates, and needs two XR buffers in tensor memory
    assert len(list(gen.candidates(128))) < len(rows)
    assert all((512 - c["bN"]) // 128 >= 2 for c in gen.candidates(128))


def test_smem_formula_matches_the_library(lib):
    from cute_mma_b200 import ops

    info = ops.kernel_info(lib)["oft"]
    assert gen.smem_bytes(info["bN"], info["bP1"], info["bP2"], 64, info["ctas"]) == info["b64"]["smem"]
    assert gen.smem_bytes(info["bN"], info["bP1"], info["bP2"], 128, info["ctas"]) == info["b128"]["smem"]


def test_stdout_contract_is_parsed_like_the_reference():
    line = "TFLOPS/s (AR_W): [1012.34], (AR_W_sparse): 1990.10, (A_RW): 998.20, Time: 0.551 ms\n"
    assert runner_oft.get_flops("M = 4096\n" + line) == 1012.34
    assert math.isnan(runner_oft.get_flops("CUDA call failed with status 1"))


def _fake_exe(path, body):
    path.write_text("#!/bin/sh\n" + body)
    path.chmod(path.stat().st_mode | stat.S_IEXEC)
    return str(path)


def test_sweep_checkpoints_and_resumes(tmp_path):
    good = _fake_exe(tmp_path / "good", 'echo "gpu=$CUDA_VISIBLE_DEVICES"; echo "TFLOPS/s (AR_W): [123.45], x"\n')
    bad = _fake_exe(tmp_path / "bad", 'echo "launch failed" 1>&2; exit 1\n')
    results = str(tmp_path / "r.jsonl")
    out = asyncio.run(runner_oft.sweep({"a": good, "b": bad}, ["-t", "1"], 2, results, 30.0))
    assert out["a"]["value"] == 123.45 and math.isnan(out["b"]["value"]) and "launch failed" in out["b"]["stderr"]
    assert "gpu=" in out["a"]["stdout"]
    lines = [json.loads(x) for x in open(results)]
    assert {r["key"] for r in lines} == {"a", "b"}
    # restart: finished keys are skipped, only the new one runs
    marker = tmp_path / "ran_again"
    good2 = _fake_exe(tmp_path / "good2", f'touch {marker}; echo "[1.00]"\n')
    out2 = asyncio.run(runner_oft.sweep({"a": good2, "c": good}, ["-t", "1"], 1, results, 30.0))
    assert not marker.exists() and out2["a"]["value"] == 123.45 and out2["c"]["value"] == 123.45


def test_gemm_generator_writes_all_specialisations(tmp_path):
    from cute_mma_b200.autotune import gen_autotune_config as gg

    counts = gg.generate(str(tmp_path))
    assert set(counts) == set(gg.KEYS) and all(n >= 20 for n in counts.values())
    text = (tmp_path / "float_float" / "NT" / "config0" / "gemm_config.hpp").read_text()
    assert text.count("template <> struct Params<") == 4 and "MMA_N, MMA_T" in text
    assert (tmp_path / "float_float" / "NT" / "config0" / "oft_config.hpp").exists()
    assert (tmp_path / "config_csvs" / "half_half_TN_param.csv").read_text().startswith("id,ctas,bN,bP,smem")
    for c in gg.candidates():
        assert gg.smem_bytes(**c) <= gg.SMEM_LIMIT
    assert {"ctas": 2, "bN": 256, "bP": 6} in list(gg.candidates())       # the shipped default is in the space
    assert {"ctas": 1, "bN": 256, "bP": 5} not in list(gg.candidates())   # 5 x 48 KB does not fit


def test_gemm_stdout_contract_is_parsed_like_the_reference():
    from cute_mma_b200.autotune import runner

    assert runner.get_flops("CUTE_GEMM:     [1234567.8]GFlop/s  (0.7440)ms") == 1234567.8
    assert runner.get_flops("CUTE_GEMM:     [ 912.5]GFlop/s  (0.1000)ms") == 912.5
    assert math.isnan(runner.get_flops("cute_mma_b200 call failed with status 3"))


def test_route_sweep_shape_arguments():
    import argparse

    import pytest

    from cute_mma_b200.autotune import route_sweep

    assert route_sweep.parse_shape("16384x4096x4096x64") == (16384, 4096, 4096, 64)
    for bad in ("16384x4096x4096", "0x4096x4096x64", "256x256x100x64"):
        with pytest.raises(argparse.ArgumentTypeError):
            route_sweep.parse_shape(bad)
