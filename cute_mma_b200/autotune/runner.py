"""Builds and times every generated plain-GEMM configuration (role of the reference's autotune/runner.py).

Same mechanics as runner_oft.py: one library + `gemm_<dtype>` executable per configuration directory,
one process per free GPU through CUDA_VISIBLE_DEVICES, the bracketed GFlop/s number parsed from
`CUTE_GEMM:     [%6.1f]GFlop/s` with the reference's expression (runner.py:23), JSON-lines results that
are skipped on restart.  The shape defaults to the reference's (-m 8192 -n 8192 -k 4096, runner.py:63).

    python -m cute_mma_b200.autotune.gen_autotune_config --out autotune_configs
    python -m cute_mma_b200.autotune.runner --configs autotune_configs --dtype half_half --layout TN --ngpus 1
"""
from __future__ import annotations

import argparse
import asyncio
import math
import os
import re

from .. import build as lib_build
from .runner_oft import append_result, load_results, run_one

NUMBER = re.compile(r"\[\s*\d+\.\d\]")


def get_flops(stdout: str) -> float:
    m = NUMBER.search(stdout)
    return float(m.group(0)[1:-1]) if m else math.nan


def build_config(config_dir: str, build_root: str, dtype: str) -> str:
    rel = os.path.join(*os.path.normpath(config_dir).split(os.sep)[-3:])
    out_dir = os.path.join(build_root, rel)
    os.makedirs(out_dir, exist_ok=True)
    lib = lib_build.build(config_dir=config_dir, out=os.path.join(out_dir, "libcute_mma_b200.so"))
    lib_build.build_cli(lib=lib, out_dir=out_dir)
    return os.path.join(out_dir, f"gemm_{dtype}")


async def sweep(exes: dict, argv: list[str], n_gpus: int, results_path: str, timeout_s: float) -> dict:
    done = load_results(results_path)
    gpus = list(range(n_gpus))
    sem = asyncio.Semaphore(n_gpus)
    tasks = [asyncio.create_task(run_one(k, e, argv, gpus, sem, timeout_s)) for k, e in exes.items() if k not in done]
    for fut in asyncio.as_completed(tasks):
        rec = await fut
        rec["value"] = get_flops(rec["stdout"])  # GFlop/s
        append_result(results_path, rec)
        done[rec["key"]] = rec
    return done


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--configs", default="autotune_configs")
    ap.add_argument("--build", default="build_autotune")
    ap.add_argument("--results", default="results_gemm.jsonl")
    ap.add_argument("--dtype", default="half_half", choices=["half_half", "float_float", "all"])
    ap.add_argument("--layout", default="TN", choices=["TN", "NT", "all"])
    ap.add_argument("--ngpus", type=int, default=1)
    ap.add_argument("-m", type=int, default=8192)
    ap.add_argument("-n", type=int, default=8192)
    ap.add_argument("-k", type=int, default=4096)
    ap.add_argument("--iter", type=int, default=100)
    ap.add_argument("--timeout", type=float, default=300.0)
    a = ap.parse_args()
    dtypes = ["half_half", "float_float"] if a.dtype == "all" else [a.dtype]
    layouts = ["TN", "NT"] if a.layout == "all" else [a.layout]
    for dtype in dtypes:
        for layout in layouts:
            root = os.path.join(a.configs, dtype, layout)
            exes = {}
            for d in sorted(os.listdir(root)):
                try:
                    exes[f"{dtype}/{layout}/{d}"] = build_config(os.path.join(root, d), a.build, dtype)
                except RuntimeError as e:
                    append_result(a.results, {"key": f"{dtype}/{layout}/{d}", "value": math.nan, "stdout": "", "stderr": str(e)[-2000:]})
            argv = ["-m", str(a.m), "-n", str(a.n), "-k", str(a.k), "--transA", layout[0], "--transB", layout[1], "-t", str(a.iter)]
            results = asyncio.run(sweep(exes, argv, a.ngpus, a.results, a.timeout))
            best = sorted((r for k, r in results.items() if k.startswith(f"{dtype}/{layout}/") and r["value"] == r["value"]), key=lambda r: -r["value"])
            for r in best[:3]:
                print(f"{r['key']:40s} {r['value'] / 1000:8.1f} TFLOP/s")


if __name__ == "__main__":
    main()
