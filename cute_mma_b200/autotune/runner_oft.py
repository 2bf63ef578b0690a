"""Builds and times every generated OFT configuration, one executable per configuration.

Follows the reference's autotune/runner_oft.py:21-95: a pool of GPUs handed out through
CUDA_VISIBLE_DEVICES, one benchmark process per free GPU (asyncio + semaphore), the bracketed number
parsed from the driver's stdout with the same regular expression, results checkpointed as the sweep
goes, finished keys skipped on restart, and suspiciously low results re-run with more iterations.
Differences: results are JSON lines (not a pickle holding raw bytes), and the problem shape and
block edge are flags (the library takes group_size / reconn_sz at run time).

    python -m cute_mma_b200.autotune.gen_oft_autotune_config --out autotune_configs --reconn_sz 64
    python -m cute_mma_b200.autotune.runner_oft --configs autotune_configs --ngpus 1 -m 16384 -n 4096 -k 4096 --reconn_sz 64
"""
from __future__ import annotations

import argparse
import asyncio
import json
import math
import os
import re

from .. import build as lib_build

NUMBER = re.compile(r"\[\d+\.\d{2}\]")  # the reference's pattern (runner_oft.py:32)


def get_flops(stdout: str) -> float:
    m = NUMBER.search(stdout)
    return float(m.group(0)[1:-1]) if m else math.nan


def load_results(path: str) -> dict:
    done = {}
    if os.path.exists(path):
        with open(path) as f:
            for line in f:
                line = line.strip()
                if line:
                    rec = json.loads(line)
                    done[rec["key"]] = rec  # a later record for the same key wins (re-runs)
    return done


def append_result(path: str, rec: dict) -> None:
    with open(path, "a") as f:
        f.write(json.dumps(rec) + "\n")
        f.flush()


def build_config(config_dir: str, build_root: str) -> str:
    """One library + one cute_oft_pc executable per configuration directory."""
    name = os.path.basename(os.path.normpath(config_dir))
    out_dir = os.path.join(build_root, name)
    os.makedirs(out_dir, exist_ok=True)
    lib = lib_build.build(config_dir=config_dir, out=os.path.join(out_dir, "libcute_mma_b200.so"))
    lib_build.build_cli(lib=lib, out_dir=out_dir)
    return os.path.join(out_dir, "cute_oft_pc")


async def run_one(key: str, exe: str, argv: list[str], gpus: list[int], sem: asyncio.Semaphore, timeout_s: float) -> dict:
    async with sem:
        gpu = gpus.pop()
        try:
            env = dict(os.environ, CUDA_VISIBLE_DEVICES=str(gpu))
            proc = await asyncio.create_subprocess_exec(exe, *argv, stdout=asyncio.subprocess.PIPE, stderr=asyncio.subprocess.PIPE, env=env)
            try:
                out, err = await asyncio.wait_for(proc.communicate(), timeout_s)
            except asyncio.TimeoutError:
                proc.kill()
                out, err = await proc.communicate()
                err += b"\n[runner] killed after timeout"
            out_s, err_s = out.decode(errors="replace"), err.decode(errors="replace")
            return {"key": key, "value": get_flops(out_s), "stdout": out_s[-2000:], "stderr": err_s[-2000:], "gpu": gpu, "argv": argv}
        finally:
            gpus.append(gpu)


async def sweep(exes: dict, argv: list[str], n_gpus: int, results_path: str, timeout_s: float) -> dict:
    done = load_results(results_path)
    todo = {k: e for k, e in exes.items() if k not in done}
    gpus = list(range(n_gpus))
    sem = asyncio.Semaphore(n_gpus)
    tasks = [asyncio.create_task(run_one(k, e, argv, gpus, sem, timeout_s)) for k, e in todo.items()]
    for fut in asyncio.as_completed(tasks):
        rec = await fut
        append_result(results_path, rec)  # every result is on disk as soon as it exists
        done[rec["key"]] = rec
    return done


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--configs", default="autotune_configs")
    ap.add_argument("--build", default="build_autotune")
    ap.add_argument("--results", default="results_oft.jsonl")
    ap.add_argument("--ngpus", type=int, default=1)
    ap.add_argument("--iter", type=int, default=100)
    ap.add_argument("-rt", "--rerun_threshold", type=float, default=50.0, help="results below this many TFLOP/s are run again with 100 iterations")
    ap.add_argument("-m", type=int, default=8192)
    ap.add_argument("-n", type=int, default=8192)
    ap.add_argument("-k", type=int, default=8192)
    ap.add_argument("--group_size", type=int, default=0)
    ap.add_argument("--reconn_sz", type=int, default=64)
    ap.add_argument("--timeout", type=float, default=300.0)
    a = ap.parse_args()

    dirs = sorted(d for d in os.listdir(a.configs) if d.startswith("config") and os.path.isdir(os.path.join(a.configs, d)) and d != "config_csvs")
    exes = {}
    for d in dirs:
        try:
            exes[f"autotune_{d}"] = build_config(os.path.join(a.configs, d), a.build)
        except RuntimeError as e:  # a configuration that does not compile is a data point, not a crash
            append_result(a.results, {"key": f"autotune_{d}", "value": math.nan, "stdout": "", "stderr": str(e)[-2000:]})
    shape = ["-m", str(a.m), "-n", str(a.n), "-k", str(a.k), "--group_size", str(a.group_size), "--reconn_sz", str(a.reconn_sz), "-rs", "1"]
    results = asyncio.run(sweep(exes, shape + ["-t", str(a.iter)], a.ngpus, a.results, a.timeout))
    low = {k: exes[k] for k, r in results.items() if k in exes and not (r["value"] >= a.rerun_threshold)}
    if low:
        kept = {k: r for k, r in load_results(a.results).items() if k not in low}
        with open(a.results, "w") as f:
            for r in kept.values():
                f.write(json.dumps(r) + "\n")
        results = asyncio.run(sweep(low, shape + ["-t", "100"], a.ngpus, a.results, a.timeout))
    best = sorted((r for r in load_results(a.results).values() if r["value"] == r["value"]), key=lambda r: -r["value"])
    for r in best[:5]:
        print(f"{r['key']:24s} {r['value']:8.2f} TFLOP/s")


if __name__ == "__main__":
    main()
