"""Build recipe of the CUDA library (nvcc, sm_100a only).  No JIT cache: the .so is written in-tree.

    python -m cute_mma_b200.build [--config-dir DIR] [--out PATH] [--verbose]

``--config-dir`` names the directory that holds gemm_config.hpp and oft_config.hpp (tile
hyperparameters are compile-time, one library per configuration, like the reference's one
executable per autotune configuration, CMakeLists.txt:54-67).
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
DEFAULT_CONFIG = os.path.join(PKG, "configs", "default")
DEFAULT_OUT = os.path.join(PKG, "libcute_mma_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-lineinfo",
    "-Xcompiler", "-fPIC", "-shared", "--expt-relaxed-constexpr",
]


def nvcc_path() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise FileNotFoundError("nvcc not found")


def sources() -> list[str]:
    return [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith(".cu")]


def _stale(out: str, config_dir: str) -> bool:
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(config_dir, f) for f in os.listdir(config_dir)]
    deps.append(os.path.join(PKG, "..", "include", "cute_mma_b200.h"))
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(config_dir: str = DEFAULT_CONFIG, out: str = DEFAULT_OUT, verbose: bool = False, force: bool = False,
          defines: list[str] | None = None) -> str:
    if not force and not _stale(out, config_dir):
        return out
    cmd = [nvcc_path(), *NVCC_FLAGS, f"-I{config_dir}", f"-I{CSRC}", *(defines or [])]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += sources() + ["-o", out, "-lcudart"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed: " + " ".join(cmd))
    return out


CLI_DIR = os.path.join(PKG, "cli")
BIN_DIR = os.path.join(PKG, "bin")
# executable -> (source, extra defines); names follow the reference's targets (README.md:18-21, CMakeLists.txt:69-80)
CLI_TARGETS = {
    "cute_oft_pc": ("cute_oft_pc.cu", []),
    "gemm_half_half": ("gemm_bench.cu", []),
    "gemm_float_float": ("gemm_bench.cu", ["-DGEMM_FLOAT"]),
}


def build_cli(lib: str = DEFAULT_OUT, defines: list[str] | None = None, out_dir: str = BIN_DIR, force: bool = False) -> list[str]:
    """Builds the C++ benchmark drivers against the library (found at run time through an rpath)."""
    os.makedirs(out_dir, exist_ok=True)
    outs = []
    lib_dir, lib_name = os.path.dirname(os.path.abspath(lib)), os.path.basename(lib)
    for exe, (src, defs) in CLI_TARGETS.items():
        out = os.path.join(out_dir, exe)
        src_path = os.path.join(CLI_DIR, src)
        deps = [src_path, os.path.join(CLI_DIR, "flags.hpp"), lib] + [os.path.join(PKG, "shim", f) for f in os.listdir(os.path.join(PKG, "shim"))]
        if not force and os.path.exists(out) and all(os.path.getmtime(d) <= os.path.getmtime(out) for d in deps):
            outs.append(out)
            continue
        cmd = [nvcc_path(), "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-lineinfo", *defs, *(defines or []),
               src_path, "-o", out, f"-L{lib_dir}", f"-l:{lib_name}", "-Xlinker", f"-rpath={lib_dir}", "-lcudart"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("nvcc failed: " + " ".join(cmd))
        outs.append(out)
    return outs


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--config-dir", default=DEFAULT_CONFIG)
    ap.add_argument("--out", default=DEFAULT_OUT)
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--force", action="store_true")
    ap.add_argument("-D", dest="defines", action="append", default=[], help="extra macro, e.g. -D B200_PROFILE_WAITS")
    a = ap.parse_args()
    print(build(a.config_dir, a.out, a.verbose, a.force, [f"-D{d}" for d in a.defines]))
