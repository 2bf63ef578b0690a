#!/usr/bin/env python
"""Benchmark of the fused OFT GEMM  Y = (X.R).W  on 1..8 B200s of one node.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...     # the reference's CPU routine on the host cores

One "step" is one pass of the fused product over the whole synthetic problem.  The default workload is
the large N-sharded configuration (X [65536, 8192] ~ N(0,1), W [8192, 28672] ~ N(0,0.02), R = 64
orthogonal 128x128 blocks); with N GPUs rank r owns a column slab of W and Y, X and R are replicated,
and there is no collective in the compute (strong scaling: total work is fixed).  FLOPs are counted
as 2MKN + 2MKb at every GPU count (replicated X.R work is not credited).  Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (M, K, N, b, R builder, sigma of W)
    "oft_large_m65536_k8192_n28672_b128": (65536, 8192, 28672, 128, "qr", 0.02),
    "oft_proj_m16384_k4096_n4096_b64": (16384, 4096, 4096, 64, "cayley", 0.02),
}
DEFAULT_WORKLOAD = "oft_large_m65536_k8192_n28672_b128"
METRIC = "oft_fused_gemm_tflops"
NOMINAL_FP16_TFLOPS = 2250.0  # vendor dense fp16 figure, context only

# DRAM bytes of one launch of the dominant kernel, from the ncu captures summarised under profiles/
# (dram__bytes_read.sum + dram__bytes_write.sum), keyed by workload and by the route the library takes;
# None until a capture exists.
NCU_TRAFFIC_BYTES = {
    # fused kernel, per launch at N = 1, one-pass counters on the full workload: read 29.2 GB + write 5.7 GB
    # against 5.3 GB algorithmic (every wave of 74 tiles re-reads its panels of X and W once)
    ("oft_large_m65536_k8192_n28672_b128", "fused"): 34.94e9,
    # two-pass route, GEMM pass (gemm2_kernel), same one-pass counters: read 17.86 GB + write 3.72 GB against
    # 5.3 GB algorithmic (28.05 GB read before the band operand was loaded evict-last and the streaming one
    # evict-first); the rotation pass before it moves 1.08 + 1.03 GB, its algorithmic bytes
    ("oft_large_m65536_k8192_n28672_b128", "two_pass"): 21.58e9,
    # ncu --set full capture of the same shape (read 363 MB + write 154 MB; algorithmic 303 MB)
    ("oft_proj_m16384_k4096_n4096_b64", "fused"): 517.2e6,
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"bf16_burst": float(p["bf16_tflops"]), "bf16_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "hbm_gbs": float(p["hbm_gbs"]), "source": "measured"}
    return {"bf16_burst": 1590.0, "bf16_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


def flops_of(m, k, n, b):
    return 2.0 * m * k * n + 2.0 * m * k * b


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.out = None

    def start(self):
        try:
            self.out = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "20"], stdout=self.out, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.out.flush()
        self.out.seek(0)
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.out.read().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for nm, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        self.out.close()
        os.unlink(self.out.name)
        sm.sort()
        # the busiest half of the samples: the sampler also sees the idle moments around the region
        busy = sm[len(sm) // 2:] if sm else []
        med = busy[len(busy) // 2] if busy else None
        return {"sm_mhz": med, "sm_max_mhz": (max(mx) if mx else None), "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------------------- CPU arm


def cpu_reference_rate(m, k, n, b, kind, seconds: float, seed: int = 0):
    """Times the reference's CPU routine (oracle/_ref when built, else the plain-C port) on a bounded
    sample of the workload: `rows` rows of X against `cols` columns of W, all K, all R.  An output
    element depends only on its row of X, on R and on its column of W, so the sample is exact work of
    the full problem.  The unmodified reference routine is single-threaded; it is run on disjoint row
    samples from one Python thread per host core (ctypes releases the GIL).  Returns a dict."""
    import numpy as np

    from cute_mma_b200 import inputs
    from oracle import oracle

    use_ref = oracle.have_reference()
    cores = os.cpu_count() or 1
    cols = min(n, 1792)
    rng = np.random.default_rng(seed)
    R = inputs.pack_r(inputs.blocks_qr(1, k // b, b, seed) if kind == "qr" else inputs.blocks_cayley(1, k // b, b, seed))
    Bs = (rng.standard_normal((cols, k)) * 0.02).astype(np.float16)

    def run(rows_per_thread: int) -> float:
        As = [rng.standard_normal((rows_per_thread, k)).astype(np.float16) for _ in range(cores)]

        def work(i):
            if use_ref:
                oracle.ref_cpu_oft_tn(As[i], R, Bs, rows_per_thread, cols, 1, k, b)
            else:
                oracle.cpu_oft_tn(As[i], R, Bs, rows_per_thread, cols, 1, k, b, threads=1)

        ts = [threading.Thread(target=work, args=(i,)) for i in range(cores)]
        t0 = time.perf_counter()
        for t in ts:
            t.start()
        for t in ts:
            t.join()
        return time.perf_counter() - t0

    probe_rows = 2
    t_probe = run(probe_rows)
    rows = max(probe_rows, min(4096, int(probe_rows * seconds / max(t_probe, 1e-3))))
    t = run(rows)
    fl = flops_of(rows * cores, k, cols, b)
    return {"value": fl / t * 1e-12, "unit": "TFLOP/s", "cores": cores, "kind": "reference" if use_ref else "port",
            "sample": f"{rows * cores} of {m} rows x {cols} of {n} columns, all K, {cores} threads x {rows} rows, {t:.1f} s",
            "seconds": t}


def run_reference_arm(args, workload):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    m, k, n, b, kind, _ = WORKLOADS[workload]
    per_step = 4.0
    for _ in range(args.warmup):
        cpu_reference_rate(m, k, n, b, kind, per_step / 4)
    vals, secs = [], []
    info = None
    for _ in range(args.steps):
        info = cpu_reference_rate(m, k, n, b, kind, per_step)
        vals.append(info["value"])
        secs.append(info["seconds"])
    value = sum(vals) / len(vals)
    full_ms = flops_of(m, k, n, b) / (value * 1e12) * 1e3
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": full_ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": {"workload": workload, "note": "ms_per_step extrapolates the sampled rate to the full problem"},
            "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": info["cores"], "kind": info["kind"], "sample": info["sample"]},
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    emit(line)


# --------------------------------------------------------------------------------------- GPU arm


def projection_shape_rate(lib, dev, stream):
    """Device-timed rate of the single-GPU projection shape (M 16384, K = N 4096, b 64, Cayley blocks),
    reported beside the headline workload at N = 1: 50 launches after 5 warm-up launches."""
    import torch

    from cute_mma_b200 import inputs, ops

    name = "oft_proj_m16384_k4096_n4096_b64"
    m, k, n, b, _, wsigma = WORKLOADS[name]
    g = torch.Generator(device=dev).manual_seed(99)
    dX = torch.randn((m, k), generator=g, device=dev, dtype=torch.float32).to(torch.float16)
    dW = (torch.randn((n, k), generator=g, device=dev, dtype=torch.float32) * wsigma).to(torch.float16)
    dR = torch.from_numpy(inputs.pack_r(inputs.blocks_cayley(1, k // b, b, 7))).to(dev)
    dY = torch.empty((m, n), dtype=torch.float16, device=dev)
    for _ in range(5):
        ops.oft_tn(m, n, k, dX, k, dW, k, dR, k, dY, n, stream, reconn_sz=b, lib=lib)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(50):
        ops.oft_tn(m, n, k, dX, k, dW, k, dR, k, dY, n, stream, reconn_sz=b, lib=lib)
    e1.record(stream)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 50
    assert ops.device_status(lib)[0] == 0
    os.environ["B200_OFT_PATH"] = "1"  # the fused kernel on the same shape
    try:
        for _ in range(5):
            ops.oft_tn(m, n, k, dX, k, dW, k, dR, k, dY, n, stream, reconn_sz=b, lib=lib)
        torch.cuda.synchronize()
        e0.record(stream)
        for _ in range(50):
            ops.oft_tn(m, n, k, dX, k, dW, k, dR, k, dY, n, stream, reconn_sz=b, lib=lib)
        e1.record(stream)
        torch.cuda.synchronize()
        ms_fused = e0.elapsed_time(e1) / 50
    finally:
        del os.environ["B200_OFT_PATH"]
    assert ops.device_status(lib)[0] == 0
    tf = flops_of(m, k, n, b) / (ms * 1e-3) * 1e-12
    peaks = measured_peaks()
    return {"workload": name, "value": tf, "unit": "TFLOP/s", "ms_per_step": ms, "steps": 50, "route": ops.oft_plan(m, n, k, reconn_sz=b, lib=lib)["path"],
            "fused_route": {"ms_per_step": ms_fused, "value": flops_of(m, k, n, b) / (ms_fused * 1e-3) * 1e-12, "unit": "TFLOP/s"},
            "frac_of_measured_bf16_burst": tf / peaks["bf16_burst"], "frac_of_nominal_fp16": tf / NOMINAL_FP16_TFLOPS}



def run_gpu_arm(args, workload):
    import numpy as np
    import torch
    import torch.distributed as dist

    from cute_mma_b200 import inputs, ops, sharded

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch N>1 with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    lib = ops.load_library()  # raises if the CUDA library is missing: there is no fallback

    m, k, n, b, kind, wsigma = WORKLOADS[workload]
    n0, n1 = sharded.my_slab(n, n, world, rank, lib=lib)
    n_loc = n1 - n0
    g = torch.Generator(device=dev).manual_seed(1234)             # X identical on every rank
    dX = torch.randn((m, k), generator=g, device=dev, dtype=torch.float32).to(torch.float16)
    gw = torch.Generator(device=dev).manual_seed(4321 + rank)     # this rank's slab of W^T
    dW = (torch.randn((n_loc, k), generator=gw, device=dev, dtype=torch.float32) * wsigma).to(torch.float16)
    blocks = inputs.blocks_qr(1, k // b, b, 7) if kind == "qr" else inputs.blocks_cayley(1, k // b, b, 7)
    R = inputs.pack_r(blocks)
    dR = torch.from_numpy(R).to(dev)
    dY = torch.empty((m, n_loc), dtype=torch.float16, device=dev)
    stream = torch.cuda.current_stream()

    def step():
        sharded.oft_tn_slab(m, n, k, dX, k, dW, k, dR, k, dY, n_loc, n0, n1, stream, reconn_sz=b, lib=lib)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    st = ops.device_status(lib)
    sampler = ClockSampler(local_rank if "CUDA_VISIBLE_DEVICES" not in os.environ else int(os.environ["CUDA_VISIBLE_DEVICES"].split(",")[local_rank]))
    if rank == 0:
        sampler.start()
        time.sleep(0.15)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    barrier()
    ms_local = e0.elapsed_time(e1) / args.steps
    clocks = sampler.stop() if rank == 0 else None
    st = ops.device_status(lib)
    assert st[0] == 0, st
    t = torch.tensor([ms_local], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    total_flops = flops_of(m, k, n, b)
    value = total_flops / (ms * 1e-3) * 1e-12

    # which route the library took, and for the two-pass route the duration of each pass on its own
    plan = ops.oft_plan(m, n_loc, k, reconn_sz=b, lib=lib)
    passes = None
    gemm_ms = ms_local
    if plan["path"] == "two_pass":
        dXR = torch.empty((m, k), dtype=torch.float16, device=dev)

        def timed(fn, reps):
            for _ in range(2):
                fn()
            torch.cuda.synchronize()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record(stream)
            for _ in range(reps):
                fn()
            t1.record(stream)
            torch.cuda.synchronize()
            return t0.elapsed_time(t1) / reps

        rot_ms = timed(lambda: ops.rotate(m, k, dX, k, dR, k, dXR, k, stream, reconn_sz=b, lib=lib), max(args.steps, 5))
        gemm_ms = timed(lambda: ops.gemm_tn(n_loc, m, k, dW, k, dXR, k, dY, n_loc, stream, lib=lib), args.steps)
        passes = {"rotate_ms": rot_ms, "rotate_gbs": 4.0 * m * k / (rot_ms * 1e-3) * 1e-9, "rotate_frac_of_measured_hbm": None,
                  "gemm_ms": gemm_ms, "gemm_tflops": 2.0 * m * n_loc * k / (gemm_ms * 1e-3) * 1e-12}
        del dXR
        assert ops.device_status(lib)[0] == 0

    # the fused kernel (X.R never leaves the SM) on the same workload, for comparison with the route taken
    fused = None
    if plan["path"] == "two_pass":
        os.environ["B200_OFT_PATH"] = "1"
        try:
            fsteps = max(3, min(args.steps, 5))
            for _ in range(2):
                step()
            barrier()
            f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            f0.record(stream)
            for _ in range(fsteps):
                step()
            f1.record(stream)
            barrier()
            tf_ = torch.tensor([f0.elapsed_time(f1) / fsteps], device=dev, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(tf_, op=dist.ReduceOp.MAX)
            fused = {"ms_per_step": float(tf_.item()), "value": total_flops / (float(tf_.item()) * 1e-3) * 1e-12, "unit": "TFLOP/s", "steps": fsteps,
                     "kernel": "oft2_kernel (B200_OFT_PATH=1)"}
        finally:
            del os.environ["B200_OFT_PATH"]
        assert ops.device_status(lib)[0] == 0

    # optional exchange, timed on its own
    allgather_ms = None
    if args.allgather and world > 1:
        for _ in range(2):
            sharded.all_gather_c(dY, world)
        barrier()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record(stream)
        out = sharded.all_gather_c(dY, world)
        a1.record(stream)
        barrier()
        ta = torch.tensor([a0.elapsed_time(a1)], device=dev, dtype=torch.float64)
        dist.all_reduce(ta, op=dist.ReduceOp.MAX)
        allgather_ms = float(ta.item())
        # the same exchange overlapped with the product (copy engines push finished row chunks to the peers)
        ag = sharded.SlabProductAllGather(m, n, k, n0, n1, reconn_sz=b, world=world, rank=rank, device=dev, lib=lib)
        for _ in range(2):
            y_all = ag(dX, dW, dR)
        overlapped_ok = bool(torch.equal(y_all.view(world * m, n_loc), out.view(world * m, n_loc)))
        barrier()
        t0 = time.perf_counter()
        for _ in range(5):
            ag(dX, dW, dR)
        tov = torch.tensor([(time.perf_counter() - t0) / 5 * 1e3], device=dev, dtype=torch.float64)
        dist.all_reduce(tov, op=dist.ReduceOp.MAX)
        overlapped_ms = float(tov.item())
        del out, ag, y_all

    # end to end from pinned host buffers, H2D + product + D2H inside the timed region.  One GPU: the C ABI's
    # host-buffer entry point.  Several GPUs: sharded.HostSlabRunner, in which X crosses the host link once per
    # node (each rank uploads 1/N of its rows, the slices are all-gathered over NVLink) instead of once per GPU.
    hW = dW.cpu().pin_memory()
    hR = torch.from_numpy(R).pin_memory()
    hY = torch.empty((m, n_loc), dtype=torch.float16).pin_memory()
    if world == 1:
        hX = dX.cpu().pin_memory()
        e2e_api = "b200_oft_tn_f16_host (pinned host buffers, synchronous)"
        h2d = (hX.numel() + hW.numel() + hR.numel()) * 2
        d2h = hY.numel() * 2

        def e2e_step():
            ops.oft_tn_host(m, n_loc, k, hX, k, hW, k, hR, k, hY, n_loc, reconn_sz=b, lib=lib)
    else:
        r0, r1 = sharded.row_slice(m, world, rank)
        hX = dX[r0:r1].cpu().pin_memory()
        runner = sharded.HostSlabRunner(m, n, k, n0, n1, reconn_sz=b, world=world, rank=rank, device=dev, lib=lib)
        e2e_api = "sharded.HostSlabRunner (pinned host buffers; X uploaded once per node, all-gathered over NVLink; synchronous)"
        h2d, d2h = runner.bytes_per_step()

        def e2e_step():
            runner(hX, hW, hR, hY)

    for _ in range(2):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.e2e_steps):
        e2e_step()  # synchronous: returns when Y is back in host memory
    e2e_s_local = (time.perf_counter() - t0) / args.e2e_steps
    te = torch.tensor([e2e_s_local], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_s = float(te.item())
    th = torch.tensor([h2d, d2h], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(th)
    same = bool(torch.equal(hY, dY.cpu()))  # the host-buffer path must reproduce the device path bit for bit

    if rank == 0:
        peaks = measured_peaks()
        # dominant kernel: the fused kernel (its launch is the step), or the GEMM pass of the two-pass route
        # (timed on its own above; algorithmic FLOPs 2 M N K, the rotation's 2 M K b belong to the other pass)
        two = plan["path"] == "two_pass"
        flops_launch = 2.0 * m * n_loc * k if two else flops_of(m, k, n_loc, b)
        achieved = flops_launch / (gemm_ms * 1e-3) * 1e-12
        timed_s = ms * args.steps * 1e-3
        peak = peaks["bf16_sustained"] if timed_s >= 2.0 else peaks["bf16_burst"]
        if passes is not None:
            passes["rotate_frac_of_measured_hbm"] = passes["rotate_gbs"] / peaks["hbm_gbs"]
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic",
            "config": {"workload": workload, "M": m, "K": k, "N": n, "b": b, "n_per_gpu": n_loc, "sharding": f"N over {world} GPU(s), X and R replicated",
                       "flops": "2MKN + 2MKb", "l2": "inputs larger than L2 (X alone exceeds 126 MB); no flush between steps",
                       "route": plan["path"], "kernel": ops.kernel_info(lib)["gemm_half_tn" if two else "oft"]},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                         "peak_source": f"{peaks['source']} bf16 {'sustained' if timed_s >= 2.0 else 'burst'} (cuBLAS matmul on this pool)",
                         "traffic": (NCU_TRAFFIC_BYTES.get((workload, plan["path"])) if world == 1 else None),
                         "frac_of_nominal_fp16": achieved / NOMINAL_FP16_TFLOPS,
                         "kernel": "gemm2_kernel (GEMM pass of the two-pass route)" if two else "oft2_kernel", "launch_ms": gemm_ms},
            "e2e": {"value": total_flops / e2e_s * 1e-12, "unit": "TFLOP/s", "h2d_bytes_per_step": int(th[0].item()),
                    "d2h_bytes_per_step": int(th[1].item()), "ms_per_step": e2e_s * 1e3, "steps": args.e2e_steps,
                    "api": e2e_api, "matches_device_path": same},
            "gpu_launches": args.steps * world * plan["kernel_launches"], "clocks": clocks,
        }
        if passes is not None:
            line["passes"] = passes
        if fused is not None:
            fused["frac_of_measured_bf16_burst"] = fused["value"] / world / peaks["bf16_burst"]  # per GPU
            line["fused_route"] = fused
        if allgather_ms is not None:
            line["allgather_y_ms"] = allgather_ms
            line["product_with_overlapped_allgather"] = {"ms_per_step": overlapped_ms, "sequential_ms": ms + allgather_ms,
                                                         "matches_nccl_allgather": overlapped_ok,
                                                         "api": "sharded.SlabProductAllGather (row chunks pushed into the peers' symmetric-memory buffers by copy engines)"}
        if world == 1 and workload == DEFAULT_WORKLOAD:
            line["also"] = projection_shape_rate(lib, dev, stream)
        if world == 1 and not args.no_cpu_baseline:
            cb = cpu_reference_rate(m, k, n, b, kind, 12.0)
            cb.pop("seconds", None)
            line["cpu_baseline"] = cb
        emit(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


_RESULT_FD = None


def emit(line):
    """The one JSON line of the run, written to the process's original stdout."""
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


def main():
    # stdout carries exactly one JSON line.  Libraries that write to file descriptor 1 on their own (NCCL prints its
    # version banner there whatever NCCL_DEBUG_FILE says) are sent to stderr: fd 1 is pointed at fd 2 for the whole
    # run and the result goes to a duplicate of the original stdout.
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--allgather", action="store_true", help="also time the optional NCCL all-gather of Y (N > 1)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args, args.workload)
    else:
        run_gpu_arm(args, args.workload)


if __name__ == "__main__":
    main()
