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

`value` times b200_oft_tn_f16 on the route it takes by itself (the fused kernel that shares one X.R per row
block among the N tiles through an L2-resident ring).  `roofline` carries, beside the figures of that kernel,
the other routes on the same workload (`routes`), the single-GPU projection shape M 16384, K = N 4096, b 64
(`projection_shape`) and the two plain GEMM configurations (`gemm_half_tn_8192`, `gemm_float_nt_4096`), each
with a same-process torch.matmul figure beside it.
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
    # Shared-X.R kernel (oft3_kernel).  Large workload: captured at M 16384 (one kernel, two launches: read 5.79 GB +
    # write 1.26 GB against 1.68 GB algorithmic) and scaled by 4 to M 65536 -- W is re-streamed once per band of 8 row
    # blocks, X and Y once, so traffic grows in proportion to M.  Projection shape: captured whole (584.5 + 295.3 MB
    # against 303 MB algorithmic; the extra is X.R leaving L2 once and W read again by later bands).
    ("oft_large_m65536_k8192_n28672_b128", "fused_ring"): 28.2e9,
    # The same ring with the rotation on SM pairs of its own (oft4_kernel), captured the same way at M 16384:
    # read 4.79 GB + write 1.17 GB, times 4.
    ("oft_large_m65536_k8192_n28672_b128", "fused_ring_split"): 23.9e9,
    ("oft_proj_m16384_k4096_n4096_b64", "fused_ring"): 879.8e6,
    # two-pass route, GEMM pass (gemm2_kernel): read 17.86 GB + write 3.72 GB against 5.3 GB algorithmic; the
    # rotation pass before it moves 1.08 + 1.03 GB, its algorithmic bytes
    ("oft_large_m65536_k8192_n28672_b128", "two_pass"): 21.58e9,
    # kernel that keeps X.R in tensor memory (oft2_kernel): read 29.2 GB + write 5.7 GB
    ("oft_large_m65536_k8192_n28672_b128", "fused_tmem"): 34.94e9,
    ("oft_proj_m16384_k4096_n4096_b64", "fused_tmem"): 517.2e6,
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


def config_of(workload: str, gpus: int) -> dict:
    """The `config` object of the JSON line: the same for this repo's arm and for the reference arm."""
    m, k, n, b, kind, wsigma = WORKLOADS[workload]
    return {"workload": workload, "M": m, "K": k, "N": n, "b": b, "blocks": kind, "w_sigma": wsigma, "gpus": gpus,
            "sharding": f"N over {gpus} GPU(s), X and R replicated", "flops": "2MKN + 2MKb",
            "l2": "inputs larger than L2 (X alone exceeds 126 MB); no flush between steps"}


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
            "config": config_of(workload, args.gpus),
            "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": info["cores"], "kind": info["kind"], "sample": info["sample"],
                             "note": "ms_per_step extrapolates the sampled rate to the full problem"},
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    emit(line)


# --------------------------------------------------------------------------------------- GPU arm


def _device_timer(stream):
    """timed(fn, reps, warm) -> ms per call, CUDA events on `stream` (the stream the kernels are launched on)."""
    import torch

    def timed(fn, reps, warm=2):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record(stream)
        for _ in range(reps):
            fn()
        t1.record(stream)
        torch.cuda.synchronize()
        return t0.elapsed_time(t1) / reps

    return timed


def _interleaved(timed, fns, reps, rounds=4, warm=3):
    """Median ms per call of each function in `fns`, each timed once per round (`reps` calls per timing) in a freshly
    shuffled order, so that clock and temperature drift hits all of them alike (on a power-capped GPU the clock a kernel
    gets depends on what ran just before it)."""
    import random
    import statistics

    for fn in fns:
        for _ in range(warm):
            fn()
    samples = [[] for _ in fns]
    rng = random.Random(len(fns) * 1000 + reps)
    for _ in range(rounds):
        order = list(range(len(fns)))
        rng.shuffle(order)  # a fixed order would favour whoever runs behind the coolest neighbour
        for i in order:
            samples[i].append(timed(fns[i], reps, warm=0))
    return [statistics.median(x) for x in samples]


def projection_shape_rates(lib, dev, stream, peaks):
    """Device-timed rates of the single-GPU projection shape (M 16384, K = N 4096, b 64, Cayley blocks) on every
    route of the library, beside the plain GEMM of the same size and cuBLAS on it: medians of 5 interleaved timings of
    10 launches each."""
    import torch

    from cute_mma_b200 import inputs, ops

    name = "oft_proj_m16384_k4096_n4096_b64"
    m, k, n, b, _, wsigma = WORKLOADS[name]
    g = torch.Generator(device=dev).manual_seed(99)
    dX = torch.randn((m, k), generator=g, device=dev, dtype=torch.float32).to(torch.float16)
    dW = (torch.randn((n, k), generator=g, device=dev, dtype=torch.float32) * wsigma).to(torch.float16)
    dR = torch.from_numpy(inputs.pack_r(inputs.blocks_cayley(1, k // b, b, 7))).to(dev)
    dY = torch.empty((m, n), dtype=torch.float16, device=dev)
    timed = _device_timer(stream)
    fl = flops_of(m, k, n, b)
    chosen = ops.oft_plan(m, n, k, reconn_sz=b, lib=lib)["path"]
    # every route, the plain GEMM of the same size (W . X^T, no rotation: the ceiling of any route) and cuBLAS on it, all
    # timed in turn (5 rounds of 10 launches each, medians), so that clock drift hits them alike
    order = sorted(ops.ROUTES.items(), key=lambda kv: kv[1] != chosen)

    def on_route(code):
        def call():
            ops.set_option("oft_route", code, lib)
            ops.oft_tn(m, n, k, dX, k, dW, k, dR, k, dY, n, stream, reconn_sz=b, lib=lib)
        return call

    fns = [on_route(code) for code, _ in order]
    fns += [lambda: ops.gemm_tn(n, m, k, dW, k, dX, k, dY, n, stream, lib=lib), lambda: torch.matmul(dX, dW.t())]
    try:
        times = _interleaved(timed, fns, 10, rounds=5)
    finally:
        ops.set_option("oft_route", 0, lib)
    assert ops.device_status(lib)[0] == 0
    routes = {}
    for (code, rname), ms in zip(order, times):
        tf = fl / (ms * 1e-3) * 1e-12
        routes[rname] = {"ms_per_step": ms, "value": tf, "unit": "TFLOP/s", "steps": 50,
                         "frac_of_measured_bf16_burst": tf / peaks["bf16_burst"], "frac_of_nominal_fp16": tf / NOMINAL_FP16_TFLOPS}
    ms_g, ms_t = times[-2], times[-1]
    out = {"workload": name, "M": m, "K": k, "N": n, "b": b, "route": chosen, "routes": routes,
           "value": routes[chosen]["value"], "unit": "TFLOP/s", "ms_per_step": routes[chosen]["ms_per_step"],
           "frac_of_measured_bf16_burst": routes[chosen]["frac_of_measured_bf16_burst"],
           "frac_of_nominal_fp16": routes[chosen]["frac_of_nominal_fp16"],
           "plain_gemm_same_size": {"ms": ms_g, "value": 2.0 * m * n * k / (ms_g * 1e-3) * 1e-12, "torch_matmul_ms": ms_t,
                                    "torch_matmul_value": 2.0 * m * n * k / (ms_t * 1e-3) * 1e-12, "unit": "TFLOP/s"}}
    return out


def plain_gemm_rates(lib, dev, stream, peaks):
    """The two plain GEMM configurations: gemm_half TN 8192^3 (fp16, U(-1,1)) and gemm_float NT 4096^3 (TF32, N(0,1)),
    device-timed, each with torch.matmul (cuBLAS) on the same operands in the same process beside it."""
    import torch

    from cute_mma_b200 import ops

    timed = _device_timer(stream)
    out = {}
    g = torch.Generator(device=dev).manual_seed(5)
    m = 8192
    A = (torch.rand((m, m), generator=g, device=dev) * 2 - 1).to(torch.float16)
    B = (torch.rand((m, m), generator=g, device=dev) * 2 - 1).to(torch.float16)
    C = torch.empty((m, m), dtype=torch.float16, device=dev)
    fl = 2.0 * m ** 3
    ms, ms_t = _interleaved(timed, [lambda: ops.gemm_tn(m, m, m, A, m, B, m, C, m, stream, lib=lib), lambda: torch.matmul(A, B.t())], 8)
    tf = fl / (ms * 1e-3) * 1e-12
    out["gemm_half_tn_8192"] = {"ms": ms, "value": tf, "unit": "TFLOP/s", "frac_of_measured_bf16_burst": tf / peaks["bf16_burst"],
                                "frac_of_nominal_fp16": tf / NOMINAL_FP16_TFLOPS,
                                "torch_matmul_fp16": {"ms": ms_t, "value": fl / (ms_t * 1e-3) * 1e-12}}
    del A, B, C
    m = 4096
    A = torch.randn((m, m), generator=g, device=dev)   # [K][M], M contiguous
    B = torch.randn((m, m), generator=g, device=dev)   # [K][N], N contiguous
    C = torch.empty((m, m), dtype=torch.float32, device=dev)
    fl = 2.0 * m ** 3
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        ms, ms_t = _interleaved(timed, [lambda: ops.gemm_nt(m, m, m, A, m, B, m, C, m, stream, dtype="float", lib=lib), lambda: torch.matmul(A.t(), B)], 15)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    tf, tf_t = fl / (ms * 1e-3) * 1e-12, fl / (ms_t * 1e-3) * 1e-12
    out["gemm_float_nt_4096"] = {"ms": ms, "value": tf, "unit": "TFLOP/s", "dtype": "tf32",
                                 "torch_matmul_tf32": {"ms": ms_t, "value": tf_t, "note": "the measured TF32 figure of this box: the reported denominator"},
                                 "frac_of_torch_matmul_tf32": tf / tf_t, "frac_of_nominal_tf32": tf / (NOMINAL_FP16_TFLOPS / 2)}
    assert ops.device_status(lib)[0] == 0
    return out


def run_gpu_arm(args, workload):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch N>1 with torch.distributed.run")
    m, k, n, b, kind, wsigma = WORKLOADS[workload]

    # The CPU leg runs first, on an otherwise idle host: no pinned buffers yet, no clock sampler, no CUDA context
    # (measured after the GPU legs, beside ~5 GB of freshly pinned memory, the same routine ran at 0.6 of this rate).
    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        cpu_reference_rate(m, k, n, b, kind, 1.0)  # warm-up: library load, thread start, page faults
        cpu_baseline = cpu_reference_rate(m, k, n, b, kind, 12.0)
        cpu_baseline.pop("seconds", None)

    from cute_mma_b200 import inputs, ops, sharded

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    lib = ops.load_library()  # raises if the CUDA library is missing: there is no fallback

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
    total_flops = flops_of(m, k, n, b)

    def step():
        sharded.oft_tn_slab(m, n, k, dX, k, dW, k, dR, k, dY, n_loc, n0, n1, stream, reconn_sz=b, lib=lib)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed_steps(steps: int, warm: int) -> float:
        """ms per step of `step`, CUDA events on the launch stream, barrier + synchronize on both sides, max over ranks."""
        for _ in range(warm):
            step()
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record(stream)
        for _ in range(steps):
            step()
        t1.record(stream)
        barrier()
        return max_over_ranks(t0.elapsed_time(t1) / steps)

    warm = max(args.warmup, 3)
    plan = ops.oft_plan(m, n_loc, k, reconn_sz=b, lib=lib)
    for _ in range(warm):
        step()
    barrier()
    assert ops.device_status(lib)[0] == 0
    sampler = ClockSampler(local_rank if "CUDA_VISIBLE_DEVICES" not in os.environ else int(os.environ["CUDA_VISIBLE_DEVICES"].split(",")[local_rank]))
    if rank == 0:
        sampler.start()
        time.sleep(0.15)
    ms = timed_steps(args.steps, 0)   # the headline: the route the library takes by itself
    clocks = sampler.stop() if rank == 0 else None
    st = ops.device_status(lib)
    assert st[0] == 0, st
    value = total_flops / (ms * 1e-3) * 1e-12
    y_chosen = dY.clone() if n_loc * m <= (1 << 31) else None

    # every route of the library on the same workload, same steps, max over ranks
    peaks = measured_peaks()
    routes = {plan["path"]: {"ms_per_step": ms, "value": value, "unit": "TFLOP/s", "steps": args.steps, "chosen": True}}
    for code, rname in ops.ROUTES.items():
        if rname == plan["path"]:
            continue
        with ops.option("oft_route", code, lib):
            r_ms = timed_steps(args.steps, 2)
        assert ops.device_status(lib)[0] == 0
        routes[rname] = {"ms_per_step": r_ms, "value": total_flops / (r_ms * 1e-3) * 1e-12, "unit": "TFLOP/s", "steps": args.steps, "chosen": False}
        if y_chosen is not None:
            routes[rname]["same_bits_as_chosen"] = bool(torch.equal(y_chosen.view(torch.int16), dY.view(torch.int16)))
    del y_chosen
    # the chosen route once more, after the others: the first timing ran on the coolest GPU of this process
    routes[plan["path"]]["ms_per_step_after_the_others"] = timed_steps(args.steps, 2)
    for r in routes.values():
        r["frac_of_measured_bf16_burst_per_gpu"] = r["value"] / world / peaks["bf16_burst"]
    # the two passes of the two-pass route on their own (rank 0's GPU)
    timed = _device_timer(stream)
    dXR = torch.empty((m, k), dtype=torch.float16, device=dev)
    rot_ms = timed(lambda: ops.rotate(m, k, dX, k, dR, k, dXR, k, stream, reconn_sz=b, lib=lib), max(args.steps, 5))
    gemm_ms = timed(lambda: ops.gemm_tn(n_loc, m, k, dW, k, dXR, k, dY, n_loc, stream, lib=lib), args.steps)
    routes["two_pass"]["passes"] = {"rotate_ms": rot_ms, "rotate_gbs": 4.0 * m * k / (rot_ms * 1e-3) * 1e-9,
                                    "rotate_frac_of_measured_hbm": 4.0 * m * k / (rot_ms * 1e-3) * 1e-9 / peaks["hbm_gbs"],
                                    "gemm_ms": gemm_ms, "gemm_tflops": 2.0 * m * n_loc * k / (gemm_ms * 1e-3) * 1e-12}
    del dXR
    step()  # dY holds the chosen route's result again
    barrier()
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
        allgather_ms = max_over_ranks(a0.elapsed_time(a1))
        # the same exchange overlapped with the product (copy engines push finished row chunks to the peers)
        ag = sharded.SlabProductAllGather(m, n, k, n0, n1, reconn_sz=b, world=world, rank=rank, device=dev, lib=lib, mode="copy_engines")
        for _ in range(2):
            y_all = ag(dX, dW, dR)
        overlapped_ok = bool(torch.equal(y_all.view(world * m, n_loc), out.view(world * m, n_loc)))
        barrier()
        t0 = time.perf_counter()
        for _ in range(5):
            ag(dX, dW, dR)
        overlapped_ms = max_over_ranks((time.perf_counter() - t0) / 5 * 1e3)
        del ag, y_all
        # ... and with the exchange done by the kernel's own epilogue (plain stores into the peers' buffers)
        ag = sharded.SlabProductAllGather(m, n, k, n0, n1, reconn_sz=b, world=world, rank=rank, device=dev, lib=lib, mode="stores")
        for _ in range(2):
            y_all = ag(dX, dW, dR)
        stores_ok = bool(torch.equal(y_all.view(world * m, n_loc), out.view(world * m, n_loc)))
        barrier()
        t0 = time.perf_counter()
        for _ in range(5):
            ag(dX, dW, dR)
        stores_ms = max_over_ranks((time.perf_counter() - t0) / 5 * 1e3)
        del out, ag, y_all

    # end to end from pinned host buffers, H2D + product + D2H inside the timed region.  One GPU: the C ABI's
    # host-buffer entry point.  Several GPUs: sharded.HostSlabRunner, in which X crosses the host link once per
    # node (each rank uploads 1/N of its rows, the slices are all-gathered over NVLink) instead of once per GPU.
    hW = dW.cpu().pin_memory()
    hR = torch.from_numpy(R).pin_memory()
    hY = torch.empty((m, n_loc), dtype=torch.float16).pin_memory()
    e2e_legs = None
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
        e2e_api = "sharded.HostSlabRunner (pinned host buffers; X uploaded once per node, all-gathered over NVLink in row chunks; synchronous)"
        h2d, d2h = runner.bytes_per_step()

        def e2e_step():
            runner(hX, hW, hR, hY)

    for _ in range(2):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.e2e_steps):
        e2e_step()  # synchronous: returns when Y is back in host memory
    e2e_s = max_over_ranks((time.perf_counter() - t0) / args.e2e_steps)
    if world > 1:
        e2e_legs = runner.leg_times(hX, hW, hR, hY)  # each leg on its own, max over ranks (ms)
        e2e_legs = {name: max_over_ranks(v) for name, v in e2e_legs.items()}
    th = torch.tensor([h2d, d2h], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(th)
    same = bool(torch.equal(hY, dY.cpu()))  # the host-buffer path must reproduce the device path bit for bit

    if rank == 0:
        # dominant kernel = the one launch of the route taken: algorithmic FLOPs of this GPU's slab per launch
        flops_launch = flops_of(m, k, n_loc, b)
        achieved = flops_launch / (ms * 1e-3) * 1e-12
        timed_s = ms * args.steps * 1e-3
        peak = peaks["bf16_sustained"] if timed_s >= 2.0 else peaks["bf16_burst"]
        kernel_of = {"fused_ring": "oft3_kernel", "fused_ring_split": "oft4_kernel", "fused_tmem": "oft2_kernel", "two_pass": "xr_kernel + gemm2_kernel"}
        config_of_route = {"fused_ring": "oft_ring", "fused_ring_split": "oft_ring_split"}
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                    "peak_source": f"{peaks['source']} bf16 {'sustained' if timed_s >= 2.0 else 'burst'} (cuBLAS matmul on this pool)",
                    "traffic": (NCU_TRAFFIC_BYTES.get((workload, plan["path"])) if world == 1 else None),
                    "frac_of_nominal_fp16": achieved / NOMINAL_FP16_TFLOPS, "route": plan["path"], "kernel": kernel_of[plan["path"]],
                    "launch_ms": ms, "kernel_config": ops.kernel_info(lib)[config_of_route.get(plan["path"], "oft")], "n_per_gpu": n_loc,
                    "routes": routes}
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": warm,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic", "config": config_of(workload, world), "roofline": roofline,
            "e2e": {"value": total_flops / e2e_s * 1e-12, "unit": "TFLOP/s", "h2d_bytes_per_step": int(th[0].item()),
                    "d2h_bytes_per_step": int(th[1].item()), "ms_per_step": e2e_s * 1e3, "steps": args.e2e_steps,
                    "api": e2e_api, "matches_device_path": same},
            "gpu_launches": args.steps * world * plan["kernel_launches"], "clocks": clocks,
        }
        if e2e_legs is not None:
            line["e2e"]["legs_ms"] = e2e_legs
        if allgather_ms is not None:
            line["allgather_y_ms"] = allgather_ms
            line["product_with_overlapped_allgather"] = {"ms_per_step": overlapped_ms, "sequential_ms": ms + allgather_ms,
                                                         "matches_nccl_allgather": overlapped_ok,
                                                         "api": "sharded.SlabProductAllGather (row chunks pushed into the peers' symmetric-memory buffers by copy engines)"}
            # fused product + exchange: the slower of the slab's FLOPs at the measured GEMM peak and the bytes that must
            # leave this GPU over NVLink ((N - 1) copies of its slab of Y) at the measured 770 GB/s peer-copy rate
            nvlink_ms = (world - 1) * m * n_loc * 2 / 770e9 * 1e3
            tensor_ms = flops_launch / (peaks["bf16_burst"] * 1e12) * 1e3
            line["product_with_epilogue_allgather"] = {"ms_per_step": stores_ms, "matches_nccl_allgather": stores_ok,
                                                       "api": "b200_oft_tn_f16_gather (the kernel's epilogue stores every tile into all GPUs' buffers)",
                                                       "roofline": {"bound": "nvlink" if nvlink_ms > tensor_ms else "tensor", "nvlink_ms": nvlink_ms,
                                                                    "tensor_ms": tensor_ms, "frac": max(nvlink_ms, tensor_ms) / stores_ms,
                                                                    "nvlink_gbs_per_gpu": (world - 1) * m * n_loc * 2 / (stores_ms * 1e-3) * 1e-9}}
        if world == 1 and workload == DEFAULT_WORKLOAD:
            del hX, hW, hY
            roofline["projection_shape"] = projection_shape_rates(lib, dev, stream, peaks)
            roofline.update(plain_gemm_rates(lib, dev, stream, peaks))
        if cpu_baseline is not None:
            line["cpu_baseline"] = cpu_baseline
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
