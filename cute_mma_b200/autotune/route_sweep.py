"""Times every route of the OFT product on given shapes, in turn, on one GPU.

The library picks a route per call from the shape (b200_oft_plan); this tool is how that choice is checked: for
each shape the library's own choice (route 0) and every forced route are timed in rounds, one timing of each per
round in a freshly shuffled order, and the medians are printed with their ratio to the library's choice.  The order
matters on a power-capped GPU: the clock a kernel gets depends on what ran in the 100 ms before it (the same kernel
timed behind the rotation pass + GEMM ran 16 % faster than behind a fused kernel), so a fixed order favours whoever
follows the coolest neighbour.  No counterpart in the reference, whose kernel has one route.

    python -m cute_mma_b200.autotune.route_sweep 16384x4096x4096x64 65536x28672x8192x128 [--routes 0,1,2,3,4]
        [--rounds 6] [--ms 30] [--json]

A shape is MxNxKxB (rows of X, columns of Y, inner dimension, block edge of R; one N-group).
"""
from __future__ import annotations

import argparse
import json
import random
import statistics
import sys


def parse_shape(text: str):
    parts = text.lower().split("x")
    if len(parts) != 4:
        raise argparse.ArgumentTypeError(f"shape {text!r} is not MxNxKxB")
    m, n, k, b = (int(p) for p in parts)
    if min(m, n, k, b) <= 0 or k % b != 0:
        raise argparse.ArgumentTypeError(f"shape {text!r}: all positive, K a multiple of B")
    return m, n, k, b


def sweep(shape, routes, rounds: int, target_ms: float, lib=None):
    """[{route, name, ms, tflops, ratio_to_choice}] for one shape; raises if a kernel reported a timed-out wait."""
    import torch

    from .. import inputs, ops

    lib = lib or ops.load_library()
    m, n, k, b = shape
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(m + n + k + b)
    dX = torch.randn((m, k), generator=g, device=dev, dtype=torch.float32).to(torch.float16)
    dW = (torch.randn((n, k), generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.float16)
    dR = torch.from_numpy(inputs.pack_r(inputs.blocks_cayley(1, k // b, b, 11))).to(dev)
    dY = torch.empty((m, n), dtype=torch.float16, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    flops = 2.0 * m * n * k + 2.0 * m * k * b

    def call(route):
        ops.set_option("oft_route", route, lib)
        ops.oft_tn(m, n, k, dX, k, dW, k, dR, k, dY, n, stream, reconn_sz=b, lib=lib)

    def timed(route, reps):
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0.record()
        for _ in range(reps):
            call(route)
        t1.record()
        torch.cuda.synchronize()
        return t0.elapsed_time(t1) / reps

    try:
        for r in routes:
            call(r)
        reps = max(1, int(target_ms / max(timed(routes[0], 1), 1e-3)))
        samples = {r: [] for r in routes}
        rng = random.Random(m * 31 + n * 17 + k)
        for _ in range(rounds):
            order = list(routes)
            rng.shuffle(order)
            for r in order:
                samples[r].append(timed(r, reps))
    finally:
        ops.set_option("oft_route", 0, lib)
    status = ops.device_status(lib, raise_on_error=False)
    if status[0] != 0:
        raise RuntimeError(f"a bounded wait ran out: {status}")
    chosen = ops.oft_plan(m, n, k, reconn_sz=b, lib=lib)["path"]
    base = statistics.median(samples[routes[0]])
    rows = []
    for r in routes:
        ms = statistics.median(samples[r])
        rows.append({"route": r, "name": chosen if r == 0 else ops.ROUTES[r], "ms": ms, "tflops": flops / ms * 1e-9,
                     "ratio_to_choice": ms / base, "launches_per_timing": reps})
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("shapes", nargs="+", type=parse_shape, help="MxNxKxB")
    ap.add_argument("--routes", default="0,1,2,3,4", help="routes to time, the reference for the ratios first (0 = the library's choice)")
    ap.add_argument("--rounds", type=int, default=6)
    ap.add_argument("--ms", type=float, default=30.0, help="kernel time per timing (sets the launches per timing)")
    ap.add_argument("--json", action="store_true")
    args = ap.parse_args(argv)
    routes = [int(r) for r in args.routes.split(",")]
    out = {}
    for shape in args.shapes:
        rows = sweep(shape, routes, args.rounds, args.ms)
        out["x".join(str(v) for v in shape)] = rows
        if not args.json:
            for row in rows:
                label = f"{row['route']} ({row['name']})" if row["route"] == 0 else f"{row['route']} {row['name']}"
                print(f"{'x'.join(str(v) for v in shape):>24}  route {label:<28} {row['ms']:9.4f} ms {row['tflops']:7.0f} TFLOP/s  x{row['ratio_to_choice']:.3f}",
                      flush=True)
    if args.json:
        json.dump(out, sys.stdout)
        print()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
