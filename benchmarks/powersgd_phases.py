#!/usr/bin/env python
"""Where the fused PowerSGD exchange spends its time: the three parts of the kernel, timed one by one.

On one GPU the kernel can run its parts as separate launches (the same code path a multi-rank emulation uses):

    part 1   M' = G + R, P = M' Q              (stage 1: 12 B per element: read G, R, write M')
    part 2   mean P, Gram, Cholesky, Q = M'^T P (stage 2: 4 B per element: read M')
    part 3   mean Q, out = P Q^T, R = M' - out  (stage 3: 12 B per element: read M', write R, out)

Each part is timed with CUDA events around its launch, L2 flushed before every launch (a 256 MiB write), median
over ``--iters``; the bytes above over the time give the achieved HBM rate, shown next to the measured copy
bandwidth of MEASURED_PEAKS.json.  ``--whole`` also times the one-launch exchange.

    python benchmarks/powersgd_phases.py --rows 4096 --cols 4096 --rank 4
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=4096)
    ap.add_argument("--cols", type=int, default=4096)
    ap.add_argument("--rank", type=int, default=4)
    ap.add_argument("--iters", type=int, default=7, help="timed iterations at least")
    ap.add_argument("--min-seconds", type=float, default=1.2,
                    help="keep iterating until the timed loop has run this long (so that the 100 ms clock sampler "
                         "sees the GPU under load); 0 = exactly --iters")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-memory", action="store_true", help="no error feedback (stage 1 reads G only)")
    ap.add_argument("--whole", action="store_true")
    args = ap.parse_args()

    import torch

    import grace_b200
    from grace_b200.communicator.fused import VirtualWorld
    from grace_b200.utils.clocks import ClockSampler

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    try:
        bw = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"])
        bw_src = "measured"
    except Exception:
        bw, bw_src = 6650.0, "fallback"
    params = {"compressor": "powersgd", "memory": "none" if args.no_memory else "powersgd", "communicator": "allreduce",
              "compress_rank": args.rank, "use_memory": True, "world_size": 1, "fused": True}
    vw = VirtualWorld(1, lambda r: grace_b200.grace_from_params(dict(params)), dev)
    n, m = args.rows, args.cols
    g = torch.randn(n, m, device=dev) * 1e-3
    vw.step([g.clone()], "w")
    vw.check()
    plan = next(iter(vw.comms[0]._plans.values()))
    flat = g.reshape(-1).clone()
    out = torch.empty_like(flat)
    flush = torch.empty(64 << 20, dtype=torch.float32, device=dev)
    sampler = ClockSampler(0, period_ms=100).start()
    t_start = time.time()
    times = {1: [], 2: [], 3: [], 0: []}
    it = -1
    while True:
        it += 1
        if it >= args.warmup + args.iters and time.time() - t_start >= args.min_seconds:
            break
        seq = None
        for part in (1, 2, 3):
            flush.fill_(float(it))
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            seq = plan.launch(flat, out, part=part, seq=seq)
            e1.record()
            torch.cuda.synchronize()
            if it >= args.warmup:
                times[part].append(e0.elapsed_time(e1))
        if args.whole:
            flush.fill_(float(it))
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            plan.launch(flat, out)
            e1.record()
            torch.cuda.synchronize()
            if it >= args.warmup:
                times[0].append(e0.elapsed_time(e1))
    plan.check()
    clocks = sampler.summary(t_start, time.time())
    sampler.stop()
    elems = n * m
    per_elem = {1: 4 if args.no_memory else 12, 2: 4, 3: 8 if args.no_memory else 12, 0: 16 if args.no_memory else 28}
    rows = []
    for part in (1, 2, 3, 0):
        if not times[part]:
            continue
        ms = sorted(times[part])[len(times[part]) // 2]
        gbs = per_elem[part] * elems / ms / 1e6
        rows.append({"part": part or "whole", "ms": round(ms, 4), "bytes_per_element": per_elem[part],
                     "achieved_gbs": round(gbs, 1), "fraction_of_copy_bandwidth": round(gbs / bw, 3)})
    print(json.dumps({"shape": [n, m], "rank": args.rank, "error_feedback": not args.no_memory, "parts": rows,
                      "hbm_gbs": bw, "hbm_source": bw_src, "clocks": clocks,
                      "timing": "cuda events per launch, median of %d, L2 flushed before every launch" % len(times[1])}))


if __name__ == "__main__":
    main()
