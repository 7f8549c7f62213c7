#!/usr/bin/env python
"""CPU ranks: the host engine of the exchange protocol against the library communicators over gloo.

    python benchmarks/host_bench.py --world 2 --elems 1048576 --iters 10

One process per rank (gloo, 127.0.0.1).  For every case both communicators exchange the same gradients; the line
reports the median wall-clock time of ``grc.step`` (max over ranks) for each and the largest difference of the
results (0 for the deterministic codecs; the stochastic one draws different random numbers on the two paths).
No GPU is involved: these numbers say what the native path buys on CPU tensors, nothing about the kernels.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

CASES = {
    "topk1": dict(compressor="topk", memory="residual", communicator="allgather", compress_ratio=0.01),
    "threshold": dict(compressor="threshold", memory="residual", communicator="allgather", threshold=2e-3),
    "qsgd8": dict(compressor="qsgd", memory="residual", communicator="allgather", quantum_num=127),
    "signsgd": dict(compressor="signsgd", memory="none", communicator="allgather"),
    "efsign": dict(compressor="efsignsgd", memory="efsignsgd", communicator="allgather", lr=0.1),
    "dense": dict(compressor="none", memory="none", communicator="allgather"),
    # two-phase mode (compressed reduce-scatter, re-encode, compressed all-gather); the library AllToAll communicator
    # needs a backend with all_to_all, which gloo is not: its column then reads null
    "qsgd8_a2a": dict(compressor="qsgd", memory="none", communicator="alltoall", quantum_num=127),
    "natural_a2a": dict(compressor="natural", memory="none", communicator="alltoall"),
    "powersgd4": dict(compressor="powersgd", memory="powersgd", communicator="allreduce", compress_rank=4, use_memory=True),
}


def _rank_main(rank, world, port, args, ret):
    import torch
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.set_num_threads(max(1, args.threads))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from grace_b200 import grace_from_params

    rows = []
    for case in args.cases.split(","):
        for n in [int(e) for e in args.elems.split(",")]:
            shape = (n,)
            if case == "powersgd4":   # a matrix: rows x 1024
                shape = (max(1, n // 1024), 1024)
            grads = [torch.randn(shape, generator=torch.Generator().manual_seed(100 * s + rank)) * 1e-3
                     for s in range(args.warmup + args.iters)]
            result = {}
            outs = {}
            for impl in ("library", "host"):
                p = dict(CASES[case], world_size=world)
                if impl == "host":
                    p.update(host_protocol=True, timeout_ms=60000)
                grc = grace_from_params(p)
                times = []
                failed = 0.0
                for s, g in enumerate(grads):
                    dist.barrier()
                    t0 = time.perf_counter()
                    try:
                        out = grc.step(g.clone(), "w")
                    except RuntimeError:      # a collective the backend does not have
                        failed = 1.0
                        break
                    t1 = time.perf_counter()
                    if s == 0:
                        outs[impl] = out   # compared on the first exchange: later ones amplify rounding differences
                    if s >= args.warmup:
                        times.append((t1 - t0) * 1e3)
                flag = torch.tensor([failed])
                dist.all_reduce(flag, op=dist.ReduceOp.MAX)
                if float(flag) > 0:
                    result[impl] = None
                    continue
                t = torch.tensor([sorted(times)[len(times) // 2]])
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                result[impl] = float(t)
                if hasattr(grc, "close"):
                    grc.close()
            lib_ms = result["library"]
            diff = float((outs["library"] - outs["host"]).abs().max()) if lib_ms is not None else None
            rows.append({"case": case, "elems": n, "world": world,
                         "library_gloo_ms": round(lib_ms, 3) if lib_ms is not None else None,
                         "host_engine_ms": round(result["host"], 3),
                         "speedup": round(lib_ms / result["host"], 2) if lib_ms is not None else None,
                         "max_abs_diff_first_exchange": diff,
                         "timing": "perf_counter around grc.step, median of %d, max over ranks" % args.iters})
    if rank == 0:
        ret.extend(rows)
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--world", type=int, default=2)
    ap.add_argument("--elems", default="65536,1048576")
    ap.add_argument("--cases", default=",".join(CASES))
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--threads", type=int, default=1, help="torch intra-op threads per rank")
    args = ap.parse_args()

    import socket

    import torch.multiprocessing as mp

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.list()
        procs = [ctx.Process(target=_rank_main, args=(r, args.world, port, args, ret)) for r in range(args.world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join()
        for row in ret:
            print(json.dumps(row))
    if any(p.exitcode != 0 for p in procs):
        sys.exit(1)


if __name__ == "__main__":
    main()
