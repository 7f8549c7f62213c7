#!/usr/bin/env python
"""Compressed-exchange microbenchmark (no model).

fp32 gradients of 1M .. 256M elements drawn from N(0, 1e-3) with seed = rank;
TopK 1 %, DGC 0.1 %, QSGD 8-bit (all-gather and two-phase "alltoall" mode), EF-signSGD (majority-style scaled vote),
natural compression, each with its error-feedback memory, and PowerSGD rank 4
on 4096 x 4096.  Measures compensate + compress + exchange + decompress for

    --impl ours       one fused kernel per exchange (FusedExchange)
    --impl library    this package's torch.distributed communicators
    --impl reference  the unmodified reference under baseline/_ref (NCCL)

Device-timed with CUDA events, max over ranks; L2 is flushed between timed
iterations (a 256 MiB write).  For the fused path the achieved time is also
reported as a fraction of the roofline

    max( minimal HBM bytes / measured copy bandwidth ,
         compressed bytes received / 770 GB/s per direction )

with the copy bandwidth taken from MEASURED_PEAKS.json when present.

    python benchmarks/microbench.py --sizes 1,4,16,64,256 --iters 5
    python -m torch.distributed.run --nproc-per-node 8 benchmarks/microbench.py ...
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

NVLINK_GBS = 770.0

CASES = {
    "topk1": dict(compressor="topk", memory="residual", communicator="allgather", compress_ratio=0.01),
    "dgc01": dict(compressor="dgc", memory="dgc", communicator="allgather", compress_ratio=0.001, momentum=0.9),
    "qsgd8": dict(compressor="qsgd", memory="residual", communicator="allgather", quantum_num=127),
    "qsgd8_a2a": dict(compressor="qsgd", memory="residual", communicator="alltoall", quantum_num=127),
    "efsign": dict(compressor="efsignsgd", memory="efsignsgd", communicator="allgather", lr=0.1),
    # *_push: same codec, encoded slots replicated to every GPU with multimem.st, decode from local memory
    "qsgd8_push": dict(compressor="qsgd", memory="residual", communicator="allgather", quantum_num=127, nvls=True,
                       nvls_min_world=2),
    "efsign_push": dict(compressor="efsignsgd", memory="efsignsgd", communicator="allgather", lr=0.1, nvls=True,
                        nvls_min_world=2),
    "natural_push": dict(compressor="natural", memory="residual", communicator="allgather", nvls=True,
                         nvls_min_world=2),
    "natural": dict(compressor="natural", memory="residual", communicator="allgather"),
    # *_phased: the phase-by-phase kernel instead of the pipelined one (encode of chunk c + 1 next to the pull of chunk c)
    "qsgd8_phased": dict(compressor="qsgd", memory="residual", communicator="allgather", quantum_num=127, pipeline=False),
    "natural_phased": dict(compressor="natural", memory="residual", communicator="allgather", pipeline=False),
    # the pipelined kernel on a single rank (queue, chunk counters and flags to itself): for profiling on one GPU
    "qsgd8_forced": dict(compressor="qsgd", memory="residual", communicator="allgather", quantum_num=127,
                         pipeline="force"),
    # uncompressed mean: "dense" = one-shot peer loads + two-phase option, "dense_nvls" = NVSwitch multicast kernel
    "dense": dict(compressor="none", memory="none", communicator="alltoall"),
    "dense_nvls": dict(compressor="none", memory="none", communicator="allreduce", nvls=True, nvls_min_world=2),
    # same, with the gradient living in the symmetric buffer (FlatParams(grad_buffer=...)): no staging copies
    "dense_nvls_inplace": dict(compressor="none", memory="none", communicator="allreduce", nvls=True,
                               nvls_min_world=2),
    "powersgd4": dict(compressor="powersgd", memory="powersgd", communicator="allreduce", compress_rank=4,
                      use_memory=True),
}


def hbm_gbs():
    try:
        return float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def roofline_ms(case, n, world, bw):
    """(hbm_bytes, link_bytes) -> ms.  Minimal traffic of the fused algorithm."""
    if case in ("topk1", "dgc01"):
        ratio = 0.01 if case == "topk1" else 0.001
        per_elem = 20 if case == "topk1" else 28          # g,r read; r,out write; one re-read (+u read/write for DGC)
        hbm = per_elem * n
        link = (world - 1) * ratio * n * 8
    elif case in ("qsgd8", "natural", "qsgd8_push", "natural_push", "qsgd8_phased", "natural_phased", "qsgd8_forced"):
        hbm = (12 + 1 + world + 4) * n                       # g,r read, r write, code write, W code reads, out write
        link = (world - 1) * n * (1 + 4.0 / 128)
    elif case == "qsgd8_a2a":
        hbm = 19 * n                                         # encode 13 B, reduce my chunk 1 + 1/W B, gather 1 + 4 B
        link = 2.0 * (world - 1) / world * n * (1 + 4.0 / 128)
    elif case in ("dense", "dense_nvls", "dense_nvls_inplace"):
        hbm = 8 * n                                          # read g, write the mean
        # two-phase peer loads: reduce-scatter + all-gather; multicast: all W copies of every slice leave through
        # the switch once (the requester's own copy included) plus the broadcast of this rank's slice
        link = (2.0 * (world - 1) / world if case == "dense" else 1.0 + 1.0 / world) * n * 4
    elif case in ("efsign", "efsign_push"):
        hbm = (12 + 8 + 4) * n + (1 + world) * n / 8
        link = (world - 1) * n / 8
    else:  # powersgd on sqrt(n) x sqrt(n)
        hbm = 28 * n
        side = int(n ** 0.5)                                 # P and Q of rank 4, padded to 16 columns
        link = (world - 1) * 2 * side * 16 * 4
    return max(hbm / (bw * 1e9), link / (NVLINK_GBS * 1e9)) * 1e3, hbm, link


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", default="1,4,16,64", help="millions of elements (2^20)")
    ap.add_argument("--elems", default="", help="further sizes as plain element counts (small tensors), e.g. 256,4096,8192")
    ap.add_argument("--cases", default=",".join(CASES))
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--min-iters", type=int, default=5,
                    help="timed iterations for sizes of 16 Mi elements and more (keeps the clock sampler busy long "
                         "enough to see the GPU under load)")
    ap.add_argument("--impl", default="ours", choices=["ours", "library", "reference"])
    ap.add_argument("--min-seconds", type=float, default=0.8,
                    help="keep iterating a case until it has run this long (the clock sampler needs to see the GPU "
                         "under load); 0 = the iteration counts only")
    ap.add_argument("--timeout-ms", type=float, default=3000.0,
                    help="limit of every device-side wait of the fused exchanges; a case that runs into it is "
                         "reported as an error after its first failing iteration")
    ap.add_argument("--virtual-ranks", type=int, default=0,
                    help="one GPU only: run W ranks of the fused exchange on this GPU, phase by phase (all ranks "
                         "compress and publish, then all ranks exchange); reports the time of all W ranks divided by W")
    args = ap.parse_args()

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29541")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    bw, bw_src = hbm_gbs()
    flush = torch.empty(64 << 20, dtype=torch.float32, device=dev)
    from grace_b200.utils.clocks import ClockSampler

    import time

    sampler = ClockSampler(local, period_ms=100)   # one sampler for the run; every line gets the samples of its window
    if rank == 0:
        sampler.start()

    if args.impl == "reference":
        for mod in [m for m in sys.modules if m.startswith("grace_dl")]:
            del sys.modules[mod]
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))

    def build(case):
        p = dict(CASES[case])
        p["world_size"] = world
        if args.impl == "ours":
            import grace_b200

            p["fused"] = True
            p["timeout_ms"] = args.timeout_ms
            return grace_b200.grace_from_params(p)
        if args.impl == "library":
            import grace_b200

            p.pop("nvls", None)
            p.pop("nvls_min_world", None)
            if case.startswith("dense"):
                p["communicator"] = "allreduce"
            return grace_b200.grace_from_params(p)
        # reference: construct the classes directly where its helper cannot
        if case == "dgc01":
            from grace_dl.dist.communicator.allgather import Allgather
            from grace_dl.dist.compressor.dgc import DgcCompressor
            from grace_dl.dist.memory.dgc import DgcMemory

            return Allgather(DgcCompressor(p["compress_ratio"]), DgcMemory(0.9, False, world), world)
        if case == "powersgd4":
            from grace_dl.dist.communicator.allreduce import Allreduce
            from grace_dl.dist.compressor.powersgd import PowerSGDCompressor
            from grace_dl.dist.memory.powersgd import PowerSGDMemory

            comp = PowerSGDCompressor(rank=4, use_memory=True, world_size=world)
            return Allreduce(comp, PowerSGDMemory(comp.q_memory, 4), world)
        if case.startswith("natural"):
            raise RuntimeError("reference natural compression needs cupy (not installed)")
        from grace_dl.dist.helper import grace_from_params

        p.pop("nvls", None)
        p.pop("nvls_min_world", None)
        if case.startswith("dense"):
            p["communicator"] = "allreduce"
        return grace_from_params(p)

    rows = []
    for case in args.cases.split(","):
        sizes = [(int(s), int(s) << 20) for s in args.sizes.split(",") if s]
        sizes += [(int(e) / float(1 << 20), int(e)) for e in args.elems.split(",") if e]
        for size_m, n in sizes:
            if case == "powersgd4":
                # matrices: 16 -> 4096 x 4096, 64 -> 8192 x 8192, 98 -> 4096 x 25088 (the first FC layer of VGG-16)
                shape = {16: (4096, 4096), 64: (8192, 8192), 98: (4096, 25088)}.get(size_m)
                if shape is None:
                    continue
                n = shape[0] * shape[1]
            else:
                shape = (n,)
            try:
                if args.virtual_ranks > 1:
                    if world != 1 or args.impl != "ours" or case.startswith("dense_nvls"):
                        raise RuntimeError("--virtual-ranks needs one process, --impl ours and a peer-load case")
                    import grace_b200
                    from grace_b200.communicator.fused import VirtualWorld

                    vp = dict(CASES[case], world_size=args.virtual_ranks, fused=True)
                    grc = VirtualWorld(args.virtual_ranks, lambda r: grace_b200.grace_from_params(dict(vp)), dev)
                else:
                    grc = build(case)
            except Exception as e:
                if rank == 0:
                    print(json.dumps({"case": case, "impl": args.impl, "unavailable": str(e)[:120]}))
                break
            gen = torch.Generator(device=dev).manual_seed(rank)
            base = torch.randn(shape, generator=gen, device=dev) * 1e-3
            vranks = args.virtual_ranks if args.virtual_ranks > 1 else 0
            vbase = [base.roll(1001 * r) for r in range(vranks)]   # a different gradient per virtual rank
            times = []
            resident = None
            if case.endswith("_inplace") and args.impl == "ours" and hasattr(grc, "buffer"):
                resident = grc.buffer(n)
            t_case = time.time()
            try:
                n_iters = args.warmup + max(args.iters, args.min_iters if size_m >= 16 else args.iters)
                it = -1
                while True:
                    it += 1
                    if it >= n_iters:
                        # every rank must take the same decision: rank 0's clock decides
                        more = torch.tensor([1.0 if time.time() - t_case < args.min_seconds else 0.0], device=dev)
                        dist.broadcast(more, 0)
                        if float(more) == 0.0 or it >= 400:
                            break
                    g = base.clone() if resident is None else resident.copy_(base)
                    vg = [b.clone() for b in vbase]
                    flush.fill_(float(it))
                    dist.barrier()
                    torch.cuda.synchronize()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    if vranks:
                        out = grc.step(vg, "w")
                    else:
                        out = grc.step(g, "w") if resident is None else grc.step_flat(g)
                    e1.record()
                    torch.cuda.synchronize()
                    if it == 0 and hasattr(grc, "check"):
                        grc.check()          # a transport that does not work here fails once, not in every iteration
                    if it >= args.warmup:
                        times.append(e0.elapsed_time(e1))
                if hasattr(grc, "check"):
                    grc.check()
            except Exception as e:
                if rank == 0:
                    print(json.dumps({"case": case, "impl": args.impl, "size_m": size_m,
                                      "error": "%s: %s" % (type(e).__name__, str(e).splitlines()[0][:160])}))
                continue
            clocks = sampler.summary(t_case, time.time()) if rank == 0 else None
            t = torch.tensor([sorted(times)[len(times) // 2]], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t) / (vranks or 1)
            roof, hbm, link = roofline_ms(case, n, vranks or world, bw)
            if vranks:                       # emulated ranks share one GPU: nothing crosses a link, HBM is the bound
                link = 0
                roof = hbm / (bw * 1e9) * 1e3
            row = {"case": case, "impl": args.impl, "size_m": size_m, "elems": n, "n_gpus": world, "ms": round(ms, 4),
                   "roofline_ms": round(roof, 4), "fraction_of_roofline": round(roof / ms, 3) if args.impl == "ours" else None,
                   "hbm_bytes": int(hbm), "link_bytes": int(link), "hbm_gbs": bw, "hbm_source": bw_src,
                   "timing": "cuda events, median of %d, max over ranks, L2 flushed" % len(times),
                   "clocks": clocks}
            if len(times) >= 10:   # error feedback changes the value distribution over the iterations of a case
                row["ms_first5"] = round(sorted(times[:5])[2] / (vranks or 1), 4)
                row["ms_last5"] = round(sorted(times[-5:])[2] / (vranks or 1), 4)
            if vranks:
                row["virtual_ranks"] = vranks
                row["timing"] += "; %d ranks emulated on one GPU phase by phase, time of all ranks / %d" % (vranks, vranks)
            rows.append(row)
            if rank == 0:
                print(json.dumps(row), flush=True)
            del grc, base, out, g, vbase, vg
            torch.cuda.empty_cache()
    if rank == 0:
        sampler.stop()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
