#!/usr/bin/env python
"""How should the exchange share the GPU with backward?  Sweep for one training config.

For a config of ``bench.py`` (default ``bert_qsgd``) the model is built once per
process and the training step is then timed under several settings of

    bucket size (MiB of fp32 gradients per fused exchange; 0 = one exchange after backward),
    overlap_sms (SMs an exchange may use while backward is still running),
    transport   (pull = peers' slots are read over NVLink, push = multimem.st through the switch),
    launches    (default: an overlapped exchange is split into a full-width compress launch and an exchange launch
                 on ``overlap_sms`` SMs; ``:whole`` keeps it one launch on ``overlap_sms`` SMs),

given as ``--settings 0:0:pull,64:32:pull,64:32:push:whole``.  Every setting gets
its own communicator, flat buffers and optimizer; device-timed with CUDA events
around ``--steps`` steps after ``--warmup`` steps, max over ranks; the batch
(and the activations it produces) is larger than L2, so nothing stays cached
from step to step.  One JSON line per setting, with the clocks seen.

    python -m torch.distributed.run --nproc-per-node 8 benchmarks/overlap_sweep.py --config bert_qsgd
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
    ap.add_argument("--config", default="bert_qsgd")
    ap.add_argument("--settings", default="0:0:pull,128:32:pull,64:32:pull,64:16:pull,64:48:pull")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--bert-impl", default="hf", choices=["hf", "own"])
    args = ap.parse_args()

    import torch
    import torch.distributed as dist

    import bench
    import grace_b200
    from grace_b200 import models
    from grace_b200.optim import FusedSGD
    from grace_b200.parallel import DistributedOptimizer
    from grace_b200.parallel.flat import FlatParams
    from grace_b200.utils.clocks import ClockSampler

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29547")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    torch.backends.cudnn.benchmark = True
    cfg = dict(bench.CONFIGS[args.config])
    amp = cfg["dtype"] == "bf16"
    torch.manual_seed(0)
    if cfg["model"] == "bert_large" and args.bert_impl == "hf":
        model = bench.hf_bert_large().to(dev)
    else:
        model = getattr(models, cfg["model"])().to(dev)
    if cfg["model"] in ("resnet50", "resnet20"):
        model = model.to(memory_format=torch.channels_last)
    named = list(model.named_parameters())
    batches = [bench.make_batch(cfg, dev, seed=1000 * rank + i) for i in range(2)]
    sampler = ClockSampler(local, period_ms=100)
    if rank == 0:
        sampler.start()

    for setting in args.settings.split(","):
        fields = setting.split(":")
        bucket_mb, sms, transport = fields[:3]
        whole = len(fields) > 3 and fields[3] == "whole"
        params = dict(cfg["grace"], world_size=world, fused=True, split_overlap=not whole)
        if int(sms) > 0:
            params["overlap_sms"] = int(sms)
        if transport == "push":
            params.update(nvls=True, nvls_min_world=2)
        grc = grace_b200.grace_from_params(params)
        flat = FlatParams(named, bucket_bytes=int(float(bucket_mb) * (1 << 20)) or None)
        opt = FusedSGD(model.parameters(), lr=0.01, momentum=0.9, flat=flat)
        opt = DistributedOptimizer(opt, grace=grc, named_parameters=named, flat=flat, always_hook=True)

        def step(batch):
            opt.zero_grad()
            loss = bench.forward_loss(model, cfg, batch, amp)
            loss.backward()
            opt.step()
            return loss

        row = {"config": args.config, "bucket_mb": float(bucket_mb), "overlap_sms": int(sms), "transport": transport,
               "launches_per_exchange": 1 if (whole or float(bucket_mb) == 0) else 2,
               "n_gpus": world, "buckets": len(flat.buckets)}
        try:
            for i in range(args.warmup):
                step(batches[i % 2])
            dist.barrier()
            torch.cuda.synchronize()
            t0 = time.time()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(args.steps):
                step(batches[i % 2])
            e1.record()
            dist.barrier()
            torch.cuda.synchronize()
            grc.check()
            ms = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev)
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            row.update(ms_per_step=round(float(ms), 3), samples_per_s=round(cfg["batch"] * world / float(ms) * 1e3, 1),
                       clocks=sampler.summary(t0, time.time()) if rank == 0 else None,
                       timing="cuda events over %d steps after %d warm-up steps, max over ranks" % (args.steps, args.warmup))
        except Exception as e:  # a setting that cannot run (no multicast support, ...) is reported, the sweep goes on
            row["error"] = "%s: %s" % (type(e).__name__, str(e).splitlines()[0][:160])
        if rank == 0:
            print(json.dumps(row), flush=True)
        for h in getattr(opt, "_hook_handles", []):
            if hasattr(h, "remove"):
                h.remove()
        torch.cuda.synchronize()
        if hasattr(grc, "close"):
            grc.close()
        del opt, flat, grc
        torch.cuda.empty_cache()
    if rank == 0:
        sampler.stop()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
