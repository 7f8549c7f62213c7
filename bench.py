#!/usr/bin/env python
"""Headline benchmark: training samples/sec with compressed gradient exchange.

Default config (the reference's headline workload as named by the baseline
file): ResNet-50, bf16 autocast + channels_last, 256 synthetic 3x224x224 images
per GPU, SGD(0.1, momentum 0.9), DGC 0.1 % with momentum-corrected memory,
sparse values+indices all-gather.  Weak scaling: per-GPU batch is fixed.

    python bench.py --gpus N --steps K --warmup W            # this framework
    python bench.py --impl reference --gpus N ...             # unmodified reference (baseline/_ref)

For N > 1 launch through ``python -m torch.distributed.run --nproc-per-node N``.
Rank 0 prints one JSON line.  ``value`` is device-timed (CUDA events, max over
ranks) with inputs resident on the GPU; ``e2e`` repeats the measurement through
the public API with a pinned-host -> device copy of every batch (prefetched on
a copy stream) and a device -> host copy of every step's loss into pinned
memory, read on the host one step later so that the host keeps queueing work
(the last one is read before the closing event); both arms use the same loop.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CONFIGS = {
    "resnet50_dgc": dict(model="resnet50", batch=256, shape=(3, 224, 224), classes=1000, dtype="bf16",
                         grace=dict(compressor="dgc", memory="dgc", communicator="allgather", compress_ratio=0.001,
                                    momentum=0.9)),
    "resnet50_topk": dict(model="resnet50", batch=256, shape=(3, 224, 224), classes=1000, dtype="bf16",
                          grace=dict(compressor="topk", memory="residual", communicator="allgather",
                                     compress_ratio=0.01)),
    "vgg16_powersgd": dict(model="vgg16", batch=128, shape=(3, 224, 224), classes=1000, dtype="fp32",
                           grace=dict(compressor="powersgd", memory="powersgd", communicator="allreduce",
                                      compress_rank=4, use_memory=True)),
    # the config where the exchange shows; `--bucket-mb 336 --overlap-sms 64` exchanges four buckets from gradient
    # hooks next to backward (measured at 4 GPUs: between 2.5 ms faster and 2 ms slower than one exchange after
    # backward, inside the run-to-run spread of the shared hosts, so one exchange stays the default)
    "bert_qsgd": dict(model="bert_large", batch=32, seq=128, vocab=30522, dtype="bf16",
                      grace=dict(compressor="qsgd", memory="none", communicator="allgather", quantum_num=64)),
    "resnet20_topk": dict(model="resnet20", batch=32, shape=(3, 32, 32), classes=10, dtype="fp32",
                          grace=dict(compressor="topk", memory="residual", communicator="allgather",
                                     compress_ratio=0.01)),
}


# ----------------------------------------------------------------------------- clocks
def _load_clock_sampler():
    # the sampler lives in the package, but is loaded by file so that the reference arm imports nothing else of it
    import importlib.util

    spec = importlib.util.spec_from_file_location("_grace_clocks", os.path.join(ROOT, "grace_b200", "utils", "clocks.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.ClockSampler


ClockSampler = _load_clock_sampler()   # read-only nvidia-smi sampling during the timed region


# ----------------------------------------------------------------------------- data
def make_batch(cfg, device, seed, pinned=False):
    import torch

    g = torch.Generator().manual_seed(seed)
    if cfg["model"] == "bert_large":
        ids = torch.randint(0, cfg["vocab"], (cfg["batch"], cfg["seq"]), generator=g)
        labels = ids.clone()
        mask = torch.rand(ids.shape, generator=g) < 0.15
        labels[~mask] = -100
        nsp = torch.randint(0, 2, (cfg["batch"],), generator=g)
        tensors = [ids, labels, nsp]
    else:
        x = torch.randn(cfg["batch"], *cfg["shape"], generator=g)
        y = torch.randint(0, cfg["classes"], (cfg["batch"],), generator=g)
        tensors = [x, y]
    if pinned:
        return [t.pin_memory() for t in tensors]
    return [t.to(device) for t in tensors]


def forward_loss(model, cfg, batch, amp):
    import torch
    import torch.nn.functional as F

    with torch.autocast("cuda", dtype=torch.bfloat16, enabled=amp):
        if cfg["model"] == "bert_large":
            ids, labels, nsp = batch
            if hasattr(model, "mlm_bias"):
                return model(ids, mlm_labels=labels, nsp_labels=nsp)
            out = model(input_ids=ids, labels=labels, next_sentence_label=nsp)
            return out.loss
        x, y = batch
        if x.dim() == 4:
            x = x.contiguous(memory_format=torch.channels_last)
        return F.cross_entropy(model(x).float(), y)


# ----------------------------------------------------------------------------- arms
def build_ours_loop(cfg, device, world):
    """Drop-in usage: the reference's training loop with this package's fused communicator."""
    import torch

    import grace_b200
    from grace_b200 import models

    torch.manual_seed(0)
    if cfg["model"] == "bert_large" and cfg.get("bert_impl", "hf") == "hf":
        model = hf_bert_large().to(device)
    else:
        model = getattr(models, cfg["model"])().to(device)
    if cfg["model"] in ("resnet50", "resnet20"):
        model = model.to(memory_format=torch.channels_last)
    params = dict(cfg["grace"])
    params.update(world_size=world, fused=True)
    grc = grace_b200.grace_from_params(params)
    opt = torch.optim.SGD(model.parameters(), lr=0.01, momentum=0.9)
    named = list(model.named_parameters())

    def step(batch, amp):
        opt.zero_grad()
        loss = forward_loss(model, cfg, batch, amp)
        loss.backward()
        for name, p in named:
            if p.grad is not None:
                new = grc.step(p.grad.data, name)
                if new.data_ptr() != p.grad.data_ptr():
                    p.grad.data.copy_(new.view_as(p.grad))
        opt.step()
        return loss

    return step, len(named), grc


def build_ours(cfg, device, world):
    import torch

    import grace_b200
    from grace_b200 import models
    from grace_b200.optim import FusedSGD
    from grace_b200.parallel import DistributedOptimizer
    from grace_b200.parallel.flat import FlatParams

    torch.manual_seed(0)
    if cfg["model"] == "bert_large" and cfg.get("bert_impl", "hf") == "hf":
        model = hf_bert_large().to(device)      # the same model class as the reference arm
    else:
        model = getattr(models, cfg["model"])().to(device)
    if cfg["model"] in ("resnet50", "resnet20"):   # VGG-16 stays NCHW: the reference arm's PowerSGD needs it
        model = model.to(memory_format=torch.channels_last)
    named = list(model.named_parameters())
    params = dict(cfg["grace"])
    params.update(world_size=world, fused=True)
    for key in ("overlap_sms", "comm_sms", "nvls", "nvls_min_world"):
        if cfg.get(key) is not None:
            params[key] = cfg[key]
    grc = grace_b200.grace_from_params(params)
    fused_flat = getattr(grc, "_kind", None) in ("sparse", "quant", "powersgd")
    if fused_flat:
        flat = FlatParams(named, bucket_bytes=cfg.get("bucket_bytes"))
        opt = FusedSGD(model.parameters(), lr=0.01, momentum=0.9, flat=flat)
        opt = DistributedOptimizer(opt, grace=grc, named_parameters=named, flat=flat, always_hook=True)
        launches = len(flat.buckets) + 1
    else:
        opt = FusedSGD(model.parameters(), lr=0.01, momentum=0.9)
        opt = DistributedOptimizer(opt, grace=grc, named_parameters=named, always_hook=True)
        launches = 1 + len(named)

    def step(batch, amp):
        opt.zero_grad()
        loss = forward_loss(model, cfg, batch, amp)
        loss.backward()
        opt.step()
        return loss

    return step, launches, grc


def hf_bert_large():
    """BERT-large for pre-training (MLM + NSP heads) from the transformers package, random weights."""
    from transformers import BertConfig, BertForPreTraining

    return BertForPreTraining(BertConfig(vocab_size=30522, hidden_size=1024, num_hidden_layers=24,
                                         num_attention_heads=16, intermediate_size=4096,
                                         max_position_embeddings=512))


def build_reference(cfg, device, world):
    """The unmodified reference from baseline/_ref: its compressor, memory and
    communicator classes over torch.distributed (NCCL), applied per parameter
    after backward as in its own example loop, with torch.optim.SGD."""
    import torch

    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "grace_dl", "dist")):
        raise RuntimeError("baseline/_ref/grace_dl/dist is missing (reference not installed)")
    for mod in [m for m in sys.modules if m == "grace_dl" or m.startswith("grace_dl.")]:
        del sys.modules[mod]
    sys.path.insert(0, ref_root)
    import grace_dl  # noqa: F401
    assert os.path.abspath(grace_dl.__file__).startswith(os.path.abspath(ref_root)), grace_dl.__file__

    g = cfg["grace"]
    if g["compressor"] == "dgc":
        from grace_dl.dist.communicator.allgather import Allgather
        from grace_dl.dist.compressor.dgc import DgcCompressor
        from grace_dl.dist.memory.dgc import DgcMemory

        grc = Allgather(DgcCompressor(g["compress_ratio"]), DgcMemory(g["momentum"], False, world), world)
    elif g["compressor"] == "powersgd":
        from grace_dl.dist.communicator.allreduce import Allreduce
        from grace_dl.dist.compressor.powersgd import PowerSGDCompressor
        from grace_dl.dist.memory.powersgd import PowerSGDMemory

        comp = PowerSGDCompressor(rank=g["compress_rank"], use_memory=True, world_size=world)
        grc = Allreduce(comp, PowerSGDMemory(comp.q_memory, g["compress_rank"]), world)
    else:
        from grace_dl.dist.helper import grace_from_params

        p = dict(g)
        p["world_size"] = world
        grc = grace_from_params(p)

    torch.manual_seed(0)
    if cfg["model"] == "bert_large":
        model = hf_bert_large().to(device)
    elif cfg["model"] == "resnet20":
        from grace_b200.models import resnet20  # torchvision has no CIFAR ResNet-20

        model = resnet20().to(device)
    else:
        import torchvision

        model = getattr(torchvision.models, cfg["model"])(weights=None).to(device)
        if g["compressor"] != "powersgd":  # the reference's PowerSGD calls .view() on the gradient: needs NCHW weights
            model = model.to(memory_format=torch.channels_last)
    opt = torch.optim.SGD(model.parameters(), lr=0.01, momentum=0.9)

    def step(batch, amp):
        opt.zero_grad()
        loss = forward_loss(model, cfg, batch, amp)
        loss.backward()
        for name, p in model.named_parameters():
            if p.grad is None:
                continue
            new = grc.step(p.grad.data, name)
            p.grad.data.copy_(new.view_as(p.grad))
        opt.step()
        return loss

    return step, 0, grc


# ----------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="resnet50_dgc", choices=sorted(CONFIGS))
    ap.add_argument("--batch", type=int, default=None, help="override the per-GPU batch (invalidates the headline)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--api", default="optimizer", choices=["optimizer", "loop"],
                    help="ours: DistributedOptimizer over flat buckets (default) or the reference-style "
                         "per-parameter grc.step loop with torch.optim.SGD (drop-in usage)")
    ap.add_argument("--bucket-mb", type=float, default=None,
                    help="exchange gradients in buckets of this size from backward hooks, next to the rest of backward "
                         "(default: the config's own bucket size; 0 = one bucket after backward)")
    ap.add_argument("--overlap-sms", type=int, default=None, help="SMs of an exchange that runs next to backward")
    ap.add_argument("--nvls", action="store_true", help="push transport (multimem.st) for the quantised codecs")
    ap.add_argument("--bert-impl", default="hf", choices=["hf", "own"],
                    help="ours, bert_qsgd: transformers' BertForPreTraining as in the reference arm (default) or "
                         "this package's own BERT")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    try:
        import torch
    except Exception as e:  # pragma: no cover
        print(json.dumps({"impl": args.impl, "unavailable": "torch import failed: %s" % e}))
        return 0
    import torch.distributed as dist

    cfg = dict(CONFIGS[args.config])
    if args.batch:
        cfg["batch"] = args.batch
    if args.bucket_mb is not None:
        cfg["bucket_bytes"] = int(args.bucket_mb * (1 << 20)) or None
    elif cfg.get("bucket_mb"):
        cfg["bucket_bytes"] = int(cfg["bucket_mb"] * (1 << 20))
    cfg["bert_impl"] = args.bert_impl
    if args.overlap_sms is not None:
        cfg["overlap_sms"] = args.overlap_sms
    if args.nvls:
        cfg["nvls"], cfg["nvls_min_world"] = True, 2
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        if rank == 0:
            print(json.dumps({"impl": args.impl, "unavailable": "no CUDA device"}))
        return 0
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    torch.backends.cudnn.benchmark = True
    amp = cfg["dtype"] == "bf16"

    try:
        if args.impl == "reference":
            step, launches, grc = build_reference(cfg, device, world)
        elif args.api == "loop":
            step, launches, grc = build_ours_loop(cfg, device, world)
        else:
            step, launches, grc = build_ours(cfg, device, world)
    except Exception as e:
        if rank == 0:
            print(json.dumps({"impl": args.impl, "unavailable": "%s: %s" % (type(e).__name__, str(e).splitlines()[0][:200])}))
        dist.destroy_process_group()
        return 0

    def barrier_sync():
        dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident inputs: kernel-side number ----
    batches = [make_batch(cfg, device, seed=1000 * rank + i) for i in range(2)]
    try:
        for i in range(args.warmup):
            step(batches[i % 2], amp)
        torch.cuda.synchronize()
    except Exception as e:
        if rank == 0:
            print(json.dumps({"impl": args.impl, "unavailable": "%s during warm-up: %s" % (
                type(e).__name__, str(e).splitlines()[0][:200])}))
        dist.destroy_process_group()
        return 0
    barrier_sync()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(batches[i % 2], amp)
    e1.record()
    barrier_sync()
    ms = torch.tensor([e0.elapsed_time(e1)], device=device)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_total = float(ms)
    clocks = sampler.stop() if rank == 0 else None
    if hasattr(grc, "check"):
        grc.check()

    # ---- end to end: pinned host batches -> H2D every step, loss read back every step ----
    e2e = None
    if not args.no_e2e:
        host = [make_batch(cfg, device, seed=77 + 1000 * rank + i, pinned=True) for i in range(3)]
        h2d_bytes = sum(t.numel() * t.element_size() for t in host[0])
        copy_stream = torch.cuda.Stream()

        def fetch(i):
            with torch.cuda.stream(copy_stream):
                dev = [t.to(device, non_blocking=True) for t in host[i % len(host)]]
                ev = torch.cuda.Event()
                ev.record(copy_stream)
            return dev, ev

        for i in range(2):  # warm the copy path
            dev, ev = fetch(i)
            torch.cuda.current_stream().wait_event(ev)
            float(step(dev, amp))
        barrier_sync()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        nxt = fetch(0)
        # every step's loss is copied to pinned host memory and read there; the read of step i happens after
        # step i + 1 has been queued, so the host never drains the GPU between steps (the last one is read
        # before the closing event)
        loss_pin = [torch.zeros((), dtype=torch.float32).pin_memory() for _ in range(2)]
        loss_ev = [torch.cuda.Event(), torch.cuda.Event()]
        loss_host = float("nan")
        for i in range(args.steps):
            dev, ev = nxt
            torch.cuda.current_stream().wait_event(ev)
            if i + 1 < args.steps:
                nxt = fetch(i + 1)  # prefetch the next batch while this one trains
            loss = step(dev, amp)
            for t in dev:
                t.record_stream(torch.cuda.current_stream())
            loss_pin[i & 1].copy_(loss.detach().float(), non_blocking=True)   # device -> host copy of the step's result
            loss_ev[i & 1].record()
            if i > 0:
                loss_ev[(i - 1) & 1].synchronize()
                loss_host = float(loss_pin[(i - 1) & 1])
        loss_ev[(args.steps - 1) & 1].synchronize()
        loss_host = float(loss_pin[(args.steps - 1) & 1])
        f1.record()
        barrier_sync()
        ms2 = torch.tensor([f0.elapsed_time(f1)], device=device)
        dist.all_reduce(ms2, op=dist.ReduceOp.MAX)
        e2e = {"value": cfg["batch"] * world * args.steps / (float(ms2) / 1e3), "unit": "samples/s",
               "ms_per_step": float(ms2) / args.steps, "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": 4,
               "last_loss": loss_host}

    if rank == 0:
        value = cfg["batch"] * world * args.steps / (ms_total / 1e3)
        line = {
            "metric": "training samples/sec (%s)" % args.config, "value": value, "unit": "samples/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_total / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": cfg["dtype"],
            "data": "synthetic N(0,1) inputs, uniform labels, random-init weights", "impl": args.impl, "api": args.api,
            "config": {"model": cfg["model"], "global_batch": cfg["batch"] * world,
                       "seq_len": cfg.get("seq"), "parallelism": "dp%d" % world, "compression": cfg["grace"],
                       "bucket_mb": (cfg["bucket_bytes"] / (1 << 20)) if cfg.get("bucket_bytes") else None,
                       "exchange": "buckets launched from gradient hooks next to backward" if cfg.get("bucket_bytes")
                                   else "one fused exchange after backward",
                       "l2": "no flush: a step streams its batch (%.1f MB), parameters, gradients, optimizer state "
                             "and activations (%.0f MB of device memory in use), far beyond the 126 MB L2" % (
                           sum(t.numel() * t.element_size() for t in batches[0]) / 1e6,
                           torch.cuda.max_memory_allocated() / 1e6)},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches * args.steps,
        }
        print(json.dumps(line))
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
