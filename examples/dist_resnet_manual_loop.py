#!/usr/bin/env python
"""The reference's "dist" usage pattern: train, then loop over the named
parameters and pass each gradient through ``grc.step`` before the optimizer
step (cf. ``examples/dist/CIFAR10-dawndist/core.py:195-209`` and
``dawn.py:119-127`` of the reference).  Synthetic CIFAR-shaped data.

    python examples/dist_resnet_manual_loop.py --compressor topk --memory residual --communicator allgather
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/dist_resnet_manual_loop.py --fused
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/dist_resnet_manual_loop.py --host-protocol
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from grace_dl.dist.helper import grace_from_params
from grace_b200.models import resnet20, resnet9


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--compressor", default="topk")
    ap.add_argument("--memory", default="residual")
    ap.add_argument("--communicator", default="allgather")
    ap.add_argument("--compress-ratio", type=float, default=0.01)
    ap.add_argument("--model", default="resnet20", choices=["resnet20", "resnet9"])
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--fused", action="store_true", help="single-kernel exchange on CUDA")
    ap.add_argument("--host-protocol", action="store_true",
                    help="CPU ranks: the exchange protocol in native code over shared memory instead of gloo collectives")
    args = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    cuda = torch.cuda.is_available()
    if world > 1 or cuda:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        dist.init_process_group("nccl" if cuda else "gloo", rank=rank, world_size=world)
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(device)

    torch.manual_seed(0)  # identical replicas (the reference's example never broadcasts its parameters)
    model = (resnet20() if args.model == "resnet20" else resnet9()).to(device)
    optimizer = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9, nesterov=True, weight_decay=5e-4)
    grc = grace_from_params({"compressor": args.compressor, "memory": args.memory, "communicator": args.communicator,
                             "compress_ratio": args.compress_ratio, "world_size": world, "fused": args.fused,
                             "host_protocol": args.host_protocol and not cuda})
    if hasattr(grc, "prepare"):   # shared heaps are created by all ranks together, before the first backward pass
        grc.prepare(list(model.named_parameters()))
    gen = torch.Generator().manual_seed(100 + rank)
    for step in range(args.steps):
        x = torch.randn(args.batch, 3, 32, 32, generator=gen).to(device)
        y = torch.randint(0, 10, (args.batch,), generator=gen).to(device)
        optimizer.zero_grad()
        loss = torch.nn.functional.cross_entropy(model(x), y)
        loss.backward()
        for name, p in model.named_parameters():
            p.grad.copy_(grc.step(p.grad, name))
        optimizer.step()
        if rank == 0 and step % 5 == 0:
            print("step %3d  loss %.4f  %s" % (step, loss.item(), grc.stats()))
    if hasattr(grc, "close"):
        grc.close()
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
