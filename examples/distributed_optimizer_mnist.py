#!/usr/bin/env python
"""Horovod-style usage (cf. ``examples/torch/pytorch_mnist.py:106-131`` of the
reference): wrap the optimizer, gradients are exchanged from backward hooks and
collected in ``optimizer.step()``.  Synthetic MNIST-shaped data, no Horovod.

    python examples/distributed_optimizer_mnist.py
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/distributed_optimizer_mnist.py
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from grace_dl.torch.helper import grace_from_params
from grace_dl.torch.optimizer import DistributedOptimizer
from grace_b200.models import MnistNet


def main():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    cuda = torch.cuda.is_available()
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29501")
        dist.init_process_group("nccl" if cuda else "gloo", rank=rank, world_size=world)
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if cuda else torch.device("cpu")
    torch.manual_seed(42)
    model = MnistNet().to(device)
    optimizer = torch.optim.SGD(model.parameters(), lr=0.01 * world, momentum=0.5)
    if world > 1:  # hvd.broadcast_parameters equivalent
        for p in model.parameters():
            dist.broadcast(p.data, 0)
    grc = grace_from_params({"compressor": "topk", "memory": "residual", "communicator": "allgather",
                             "compress_ratio": 0.3, "world_size": world})
    optimizer = DistributedOptimizer(optimizer, grace=grc, named_parameters=model.named_parameters(), always_hook=True)
    gen = torch.Generator().manual_seed(rank)
    for step in range(30):
        x = torch.randn(64, 1, 28, 28, generator=gen).to(device)
        y = torch.randint(0, 10, (64,), generator=gen).to(device)
        optimizer.zero_grad()
        loss = torch.nn.functional.nll_loss(model(x), y)
        loss.backward()
        optimizer.step()
        if rank == 0 and step % 10 == 0:
            print("step %2d loss %.4f" % (step, loss.item()))
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
