#!/usr/bin/env python
"""DistributedDataParallel with GRACE as its communication hook.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/ddp_hook_example.py
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist
from torch.nn.parallel import DistributedDataParallel as DDP

from grace_b200 import grace_from_params
from grace_b200.models import resnet20
from grace_b200.parallel.ddp_hook import register_grace_hook


def main():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    cuda = torch.cuda.is_available()
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29502")
    dist.init_process_group("nccl" if cuda else "gloo", rank=rank, world_size=world)
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(device)
    torch.manual_seed(0)
    model = DDP(resnet20().to(device), device_ids=[device.index] if cuda else None)
    grc = grace_from_params({"compressor": "qsgd", "memory": "residual", "communicator": "allgather",
                             "quantum_num": 64, "world_size": world, "fused": cuda})
    register_grace_hook(model, grc)
    opt = torch.optim.SGD(model.parameters(), lr=0.05, momentum=0.9)
    gen = torch.Generator().manual_seed(rank)
    for step in range(10):
        x = torch.randn(32, 3, 32, 32, generator=gen).to(device)
        y = torch.randint(0, 10, (32,), generator=gen).to(device)
        opt.zero_grad()
        loss = torch.nn.functional.cross_entropy(model(x), y)
        loss.backward()
        opt.step()
        if rank == 0:
            print("step %d loss %.4f" % (step, loss.item()))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
