#!/usr/bin/env python
"""cifar10-fast (DAWNBench ResNet-9) with compressed gradient exchange, after the reference's
``examples/dist/CIFAR10-dawndist/dawn.py``: batch 512, piecewise-linear learning rate peaking at epoch 5, nesterov
SGD with weight decay, random crop + flip + cutout, gradients passed through ``grc.step`` parameter by parameter.
Unlike the reference's script every flag is honoured.  Data: CIFAR-10 tensors from ``--data`` (a ``.pt`` file with
``x_train`` uint8 N x 32 x 32 x 3, ``y_train``, ``x_test``, ``y_test``) or, without it, a synthetic set of the same shape.

    python examples/cifar10_fast_dawn.py --epochs 2 --train-size 2048
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/cifar10_fast_dawn.py \
        --compressor dgc --memory dgc --communicator allgather --compress-ratio 0.01 --fused
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from grace_dl.dist.helper import grace_from_params
from grace_b200.models import resnet9
from grace_b200.utils.metrics import DeviceTimer, TableLogger
from grace_b200.utils.training import PiecewiseLinear, cutout, evaluate, random_crop, random_flip, train_epoch

MEAN = torch.tensor([0.4914, 0.4822, 0.4465]).view(1, 3, 1, 1)
STD = torch.tensor([0.2471, 0.2435, 0.2616]).view(1, 3, 1, 1)


def load_data(path, train_size, test_size, seed):
    if path:
        blob = torch.load(path)
        xs = [blob["x_train"], blob["x_test"]]
        ys = [blob["y_train"].long(), blob["y_test"].long()]
        xs = [(x.permute(0, 3, 1, 2).float() / 255.0 - MEAN) / STD for x in xs]
        return xs[0], ys[0], xs[1], ys[1]
    g = torch.Generator().manual_seed(seed)          # synthetic: class-dependent mean so that there is signal to learn
    def make(n):
        y = torch.randint(0, 10, (n,), generator=g)
        x = torch.randn(n, 3, 32, 32, generator=g) + 0.5 * torch.randn(10, 3, 1, 1, generator=torch.Generator().manual_seed(7))[y]
        return x, y
    xtr, ytr = make(train_size)
    xte, yte = make(test_size)
    return xtr, ytr, xte, yte


def batches(x, y, batch, device, perm=None):
    idx = perm if perm is not None else torch.arange(x.shape[0])
    for i in range(0, idx.numel() - batch + 1, batch):
        sel = idx[i : i + batch]
        yield x[sel].to(device, non_blocking=True), y[sel].to(device, non_blocking=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--compressor", default="none")
    ap.add_argument("--memory", default="none")
    ap.add_argument("--communicator", default="allreduce")
    ap.add_argument("--compress-ratio", type=float, default=0.01)
    ap.add_argument("--fused", action="store_true")
    ap.add_argument("--epochs", type=int, default=24)
    ap.add_argument("--batch", type=int, default=512, help="global batch, split over the ranks")
    ap.add_argument("--peak-lr", type=float, default=0.4)
    ap.add_argument("--peak-epoch", type=float, default=5)
    ap.add_argument("--momentum", type=float, default=0.9)
    ap.add_argument("--weight-decay", type=float, default=5e-4)
    ap.add_argument("--data", default="")
    ap.add_argument("--train-size", type=int, default=50000)
    ap.add_argument("--test-size", type=int, default=10000)
    ap.add_argument("--seed", type=int, default=0)
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

    xtr, ytr, xte, yte = load_data(args.data, args.train_size, args.test_size, args.seed)
    shard = torch.arange(rank, xtr.shape[0], world)          # every rank trains on its own shard
    xtr, ytr = xtr[shard], ytr[shard]
    local_batch = max(1, args.batch // world)
    steps_per_epoch = xtr.shape[0] // local_batch

    torch.manual_seed(args.seed)                              # identical replicas
    model = resnet9().to(device)
    optimizer = torch.optim.SGD(model.parameters(), lr=0.0, momentum=args.momentum, nesterov=True,
                                weight_decay=args.weight_decay)
    schedule = PiecewiseLinear([0, args.peak_epoch, args.epochs], [0.0, args.peak_lr, 0.0])
    grc = grace_from_params({"compressor": args.compressor, "memory": args.memory, "communicator": args.communicator,
                             "compress_ratio": args.compress_ratio, "world_size": world, "fused": args.fused,
                             "momentum": args.momentum})
    gen = torch.Generator().manual_seed(1000 + rank)
    augment = lambda x: cutout(random_flip(random_crop(x, 32, 4, gen), gen), 8, gen)   # noqa: E731
    log = TableLogger()
    step = 0
    for epoch in range(args.epochs):
        perm = torch.randperm(xtr.shape[0], generator=gen)
        with DeviceTimer(device) as timer:
            tr = train_epoch(model, batches(xtr, ytr, local_batch, device, perm), optimizer,
                             grace=grc if world > 1 or args.fused else None, lr_schedule=schedule, step0=step,
                             steps_per_epoch=steps_per_epoch, augment=augment)
        secs = timer.ms / 1e3
        step += tr["steps"]
        te = evaluate(model, batches(xte, yte, 1000 if xte.shape[0] >= 1000 else xte.shape[0], device))
        if rank == 0:
            log.append({"epoch": epoch + 1, "lr": schedule(step / max(steps_per_epoch, 1)), "train loss": tr["loss"],
                        "train acc": tr["acc"], "test acc": te["acc"], "epoch s": secs})
    if hasattr(grc, "check"):
        grc.check()
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
