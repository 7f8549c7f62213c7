"""Training-loop helpers for the CIFAR-style examples.

The reference's DAWNBench example carries its own small training library
(``examples/dist/CIFAR10-dawndist/core.py``: ``PiecewiseLinear`` ``:~60``, ``Crop`` / ``FlipLR`` / ``Cutout``
transforms applied per sample on the host, ``train_epoch`` / ``run_batches`` ``:195-220``; ``dawn.py:90-117``:
24 epochs, learning rate 0 -> 0.4 at epoch 5 -> 0 at the end, per-step updates, weight decay 5e-4 x batch).
Equivalents, written for batched tensors so that augmentation runs on the GPU in a handful of kernels instead of
per-sample NumPy code:

* ``PiecewiseLinear(knots, values)`` - schedule evaluated per step;
* ``random_crop`` / ``random_flip`` / ``cutout`` - batched augmentations, reproducible through a ``torch.Generator``;
* ``train_epoch`` / ``evaluate`` - the manual-loop pattern ``backward -> grc.step per parameter -> optimizer.step``
  (``core.py:202-208``), or a ``DistributedOptimizer`` when one is passed.
"""
from __future__ import annotations

from bisect import bisect_right
from typing import Callable, Dict, Iterable, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F


class PiecewiseLinear:
    """Linear interpolation between ``(knot, value)`` pairs; constant outside the knots."""

    def __init__(self, knots: Sequence[float], values: Sequence[float]):
        if len(knots) != len(values) or len(knots) < 1 or list(knots) != sorted(knots):
            raise ValueError("knots must be sorted and as many as values")
        self.knots, self.values = [float(k) for k in knots], [float(v) for v in values]

    def __call__(self, t: float) -> float:
        k, v = self.knots, self.values
        if t <= k[0]:
            return v[0]
        if t >= k[-1]:
            return v[-1]
        i = bisect_right(k, t)
        w = (t - k[i - 1]) / (k[i] - k[i - 1])
        return v[i - 1] + w * (v[i] - v[i - 1])


def set_lr(optimizer: torch.optim.Optimizer, lr: float) -> None:
    for group in optimizer.param_groups:
        group["lr"] = lr


def random_crop(x: torch.Tensor, size: int, pad: int = 4, generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """Pad by reflection and cut one ``size x size`` window per image (N, C, H, W)."""
    n = x.shape[0]
    xp = F.pad(x, (pad, pad, pad, pad), mode="reflect")
    hi = xp.shape[-1] - size + 1
    ox = torch.randint(0, hi, (n,), generator=generator, device=generator.device if generator else "cpu").to(x.device)
    oy = torch.randint(0, hi, (n,), generator=generator, device=generator.device if generator else "cpu").to(x.device)
    ar = torch.arange(size, device=x.device)
    rows = (oy[:, None] + ar[None, :])[:, :, None].expand(n, size, size)
    cols = (ox[:, None] + ar[None, :])[:, None, :].expand(n, size, size)
    idx = torch.arange(n, device=x.device)[:, None, None].expand(n, size, size)
    return xp.permute(0, 2, 3, 1)[idx, rows, cols].permute(0, 3, 1, 2).contiguous()


def random_flip(x: torch.Tensor, generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """Mirror each image left-right with probability one half."""
    flip = torch.rand(x.shape[0], generator=generator, device=generator.device if generator else "cpu").to(x.device) < 0.5
    return torch.where(flip[:, None, None, None], x.flip(-1), x)


def cutout(x: torch.Tensor, size: int = 8, generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """Zero one ``size x size`` square per image."""
    n, _, h, w = x.shape
    dev = generator.device if generator else "cpu"
    oy = torch.randint(0, h - size + 1, (n,), generator=generator, device=dev).to(x.device)
    ox = torch.randint(0, w - size + 1, (n,), generator=generator, device=dev).to(x.device)
    yy = torch.arange(h, device=x.device)[None, :, None]
    xx = torch.arange(w, device=x.device)[None, None, :]
    hole = (yy >= oy[:, None, None]) & (yy < oy[:, None, None] + size) & (xx >= ox[:, None, None]) & (xx < ox[:, None, None] + size)
    return x.masked_fill(hole[:, None, :, :], 0.0)


def train_epoch(model: torch.nn.Module, batches: Iterable[Tuple[torch.Tensor, torch.Tensor]],
                optimizer: torch.optim.Optimizer, grace=None, lr_schedule: Optional[Callable[[float], float]] = None,
                step0: int = 0, steps_per_epoch: Optional[int] = None,
                augment: Optional[Callable[[torch.Tensor], torch.Tensor]] = None) -> Dict[str, float]:
    """One pass over ``batches``.  With ``grace`` every gradient goes through ``grace.step(grad, name)`` before the
    optimizer step (the reference's manual loop); pass ``grace=None`` when ``optimizer`` is a ``DistributedOptimizer``
    (it exchanges the gradients itself).  Returns mean loss, accuracy and the number of steps taken."""
    model.train()
    named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
    loss_sum = correct = seen = 0.0
    step = step0
    for x, y in batches:
        if lr_schedule is not None:
            set_lr(optimizer, lr_schedule(step / steps_per_epoch if steps_per_epoch else step))
        if augment is not None:
            x = augment(x)
        optimizer.zero_grad()
        logits = model(x)
        loss = F.cross_entropy(logits, y)
        loss.backward()
        if grace is not None:
            for name, p in named:
                if p.grad is not None:
                    new = grace.step(p.grad.data, name)
                    if new.data_ptr() != p.grad.data_ptr():
                        p.grad.data.copy_(new.view_as(p.grad))
        optimizer.step()
        loss_sum += float(loss.detach()) * y.numel()
        correct += float((logits.detach().argmax(1) == y).sum())
        seen += y.numel()
        step += 1
    return {"loss": loss_sum / max(seen, 1), "acc": correct / max(seen, 1), "steps": step - step0}


@torch.no_grad()
def evaluate(model: torch.nn.Module, batches: Iterable[Tuple[torch.Tensor, torch.Tensor]]) -> Dict[str, float]:
    model.eval()
    loss_sum = correct = seen = 0.0
    for x, y in batches:
        logits = model(x)
        loss_sum += float(F.cross_entropy(logits, y, reduction="sum"))
        correct += float((logits.argmax(1) == y).sum())
        seen += y.numel()
    return {"loss": loss_sum / max(seen, 1), "acc": correct / max(seen, 1)}
