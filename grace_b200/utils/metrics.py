"""Timing, throughput and logging helpers.

The reference only prints: a wall-clock ``Timer`` that synchronises CUDA
(``examples/dist/CIFAR10-dawndist/core.py:14-27``), table / TSV loggers
(``core.py:33-39``, ``dawn.py:72-81``) and ad-hoc ``print`` calls.  Here:

* ``DeviceTimer``: CUDA-event timing of a region on the current stream (falls
  back to ``perf_counter`` on CPU), the way every number in this repository is
  taken;
* ``ThroughputMeter``: samples/s over a window, optionally the max over ranks;
* ``JsonlLogger``: one JSON object per line, rank-0 only by default;
* ``TableLogger``: fixed-width console table like the reference's.
"""
from __future__ import annotations

import json
import time
from typing import Any, Dict, List, Optional

import torch


class DeviceTimer:
    """``with DeviceTimer() as t: ...; t.ms`` (device time of the enclosed work)."""

    def __init__(self, device: Optional[torch.device] = None):
        self.cuda = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
        self.ms = 0.0

    def __enter__(self):
        if self.cuda:
            self._e0 = torch.cuda.Event(enable_timing=True)
            self._e1 = torch.cuda.Event(enable_timing=True)
            self._e0.record()
        else:
            self._t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        if self.cuda:
            self._e1.record()
            self._e1.synchronize()
            self.ms = self._e0.elapsed_time(self._e1)
        else:
            self.ms = (time.perf_counter() - self._t0) * 1e3
        return False


class ThroughputMeter:
    def __init__(self):
        self.samples = 0
        self.ms = 0.0

    def update(self, samples: int, ms: float) -> None:
        self.samples += samples
        self.ms += ms

    def rate(self, across_ranks: bool = False) -> float:
        """samples/s; with ``across_ranks`` the slowest rank's time and the summed sample count."""
        ms, n = self.ms, float(self.samples)
        if across_ranks and torch.distributed.is_available() and torch.distributed.is_initialized():
            dev = "cuda" if torch.cuda.is_available() and torch.distributed.get_backend() == "nccl" else "cpu"
            t = torch.tensor([ms, n], dtype=torch.float64, device=dev)
            tmax = t.clone()
            torch.distributed.all_reduce(tmax, op=torch.distributed.ReduceOp.MAX)
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.SUM)
            ms, n = float(tmax[0]), float(t[1])
        return n / (ms / 1e3) if ms > 0 else 0.0


class JsonlLogger:
    def __init__(self, path: str, rank: int = 0, only_rank0: bool = True):
        self.enabled = (rank == 0) or not only_rank0
        self.path = path
        self.rank = rank

    def log(self, **fields: Any) -> None:
        if not self.enabled:
            return
        fields.setdefault("time", time.time())
        fields.setdefault("rank", self.rank)
        with open(self.path, "a") as f:
            f.write(json.dumps(fields) + "\n")


class TableLogger:
    def __init__(self, width: int = 12):
        self.keys: Optional[List[str]] = None
        self.width = width

    def append(self, row: Dict[str, Any]) -> str:
        lines = []
        if self.keys is None:
            self.keys = list(row.keys())
            lines.append("".join(str(k).rjust(self.width) for k in self.keys))
        cells = []
        for k in self.keys:
            v = row.get(k, "")
            cells.append(("%.4f" % v if isinstance(v, float) else str(v)).rjust(self.width))
        lines.append("".join(cells))
        out = "\n".join(lines)
        print(out)
        return out
