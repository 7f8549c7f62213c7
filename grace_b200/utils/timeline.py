"""Timeline of gradient exchanges in the Chrome trace format (open with chrome://tracing or Perfetto).

The reference only re-exports Horovod's ``start_timeline`` / ``stop_timeline``
(``patch_files/horovod/torch/__init__.py:37``, ``mpi_ops.py:36-37``), which trace Horovod's own negotiation
and collectives.  Here the communicators themselves report every exchange:

    from grace_b200.utils import timeline
    timeline.start_timeline("trace_rank%d.json" % rank)
    ... training steps ...
    timeline.stop_timeline()

Each exchange becomes two complete ("X") events of process ``rank``: on the *host* track the time the call
spent queueing work, on the *device* track the time between two CUDA events recorded on the launching stream
around the exchange (resolved when the timeline is stopped, so recording never synchronises).  Arguments carry
the tensor / bucket name, element count, payload bytes and the kernel family.
"""
from __future__ import annotations

import json
import os
import threading
import time
from typing import Any, Dict, List, Optional

import torch

_HOST_TID, _DEVICE_TID = 0, 1


class Timeline:
    def __init__(self, path: str, rank: Optional[int] = None):
        self.path = path
        if rank is None:
            rank = int(os.environ.get("RANK", "0"))
        self.rank = rank
        self._lock = threading.Lock()
        self._events: List[Dict[str, Any]] = []
        self._pending = []            # (name, cat, args, ev0, ev1)
        self._t0 = time.perf_counter()
        self._base = None             # CUDA event recorded at _t0_dev (host time) on first device use
        self._t0_dev = 0.0

    def _now_us(self) -> float:
        return (time.perf_counter() - self._t0) * 1e6

    def begin(self, name: str, cat: str = "exchange", device: bool = False, **args):
        tok = {"name": name, "cat": cat, "args": args, "ts": self._now_us(), "ev0": None}
        if device and torch.cuda.is_available():
            if self._base is None:
                self._base = torch.cuda.Event(enable_timing=True)
                self._base.record()
                self._t0_dev = self._now_us()
            tok["ev0"] = torch.cuda.Event(enable_timing=True)
            tok["ev0"].record()
        return tok

    def end(self, tok, **more_args) -> None:
        args = dict(tok["args"], **more_args)
        ts = tok["ts"]
        ev = {"name": tok["name"], "cat": tok["cat"], "ph": "X", "pid": self.rank, "tid": _HOST_TID, "ts": ts,
              "dur": max(self._now_us() - ts, 0.0), "args": args}
        with self._lock:
            self._events.append(ev)
            if tok["ev0"] is not None:
                ev1 = torch.cuda.Event(enable_timing=True)
                ev1.record()
                self._pending.append((tok["name"], tok["cat"], args, tok["ev0"], ev1))

    def instant(self, name: str, **args) -> None:
        with self._lock:
            self._events.append({"name": name, "ph": "i", "s": "p", "pid": self.rank, "tid": _HOST_TID,
                                 "ts": self._now_us(), "args": args})

    def close(self) -> str:
        with self._lock:
            if self._pending:
                torch.cuda.synchronize()
                for name, cat, args, ev0, ev1 in self._pending:
                    start = self._t0_dev + self._base.elapsed_time(ev0) * 1e3
                    self._events.append({"name": name, "cat": cat, "ph": "X", "pid": self.rank, "tid": _DEVICE_TID,
                                         "ts": start, "dur": ev0.elapsed_time(ev1) * 1e3, "args": args})
                self._pending = []
            meta = [
                {"name": "process_name", "ph": "M", "pid": self.rank, "args": {"name": "rank %d" % self.rank}},
                {"name": "thread_name", "ph": "M", "pid": self.rank, "tid": _HOST_TID, "args": {"name": "host (queueing)"}},
                {"name": "thread_name", "ph": "M", "pid": self.rank, "tid": _DEVICE_TID, "args": {"name": "device (CUDA events)"}},
            ]
            with open(self.path, "w") as f:
                json.dump({"traceEvents": meta + self._events, "displayTimeUnit": "ms"}, f)
        return self.path


_active: Optional[Timeline] = None


def start_timeline(file_path: str, mark_cycles: bool = False, rank: Optional[int] = None) -> Timeline:
    """Start recording (``mark_cycles`` is accepted for signature parity with Horovod and ignored)."""
    global _active
    if _active is not None:
        _active.close()
    _active = Timeline(file_path, rank)
    return _active


def stop_timeline() -> Optional[str]:
    """Stop recording and write the trace; returns its path (None when no timeline was active)."""
    global _active
    tl, _active = _active, None
    return tl.close() if tl is not None else None


def active() -> Optional[Timeline]:
    return _active
