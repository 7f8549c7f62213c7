"""Failure detection and host-side fault injection.

The reference has no failure handling of its own (it inherits Horovod's
elastic hooks and a 20 s process-group timeout,
``examples/dist/CIFAR10-dawndist/core.py:225-226``).  Here:

* on the device every wait is bounded and reports a status word that surfaces
  as ``GraceCommError`` (see ``ops/exchange.py``);
* on the host ``HeartbeatMonitor`` keeps one key per rank in the process
  group's store; a rank that stops beating is reported by ``dead_ranks()`` so
  the others can stop launching exchanges that would time out;
* ``FaultPlan`` parses ``GRACE_FAULT`` (for example
  ``skip_publish:rank1:step3``) so tests can make one rank skip a protocol step
  without touching the GPU's health: the peers then see a bounded-wait timeout.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass
from typing import List, Optional


class HeartbeatMonitor:
    def __init__(self, store, rank: int, world: int, interval_s: float = 1.0, timeout_s: float = 10.0,
                 prefix: str = "grace/heartbeat"):
        self.store, self.rank, self.world = store, rank, world
        self.interval_s, self.timeout_s, self.prefix = interval_s, timeout_s, prefix
        self._last = 0.0

    def _key(self, r: int) -> str:
        return "%s/%d" % (self.prefix, r)

    def beat(self, force: bool = True) -> None:
        now = time.time()
        if force or now - self._last >= self.interval_s:
            self.store.set(self._key(self.rank), repr(now))
            self._last = now

    def last_seen(self, r: int) -> Optional[float]:
        try:
            if hasattr(self.store, "check") and not self.store.check([self._key(r)]):
                return None
            return float(self.store.get(self._key(r)).decode())
        except Exception:
            return None

    def dead_ranks(self) -> List[int]:
        now = time.time()
        dead = []
        for r in range(self.world):
            if r == self.rank:
                continue
            seen = self.last_seen(r)
            if seen is None or now - seen > self.timeout_s:
                dead.append(r)
        return dead


class ErrorBoard:
    """Agreement about failures through the process group's store (host side only, no collective).

    A bounded wait that expires is seen by ONE rank; its peers may have finished the same exchange without a
    complaint.  ``vote`` lets every rank learn, at a step boundary, whether any rank failed, so that all of them
    recover together; ``barrier`` is the re-rendezvous after the reset.  Keys carry an epoch number, so the
    records of an earlier recovery are never read again.  (The reference has only the 20 s process-group
    timeout of ``examples/dist/CIFAR10-dawndist/core.py:225-226``.)"""

    def __init__(self, store, rank: int, world: int, prefix: str = "grace/error"):
        self.store, self.rank, self.world, self.prefix = store, rank, world, prefix
        self._votes = 0   # votes are numbered: every rank calls vote() the same number of times

    def _wait(self, keys, timeout_s: float):
        from datetime import timedelta

        self.store.wait(list(keys), timedelta(seconds=timeout_s))

    def vote(self, epoch: int, failed: bool, timeout_s: float = 30.0, info: str = "") -> List[int]:
        """Post this rank's verdict, wait for all others, return the ranks that failed (sorted)."""
        self._votes += 1
        base = "%s/%d/vote%d" % (self.prefix, epoch, self._votes)
        self.store.set("%s/%d" % (base, self.rank), ("1" + info) if failed else "0")
        keys = ["%s/%d" % (base, r) for r in range(self.world)]
        self._wait(keys, timeout_s)
        return [r for r, k in enumerate(keys) if self.store.get(k).decode()[:1] == "1"]

    def barrier(self, epoch: int, timeout_s: float = 30.0, tag: str = "") -> None:
        """Every rank sets its key and waits for all W keys of this epoch (and ``tag``)."""
        base = "%s/%d/barrier%s" % (self.prefix, epoch, tag)
        self.store.set("%s/%d" % (base, self.rank), "1")
        self._wait(["%s/%d" % (base, r) for r in range(self.world)], timeout_s)


@dataclass
class FaultPlan:
    """``action:rankR:stepS`` from the ``GRACE_FAULT`` environment variable."""

    action: str = ""
    rank: int = -1
    step: int = -1

    @classmethod
    def from_env(cls) -> "FaultPlan":
        spec = os.environ.get("GRACE_FAULT", "")
        if not spec:
            return cls()
        parts = spec.split(":")
        plan = cls(action=parts[0])
        for part in parts[1:]:
            if part.startswith("rank"):
                plan.rank = int(part[4:])
            elif part.startswith("step"):
                plan.step = int(part[4:])
        return plan

    def hits(self, action: str, rank: int, step: int) -> bool:
        return self.action == action and (self.rank < 0 or self.rank == rank) and (self.step < 0 or self.step == step)
