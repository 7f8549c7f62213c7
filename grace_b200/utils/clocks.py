"""SM clock and throttle-reason sampling during a timed region.

Reads ``nvidia-smi --query-gpu`` every 200 ms in a child process (read-only: no
clock, power or mode setting is touched) and condenses the samples into the
record that accompanies a measured number: median SM MHz under load, the
maximum SM clock, and which throttle reasons were seen active.  One sampler can
serve many short measurements: ``summary(t0, t1)`` condenses only the samples
taken between two ``time.time()`` stamps.
"""
from __future__ import annotations

import datetime
import os
import statistics
import subprocess
import tempfile
import time
from typing import Optional


class ClockSampler:
    FIELDS = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASONS = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, device_index: int, period_ms: int = 200):
        self.device_index = device_index
        self.period_ms = period_ms
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits", "-lms",
                 str(self.period_ms), "-i", str(self.device_index)],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None
        return self

    @staticmethod
    def _stamp(text: str) -> Optional[float]:
        try:
            return datetime.datetime.strptime(text.strip(), "%Y/%m/%d %H:%M:%S.%f").timestamp()
        except Exception:
            return None

    def _rows(self):
        rows = []
        try:
            for line in open(self.path).read().strip().splitlines():
                r = [c.strip() for c in line.split(", ")]
                if len(r) >= 10:
                    rows.append(r)
        except Exception:
            pass
        return rows

    def summary(self, t0: Optional[float] = None, t1: Optional[float] = None, slack_s: float = 0.3):
        """Condense the samples taken so far; with ``t0`` / ``t1`` only those stamped inside
        ``[t0 - slack_s, t1 + slack_s]`` (``time.time()`` values)."""
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        rows = self._rows()
        if t0 is not None and t1 is not None:
            rows = [r for r in rows if (lambda s: s is not None and t0 - slack_s <= s <= t1 + slack_s)(self._stamp(r[0]))]
        try:
            sm = [float(r[2]) for r in rows]
            reasons = set()
            for r in rows:
                for name, val in zip(self.REASONS, r[6:10]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            if sm:
                out = {"sm_mhz": statistics.median(sm), "sm_max_mhz": float(rows[0][3]), "reasons": sorted(reasons),
                       "samples": len(sm)}
        except Exception:
            pass
        return out

    def stop(self):
        """Stop sampling and return the summary of all samples."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        try:
            self.proc.terminate()
            self.proc.wait(timeout=5)
        except Exception:
            pass
        out = self.summary()
        try:
            os.unlink(self.path)
        except Exception:
            pass
        self.proc = None
        return out


def now() -> float:
    return time.time()
