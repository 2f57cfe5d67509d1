"""SM clock and throttle-reason sampling with ``nvidia-smi`` while a measurement runs (read-only queries).

``ClockSampler(index).start()`` streams one sample every 200 ms; every sample is stamped with the host time at
which it was read, so one sampler can serve many consecutive measurements: ``window(t0, t1)`` summarises the
samples that fall into a timed region (median SM MHz of the busiest half, maximum clock, reasons seen)."""
from __future__ import annotations

import statistics
import subprocess
import threading
import time


class ClockSampler:
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    REASONS = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index=0, period_ms=200):
        self.index, self.period_ms = index, period_ms
        self.proc = None
        self.samples = []          # (host time, sm MHz, max MHz, power W, set(reasons))

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", str(self.period_ms)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm, mx, pw = float(f[0]), float(f[1]), float(f[2])
            except ValueError:
                continue
            rs = {n for n, v in zip(self.REASONS, f[3:7]) if v.lower().startswith("active")}
            self.samples.append((time.time(), sm, mx, pw, rs))

    def window(self, t0, t1):
        got = [s for s in self.samples if t0 <= s[0] <= t1]
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        if not got:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm = sorted(s[1] for s in got)
        load = sm[len(sm) // 2:]
        reasons = set()
        for s in got:
            reasons |= s[4]
        return {"sm_mhz": statistics.median(load), "sm_max_mhz": max(s[2] for s in got), "reasons": sorted(reasons),
                "power_w": round(max(s[3] for s in got), 1), "samples": len(got)}

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
