"""Sample a GPU's SM clock and throttle reasons with ``nvidia-smi`` while a benchmark runs.

Only reads settings; nothing about the GPU is changed.  Used by ``bench.py`` and the scripts
under ``benchmarks/`` so that every reported time comes with the clocks it was measured at.
"""

from __future__ import annotations

import statistics
import subprocess
import tempfile
from pathlib import Path


class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASONS = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, gpu_index: int = 0, period_ms: int = 200):
        self.path = Path(tempfile.mkstemp(prefix="clocks_", suffix=".csv")[1])
        self.gpu = gpu_index
        self.period_ms = period_ms
        self.proc = None

    def start(self) -> "ClockSampler":
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms",
                 str(self.period_ms), "-i", str(self.gpu)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        return self

    def stop(self) -> dict:
        """``{"sm_mhz": median, "sm_max_mhz": ..., "samples": n, "reasons": [...]}``."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, power, reasons = [], [], [], set()
        for line in self.path.read_text().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, flag in zip(self.REASONS, parts[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        self.path.unlink(missing_ok=True)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}

    def __enter__(self):
        return self.start()

    def __exit__(self, *exc):
        self.result = self.stop()
        return False
