"""SM clock and throttle-reason sampling during a timed region (read-only use of ``nvidia-smi``)."""

from __future__ import annotations

import os
import signal
import statistics
import subprocess
import tempfile

_QUERY = (
    "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
    "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
    "clocks_event_reasons.sw_power_cap"
)


class ClockSampler:
    """Samples every 200 ms between ``start()`` and ``stop()``; ``summary()`` gives the JSON-able record."""

    def __init__(self, gpu_index: int = 0):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self) -> None:
        fd, self.path = tempfile.mkstemp(prefix="moodist-clocks-", suffix=".csv")
        os.close(fd)
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={_QUERY}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(self.gpu_index)],
                stdout=open(self.path, "w"),
                stderr=subprocess.DEVNULL,
            )
        except OSError:
            self.proc = None

    def stop(self) -> None:
        if self.proc is not None:
            self.proc.send_signal(signal.SIGTERM)
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.proc = None

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, val in zip(names, f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        except OSError:
            pass
        finally:
            if self.path and os.path.exists(self.path):
                os.unlink(self.path)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        # under load = the upper half of the samples (idle samples at the edges pull the median down)
        return {
            "sm_mhz": statistics.median(sm),
            "sm_max_mhz": max(mx),
            "reasons": sorted(reasons),
            "samples": len(sm),
        }
