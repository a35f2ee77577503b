"""Read-only sampling of GPU clocks and throttle reasons while a benchmark runs.

Starts ``nvidia-smi --query-gpu=... -lms`` as a child process, stops it after the timed
region and summarises: median SM clock under load, max SM clock, and which throttle
reasons were active.  Nothing here changes a GPU setting.
"""
from __future__ import annotations

import os
import shutil
import statistics
import subprocess
import tempfile

_FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
           "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
           "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    def __init__(self, gpu_index: int | None = None, period_ms: int = 100):
        self.gpu_index = gpu_index
        self.period_ms = period_ms
        self._proc = None
        self._file = None

    def start(self) -> "ClockSampler":
        exe = shutil.which("nvidia-smi")
        if exe is None:
            return self
        self._file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        cmd = [exe, f"--query-gpu={_FIELDS}", "--format=csv,noheader,nounits", "-lms", str(self.period_ms)]
        if self.gpu_index is not None:
            cmd += ["-i", str(self.gpu_index)]
        self._proc = subprocess.Popen(cmd, stdout=self._file, stderr=subprocess.DEVNULL)
        return self

    def stop(self) -> dict:
        if self._proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self._proc.terminate()
        try:
            self._proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self._proc.kill()
        self._file.flush()
        self._file.seek(0)
        sm, smax, power, reasons = [], [], [], set()
        for line in self._file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); smax.append(float(parts[2])); power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        self._file.close()
        try:
            os.unlink(self._file.name)
        except OSError:
            pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        busy = [c for c, p in zip(sm, power) if p >= 0.5 * max(power)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(smax), "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(power)}

    def __enter__(self):
        return self.start()

    def __exit__(self, *exc):
        self.result = self.stop()
