"""GPU clock / throttle-reason sampling around a timed region (read-only).

A background ``nvidia-smi`` process writes one CSV line per GPU every 200 ms;
:meth:`ClockSampler.summary` reduces the samples taken under load to the
median SM clock, the maximum clock and the throttle reasons that were active.
Nothing here changes a GPU setting.  The reference samples the same way
(comm_comp/run_all.sh:110-141) but also pins clocks with ``nvidia-smi -lgc``
(comm_comp/pick_clock.sh), which this library never does.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import tempfile

_FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
           "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
           "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    def __init__(self, period_ms: int = 200, gpu_index: int | None = None):
        self.period_ms = period_ms
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self) -> "ClockSampler":
        exe = shutil.which("nvidia-smi")
        if not exe:
            return self
        fd, self.path = tempfile.mkstemp(prefix="tileccl_clocks_", suffix=".csv")
        os.close(fd)
        cmd = [exe, f"--query-gpu={_FIELDS}", "--format=csv,noheader,nounits", "-lms", str(self.period_ms)]
        if self.gpu_index is not None:
            cmd += ["-i", str(self.gpu_index)]
        self.proc = subprocess.Popen(cmd, stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        return self

    def stop(self) -> None:
        if self.proc is not None:
            self.proc.terminate()          # the exact process started above
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
            self.proc = None

    def summary(self) -> dict:
        self.stop()
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if not self.path or not os.path.exists(self.path):
            return out
        rows = parse_samples(open(self.path).read())
        try:
            os.unlink(self.path)
        except OSError:
            pass
        return summarize(rows)


def parse_samples(text: str) -> list[dict]:
    rows = []
    for line in text.splitlines():
        parts = [p.strip() for p in line.split(",")]
        if len(parts) < 9:
            continue
        try:
            rows.append({"index": int(parts[0]), "sm": float(parts[1]), "sm_max": float(parts[2]),
                         "power": float(parts[3]), "active": parts[4],
                         "hw_slowdown": parts[5], "hw_thermal": parts[6], "sw_thermal": parts[7],
                         "sw_power_cap": parts[8]})
        except ValueError:
            continue
    return rows


def summarize(rows: list[dict]) -> dict:
    out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": len(rows)}
    if not rows:
        return out
    pmax = max(r["power"] for r in rows)
    load = [r for r in rows if r["power"] >= 0.5 * pmax] or rows
    clocks = sorted(r["sm"] for r in load)
    out["sm_mhz"] = clocks[len(clocks) // 2]
    out["sm_max_mhz"] = max(r["sm_max"] for r in rows)
    out["power_w_max"] = pmax
    reasons = set()
    for r in load:
        for key, name in (("hw_slowdown", "hw_slowdown"), ("hw_thermal", "hw_thermal_slowdown"),
                          ("sw_thermal", "sw_thermal_slowdown"), ("sw_power_cap", "sw_power_cap")):
            if r[key].lower().startswith("active"):
                reasons.add(name)
    out["reasons"] = sorted(reasons)
    return out
