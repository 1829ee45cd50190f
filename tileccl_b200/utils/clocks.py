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
            except subprocess.TimeoutExpired:
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


class NvmlSampler:
    """Same record, taken in-process through NVML (read-only queries) by a thread every few
    milliseconds: fine enough to catch a timed region that lasts a fraction of a second.
    :func:`make_sampler` falls back to :class:`ClockSampler` when NVML is not importable."""

    # nvmlClocksEventReasons bits
    _BITS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}

    def __init__(self, period_ms: int = 10, gpu_index: int = 0):
        import threading

        import pynvml
        self.n = pynvml
        pynvml.nvmlInit()
        self.h = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
        self.index = gpu_index
        self.period = period_ms / 1000.0
        self.rows: list[dict] = []
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._loop, daemon=True)

    def _loop(self):
        import time
        n, h = self.n, self.h
        try:
            sm_max = float(n.nvmlDeviceGetMaxClockInfo(h, n.NVML_CLOCK_SM))
        except Exception:  # noqa: BLE001
            sm_max = 0.0
        get_reasons = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or getattr(n, "nvmlDeviceGetCurrentClocksThrottleReasons")
        while not self._stop.is_set():
            try:
                mask = int(get_reasons(h))
                row = {"index": self.index, "sm": float(n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM)), "sm_max": sm_max,
                       "power": n.nvmlDeviceGetPowerUsage(h) / 1000.0, "active": hex(mask),
                       "hw_slowdown": "Active" if mask & 0x8 else "Not Active", "hw_thermal": "Active" if mask & 0x40 else "Not Active",
                       "sw_thermal": "Active" if mask & 0x20 else "Not Active", "sw_power_cap": "Active" if mask & 0x4 else "Not Active"}
                self.rows.append(row)
            except Exception:  # noqa: BLE001
                pass
            time.sleep(self.period)

    def start(self) -> "NvmlSampler":
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        self._thread.join(timeout=2)

    def summary(self) -> dict:
        self.stop()
        out = summarize(self.rows)
        out["source"] = "nvml"
        return out


def make_sampler(gpu_index: int, period_ms: int = 10):
    """An NVML thread sampler when possible, else the nvidia-smi subprocess sampler."""
    try:
        return NvmlSampler(period_ms=period_ms, gpu_index=gpu_index)
    except Exception:  # noqa: BLE001
        return ClockSampler(period_ms=max(50, period_ms), gpu_index=gpu_index)


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
