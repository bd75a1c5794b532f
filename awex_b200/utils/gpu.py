"""GPU diagnostics: nvidia-smi text, torch memory snapshots, and a clock /
throttle-reason sampler for benchmarks.  Everything here only *reads* device
state (`awex/util/gpu.py:29-78` in the reference covers the first two)."""

from __future__ import annotations

import os
import shutil
import statistics
import subprocess
import tempfile
import time
from typing import Dict, List, Optional

import torch

from awex_b200 import logging

logger = logging.getLogger(__name__)

_QUERY = (
    "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
    "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
)


def get_gpu_status() -> str:
    exe = shutil.which("nvidia-smi")
    if exe is None:
        return "nvidia-smi not available"
    try:
        return subprocess.run(
            [exe, "--query-gpu=name,utilization.gpu,memory.used,memory.total", "--format=csv"],
            capture_output=True, text=True, timeout=20,
        ).stdout.strip()
    except Exception as exc:  # diagnostics must never break the caller
        return f"nvidia-smi failed: {exc}"


def print_gpu_status(stage: str) -> None:
    logger.info(f"GPU status for {stage}:\n{get_gpu_status()}")


def print_current_gpu_status(stage: str) -> None:
    """What torch and the driver say about this process's GPU memory
    (`awex/util/gpu.py:57-78`)."""
    from awex_b200.utils.common import pretty_bytes

    if not torch.cuda.is_available():
        logger.info(f"Device cpu memory status for [{stage}]: no GPU")
        return
    free, total = torch.cuda.mem_get_info()
    logger.info(
        f"Device cuda memory status for [{stage}]: torch allocated {pretty_bytes(torch.cuda.memory_allocated())}, "
        f"torch reserved {pretty_bytes(torch.cuda.memory_reserved())} device mem_free {pretty_bytes(free)}, "
        f"device occupy {pretty_bytes(total - free)}"
    )


def memory_snapshot(tag: str = "") -> Dict[str, int]:
    if not torch.cuda.is_available():
        return {}
    free, total = torch.cuda.mem_get_info()
    snap = {
        "allocated": torch.cuda.memory_allocated(), "reserved": torch.cuda.memory_reserved(),
        "max_allocated": torch.cuda.max_memory_allocated(), "free": free, "total": total,
    }
    if os.environ.get("AWEX_MEM_DEBUG") == "1":
        logger.info(f"[mem {tag}] " + " ".join(f"{k}={v / 2**30:.2f}GiB" for k, v in snap.items()))
    return snap


class ClockSampler:
    """Samples SM clocks and throttle reasons with ``nvidia-smi -lms`` while a
    timed region runs.  Read-only: never sets or resets any clock."""

    def __init__(self, gpu_indices: Optional[List[int]] = None, period_ms: int = 200):
        self.exe = shutil.which("nvidia-smi")
        self.period_ms = period_ms
        self.gpu_indices = gpu_indices
        self.proc = None
        self.path = None

    def __enter__(self):
        if self.exe is None:
            return self
        fd, self.path = tempfile.mkstemp(prefix="awex_clocks_", suffix=".csv")
        os.close(fd)
        cmd = [self.exe, f"--query-gpu={_QUERY}", "--format=csv,noheader,nounits", "-lms", str(self.period_ms)]
        if self.gpu_indices:
            cmd += ["-i", ",".join(str(i) for i in self.gpu_indices)]
        self.proc = subprocess.Popen(cmd, stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        time.sleep(0.05)
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(self.period_ms / 1000.0)  # let one more sample land
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        return False

    def summary(self) -> Dict[str, object]:
        out: Dict[str, object] = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if not self.path or not os.path.exists(self.path):
            out["reasons"] = ["nvidia-smi unavailable"]
            return out
        clocks, maxes, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    clocks.append(float(parts[1]))
                    maxes.append(float(parts[2]))
                    power.append(float(parts[3]))
                except ValueError:
                    continue
                for name, val in zip(names, parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        try:
            os.unlink(self.path)
        except OSError:
            pass
        if clocks:
            out.update(sm_mhz=statistics.median(clocks), sm_max_mhz=max(maxes), power_w_max=max(power), samples=len(clocks))
        out["reasons"] = sorted(reasons)
        return out
