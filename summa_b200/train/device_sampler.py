"""Fail-soft asynchronous GPU telemetry through one persistent `nvidia-smi` child.

The trainer stays the only writer of the metric journal: this module owns the child process
and a reader thread, and hands out bounded, non-blocking batches of samples (`drain`) at
safe boundaries. A missing tool, malformed line, process exit or a full queue becomes a
diagnostic, never an exception in the training loop and never a blocked step
(`summa-train/src/device_sampler.rs:1-120`). The query only READS device state; nothing
here changes a clock, power or mode setting.
"""
from __future__ import annotations

import collections
import queue
import re
import subprocess
import threading
import time
from dataclasses import dataclass, field
from typing import List, Optional

DEFAULT_CAPACITY = 256
MAX_CAPACITY = 4096
MAX_DIAGNOSTICS = 16
MAX_LINE_BYTES = 64 * 1024
QUERY = "index,utilization.gpu,memory.used,memory.total,power.draw,temperature.gpu,clocks.sm"
_SELECTOR = re.compile(r"^(\d{1,4}|GPU-[0-9a-fA-F-]{8,64}|[0-9a-fA-F]{4,8}:[0-9a-fA-F]{2}:[0-9a-fA-F]{2}\.[0-9a-fA-F])$")


class SamplerConfigError(ValueError):
    pass


@dataclass
class DeviceSample:
    collected_at_unix_ms: int
    gpu_utilization: float
    memory_used_mib: float
    memory_total_mib: float
    power_watts: Optional[float]
    temperature_c: Optional[float]
    sm_clock_mhz: Optional[float]

    def as_metric(self, device_index: int = 0, sample_window_seconds: float = 1.0) -> dict:
        """Values of a `device_utilization` metric event (`summa-train/src/metrics.rs:307-329`); the fields
        nvidia-smi cannot report (SM / tensor-core / memory-bandwidth activity) stay absent."""
        return {"sampled_at_unix_ms": int(self.collected_at_unix_ms), "device_index": int(device_index),
                "sample_window_seconds": float(sample_window_seconds),
                "gpu_utilization_percent": float(self.gpu_utilization),
                "memory_used_bytes": int(self.memory_used_mib * 1024 * 1024),
                "memory_total_bytes": int(self.memory_total_mib * 1024 * 1024),
                "power_watts": self.power_watts, "temperature_celsius": self.temperature_c}


@dataclass
class Drain:
    samples: List[DeviceSample] = field(default_factory=list)
    diagnostics: List[str] = field(default_factory=list)


def validate_selector(sel: str) -> str:
    """A physical index, GPU UUID or PCI bus id; passed as ONE argv entry, never via a shell."""
    if not _SELECTOR.match(sel):
        raise SamplerConfigError(f"invalid physical device selector `{sel}`")
    return sel


def _opt(x: str) -> Optional[float]:
    x = x.strip()
    if x in ("N/A", "[N/A]", "[Not Supported]", ""):
        return None
    v = float(x)
    if v != v or v in (float("inf"), float("-inf")):
        raise ValueError("non-finite optional field")
    return v


def parse_line(line: str, now_ms: Optional[int] = None) -> DeviceSample:
    """One `csv,noheader,nounits` row. Utilisation and memory are required (N/A rejects the
    sample); power, temperature and clock stay None when the driver cannot report them."""
    if len(line) > MAX_LINE_BYTES:
        raise ValueError("sample line too long")
    f = [x.strip() for x in line.strip().split(",")]
    if len(f) != 7:
        raise ValueError(f"expected 7 fields, got {len(f)}")
    util = float(f[1])
    if not (0.0 <= util <= 100.0):
        raise ValueError("GPU utilization is outside 0..=100")
    used, total = float(f[2]), float(f[3])
    if used < 0 or total <= 0 or used > total:
        raise ValueError("GPU memory fields are inconsistent")
    return DeviceSample(now_ms if now_ms is not None else int(time.time() * 1000), util, used, total,
                        _opt(f[4]), _opt(f[5]), _opt(f[6]))


class NvidiaSmiSampler:
    def __init__(self, interval_s: float, physical_device: str = "0", capacity: int = DEFAULT_CAPACITY,
                 command: Optional[List[str]] = None):
        """`command` replaces the nvidia-smi argv (tests pass a script that prints rows)."""
        if not (interval_s > 0):
            raise SamplerConfigError("device sampling interval must be positive")
        if not (1 <= capacity <= MAX_CAPACITY):
            raise SamplerConfigError(f"device sample channel capacity must be in 1..={MAX_CAPACITY}")
        validate_selector(physical_device)
        self._q: "queue.Queue[DeviceSample]" = queue.Queue(maxsize=capacity)
        self._diag = collections.deque(maxlen=MAX_DIAGNOSTICS)
        self._dropped = 0
        self._lock = threading.Lock()
        self._stopping = False
        argv = command or ["nvidia-smi", f"--query-gpu={QUERY}", "--format=csv,noheader,nounits", "--id",
                           physical_device, f"--loop-ms={max(1, int(interval_s * 1000))}"]
        try:
            self._proc = subprocess.Popen(argv, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError as e:
            self._proc = None
            self._diag.append(f"nvidia-smi stopped: {e}")
            self._thread = None
            return
        self._thread = threading.Thread(target=self._read, name="device-sampler", daemon=True)
        self._thread.start()

    def _read(self):
        for line in self._proc.stdout:
            if self._stopping:
                break
            if not line.strip():
                continue
            try:
                s = parse_line(line)
            except ValueError as e:
                with self._lock:
                    self._diag.append(f"discarded invalid nvidia-smi sample: {e}")
                continue
            try:
                self._q.put_nowait(s)
            except queue.Full:
                with self._lock:
                    self._dropped += 1
        if not self._stopping:
            rc = self._proc.wait()
            with self._lock:
                self._diag.append(f"nvidia-smi stopped: exit status {rc}")

    def drain(self) -> Drain:
        """Everything collected since the last call; never blocks."""
        out = Drain()
        while True:
            try:
                out.samples.append(self._q.get_nowait())
            except queue.Empty:
                break
        with self._lock:
            out.diagnostics.extend(self._diag)
            self._diag.clear()
            if self._dropped:
                out.diagnostics.append(f"dropped {self._dropped} device samples because the channel was full")
                self._dropped = 0
        return out

    def close(self):
        self._stopping = True
        if self._proc is not None:
            try:
                self._proc.kill()           # the exact child we started
            except OSError:
                pass
            self._proc.wait()
        if self._thread is not None:
            self._thread.join(timeout=2.0)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
