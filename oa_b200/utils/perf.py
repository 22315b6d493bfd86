"""Rolling performance statistics, the append-only performance store and profiler ranges.

Parity: Source/Public/Oa/Core/PerfStore.h:1-64 (OaPerfRecord: timestamp, GPU name, metric name, sample count, mean,
stddev, min, max, p50, p95, p99; OaPerfStore: Load / Append / FindLatest / PrintComparison / RecordCount over
`var/perf/OaPerf.dat`), the rolling window of the reference's PerfStat, and the NVTX ranges the reference compiles in
when the header is present (CMakeLists.txt:286-291).  Records are fixed-size little-endian structs so the file can be
appended to by several runs and read back without an index.
"""
from __future__ import annotations

import contextlib
import math
import os
import struct
import time
from collections import deque
from dataclasses import dataclass
from typing import Deque, List, Optional

import torch

from ..core.types import OaStatus, OaStatusCode

_REC = struct.Struct("<q64s64sQ7d")


@dataclass
class OaPerfRecord:
    TimestampNs: int = 0
    GpuName: str = ""
    MetricName: str = ""
    SampleCount: int = 0
    Mean: float = 0.0
    Stddev: float = 0.0
    Min: float = 0.0
    Max: float = 0.0
    P50: float = 0.0
    P95: float = 0.0
    P99: float = 0.0

    def Pack(self) -> bytes:
        return _REC.pack(self.TimestampNs, self.GpuName.encode()[:63], self.MetricName.encode()[:63], self.SampleCount, self.Mean, self.Stddev,
                         self.Min, self.Max, self.P50, self.P95, self.P99)

    @staticmethod
    def Unpack(blob: bytes) -> "OaPerfRecord":
        ts, gpu, metric, n, *vals = _REC.unpack(blob)
        return OaPerfRecord(ts, gpu.split(b"\0")[0].decode(), metric.split(b"\0")[0].decode(), n, *vals)


def _percentile(sorted_vals: List[float], q: float) -> float:
    """Linear interpolation between the closest ranks."""
    if not sorted_vals:
        return 0.0
    pos = q * (len(sorted_vals) - 1)
    lo, hi = int(math.floor(pos)), int(math.ceil(pos))
    return sorted_vals[lo] + (sorted_vals[hi] - sorted_vals[lo]) * (pos - lo)


class OaPerfStat:
    """Statistics over the last `window` samples (all samples when window = 0)."""

    def __init__(self, name: str = "", window: int = 0):
        self.Name = name
        self._v: Deque[float] = deque(maxlen=window or None)
        self.TotalSamples = 0

    def Add(self, value: float) -> None:
        self._v.append(float(value))
        self.TotalSamples += 1

    def Reset(self) -> None:
        self._v.clear()
        self.TotalSamples = 0

    def Count(self) -> int: return len(self._v)
    def Mean(self) -> float: return sum(self._v) / len(self._v) if self._v else 0.0
    def Min(self) -> float: return min(self._v) if self._v else 0.0
    def Max(self) -> float: return max(self._v) if self._v else 0.0

    def Stddev(self) -> float:
        if len(self._v) < 2:
            return 0.0
        m = self.Mean()
        return math.sqrt(sum((x - m) ** 2 for x in self._v) / len(self._v))

    def Percentile(self, q: float) -> float: return _percentile(sorted(self._v), q)

    def ToRecord(self, gpu_name: str) -> OaPerfRecord:
        s = sorted(self._v)
        return OaPerfRecord(time.time_ns(), gpu_name, self.Name, len(s), self.Mean(), self.Stddev(), self.Min(), self.Max(), _percentile(s, 0.5),
                            _percentile(s, 0.95), _percentile(s, 0.99))


class OaPerfStore:
    DEFAULT_PATH = os.path.join("var", "perf", "OaPerf.dat")

    def __init__(self):
        self.Path_ = ""
        self.Records_: List[OaPerfRecord] = []

    def Load(self, path: Optional[str] = None) -> OaStatus:
        self.Path_ = path or self.DEFAULT_PATH
        self.Records_ = []
        if not os.path.exists(self.Path_):
            return OaStatus.Ok()
        with open(self.Path_, "rb") as f:
            blob = f.read()
        if len(blob) % _REC.size:
            return OaStatus(OaStatusCode.DataLoss, f"{self.Path_} is not a whole number of records")
        self.Records_ = [OaPerfRecord.Unpack(blob[i:i + _REC.size]) for i in range(0, len(blob), _REC.size)]
        return OaStatus.Ok()

    def Append(self, record: OaPerfRecord) -> OaStatus:
        if not self.Path_:
            self.Path_ = self.DEFAULT_PATH
        try:
            os.makedirs(os.path.dirname(os.path.abspath(self.Path_)), exist_ok=True)
            with open(self.Path_, "ab") as f:
                f.write(record.Pack())
        except OSError as e:
            return OaStatus(OaStatusCode.Unavailable, str(e))
        self.Records_.append(record)
        return OaStatus.Ok()

    def FindLatest(self, gpu_name: str, metric_name: str) -> Optional[OaPerfRecord]:
        for r in reversed(self.Records_):
            if r.GpuName == gpu_name and r.MetricName == metric_name:
                return r
        return None

    def RecordCount(self) -> int: return len(self.Records_)

    def Comparison(self, metric_name: str, current: OaPerfRecord, gpu_name: str) -> str:
        prev = self.FindLatest(gpu_name, metric_name)
        if prev is None or prev.Mean == 0:
            return f"{metric_name}: {current.Mean:.4f} (no earlier record on {gpu_name})"
        delta = 100.0 * (current.Mean - prev.Mean) / prev.Mean
        return f"{metric_name}: {current.Mean:.4f} vs {prev.Mean:.4f} ({delta:+.2f} %), p95 {current.P95:.4f} vs {prev.P95:.4f}"

    def PrintComparison(self, metric_name: str, current: OaPerfRecord, gpu_name: str, out=print) -> None:
        out(self.Comparison(metric_name, current, gpu_name))


@contextlib.contextmanager
def OaNvtxRange(name: str):
    """Named range for a system profiler's timeline; costs nothing without a GPU."""
    pushed = False
    if torch.cuda.is_available():
        try:
            torch.cuda.nvtx.range_push(name)
            pushed = True
        except Exception:      # the tools extension library may be absent
            pushed = False
    try:
        yield
    finally:
        if pushed:
            torch.cuda.nvtx.range_pop()
