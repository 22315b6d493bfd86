"""Column-oriented numeric containers: OaSeries, OaTimeSeries, OaDataFrame and the OHLCV records.

Parity: Source/Public/Oa/Data/Dataframe.h (OaSeries arithmetic / statistics / rolling windows / shifts, OaTimeSeries,
OaDataFrame), Source/Public/Oa/Data/Ohlcv.h (OaRecordOhlcv, OaDataOhlcv).  Columns are contiguous float64 numpy
arrays, so a frame converts to a device tensor with one copy (`ToTensor`).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Sequence, Union

import numpy as np
import torch

OaOhlcvColumns = ("Time", "Open", "High", "Low", "Close", "Volume")
OaOhlcvColumnTimeLegacy = "OaTimestamp"


class OaSeries:
    def __init__(self, data: Union[int, Iterable[float], np.ndarray, None] = None):
        if data is None:
            self._d = np.zeros(0, np.float64)
        elif isinstance(data, (int, np.integer)):
            self._d = np.zeros(int(data), np.float64)
        else:
            self._d = np.array(data, dtype=np.float64).reshape(-1)

    # -- container
    def Size(self) -> int: return self._d.size
    def IsEmpty(self) -> bool: return self._d.size == 0
    def __len__(self) -> int: return self._d.size
    def __getitem__(self, i): return float(self._d[i])
    def __setitem__(self, i, v): self._d[i] = v
    def At(self, i: int) -> float:
        if not 0 <= i < self._d.size:
            raise IndexError(i)
        return float(self._d[i])
    def Front(self) -> float: return float(self._d[0])
    def Back(self) -> float: return float(self._d[-1])
    def Data(self) -> np.ndarray: return self._d
    def Resize(self, n: int) -> None: self._d = np.resize(self._d, n) if n <= self._d.size else np.concatenate([self._d, np.zeros(n - self._d.size)])
    def Reserve(self, n: int) -> None: pass
    def PushBack(self, v: float) -> None: self._d = np.append(self._d, float(v))
    def Clear(self) -> None: self._d = np.zeros(0, np.float64)
    def Fill(self, v: float) -> None: self._d[:] = v
    def CopyFrom(self, src: Sequence[float]) -> None: self._d = np.array(src, dtype=np.float64).reshape(-1)
    def ToList(self) -> List[float]: return self._d.tolist()
    def ToTensor(self, dtype=torch.float32, device="cpu") -> torch.Tensor: return torch.from_numpy(self._d).to(device=device, dtype=dtype)

    # -- arithmetic
    def _other(self, o):
        if isinstance(o, OaSeries):
            if o.Size() != self.Size():
                raise ValueError("series lengths differ")
            return o._d
        return float(o)

    def Add(self, o) -> "OaSeries": return OaSeries(self._d + self._other(o))
    def Sub(self, o) -> "OaSeries": return OaSeries(self._d - self._other(o))
    def Mul(self, o) -> "OaSeries": return OaSeries(self._d * self._other(o))
    def Div(self, o) -> "OaSeries":
        with np.errstate(divide="ignore", invalid="ignore"):
            return OaSeries(self._d / self._other(o))
    def AddInplace(self, o) -> "OaSeries": self._d += self._other(o); return self
    def SubInplace(self, o) -> "OaSeries": self._d -= self._other(o); return self
    def MulInplace(self, o) -> "OaSeries": self._d *= self._other(o); return self
    def DivInplace(self, o) -> "OaSeries":
        with np.errstate(divide="ignore", invalid="ignore"):
            self._d /= self._other(o)
        return self
    __add__, __sub__, __mul__, __truediv__ = Add, Sub, Mul, Div
    __iadd__, __isub__, __imul__, __itruediv__ = AddInplace, SubInplace, MulInplace, DivInplace

    # -- statistics (population variance, as a running-moment implementation gives)
    def Sum(self) -> float: return float(self._d.sum())
    def Mean(self) -> float: return float(self._d.mean()) if self._d.size else 0.0
    def Var(self) -> float: return float(self._d.var()) if self._d.size else 0.0
    def Std(self) -> float: return float(self._d.std()) if self._d.size else 0.0
    def Min(self) -> float: return float(self._d.min())
    def Max(self) -> float: return float(self._d.max())
    def ArgMin(self) -> int: return int(self._d.argmin())
    def ArgMax(self) -> int: return int(self._d.argmax())

    # -- rolling windows: entry i covers [i - window + 1, i]; the first window - 1 entries are NaN
    def _rolling(self, window: int, fn) -> "OaSeries":
        n = self._d.size
        out = np.full(n, np.nan)
        if 0 < window <= n:
            view = np.lib.stride_tricks.sliding_window_view(self._d, window)
            out[window - 1:] = fn(view, axis=1)
        return OaSeries(out)

    def RollingSum(self, window: int) -> "OaSeries": return self._rolling(window, np.sum)
    def RollingMean(self, window: int) -> "OaSeries": return self._rolling(window, np.mean)
    def RollingStd(self, window: int) -> "OaSeries": return self._rolling(window, np.std)
    def RollingMin(self, window: int) -> "OaSeries": return self._rolling(window, np.min)
    def RollingMax(self, window: int) -> "OaSeries": return self._rolling(window, np.max)

    def Shift(self, periods: int, fill: float = 0.0) -> "OaSeries":
        n = self._d.size
        out = np.full(n, float(fill))
        if periods >= 0:
            if periods < n:
                out[periods:] = self._d[:n - periods]
        elif -periods < n:
            out[:n + periods] = self._d[-periods:]
        return OaSeries(out)

    def Diff(self, periods: int = 1) -> "OaSeries":
        out = self._d - self.Shift(periods, np.nan)._d
        return OaSeries(out)

    def PctChange(self, periods: int = 1) -> "OaSeries":
        prev = self.Shift(periods, np.nan)._d
        with np.errstate(divide="ignore", invalid="ignore"):
            return OaSeries((self._d - prev) / prev)

    def Slice(self, start: int, end: int) -> "OaSeries": return OaSeries(self._d[max(0, start):max(0, end)].copy())
    def Head(self, n: int) -> "OaSeries": return OaSeries(self._d[:n].copy())
    def Tail(self, n: int) -> "OaSeries": return OaSeries(self._d[self._d.size - min(n, self._d.size):].copy())


@dataclass
class OaRecordOhlcv:
    Time: float = 0.0
    Open: float = 0.0
    High: float = 0.0
    Low: float = 0.0
    Close: float = 0.0
    Volume: float = 0.0

    def IsValid(self) -> bool: return self.High >= self.Low and self.High >= self.Open and self.High >= self.Close


class OaDataOhlcv:
    """Structure-of-arrays bars."""

    def __init__(self, records: Optional[Iterable[OaRecordOhlcv]] = None):
        self._cols: Dict[str, List[float]] = {c: [] for c in OaOhlcvColumns}
        for r in records or ():
            self.PushBack(r)

    def PushBack(self, r: OaRecordOhlcv) -> None:
        for c in OaOhlcvColumns:
            self._cols[c].append(float(getattr(r, c)))

    def Clear(self) -> None:
        for c in OaOhlcvColumns:
            self._cols[c].clear()

    def Size(self) -> int: return len(self._cols["Time"])
    def IsEmpty(self) -> bool: return self.Size() == 0
    def Column(self, name: str) -> OaSeries: return OaSeries(self._cols[name])
    def GetRecord(self, i: int) -> OaRecordOhlcv: return OaRecordOhlcv(*[self._cols[c][i] for c in OaOhlcvColumns])
    def Records(self) -> List[OaRecordOhlcv]: return [self.GetRecord(i) for i in range(self.Size())]


class OaTimeSeries:
    def __init__(self, times: Optional[OaSeries] = None, values: Optional[OaSeries] = None):
        self._t, self._v = times or OaSeries(), values or OaSeries()

    @staticmethod
    def Create(times: OaSeries, values: OaSeries) -> "OaTimeSeries":
        if times.Size() != values.Size():
            raise ValueError("times and values differ in length")
        if times.Size() > 1 and np.any(np.diff(times.Data()) < 0):
            raise ValueError("times must be non-decreasing")
        return OaTimeSeries(times, values)

    @staticmethod
    def FromOhlcvClose(data: OaDataOhlcv) -> "OaTimeSeries":
        return OaTimeSeries(data.Column("Time"), data.Column("Close"))

    def Size(self) -> int: return self._v.Size()
    def HasTimeIndex(self) -> bool: return not self._t.IsEmpty()
    def Times(self) -> OaSeries: return self._t
    def Values(self) -> OaSeries: return self._v
    def Slice(self, start: int, end: int) -> "OaTimeSeries": return OaTimeSeries(self._t.Slice(start, end), self._v.Slice(start, end))


class OaDataFrame:
    """Named float64 columns of equal length, in insertion order."""

    def __init__(self):
        self._cols: Dict[str, OaSeries] = {}

    @staticmethod
    def FromOhlcvData(data: OaDataOhlcv) -> "OaDataFrame":
        df = OaDataFrame()
        for c in OaOhlcvColumns:
            df.AddColumn(c, data.Column(c))
        return df

    def AddColumn(self, name: str, series: Union[OaSeries, Sequence[float]]) -> None:
        s = series if isinstance(series, OaSeries) else OaSeries(series)
        if self._cols and s.Size() != self.NumRows():
            raise ValueError(f"column '{name}' has {s.Size()} rows, the frame has {self.NumRows()}")
        self._cols[name] = s

    def HasColumn(self, name: str) -> bool: return name in self._cols
    def GetColumn(self, name: str) -> OaSeries: return self._cols[name]
    def __getitem__(self, name: str) -> OaSeries: return self._cols[name]
    def RemoveColumn(self, name: str) -> bool: return self._cols.pop(name, None) is not None
    def ColumnNames(self) -> List[str]: return list(self._cols)
    def NumColumns(self) -> int: return len(self._cols)
    def NumRows(self) -> int: return next(iter(self._cols.values())).Size() if self._cols else 0
    def IsEmpty(self) -> bool: return self.NumRows() == 0

    def Slice(self, start: int, end: int) -> "OaDataFrame":
        df = OaDataFrame()
        for k, s in self._cols.items():
            df._cols[k] = s.Slice(start, end)
        return df

    def Head(self, n: int) -> "OaDataFrame": return self.Slice(0, n)
    def Tail(self, n: int) -> "OaDataFrame": return self.Slice(max(0, self.NumRows() - n), self.NumRows())

    def ToTensor(self, columns: Optional[Sequence[str]] = None, dtype=torch.float32, device="cpu") -> torch.Tensor:
        """[rows, columns] tensor of the chosen columns (all by default)."""
        names = list(columns) if columns is not None else self.ColumnNames()
        return torch.from_numpy(np.stack([self._cols[n].Data() for n in names], axis=1)).to(device=device, dtype=dtype)

    def ToCsv(self, path: str) -> None:
        with open(path, "w") as f:
            f.write(",".join(self._cols) + "\n")
            for row in zip(*[s.Data() for s in self._cols.values()]):
                f.write(",".join(repr(float(v)) for v in row) + "\n")

    @staticmethod
    def FromCsv(path: str) -> "OaDataFrame":
        with open(path) as f:
            names = f.readline().strip().split(",")
            rows = [[float(v) for v in line.strip().split(",")] for line in f if line.strip()]
        df = OaDataFrame()
        arr = np.array(rows, dtype=np.float64).reshape(len(rows), len(names))
        for i, n in enumerate(names):
            df.AddColumn(n, OaSeries(arr[:, i]))
        return df
