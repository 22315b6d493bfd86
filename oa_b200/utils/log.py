"""Logging and scalar-metric streams (Source/Public/Oa/Core/Log.h:16-90 OaLog: levels, components, console + dated file;
:249-313 the JSONL metric writer with LogScalar / LogScalars / Flush / SetFlushInterval).

One process-wide `OaLog`; every rank of a multi-GPU job writes its own dated file when a directory is given, and rank 0
alone writes to the console unless `OA_LOG_ALL_RANKS` is set, so an 8-GPU run does not print everything eight times.
"""
from __future__ import annotations

import datetime
import enum
import json
import os
import sys
import threading
import time
from typing import Dict, Optional, TextIO

from . import envflag


class OaLogLevel(enum.IntEnum):
    Trace = 0
    Debug = 1
    Info = 2
    Warn = 3
    Error = 4
    Fatal = 5
    Off = 6


class OaLogComponent(enum.IntEnum):
    Core = 0
    ML = 1
    Crypto = 2
    Network = 4
    Storage = 5
    Api = 6
    App = 7
    Execution = 10


_NAMES = {OaLogComponent.Core: "CORE", OaLogComponent.ML: "ML  ", OaLogComponent.Crypto: "CRYP", OaLogComponent.Network: "NET ",
          OaLogComponent.Storage: "STOR", OaLogComponent.Api: "API ", OaLogComponent.App: "APP ", OaLogComponent.Execution: "EXEC"}
_COLORS = {OaLogLevel.Trace: "\033[90m", OaLogLevel.Debug: "\033[36m", OaLogLevel.Info: "", OaLogLevel.Warn: "\033[33m",
           OaLogLevel.Error: "\033[31m", OaLogLevel.Fatal: "\033[1;31m"}


def OaGetComponentName(c: OaLogComponent) -> str:
    return _NAMES.get(c, "????")


class OaLog:
    _instance: Optional["OaLog"] = None

    def __init__(self):
        self.MinLevel_ = OaLogLevel.Info
        self._console: Optional[TextIO] = sys.stderr
        self._file: Optional[TextIO] = None
        self._lock = threading.Lock()
        self._rank = int(os.environ.get("RANK", "0") or 0)
        self.Path = ""

    @classmethod
    def Instance(cls) -> "OaLog":
        if cls._instance is None:
            cls._instance = OaLog()
        return cls._instance

    def Init(self, directory: str = "", name: str = "oa", level: OaLogLevel = OaLogLevel.Info, console: bool = True) -> None:
        """Console on rank 0 (all ranks with OA_LOG_ALL_RANKS); with a directory also `<dir>/<name>_<date>[_rankN].log`."""
        self.Close()
        self.MinLevel_ = OaLogLevel(level)
        self._console = sys.stderr if console and (self._rank == 0 or envflag.IsSet("OA_LOG_ALL_RANKS")) else None
        if directory:
            os.makedirs(directory, exist_ok=True)
            suffix = f"_rank{self._rank}" if "RANK" in os.environ else ""
            self.Path = os.path.join(directory, f"{name}_{datetime.date.today():%Y%m%d}{suffix}.log")
            self._file = open(self.Path, "a", encoding="utf-8")

    def SetLevel(self, level: OaLogLevel) -> None: self.MinLevel_ = OaLogLevel(level)
    def GetLevel(self) -> OaLogLevel: return self.MinLevel_

    def Log(self, level: OaLogLevel, component: OaLogComponent, fmt: str, *args) -> None:
        if level < self.MinLevel_ or self.MinLevel_ == OaLogLevel.Off:
            return
        now = datetime.datetime.now()
        text = (fmt % args) if args else fmt
        line = f"{now:%Y-%m-%d %H:%M:%S}.{now.microsecond // 1000:03d} [{OaLogLevel(level).name.upper():5s}] [{OaGetComponentName(component)}] {text}"
        with self._lock:
            if self._console is not None:
                color = _COLORS.get(OaLogLevel(level), "") if self._console.isatty() else ""
                self._console.write(f"{color}{line}\033[0m\n" if color else line + "\n")
            if self._file is not None:
                self._file.write(line + "\n")
                if level >= OaLogLevel.Warn:
                    self._file.flush()

    def Close(self) -> None:
        if self._file is not None:
            self._file.close()
            self._file = None


def OA_LOG_TRACE(c, fmt, *a): OaLog.Instance().Log(OaLogLevel.Trace, c, fmt, *a)
def OA_LOG_DEBUG(c, fmt, *a): OaLog.Instance().Log(OaLogLevel.Debug, c, fmt, *a)
def OA_LOG_INFO(c, fmt, *a): OaLog.Instance().Log(OaLogLevel.Info, c, fmt, *a)
def OA_LOG_WARN(c, fmt, *a): OaLog.Instance().Log(OaLogLevel.Warn, c, fmt, *a)
def OA_LOG_ERROR(c, fmt, *a): OaLog.Instance().Log(OaLogLevel.Error, c, fmt, *a)


def OaLogSummary(component: OaLogComponent, left: str, right) -> None:
    """`left .... right` padded to 60 columns; integers are grouped by thousands."""
    val = f"{right:,}" if isinstance(right, int) else str(right)
    OA_LOG_INFO(component, "%s", left + " " + "." * max(1, 58 - len(left) - len(val)) + " " + val)


class OaMetricsWriter:
    """Append-only JSONL stream of scalars: {"tag", "step", "value", "wall_time"} per line."""

    def __init__(self, path: str, flush_interval: int = 50):
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        self._f: Optional[TextIO] = open(path, "a", encoding="utf-8")
        self._interval, self._pending = max(1, flush_interval), 0
        self.Path = path

    def LogScalar(self, tag: str, step: int, value: float) -> None:
        if self._f is None:
            return
        self._f.write(json.dumps({"tag": tag, "step": int(step), "value": float(value), "wall_time": time.time()}) + "\n")
        self._pending += 1
        if self._pending >= self._interval:
            self.Flush()

    def LogScalars(self, tag: str, step: int, values: Dict[str, float]) -> None:
        for k, v in values.items():
            self.LogScalar(f"{tag}/{k}", step, v)

    def SetFlushInterval(self, n: int) -> None: self._interval = max(1, int(n))

    def Flush(self) -> None:
        if self._f is not None:
            self._f.flush()
            self._pending = 0

    def Close(self) -> None:
        if self._f is not None:
            self._f.close()
            self._f = None
