""".oad dataset archive (Source/Public/Oa/Ml/Oad.h:12-93): a 64-byte little-endian header
  u32 magic 'OAD1' | u8 major | u8 minor | u16 flags | u32 reserved | (u64 offset, u64 bytes) x {train, val, test} | u32 reserved
followed by the three payloads.  Files are memory-mapped; spans are zero-copy memoryviews."""
from __future__ import annotations

import enum
import mmap
import os
import struct
from typing import Optional

from ..core.types import OaStatus, OaStatusCode

OA_OAD_MAGIC = 0x3144414F
OA_OAD_HEADER_V1_BYTES = 64
_FMT = "<IBBHI6QI"
assert struct.calcsize(_FMT) == 64


class OaOadSplit(enum.IntEnum):
    Train = 0
    Val = 1
    Test = 2


class OaOadHeaderV1:
    def __init__(self):
        self.Magic, self.VersionMajor, self.VersionMinor, self.Flags = 0, 0, 0, 0
        self.TrainOffset = self.TrainBytes = self.ValOffset = self.ValBytes = self.TestOffset = self.TestBytes = 0


def OaOadProbeMagic(data) -> bool:
    return len(data) >= 4 and struct.unpack_from("<I", data, 0)[0] == OA_OAD_MAGIC


def OaOadParseHeader(data):
    """Returns (header | None, status).  Every span must lie inside the file, behind the header."""
    if len(data) < OA_OAD_HEADER_V1_BYTES:
        return None, OaStatus.Error(OaStatusCode.DataLoss, "oad: file shorter than its header")
    f = struct.unpack_from(_FMT, data, 0)
    if f[0] != OA_OAD_MAGIC:
        return None, OaStatus.Error(OaStatusCode.DataLoss, "oad: bad magic")
    if f[1] != 1:
        return None, OaStatus.Error(OaStatusCode.Unimplemented, f"oad: unsupported major version {f[1]}")
    h = OaOadHeaderV1()
    h.Magic, h.VersionMajor, h.VersionMinor, h.Flags = f[0], f[1], f[2], f[3]
    h.TrainOffset, h.TrainBytes, h.ValOffset, h.ValBytes, h.TestOffset, h.TestBytes = f[5:11]
    for off, n in ((h.TrainOffset, h.TrainBytes), (h.ValOffset, h.ValBytes), (h.TestOffset, h.TestBytes)):
        if n and (off < OA_OAD_HEADER_V1_BYTES or off + n > len(data)):
            return None, OaStatus.Error(OaStatusCode.DataLoss, "oad: a split lies outside the file")
    return h, OaStatus.Ok()


def OaOadWriteFile(path: str, train: bytes, val: bytes = b"", test: bytes = b"") -> OaStatus:
    off = OA_OAD_HEADER_V1_BYTES
    spans = []
    for part in (train, val, test):
        spans += [off if part else 0, len(part)]
        off += len(part)
    head = struct.pack(_FMT, OA_OAD_MAGIC, 1, 0, 0, 0, *spans, 0)
    tmp = str(path) + ".tmp"
    try:
        with open(tmp, "wb") as f:
            f.write(head)
            for part in (train, val, test):
                f.write(part)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, str(path))
    except OSError as e:
        return OaStatus.Error(OaStatusCode.PermissionDenied, f"oad: cannot write {path}: {e}")
    return OaStatus.Ok()


class OaOadFile:
    def __init__(self):
        self._f, self._map, self._hdr = None, None, None

    def TryOpen(self, path: str) -> bool:
        self.Close()
        try:
            self._f = open(path, "rb")
            self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        except (OSError, ValueError):
            self.Close()
            return False
        self._hdr, st = OaOadParseHeader(self._map)
        if not st:
            self.Close()
            return False
        return True

    def IsOpen(self) -> bool:
        return self._hdr is not None

    def Header(self) -> Optional[OaOadHeaderV1]:
        return self._hdr

    def _span(self, off: int, n: int) -> memoryview:
        return memoryview(self._map)[off:off + n] if self._hdr is not None and n else memoryview(b"")

    def TrainSpan(self) -> memoryview: return self._span(self._hdr.TrainOffset, self._hdr.TrainBytes)
    def ValSpan(self) -> memoryview: return self._span(self._hdr.ValOffset, self._hdr.ValBytes)
    def TestSpan(self) -> memoryview: return self._span(self._hdr.TestOffset, self._hdr.TestBytes)

    def Span(self, split: OaOadSplit) -> memoryview:
        return (self.TrainSpan, self.ValSpan, self.TestSpan)[int(split)]()

    def Close(self) -> None:
        self._hdr = None
        if self._map is not None:
            try:
                self._map.close()
            except BufferError:
                pass            # a span handed out earlier is still alive; the mapping goes with it
            self._map = None
        if self._f is not None:
            self._f.close()
            self._f = None
