"""OaPath / OaPaths / OaFilesystem: the small path and file helpers of the public surface
(Source/Public/Oa/Core/Filesystem.h, Paths.h).  `OaPaths.Var(sub)` is the writable tree for run products
(checkpoints, route caches, reports): $OA_VAR_DIR or ./var."""
from __future__ import annotations

import os
import shutil
from pathlib import Path

from ..core.types import OaStatus, OaStatusCode


class OaPath:
    def __init__(self, p=""):
        self._p = Path(str(p))

    def String(self) -> str:
        return str(self._p)

    __str__ = String
    __fspath__ = String

    def __truediv__(self, other) -> "OaPath":
        return OaPath(self._p / str(other))

    def Parent(self) -> "OaPath":
        return OaPath(self._p.parent)

    def Stem(self) -> "OaPath":
        return OaPath(self._p.stem)

    def Extension(self) -> "OaPath":
        return OaPath(self._p.suffix)

    def Filename(self) -> "OaPath":
        return OaPath(self._p.name)

    def Exists(self) -> bool:
        return self._p.exists()


class OaPaths:
    @staticmethod
    def Root() -> OaPath:
        return OaPath(os.getcwd())

    @staticmethod
    def Var(sub: str = "") -> OaPath:
        base = os.environ.get("OA_VAR_DIR", os.path.join(os.getcwd(), "var"))
        return OaPath(os.path.join(base, sub) if sub else base)


class OaFilesystem:
    @staticmethod
    def Exists(p) -> bool: return os.path.exists(str(p))
    @staticmethod
    def IsFile(p) -> bool: return os.path.isfile(str(p))
    @staticmethod
    def IsDirectory(p) -> bool: return os.path.isdir(str(p))

    @staticmethod
    def CreateDirectories(p) -> OaStatus:
        try:
            os.makedirs(str(p), exist_ok=True)
            return OaStatus.Ok()
        except OSError as e:
            return OaStatus.Error(OaStatusCode.PermissionDenied, str(e))

    @staticmethod
    def RemoveFile(p) -> OaStatus:
        try:
            os.remove(str(p))
            return OaStatus.Ok()
        except OSError as e:
            return OaStatus.Error(OaStatusCode.NotFound, str(e))

    @staticmethod
    def RemoveAll(p) -> OaStatus:
        shutil.rmtree(str(p), ignore_errors=True)
        return OaStatus.Ok()

    @staticmethod
    def ListFiles(p, extension: str = ""):
        try:
            return [OaPath(os.path.join(str(p), f)) for f in sorted(os.listdir(str(p))) if f.endswith(extension)]
        except OSError:
            return []

    @staticmethod
    def FileSize(p) -> int:
        return os.path.getsize(str(p))

    @staticmethod
    def ReadBytes(p) -> bytes:
        with open(str(p), "rb") as f:
            return f.read()

    @staticmethod
    def WriteBytesAtomic(p, data: bytes) -> OaStatus:
        tmp = str(p) + ".tmp"
        try:
            with open(tmp, "wb") as f:
                f.write(data)
                f.flush()
                os.fsync(f.fileno())
            os.replace(tmp, str(p))
            return OaStatus.Ok()
        except OSError as e:
            return OaStatus.Error(OaStatusCode.PermissionDenied, str(e))
