"""Scalar types, precision enums and the status codes shared by every layer.

Enum values are part of the checkpoint format and match the reference
(Source/Public/Oa/Core/Type.gen.h:17-65, Source/Public/Oa/Core/Status.h:10-60).
"""
from __future__ import annotations

import enum

import torch


class OaScalarType(enum.IntEnum):
    Float32 = 0
    BFloat16 = 1
    Float16 = 2
    Int8 = 3
    Int32 = 4
    UInt8 = 5
    Float64 = 6
    Int16 = 7
    Int64 = 8
    UInt16 = 9
    UInt32 = 10
    UInt64 = 11
    Bool = 12


class OaPrecision(enum.IntEnum):
    FP32 = 0
    TF32 = 1
    BF16 = 2
    FP16 = 3
    INT8 = 4


class OaMatMulPrecision(enum.IntEnum):
    Auto = 0
    Fp32 = 1
    Bf16 = 2


class OaNumericMode(enum.IntEnum):
    Fast = 0
    Stable = 1
    Deterministic = 2


class OaStatusCode(enum.IntEnum):
    Ok = 0
    Cancelled = 1
    Unknown = 2
    InvalidArgument = 3
    DeadlineExceeded = 4
    NotFound = 5
    AlreadyExists = 6
    PermissionDenied = 7
    ResourceExhausted = 8
    FailedPrecondition = 9
    Aborted = 10
    OutOfRange = 11
    Unimplemented = 12
    Internal = 13
    Unavailable = 14
    DataLoss = 15


class OaStatus:
    """A status value: code + message. Truthy when Ok."""

    __slots__ = ("code", "message")

    def __init__(self, code: OaStatusCode = OaStatusCode.Ok, message: str = ""):
        self.code = OaStatusCode(code)
        self.message = message

    @staticmethod
    def Ok() -> "OaStatus":
        return OaStatus()

    @staticmethod
    def Error(code: OaStatusCode, message: str) -> "OaStatus":
        return OaStatus(code, message)

    def IsOk(self) -> bool:
        return self.code == OaStatusCode.Ok

    def __bool__(self) -> bool:
        return self.IsOk()

    def __repr__(self) -> str:
        return "OaStatus(Ok)" if self.IsOk() else f"OaStatus({self.code.name}: {self.message})"


class OaError(RuntimeError):
    def __init__(self, status: OaStatus):
        super().__init__(repr(status))
        self.status = status


_TO_TORCH = {
    OaScalarType.Float32: torch.float32, OaScalarType.BFloat16: torch.bfloat16, OaScalarType.Float16: torch.float16,
    OaScalarType.Int8: torch.int8, OaScalarType.Int32: torch.int32, OaScalarType.UInt8: torch.uint8,
    OaScalarType.Float64: torch.float64, OaScalarType.Int16: torch.int16, OaScalarType.Int64: torch.int64,
    OaScalarType.UInt32: torch.int32,  # token ids: stored as 32-bit words, values < 2^31
    OaScalarType.Bool: torch.bool,
}
_FROM_TORCH = {torch.float32: OaScalarType.Float32, torch.bfloat16: OaScalarType.BFloat16, torch.float16: OaScalarType.Float16,
               torch.int8: OaScalarType.Int8, torch.int32: OaScalarType.Int32, torch.uint8: OaScalarType.UInt8,
               torch.float64: OaScalarType.Float64, torch.int16: OaScalarType.Int16, torch.int64: OaScalarType.Int64,
               torch.bool: OaScalarType.Bool}


def to_torch_dtype(t) -> torch.dtype:
    if isinstance(t, torch.dtype):
        return t
    return _TO_TORCH[OaScalarType(t)]


def from_torch_dtype(t: torch.dtype) -> OaScalarType:
    return _FROM_TORCH[t]


def element_size(t: OaScalarType) -> int:
    return torch.empty((), dtype=to_torch_dtype(t)).element_size()


class OaMatrixShape(tuple):
    """Shape of rank <= 8 (Source/Public/Oa/Core/MatrixShape.h)."""

    MaxRank = 8

    def __new__(cls, dims=()):
        dims = tuple(int(d) for d in dims)
        if len(dims) > cls.MaxRank:
            raise ValueError("OaMatrixShape: rank > 8")
        return super().__new__(cls, dims)

    def Rank(self) -> int:
        return len(self)

    def NumElements(self) -> int:
        n = 1
        for d in self:
            n *= d
        return n

    def Strides(self):
        s, acc = [], 1
        for d in reversed(self):
            s.append(acc)
            acc *= d
        return tuple(reversed(s))


# ---- string forms of every enumeration of this module (Source/Public/Oa/Core/Type.gen.h: <Type>ToString / <Type>FromString,
# which the reference generates from its type schemas; here they are derived from the IntEnum classes themselves)
def OaEnumToString(value) -> str:
    return value.name if isinstance(value, enum.Enum) else str(value)


def OaEnumFromString(cls, text: str, default=None):
    """Case-insensitive member lookup; `default` (or the first member) for an unknown string, as the reference does."""
    want = str(text).strip().lower()
    for m in cls:
        if m.name.lower() == want:
            return m
    return default if default is not None else list(cls)[0]


def _make_string_functions() -> None:
    g = globals()
    for name, obj in list(g.items()):
        if isinstance(obj, type) and issubclass(obj, enum.IntEnum) and obj is not enum.IntEnum and name.startswith("Oa"):
            g[name + "ToString"] = (lambda v, _c=obj: OaEnumToString(_c(v)))
            g[name + "FromString"] = (lambda text, _c=obj: OaEnumFromString(_c, text))


_make_string_functions()
