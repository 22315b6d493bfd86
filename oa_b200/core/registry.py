"""OaKernelRegistry and operation contracts (Source/Public/Oa/Core/KernelRegistry.h, Core/Operation.h of the reference).

The tables are native (csrc/runtime/registry.cpp).  They are filled once per process: one kernel row per exported entry
point of the kernel library, grouped by the `// ---- section (file.cu)` comments of csrc/kernels/api.h, and one operation
contract per public function of the OaFnMatrix / OaFnLoss namespaces, with kind, differentiation (does the function attach
a backward node), lowering (dispatch, GEMM, or a composition of other operations), effects and the kernels it launches -
all read from the function's own source, so the contracts cannot drift from the code.
"""
from __future__ import annotations

import ctypes
import enum
import inspect
import re
from dataclasses import dataclass, field
from pathlib import Path
from typing import List, Optional

from ..io.oam import runtime_lib


class OaOperationKind(enum.IntEnum):
    Elementwise = 0
    Reduction = 1
    Gemm = 2
    Indexing = 3
    Normalization = 4
    Attention = 5
    Loss = 6
    Shape = 7
    Factory = 8
    Other = 9


class OaDifferentiation(enum.IntEnum):
    NoGradient = 0
    Analytic = 1


class OaLowering(enum.IntEnum):
    Dispatch = 0
    Gemm = 1
    Composite = 2


class OaEffects(enum.IntEnum):
    Pure = 0
    MutatesInput = 1
    Random = 2


@dataclass
class OaKernelInfo:
    Name: str
    Id: int
    Category: str
    Provider: str


@dataclass
class OaOperationContract:
    Name: str
    Hash: int
    Kind: OaOperationKind
    Differentiation: OaDifferentiation
    Lowering: OaLowering
    Effects: OaEffects
    MutatedInputMask: int
    Kernels: List[str] = field(default_factory=list)


_ready = False


def _lib():
    global _ready
    L = runtime_lib()
    if _ready:
        return L
    u64, u32, i32, cp = ctypes.c_uint64, ctypes.c_uint32, ctypes.c_int, ctypes.c_char_p
    P = ctypes.POINTER
    sig = {"oa_registry_fnv1a": (u64, [cp]), "oa_registry_add_kernel": (u32, [cp, cp, cp]), "oa_registry_num_kernels": (i32, []),
           "oa_registry_find_kernel": (i32, [cp]), "oa_registry_find_kernel_id": (i32, [u32]), "oa_registry_kernel_name": (cp, [i32]),
           "oa_registry_kernel_category": (cp, [i32]), "oa_registry_kernel_provider": (cp, [i32]), "oa_registry_kernel_id": (u32, [i32]),
           "oa_registry_add_operation": (i32, [cp, i32, i32, i32, i32, u32]), "oa_registry_operation_add_kernel": (None, [i32, cp]),
           "oa_registry_num_operations": (i32, []), "oa_registry_find_operation": (i32, [cp]), "oa_registry_find_operation_hash": (i32, [u64]),
           "oa_registry_operation_name": (cp, [i32]), "oa_registry_operation_hash": (u64, [i32]),
           "oa_registry_operation_fields": (None, [i32, P(i32), P(i32), P(i32), P(i32), P(u32)]),
           "oa_registry_operation_num_kernels": (i32, [i32]), "oa_registry_operation_kernel": (cp, [i32, i32])}
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype, fn.argtypes = res, args
    _ready = True
    return L


def Fnv1a(name: str) -> int:
    return int(_lib().oa_registry_fnv1a(name.encode()))


_populated = False
_KIND_HINTS = (
    (OaOperationKind.Loss, ("CrossEntropy", "Mse", "L1", "SmoothL1", "Bce")),
    (OaOperationKind.Attention, ("Attention",)),
    (OaOperationKind.Normalization, ("Norm",)),
    (OaOperationKind.Gemm, ("Linear", "MatMul", "Bmm")),
    (OaOperationKind.Reduction, ("Sum", "Mean", "Max", "Argmax", "Softmax", "TopK")),
    (OaOperationKind.Indexing, ("Gather", "Embedding", "Scatter")),
    (OaOperationKind.Shape, ("Reshape", "Transpose", "Permute", "Slice", "Concat", "Split", "Repeat", "Heads", "Cast", "Detach")),
    (OaOperationKind.Factory, ("Empty", "Zeros", "Ones", "Full", "Rand", "From", "CausalMask", "Philox")),
)


def _classify(name: str) -> OaOperationKind:
    for kind, keys in _KIND_HINTS:
        if any(k in name for k in keys):
            return kind
    return OaOperationKind.Elementwise


def Populate() -> None:
    """Fills both tables (idempotent)."""
    global _populated
    if _populated:
        return
    L = _lib()
    # kernel rows come from the generated table; a table that is older than the header is ignored and the header is read
    import hashlib
    api = (Path(__file__).resolve().parent.parent / "csrc" / "kernels" / "api.h").read_text()
    rows = None
    try:
        from .._generated import kernel_table as KT
        if KT.API_SHA256 == hashlib.sha256(api.encode()).hexdigest():
            rows = [(name, section, file) for name, section, file, _, _, _ in KT.KERNELS]
    except ImportError:
        pass
    if rows is None:
        from ..utils.api_header import parse_api
        rows = [(r["name"], r["section"], r["file"]) for r in parse_api(api)[0]]
    for name, category, provider in rows:
        L.oa_registry_add_kernel(name.encode(), category.encode(), provider.encode())
    from . import fn_matrix as F
    from ..ml import fn_loss as FL
    for ns, mod in (("", F), ("Loss.", FL)):
        for name in sorted(n for n in dir(mod) if n[0].isupper() and inspect.isfunction(getattr(mod, n))):
            fn = getattr(mod, name)
            try:
                src = inspect.getsource(fn)
            except (OSError, TypeError):
                src = ""
            kernels = sorted(set(re.findall(r"\b(oa_\w+)\(", src)))
            calls_gemm = bool(re.search(r"K\.b?gemm\(|FF\.\w+\(", src))
            composite = not kernels and not re.search(r"\bK\.\w+\(", src) and bool(re.search(r"\b(?:F\.)?[A-Z]\w+\(", src))
            diff = OaDifferentiation.Analytic if ("AG.attach" in src or "_unary(" in src or "_binary(" in src or "_elem_loss(" in src) else OaDifferentiation.NoGradient
            effects = OaEffects.MutatesInput if name.endswith("InPlace") or name in ("Fill", "MultiFill", "MultiAdd") else (
                OaEffects.Random if any(k in name for k in ("Rand", "Philox", "Dropout", "Sample")) else OaEffects.Pure)
            lowering = OaLowering.Gemm if calls_gemm else (OaLowering.Composite if composite else OaLowering.Dispatch)
            kind = OaOperationKind.Loss if ns else _classify(name)
            idx = L.oa_registry_add_operation((ns + name).encode(), int(kind), int(diff), int(lowering), int(effects),
                                              1 if effects == OaEffects.MutatesInput else 0)
            for k in kernels:
                L.oa_registry_operation_add_kernel(idx, k.encode())
    _populated = True


class OaKernelRegistry:
    @staticmethod
    def Count() -> int:
        Populate()
        return int(_lib().oa_registry_num_kernels())

    @staticmethod
    def At(i: int) -> OaKernelInfo:
        L = _lib()
        return OaKernelInfo(L.oa_registry_kernel_name(i).decode(), int(L.oa_registry_kernel_id(i)), L.oa_registry_kernel_category(i).decode(),
                            L.oa_registry_kernel_provider(i).decode())

    @staticmethod
    def Find(name: str) -> Optional[OaKernelInfo]:
        Populate()
        i = _lib().oa_registry_find_kernel(name.encode())
        return OaKernelRegistry.At(i) if i >= 0 else None

    @staticmethod
    def FindById(kernel_id: int) -> Optional[OaKernelInfo]:
        Populate()
        i = _lib().oa_registry_find_kernel_id(int(kernel_id))
        return OaKernelRegistry.At(i) if i >= 0 else None

    @staticmethod
    def All() -> List[OaKernelInfo]:
        return [OaKernelRegistry.At(i) for i in range(OaKernelRegistry.Count())]


class OaOperationRegistry:
    @staticmethod
    def Count() -> int:
        Populate()
        return int(_lib().oa_registry_num_operations())

    @staticmethod
    def At(i: int) -> OaOperationContract:
        L = _lib()
        k, d, lo, e = (ctypes.c_int() for _ in range(4))
        mask = ctypes.c_uint32()
        L.oa_registry_operation_fields(i, ctypes.byref(k), ctypes.byref(d), ctypes.byref(lo), ctypes.byref(e), ctypes.byref(mask))
        kernels = [L.oa_registry_operation_kernel(i, j).decode() for j in range(L.oa_registry_operation_num_kernels(i))]
        return OaOperationContract(L.oa_registry_operation_name(i).decode(), int(L.oa_registry_operation_hash(i)), OaOperationKind(k.value),
                                   OaDifferentiation(d.value), OaLowering(lo.value), OaEffects(e.value), int(mask.value), kernels)

    @staticmethod
    def Find(name: str) -> Optional[OaOperationContract]:
        Populate()
        i = _lib().oa_registry_find_operation(name.encode())
        return OaOperationRegistry.At(i) if i >= 0 else None

    @staticmethod
    def FindByHash(h: int) -> Optional[OaOperationContract]:
        Populate()
        i = _lib().oa_registry_find_operation_hash(int(h))
        return OaOperationRegistry.At(i) if i >= 0 else None

    @staticmethod
    def All() -> List[OaOperationContract]:
        return [OaOperationRegistry.At(i) for i in range(OaOperationRegistry.Count())]
