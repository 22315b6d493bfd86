"""ctypes binding of the in-tree CUDA kernel library (`_lib/liboa_kernels.so`).

The C prototypes in `csrc/kernels/api.h` are the single source of truth: they are parsed here to set
`argtypes` / `restype`, so a prototype change cannot silently disagree with its Python caller.
On a machine with a GPU a missing library is an error (no silent fallback to PyTorch math); on a
CPU-only machine `lib()` returns None and callers use the fp32 reference math instead.
"""
from __future__ import annotations

import ctypes
import os
import re
from pathlib import Path
from typing import Optional

import torch

_ROOT = Path(__file__).resolve().parent
_API_H = _ROOT / "csrc" / "kernels" / "api.h"
# OA_KERNELS_LIB: another build of the same sources (an experiment compiled with different macros) to load instead
_LIB_PATH = Path(os.environ["OA_KERNELS_LIB"]) if os.environ.get("OA_KERNELS_LIB") else _ROOT / "_lib" / "liboa_kernels.so"

_CTYPES = {
    "int": ctypes.c_int, "float": ctypes.c_float, "size_t": ctypes.c_size_t, "long long": ctypes.c_longlong,
    "unsigned long long": ctypes.c_ulonglong, "unsigned": ctypes.c_uint, "double": ctypes.c_double,
}

OA_ERRORS = {0: "ok", 1: "bad argument", 2: "misaligned pointer or extent", 3: "driver entry point unavailable",
             4: "launch failed", 5: "unsupported dtype/shape", 6: "size beyond the supported maximum"}


class OaKernelError(RuntimeError):
    pass


def _parse_enums(text: str) -> dict[str, int]:
    out: dict[str, int] = {}
    for body in re.findall(r"enum\s*\{(.*?)\}\s*;", text, flags=re.S):
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        val = -1
        for item in body.split(","):
            item = item.strip()
            if not item:
                continue
            if "=" in item:
                name, v = item.split("=")
                val = int(v.strip(), 0)
                out[name.strip()] = val
            else:
                val += 1
                out[item] = val
    return out


def _parse_protos(text: str):
    text = re.sub(r"//.*", "", text)
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    protos = []
    for m in re.finditer(r"\b(int|size_t|void)\s+(oa_\w+)\s*\(([^)]*)\)\s*;", text, flags=re.S):
        ret, name, args = m.group(1), m.group(2), m.group(3)
        argtypes = []
        for a in args.split(","):
            a = " ".join(a.split())
            if not a or a == "void":
                continue
            if "*" in a:
                argtypes.append(ctypes.c_void_p)
                continue
            a = a.replace("const ", "")
            ty = " ".join(a.split(" ")[:-1])
            argtypes.append(_CTYPES[ty])
        restype = {"int": ctypes.c_int, "size_t": ctypes.c_size_t, "void": None}[ret]
        protos.append((name, restype, argtypes))
    return protos


_API_TEXT = _API_H.read_text()
CONST = _parse_enums(_API_TEXT)
_PROTOS = _parse_protos(_API_TEXT)

_lib: Optional[ctypes.CDLL] = None
_tried = False


def lib_path() -> Path:
    return _LIB_PATH


def lib() -> Optional[ctypes.CDLL]:
    """Returns the loaded kernel library, or None on a machine without CUDA."""
    global _lib, _tried
    if _lib is not None or _tried:
        return _lib
    _tried = True
    if not _LIB_PATH.exists():
        if torch.cuda.is_available():
            raise OaKernelError(f"{_LIB_PATH} is missing on a GPU machine: run `python -m oa_b200.build` first")
        return None
    try:
        handle = ctypes.CDLL(str(_LIB_PATH))
    except OSError as e:  # e.g. no libcudart on a CPU-only box
        if torch.cuda.is_available():
            raise OaKernelError(f"cannot load {_LIB_PATH}: {e}") from e
        return None
    for name, restype, argtypes in _PROTOS:
        fn = getattr(handle, name, None)
        if fn is None:
            raise OaKernelError(f"{name} is declared in api.h but missing from {_LIB_PATH.name}")
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = handle
    return _lib


def require() -> ctypes.CDLL:
    h = lib()
    if h is None:
        raise OaKernelError("the CUDA kernel library is not available")
    return h


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise OaKernelError(f"{what}: {OA_ERRORS.get(rc, rc)}")


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


_launch_count = 0


def count_launch(n: int = 1) -> None:
    global _launch_count
    _launch_count += n


def launches() -> int:
    """Number of kernels of this library launched so far by this process."""
    return _launch_count
