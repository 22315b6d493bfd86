"""SafeTensors reading and weight transfer into OaModule checkpoints
(Source/Public/Oa/Ml/TransferWeights.h:13-122, Source/Private/Oa/Ml/Io/SafeTensorReader.cpp).

A .safetensors file is `u64 header_len | JSON header | raw tensor bytes`; each JSON entry has dtype, shape and
data_offsets relative to the end of the header.  `OaSafeTensorReader` validates the header (offsets inside the file, sizes
matching dtype x shape, no overlap) and hands out zero-copy tensors; a sharded source is a directory with
`model.safetensors.index.json`.  `OaTransferWeights` inspects a source, maps names onto a module's parameter names with
rename rules, converts dtypes, loads and verifies."""
from __future__ import annotations

import json
import mmap
import os
import re
import struct
from typing import Callable, Optional, Sequence

import torch

from ..core.types import OaStatus, OaStatusCode

_DT = {"F32": (torch.float32, 4), "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2), "I32": (torch.int32, 4), "I64": (torch.int64, 8),
       "U8": (torch.uint8, 1), "I8": (torch.int8, 1), "F64": (torch.float64, 8), "BOOL": (torch.bool, 1)}
_NAME = {v[0]: k for k, v in _DT.items()}


class OaSafeTensorReader:
    def __init__(self):
        self._files: list = []            # (file, mmap, data_start)
        self._index: dict[str, tuple] = {}  # name -> (file idx, dtype, shape, begin, end)
        self.Metadata: dict = {}

    def Open(self, path: str) -> OaStatus:
        """A single file, or a directory with a sharded-checkpoint index."""
        if os.path.isdir(path):
            idx = os.path.join(path, "model.safetensors.index.json")
            try:
                shards = sorted(set(json.load(open(idx))["weight_map"].values()))
            except (OSError, ValueError, KeyError) as e:
                return OaStatus.Error(OaStatusCode.NotFound, f"safetensors: no usable shard index in {path}: {e}")
            for s in shards:
                st = self._open_one(os.path.join(path, s))
                if not st:
                    return st
            return OaStatus.Ok()
        return self._open_one(path)

    def _open_one(self, path: str) -> OaStatus:
        try:
            f = open(path, "rb")
            mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        except (OSError, ValueError) as e:
            return OaStatus.Error(OaStatusCode.NotFound, f"safetensors: cannot open {path}: {e}")
        bad = lambda why: OaStatus.Error(OaStatusCode.DataLoss, f"safetensors: {path}: {why}")
        if len(mm) < 8:
            return bad("shorter than the length prefix")
        n = struct.unpack_from("<Q", mm, 0)[0]
        if n > len(mm) - 8 or n > (100 << 20):
            return bad("header length exceeds the file")
        try:
            header = json.loads(bytes(mm[8:8 + n]))
        except ValueError:
            return bad("header is not valid JSON")
        start, size = 8 + n, len(mm) - 8 - n
        fi = len(self._files)
        spans = []
        for name, e in header.items():
            if name == "__metadata__":
                self.Metadata.update(e or {})
                continue
            try:
                dt, shape, (b0, b1) = e["dtype"], [int(d) for d in e["shape"]], e["data_offsets"]
            except (KeyError, TypeError, ValueError):
                return bad(f"malformed entry '{name}'")
            if dt not in _DT:
                return bad(f"unsupported dtype {dt} for '{name}'")
            numel = 1
            for d in shape:
                numel *= d
            if not (0 <= b0 <= b1 <= size) or b1 - b0 != numel * _DT[dt][1]:
                return bad(f"'{name}': byte range does not match dtype x shape or leaves the file")
            spans.append((b0, b1))
            self._index[name] = (fi, dt, shape, b0, b1)
        spans.sort()
        for (a0, a1), (c0, c1) in zip(spans, spans[1:]):
            if c0 < a1:
                return bad("tensor byte ranges overlap")
        self._files.append((f, mm, start))
        return OaStatus.Ok()

    def Names(self) -> list:
        return sorted(self._index)

    def Info(self, name: str):
        fi, dt, shape, b0, b1 = self._index[name]
        return dt, list(shape), b1 - b0

    def Tensor(self, name: str) -> torch.Tensor:
        fi, dt, shape, b0, b1 = self._index[name]
        _, mm, start = self._files[fi]
        t = torch.frombuffer(mm, dtype=_DT[dt][0], count=(b1 - b0) // _DT[dt][1], offset=start + b0) if b1 > b0 else torch.empty(0, dtype=_DT[dt][0])
        return t.reshape(shape)

    def Close(self) -> None:
        for f, mm, _ in self._files:
            try:
                mm.close()
            except BufferError:
                pass
            f.close()
        self._files, self._index = [], {}


def OaSafeTensorWrite(path: str, tensors: dict, metadata: Optional[dict] = None) -> OaStatus:
    header, blobs, off = {}, [], 0
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAME[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * (-len(hj) % 8)
    tmp = str(path) + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj)
        for b in blobs:
            f.write(b)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, str(path))
    return OaStatus.Ok()


class OaTransferRule:
    """regex -> replacement applied to source names (first match wins), plus an optional tensor transform."""

    def __init__(self, pattern: str, replacement: str, transform: Optional[Callable[[torch.Tensor], torch.Tensor]] = None):
        self.Pattern, self.Replacement, self.Transform = re.compile(pattern), replacement, transform


class OaTransferReport:
    def __init__(self):
        self.Loaded, self.Missing, self.Unused, self.ShapeMismatch = [], [], [], []

    def Ok(self) -> bool:
        return not self.Missing and not self.ShapeMismatch


class OaTransferWeights:
    def __init__(self, rules: Sequence[OaTransferRule] = ()):
        self.Rules = list(rules)

    def Inspect(self, path: str):
        r = OaSafeTensorReader()
        st = r.Open(path)
        if not st:
            return None, st
        out = {n: r.Info(n) for n in r.Names()}
        r.Close()
        return out, OaStatus.Ok()

    def Map(self, name: str):
        for rule in self.Rules:
            if rule.Pattern.search(name):
                return rule.Pattern.sub(rule.Replacement, name), rule.Transform
        return name, None

    def LoadInto(self, module, path: str, strict: bool = True):
        """Validate everything first, then copy (a failed transfer leaves the module untouched)."""
        r = OaSafeTensorReader()
        st = r.Open(path)
        rep = OaTransferReport()
        if not st:
            return rep, st
        targets = {n.Name: n.Param for n in module.AllNamedParameterPtrs()}
        staged = {}
        for src in r.Names():
            dst, tf = self.Map(src)
            if dst not in targets:
                rep.Unused.append(src)
                continue
            t = r.Tensor(src)
            t = tf(t) if tf is not None else t
            want = tuple(targets[dst].Tensor().shape)
            if tuple(t.shape) != want:
                rep.ShapeMismatch.append((dst, tuple(t.shape), want))
                continue
            staged[dst] = t
        rep.Missing = sorted(set(targets) - set(staged) - {m[0] for m in rep.ShapeMismatch})
        if rep.ShapeMismatch or (strict and rep.Missing):
            r.Close()
            return rep, OaStatus.Error(OaStatusCode.FailedPrecondition, f"transfer: {len(rep.Missing)} missing, {len(rep.ShapeMismatch)} shape mismatches")
        for dst, t in staged.items():
            p = targets[dst].Tensor()
            p.copy_(t.to(dtype=p.dtype, device=p.device))
            rep.Loaded.append(dst)
        r.Close()
        return rep, OaStatus.Ok()

    def Verify(self, module, path: str, atol: float = 0.0):
        """Max absolute difference between the module's parameters and the (mapped) source tensors."""
        r = OaSafeTensorReader()
        st = r.Open(path)
        if not st:
            return float("inf"), st
        targets = {n.Name: n.Param for n in module.AllNamedParameterPtrs()}
        worst = 0.0
        for src in r.Names():
            dst, tf = self.Map(src)
            if dst in targets:
                t = r.Tensor(src)
                t = tf(t) if tf is not None else t
                p = targets[dst].Tensor()
                worst = max(worst, float((p.float().cpu() - t.to(p.dtype).float()).abs().max()))
        r.Close()
        ok = worst <= atol
        return worst, OaStatus.Ok() if ok else OaStatus.Error(OaStatusCode.DataLoss, f"transfer: parameters differ from the source by {worst}")
