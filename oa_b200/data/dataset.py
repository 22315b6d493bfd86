"""Datasets and the batching loader (Source/Public/Oa/Data/Dataset.h:12-118).

OaDataset is the map-style interface (Size / GetItem / GetSample); OaByteDataset cuts raw files into fixed-length byte
sequences (the byte-level language-modelling input); OaOadTokenDataset reads a split of an .oad archive as next-token
pairs.  OaDataLoader shuffles with its own seeded generator, batches on the host in pinned memory and, with
`NumWorkers > 0`, assembles batches ahead of time on a thread pool; `ToDevice` stages a batch through the upload ring."""
from __future__ import annotations

import os
import warnings
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass, field
from typing import Optional

import torch

from ..core.matrix import OaMatrix
from ..io.oad import OaOadFile, OaOadSplit


class OaDataset:
    class Sample:
        def __init__(self, x: Optional[OaMatrix] = None, y: Optional[OaMatrix] = None):
            self.X, self.Y = x if x is not None else OaMatrix(), y if y is not None else OaMatrix()

        def HasLabel(self) -> bool:
            return not self.Y.IsEmpty()

    def Size(self) -> int:
        raise NotImplementedError

    def GetItem(self, index: int) -> OaMatrix:
        raise NotImplementedError

    def GetSample(self, index: int) -> "OaDataset.Sample":
        return OaDataset.Sample(self.GetItem(index))

    def __getitem__(self, index: int) -> OaMatrix:
        return self.GetItem(index)

    def __len__(self) -> int:
        return self.Size()


class OaByteDataset(OaDataset):
    """Every file under `path` (or the single file) cut into sequences of `seq_len` bytes (int32 ids on the host)."""

    def __init__(self, path: str, seq_len: int = 1024, single_file: bool = False):
        self.SeqLen = int(seq_len)
        files = [path] if (single_file or os.path.isfile(path)) else sorted(os.path.join(path, f) for f in os.listdir(path))
        self._data = []
        for f in files:
            if os.path.isfile(f):
                with open(f, "rb") as h:
                    self._data.append(torch.frombuffer(bytearray(h.read()), dtype=torch.uint8))
        self._counts = [len(d) // self.SeqLen for d in self._data]
        self.NumSequences, self.TotalBytes_ = sum(self._counts), sum(len(d) for d in self._data)

    def Size(self) -> int:
        return self.NumSequences

    def TotalBytes(self) -> int:
        return self.TotalBytes_

    def GetItem(self, index: int) -> OaMatrix:
        if not 0 <= index < self.NumSequences:
            raise IndexError(index)
        for d, n in zip(self._data, self._counts):
            if index < n:
                return OaMatrix(d[index * self.SeqLen:(index + 1) * self.SeqLen].to(torch.int32))
            index -= n
        raise IndexError(index)


class OaOadTokenDataset(OaDataset):
    """Next-token samples from one split of an .oad archive of byte tokens: X = bytes[i*S : i*S+S], Y = the same shifted by one."""

    def __init__(self, path: str, seq_len: int, split: OaOadSplit = OaOadSplit.Train):
        self._file = OaOadFile()
        if not self._file.TryOpen(path):
            raise FileNotFoundError(f"not a readable .oad archive: {path}")
        self.SeqLen = int(seq_len)
        span = self._file.Span(split)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)        # read-only mapping: the tensor is never written
            self._bytes = torch.frombuffer(span, dtype=torch.uint8) if len(span) else torch.empty(0, dtype=torch.uint8)
        self._n = max(0, (len(self._bytes) - 1) // self.SeqLen)

    def Size(self) -> int:
        return self._n

    def GetItem(self, index: int) -> OaMatrix:
        return self.GetSample(index).X

    def GetSample(self, index: int) -> OaDataset.Sample:
        if not 0 <= index < self._n:
            raise IndexError(index)
        a = index * self.SeqLen
        return OaDataset.Sample(OaMatrix(self._bytes[a:a + self.SeqLen].to(torch.int32)), OaMatrix(self._bytes[a + 1:a + self.SeqLen + 1].to(torch.int32)))


class OaDataTransform:
    def Apply(self, sample: OaDataset.Sample) -> None:
        raise NotImplementedError


@dataclass
class OaDataLoaderConfig:
    BatchSize: int = 32
    Shuffle: bool = True
    Seed: int = 0               # 0: nondeterministic
    NumWorkers: int = 0
    DropLast: bool = False
    PinMemory: bool = False
    Transforms: list = field(default_factory=list)


class OaDataLoader:
    class Batch:
        def __init__(self, x: OaMatrix, y: OaMatrix):
            self.X, self.Y = x, y

        def IsValid(self) -> bool:
            return not self.X.IsEmpty()

        __bool__ = IsValid

    def __init__(self, dataset: OaDataset, config: Optional[OaDataLoaderConfig] = None):
        self.Dataset, self.Config = dataset, config or OaDataLoaderConfig()
        self._gen = torch.Generator()
        if self.Config.Seed:
            self._gen.manual_seed(self.Config.Seed)
        else:
            self._gen.seed()
        self._pool = ThreadPoolExecutor(self.Config.NumWorkers) if self.Config.NumWorkers > 0 else None
        self._pending: list = []
        self.Reset()

    def NumBatches(self) -> int:
        n, b = self.Dataset.Size(), self.Config.BatchSize
        return n // b if self.Config.DropLast else (n + b - 1) // b

    def Reset(self) -> None:
        n = self.Dataset.Size()
        self._order = torch.randperm(n, generator=self._gen).tolist() if self.Config.Shuffle else list(range(n))
        self._cursor = 0
        self._pending = []

    def _assemble(self, idx: list) -> "OaDataLoader.Batch":
        xs, ys = [], []
        for i in idx:
            s = self.Dataset.GetSample(i)
            for t in self.Config.Transforms:
                t.Apply(s)
            xs.append(s.X.Tensor())
            if s.HasLabel():
                ys.append(s.Y.Tensor())
        x = torch.stack(xs)
        y = torch.stack(ys) if len(ys) == len(xs) else None
        if self.Config.PinMemory and torch.cuda.is_available():
            x = x.pin_memory()
            y = y.pin_memory() if y is not None else None
        return OaDataLoader.Batch(OaMatrix(x), OaMatrix(y) if y is not None else OaMatrix())

    def _next_indices(self) -> Optional[list]:
        b = self.Config.BatchSize
        idx = self._order[self._cursor:self._cursor + b]
        if not idx or (self.Config.DropLast and len(idx) < b):
            return None
        self._cursor += len(idx)
        return idx

    def NextBatch(self) -> Optional["OaDataLoader.Batch"]:
        if self._pool is None:
            idx = self._next_indices()
            return self._assemble(idx) if idx is not None else None
        while len(self._pending) < 2 * self.Config.NumWorkers:          # keep the workers busy ahead of the consumer
            idx = self._next_indices()
            if idx is None:
                break
            self._pending.append(self._pool.submit(self._assemble, idx))
        return self._pending.pop(0).result() if self._pending else None

    def Next(self) -> Optional[OaMatrix]:
        b = self.NextBatch()
        return b.X if b is not None else None

    def __iter__(self):
        self.Reset()
        while True:
            b = self.NextBatch()
            if b is None:
                return
            yield b
