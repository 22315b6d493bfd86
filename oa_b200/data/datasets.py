"""Concrete datasets, index utilities and the asynchronous file reader.

Parity (paths inside the reference): Data/DsMnist.h (IDX files), Data/DsTinyShakespeare.h and Data/DsDailyDialog.h
(byte-level next-character samples), Data/DsHumanMl3d.h (motion clips with captions, world-joint recovery and motion
metrics), Data/DsSharded.h (directory of byte shards), Data/DsSubset.h, Data/FnDataset.h (Shuffle, RandomSplit,
Collate, Normalize, ScaleToRange, Cast), Data/IoUringReader.h (here: `OaAsyncReader` over `csrc/runtime/reader.cpp`).

Batches are assembled on the host as contiguous uint8 / int32 / fp32 tensors so that they can be staged to the device
with one copy from pinned memory.
"""
from __future__ import annotations

import ctypes
import math
import os
import struct
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..core.matrix import OaMatrix
from ..core.types import OaStatus, OaStatusCode
from ..io.oam import runtime_lib
from .dataset import OaDataset


# ------------------------------------------------------------------------------------------ async reader
_reader_ready = False


def _reader_lib():
    global _reader_ready
    L = runtime_lib()
    if not _reader_ready:
        vp, i64, i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
        for name, (res, args) in {
            "oa_reader_open": (vp, [ctypes.c_char_p, i32, i32]), "oa_reader_close": (None, [vp]),
            "oa_reader_file_size": (i64, [vp]), "oa_reader_bytes_read": (i64, [vp]), "oa_reader_in_flight": (i32, [vp]),
            "oa_reader_submit": (i32, [vp, vp, i64, i64]), "oa_reader_wait": (i32, [vp, i32]),
        }.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _reader_ready = True
    return L


class OaAsyncReader:
    """Positioned reads of one file into caller-owned host memory, `queue_depth` in flight at most."""

    def __init__(self, path: str, queue_depth: int = 32, threads: int = 0):
        self._L = _reader_lib()
        self._h = self._L.oa_reader_open(os.fsencode(path), queue_depth, threads)
        self._keep: list = []

    def IsValid(self) -> bool: return bool(self._h)
    def FileSize(self) -> int: return self._L.oa_reader_file_size(self._h) if self._h else 0
    def BytesRead(self) -> int: return self._L.oa_reader_bytes_read(self._h) if self._h else 0
    def InFlight(self) -> int: return self._L.oa_reader_in_flight(self._h) if self._h else 0

    def SubmitRead(self, dst: torch.Tensor, file_offset: int, nbytes: Optional[int] = None) -> OaStatus:
        """`dst` is a contiguous CPU tensor (pinned for uploads) of at least `nbytes` bytes."""
        if not self._h:
            return OaStatus(OaStatusCode.FailedPrecondition, "reader is not open")
        cap = dst.numel() * dst.element_size()
        nbytes = cap if nbytes is None else nbytes
        if dst.device.type != "cpu" or not dst.is_contiguous() or nbytes > cap:
            return OaStatus(OaStatusCode.InvalidArgument, "destination must be a contiguous CPU tensor large enough for the read")
        rc = self._L.oa_reader_submit(self._h, dst.data_ptr(), file_offset, nbytes)
        if rc == -1:
            return OaStatus(OaStatusCode.OutOfRange, "read outside the file")
        if rc == -2:
            return OaStatus(OaStatusCode.ResourceExhausted, "queue is full: collect completions first")
        self._keep.append(dst)
        return OaStatus.Ok()

    def WaitCompletions(self, min_complete: int = 1) -> int:
        """Number of reads collected; negative when any of them failed."""
        n = self._L.oa_reader_wait(self._h, min_complete) if self._h else 0
        if self.InFlight() == 0:
            self._keep.clear()
        return n

    def Close(self) -> None:
        if self._h:
            self._L.oa_reader_close(self._h)
            self._h = None

    def __del__(self):
        self.Close()


OaIoUringReader = OaAsyncReader       # the name the reference gives the same interface


def OaReadFileParallel(path: str, pinned: bool = False, chunk_bytes: int = 8 << 20, queue_depth: int = 16) -> torch.Tensor:
    """Whole file as a uint8 tensor, read in `chunk_bytes` pieces with `queue_depth` reads in flight."""
    r = OaAsyncReader(path, queue_depth)
    if not r.IsValid():
        raise FileNotFoundError(path)
    size = r.FileSize()
    out = torch.empty(size, dtype=torch.uint8, pin_memory=pinned and torch.cuda.is_available())
    off, ok = 0, True
    while off < size:
        n = min(chunk_bytes, size - off)
        st = r.SubmitRead(out[off:off + n], off, n)
        if st.code == OaStatusCode.ResourceExhausted:
            ok &= r.WaitCompletions(1) >= 0
            continue
        if not st.IsOk():
            raise IOError(st.message)
        off += n
    while r.InFlight():
        ok &= r.WaitCompletions(r.InFlight()) >= 0
    r.Close()
    if not ok:
        raise IOError(f"short read on {path}")
    return out


# ------------------------------------------------------------------------------------------ index utilities
class OaFnDataset:
    @dataclass
    class SplitResult:
        Train: List[int] = field(default_factory=list)
        Val: List[int] = field(default_factory=list)
        Test: List[int] = field(default_factory=list)

    @dataclass
    class Batch:
        X: OaMatrix
        Y: OaMatrix

    @staticmethod
    def Shuffle(indices: List[int], seed: int = 0) -> None:
        g = torch.Generator().manual_seed(int(seed))
        perm = torch.randperm(len(indices), generator=g).tolist()
        indices[:] = [indices[i] for i in perm]

    @staticmethod
    def RandomSplit(total: int, train_ratio: float = 0.8, val_ratio: float = 0.1, seed: int = 42) -> "OaFnDataset.SplitResult":
        idx = list(range(total))
        OaFnDataset.Shuffle(idx, seed)
        n_train = int(total * train_ratio)
        n_val = int(total * val_ratio)
        return OaFnDataset.SplitResult(idx[:n_train], idx[n_train:n_train + n_val], idx[n_train + n_val:])

    @staticmethod
    def Collate(samples: Sequence[OaDataset.Sample]) -> "OaFnDataset.Batch":
        xs = torch.stack([s.X.Tensor() for s in samples])
        ys = [s.Y.Tensor() for s in samples if s.HasLabel()]
        return OaFnDataset.Batch(OaMatrix(xs), OaMatrix(torch.stack(ys)) if len(ys) == len(samples) else OaMatrix())

    @staticmethod
    def Normalize(batch: OaMatrix, mean: Sequence[float], std: Sequence[float]) -> OaStatus:
        """In place, per channel (axis 1) for rank >= 3, per feature (last axis) otherwise."""
        t = batch.Tensor()
        if not t.is_floating_point():
            return OaStatus(OaStatusCode.InvalidArgument, "Normalize needs a floating-point batch")
        m, s = torch.tensor(mean, dtype=t.dtype, device=t.device), torch.tensor(std, dtype=t.dtype, device=t.device)
        if (s == 0).any():
            return OaStatus(OaStatusCode.InvalidArgument, "zero standard deviation")
        shape = [1, -1] + [1] * (t.dim() - 2) if t.dim() >= 3 else [-1]
        t.sub_(m.view(shape)).div_(s.view(shape))
        return OaStatus.Ok()

    @staticmethod
    def ScaleToRange(batch: OaMatrix, lo: float = 0.0, hi: float = 1.0) -> OaStatus:
        t = batch.Tensor()
        if not t.is_floating_point():
            return OaStatus(OaStatusCode.InvalidArgument, "ScaleToRange needs a floating-point batch")
        mn, mx = t.min(), t.max()
        span = (mx - mn).clamp_min(1e-12)
        t.sub_(mn).mul_((hi - lo) / span).add_(lo)
        return OaStatus.Ok()

    @staticmethod
    def Cast(batch: OaMatrix, dtype: torch.dtype) -> OaMatrix:
        return OaMatrix(batch.Tensor().to(dtype))


class OaDsSubset(OaDataset):
    def __init__(self, parent: OaDataset, indices: Sequence[int]):
        self._parent, self._idx = parent, [int(i) for i in indices]
        n = parent.Size()
        if any(i < 0 or i >= n for i in self._idx):
            raise IndexError("subset index outside the parent dataset")

    def Size(self) -> int: return len(self._idx)
    def GetItem(self, index: int) -> OaMatrix: return self._parent.GetItem(self._idx[index])
    def GetSample(self, index: int) -> OaDataset.Sample: return self._parent.GetSample(self._idx[index])
    def Indices(self) -> List[int]: return list(self._idx)
    def Parent(self) -> OaDataset: return self._parent


class _BatchedMixin:
    """Shuffled mini-batch iteration shared by the in-memory datasets."""

    def _init_batches(self, num_samples: int, batch_size: int, shuffle: bool, seed: int = 0x0A5EED) -> None:
        self._n, self._bs, self._shuffle = int(num_samples), int(batch_size), shuffle
        self._gen = torch.Generator().manual_seed(seed)
        self._nb = self._n // self._bs if self._bs > 0 else 0
        self._cursor = 0
        self._order = torch.randperm(self._n, generator=self._gen) if shuffle else torch.arange(self._n)

    def NumBatches(self) -> int: return self._nb
    def BatchSize(self) -> int: return self._bs

    def Reset(self, reshuffle: bool = True) -> None:
        self._cursor = 0
        if reshuffle and self._shuffle:
            self._order = torch.randperm(self._n, generator=self._gen)

    def _next_indices(self) -> Optional[torch.Tensor]:
        if self._cursor >= self._nb:
            return None
        idx = self._order[self._cursor * self._bs:(self._cursor + 1) * self._bs]
        self._cursor += 1
        return idx


# ------------------------------------------------------------------------------------------ MNIST (IDX files)
def _read_idx(path: str) -> np.ndarray:
    with open(path, "rb") as f:
        raw = f.read()
    zero, dtype_code, rank = struct.unpack(">HBB", raw[:4])
    if zero != 0 or dtype_code != 0x08:
        raise ValueError(f"{path}: not an unsigned-byte IDX file")
    dims = struct.unpack(">" + "I" * rank, raw[4:4 + 4 * rank])
    data = np.frombuffer(raw, dtype=np.uint8, offset=4 + 4 * rank)
    if data.size != int(np.prod(dims)):
        raise ValueError(f"{path}: truncated IDX payload")
    return data.reshape(dims)


class OaDsMnist(_BatchedMixin, OaDataset):
    """`<dir>/{train,t10k}-images-idx3-ubyte` + `-labels-idx1-ubyte`; samples are 784 uint8 pixels and a uint8 label."""

    def __init__(self, data_dir: str, split: str = "train", batch_size: int = 64, shuffle: bool = True):
        stem = "train" if split == "train" else "t10k"
        images = _read_idx(os.path.join(data_dir, f"{stem}-images-idx3-ubyte"))
        labels = _read_idx(os.path.join(data_dir, f"{stem}-labels-idx1-ubyte"))
        if images.shape[0] != labels.shape[0] or images.shape[1:] != (28, 28):
            raise ValueError("MNIST images / labels do not match")
        self._images = torch.from_numpy(images.reshape(images.shape[0], 784).copy())
        self._labels = torch.from_numpy(labels.copy())
        self._init_batches(images.shape[0], batch_size, shuffle)

    def Size(self) -> int: return self._n
    def NumSamples(self) -> int: return self._n
    def InputSize(self) -> int: return 784
    def OutputSize(self) -> int: return 1
    def GetItem(self, index: int) -> OaMatrix: return OaMatrix(self._images[index])

    def GetSample(self, index: int) -> OaDataset.Sample:
        return OaDataset.Sample(OaMatrix(self._images[index]), OaMatrix(self._labels[index:index + 1]))

    def NextBatch(self) -> Optional[Tuple[OaMatrix, OaMatrix]]:
        """([B, 784] uint8, [B] uint8) or None at the end of the epoch."""
        idx = self._next_indices()
        if idx is None:
            return None
        return OaMatrix(self._images[idx]), OaMatrix(self._labels[idx])


# ------------------------------------------------------------------------------------------ byte-level text
class _ByteTextDataset(_BatchedMixin, OaDataset):
    def __init__(self, file_path: str, batch_size: int = 64, context_len: int = 128, shuffle: bool = True):
        self._text = OaReadFileParallel(file_path)
        self._ctx = int(context_len)
        self.NumChars_ = self._text.numel()
        self._init_batches(max(0, self.NumChars_ - self._ctx), batch_size, shuffle)

    def Size(self) -> int: return self._n
    def NumChars(self) -> int: return self.NumChars_
    def ContextLen(self) -> int: return self._ctx

    def GetItem(self, index: int) -> OaMatrix:
        if not 0 <= index < self._n:
            return OaMatrix()
        return OaMatrix(self._text[index:index + self._ctx])

    def GetSample(self, index: int) -> OaDataset.Sample:
        if not 0 <= index < self._n:
            return OaDataset.Sample()
        return OaDataset.Sample(OaMatrix(self._text[index:index + self._ctx]), OaMatrix(self._text[index + self._ctx:index + self._ctx + 1]))

    def NextBatch(self) -> Optional[Tuple[OaMatrix, OaMatrix]]:
        """([B, context] uint8, [B] uint8 next byte) or None at the end of the epoch."""
        idx = self._next_indices()
        if idx is None:
            return None
        win = idx[:, None] + torch.arange(self._ctx + 1)[None, :]
        block = self._text[win]
        return OaMatrix(block[:, :-1].contiguous()), OaMatrix(block[:, -1].contiguous())


class OaDsTinyShakespeare(_ByteTextDataset):
    """One text file; sample i is bytes [i, i + context) with byte i + context as the label."""


class OaDsDailyDialog(_ByteTextDataset):
    """Dialogue transcript with conversations separated by blank lines; samples as for any byte text."""

    def __init__(self, file_path: str, batch_size: int = 64, context_len: int = 128, shuffle: bool = True):
        super().__init__(file_path, batch_size, context_len, shuffle)
        blocks = [b for b in bytes(self._text.numpy().tobytes()).replace(b"\r", b"").split(b"\n\n") if b.strip()]
        self._conversations = len(blocks)

    def NumConversations(self) -> int: return self._conversations


# ------------------------------------------------------------------------------------------ sharded bytes
class OaDsSharded(OaDataset):
    """Every regular file of a directory is a shard of raw bytes (memory-mapped); sequences never cross shards."""

    def __init__(self, directory: str, seq_len: int):
        self._seq = int(seq_len)
        files = sorted(os.path.join(directory, f) for f in os.listdir(directory))
        self._shards = [np.memmap(f, dtype=np.uint8, mode="r") for f in files if os.path.isfile(f) and os.path.getsize(f) > 0]
        self._counts = [len(s) // self._seq for s in self._shards]
        self._prefix = np.concatenate([[0], np.cumsum(self._counts)]).astype(np.int64)
        self.TotalBytes_ = int(sum(len(s) for s in self._shards))

    def Size(self) -> int: return int(self._prefix[-1])
    def TotalBytes(self) -> int: return self.TotalBytes_
    def NumShards(self) -> int: return len(self._shards)
    def SeqLen(self) -> int: return self._seq
    def ShardBytes(self, shard: int) -> int: return len(self._shards[shard])
    def ShardData(self, shard: int) -> np.ndarray: return self._shards[shard]

    def GetItem(self, index: int) -> OaMatrix:
        if not 0 <= index < self.Size():
            raise IndexError(index)
        shard = int(np.searchsorted(self._prefix, index, side="right") - 1)
        local = index - int(self._prefix[shard])
        return OaMatrix(torch.from_numpy(np.array(self._shards[shard][local * self._seq:(local + 1) * self._seq])))

    def SampleSequence(self, rng_state: int) -> Tuple[np.ndarray, int]:
        """A random window of `seq_len` bytes (any offset) with a 64-bit xorshift state; returns (bytes, new state)."""
        x = rng_state & (2 ** 64 - 1) or 0x9E3779B97F4A7C15
        def step(v):
            v ^= (v << 13) & (2 ** 64 - 1); v ^= v >> 7; v ^= (v << 17) & (2 ** 64 - 1)
            return v
        x = step(x)
        shard = x % len(self._shards)
        x = step(x)
        span = len(self._shards[shard]) - self._seq
        if span < 0:
            raise ValueError("shard shorter than the sequence length")
        off = x % (span + 1)
        return np.array(self._shards[shard][off:off + self._seq]), x


# ------------------------------------------------------------------------------------------ HumanML3D
@dataclass
class OaHumanMl3dCaption:
    Text: str = ""
    StartSec: float = 0.0
    EndSec: float = 0.0
    HasRange: bool = False


@dataclass
class OaHumanMl3dMotionMetrics:
    MpjpeCm: float = 0.0
    VelocityErrorCmPerFrame: float = 0.0
    ContactAccuracy: float = 0.0
    FootSkateCmPerFrame: float = 0.0
    Ok: bool = False


def _joints_for_feat_dim(feat_dim: int) -> int:
    """feat_dim = 4 root + 3 (J-1) positions + 6 (J-1) rotations + 3 J velocities + 4 contacts = 12 J - 1."""
    return (feat_dim + 1) // 12 if feat_dim > 0 and (feat_dim + 1) % 12 == 0 else 0


def OaHumanMl3dRecoverWorldJoints(features, frames: int, feat_dim: int = 263) -> torch.Tensor:
    """[frames, J, 3] world positions from the root-relative feature vectors (DsHumanMl3d.cpp:148-208).

    Feature 0 is the per-frame change of the root's half yaw angle, 1-2 the root's planar velocity in its own frame,
    3 the root height, 4.. the other joints relative to the root.  Angles and positions integrate from frame 0."""
    f = torch.as_tensor(features, dtype=torch.float32).reshape(-1)
    joints = _joints_for_feat_dim(feat_dim)
    if frames <= 0 or joints <= 0 or f.numel() < frames * feat_dim:
        return torch.empty(0)
    f = f[:frames * feat_dim].view(frames, feat_dim)
    half = torch.zeros(frames)
    half[1:] = torch.cumsum(f[:-1, 0], 0)
    # rotation by the quaternion (w = cos a, y = -sin a): a turn of -2a about the vertical axis
    c, s = torch.cos(-2.0 * half), torch.sin(-2.0 * half)

    def rotate(x, z):
        return x * c + z * s, -x * s + z * c

    dx, dz = torch.zeros(frames), torch.zeros(frames)
    dx[1:], dz[1:] = f[:-1, 1], f[:-1, 2]
    rx, rz = rotate(dx, dz)
    root = torch.stack([torch.cumsum(rx, 0), f[:, 3], torch.cumsum(rz, 0)], dim=1)
    ric = f[:, 4:4 + (joints - 1) * 3].view(frames, joints - 1, 3)
    c, s = c[:, None], s[:, None]
    wx, wz = rotate(ric[..., 0], ric[..., 2])
    world = torch.stack([wx + root[:, None, 0], ric[..., 1], wz + root[:, None, 2]], dim=-1)
    return torch.cat([root[:, None, :], world], dim=1)


def OaHumanMl3dMpjpeCm(pred_world, target_world) -> float:
    p, t = torch.as_tensor(pred_world, dtype=torch.float64).reshape(-1, 3), torch.as_tensor(target_world, dtype=torch.float64).reshape(-1, 3)
    if p.numel() == 0 or p.shape != t.shape:
        return float("nan")
    return float(100.0 * (p - t).norm(dim=1).mean())


def OaHumanMl3dEvaluateMotion(pred_features, target_features, frames: int, feat_dim: int = 263,
                              contact_threshold: float = 0.5) -> OaHumanMl3dMotionMetrics:
    out = OaHumanMl3dMotionMetrics()
    pw, tw = OaHumanMl3dRecoverWorldJoints(pred_features, frames, feat_dim), OaHumanMl3dRecoverWorldJoints(target_features, frames, feat_dim)
    if pw.numel() == 0 or pw.shape != tw.shape:
        return out
    joints = pw.shape[1]
    out.MpjpeCm = OaHumanMl3dMpjpeCm(pw, tw)
    if frames > 1:
        dv = (pw[1:] - pw[:-1]) - (tw[1:] - tw[:-1])
        out.VelocityErrorCmPerFrame = float(100.0 * dv.double().norm(dim=-1).mean())
    pf = torch.as_tensor(pred_features, dtype=torch.float32).reshape(-1)[:frames * feat_dim].view(frames, feat_dim)
    tf = torch.as_tensor(target_features, dtype=torch.float32).reshape(-1)[:frames * feat_dim].view(frames, feat_dim)
    pc, tc = pf[:, -4:] >= contact_threshold, tf[:, -4:] >= contact_threshold
    out.ContactAccuracy = float((pc == tc).double().mean())
    skate, count = 0.0, 0
    for k, j in enumerate((7, 10, 8, 11)):            # left ankle, left foot, right ankle, right foot
        if j >= joints or frames < 2:
            continue
        step = (pw[1:, j, [0, 2]] - pw[:-1, j, [0, 2]]).double().norm(dim=-1)
        mask = tc[1:, k]
        skate += float(step[mask].sum())
        count += int(mask.sum())
    out.FootSkateCmPerFrame = 100.0 * skate / count if count else 0.0
    out.Ok = all(math.isfinite(v) for v in (out.MpjpeCm, out.VelocityErrorCmPerFrame, out.ContactAccuracy, out.FootSkateCmPerFrame))
    return out


def _read_captions(path: str) -> List[OaHumanMl3dCaption]:
    """Lines of `text#part-of-speech tags#start#end`; a 0 / 0 range means the caption covers the whole clip."""
    caps: List[OaHumanMl3dCaption] = []
    if not os.path.isfile(path):
        return caps
    with open(path, "r", encoding="utf-8", errors="replace") as f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            parts = line.split("#")
            cap = OaHumanMl3dCaption(parts[0].strip())
            if len(parts) >= 4:
                try:
                    cap.StartSec, cap.EndSec = float(parts[2]), float(parts[3])
                    cap.HasRange = cap.EndSec > cap.StartSec
                except ValueError:
                    pass
            caps.append(cap)
    return caps


class OaDsHumanMl3d(OaDataset):
    """`<dir>/<split>.txt` lists clip ids; `<dir>/new_joint_vecs/<id>.npy` holds [frames, feat_dim] fp32 features,
    `<dir>/texts/<id>.txt` the captions, `<dir>/Mean.npy` / `Std.npy` the feature statistics.  Items are normalised."""

    def __init__(self, data_dir: str, split: str = "train", max_clips: int = 0, feat_dim: int = 263):
        self.FeatDim_, self.NumJoints_ = feat_dim, _joints_for_feat_dim(feat_dim)
        self._clips: List[torch.Tensor] = []
        self._ids: List[str] = []
        self._caps: List[List[OaHumanMl3dCaption]] = []
        self.Ok_ = False
        try:
            self.Mean = torch.from_numpy(np.load(os.path.join(data_dir, "Mean.npy")).astype(np.float32))
            self.Std = torch.from_numpy(np.load(os.path.join(data_dir, "Std.npy")).astype(np.float32))
            with open(os.path.join(data_dir, f"{split}.txt")) as f:
                ids = [l.strip() for l in f if l.strip()]
        except OSError:
            return
        if self.Mean.numel() != feat_dim or self.Std.numel() != feat_dim:
            return
        for cid in ids:
            p = os.path.join(data_dir, "new_joint_vecs", cid + ".npy")
            if not os.path.isfile(p):
                continue
            arr = np.load(p)
            if arr.ndim != 2 or arr.shape[1] != feat_dim or arr.shape[0] == 0:
                continue
            self._clips.append(torch.from_numpy(arr.astype(np.float32)))
            self._ids.append(cid)
            self._caps.append(_read_captions(os.path.join(data_dir, "texts", cid + ".txt")))
            if max_clips and len(self._clips) >= max_clips:
                break
        self.Ok_ = len(self._clips) > 0

    def Ok(self) -> bool: return self.Ok_
    def Name(self) -> str: return "HumanML3D"
    def Size(self) -> int: return len(self._clips)
    def NumClips(self) -> int: return len(self._clips)
    def FeatDim(self) -> int: return self.FeatDim_
    def NumJoints(self) -> int: return self.NumJoints_
    def TotalFrames(self) -> int: return sum(c.shape[0] for c in self._clips)
    def ClipFrames(self, index: int) -> int: return self._clips[index].shape[0]
    def ClipData(self, index: int) -> torch.Tensor: return self._clips[index]
    def ClipId(self, index: int) -> str: return self._ids[index]
    def ClipCaptions(self, index: int) -> List[OaHumanMl3dCaption]: return self._caps[index]
    def ClipText(self, index: int) -> str: return self._caps[index][0].Text if self._caps[index] else ""

    def GetItem(self, index: int) -> OaMatrix:
        return OaMatrix((self._clips[index] - self.Mean) / self.Std.clamp_min(1e-8))

    def Denormalize(self, features: torch.Tensor) -> torch.Tensor:
        return features * self.Std.clamp_min(1e-8) + self.Mean
