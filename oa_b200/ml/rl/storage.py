"""Fixed-capacity device-resident RL storage: the time-major on-policy rollout and the circular off-policy replay.

Reference: Source/Public/Oa/Ml/Rl/Rollout.h:9-82 and Replay.h:7-61 (Rl/Rollout.cpp, Rl/Replay.cpp; kernels
RlRolloutAppend / RlRolloutReset / RlReplayAppend / RlReplaySample).  Size and Cursor are host control metadata; tensor
data never crosses the host.  Every Append is one fused kernel launch.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch

from ...core import fn_matrix as F
from ...core.matrix import OaMatrix
from ...core.types import OaScalarType, OaStatus, OaStatusCode, to_torch_dtype
from ...ops import rl as R
from ...runtime import engine as RT
from .fn_rl import OaGaeConfig, GaeInto


def _err(code, msg):
    return OaStatus.Error(code, msg)


@dataclass
class OaRlRolloutConfig:
    Time: int = 0
    Environments: int = 0
    ObservationShape: tuple = ()


@dataclass
class OaRlTransition:
    Observation: Optional[OaMatrix] = None       # fp32 [E, ...ObservationShape]
    Action: Optional[OaMatrix] = None            # Int32 [E]
    Reward: Optional[OaMatrix] = None            # fp32 [E]
    Value: Optional[OaMatrix] = None
    NextValue: Optional[OaMatrix] = None
    LogProbability: Optional[OaMatrix] = None
    Terminated: Optional[OaMatrix] = None        # UInt8 [E]
    Truncated: Optional[OaMatrix] = None


@dataclass
class OaRlRolloutBatch:
    """Time-major carrier; reshape the leading [Time, Environments] axes for minibatch views without copying."""
    Observation: Optional[OaMatrix] = None
    Action: Optional[OaMatrix] = None
    Reward: Optional[OaMatrix] = None
    Value: Optional[OaMatrix] = None
    NextValue: Optional[OaMatrix] = None
    OldLogProbability: Optional[OaMatrix] = None
    Terminated: Optional[OaMatrix] = None
    Truncated: Optional[OaMatrix] = None
    Valid: Optional[OaMatrix] = None
    Advantage: Optional[OaMatrix] = None
    Return: Optional[OaMatrix] = None

    def IsValid(self) -> bool:
        return all(getattr(self, k) is not None for k in ("Observation", "Action", "Reward", "Value", "NextValue", "OldLogProbability",
                                                          "Terminated", "Truncated", "Valid", "Advantage", "Return"))


class OaRlRolloutBuffer:
    def __init__(self):
        self.Config_ = OaRlRolloutConfig()
        self.Batch_ = OaRlRolloutBatch()
        self.Size_ = 0
        self.Finalized_ = False
        self._obs_elems = 0

    @staticmethod
    def Create(config: OaRlRolloutConfig):
        """Returns (buffer, status)."""
        if config.Time <= 0 or config.Environments <= 0 or not config.ObservationShape or any(int(s) <= 0 for s in config.ObservationShape):
            return None, _err(OaStatusCode.InvalidArgument, "rollout needs positive Time, Environments and observation extents")
        b = OaRlRolloutBuffer()
        b.Config_ = config
        T, E, dev = config.Time, config.Environments, RT.get_engine().Device()
        z = lambda shape, dt: OaMatrix(torch.zeros(shape, dtype=dt, device=dev))
        b.Batch_ = OaRlRolloutBatch(
            Observation=z((T, E) + tuple(config.ObservationShape), torch.float32), Action=z((T, E), torch.int32),
            Reward=z((T, E), torch.float32), Value=z((T, E), torch.float32), NextValue=z((T, E), torch.float32),
            OldLogProbability=z((T, E), torch.float32), Terminated=z((T, E), torch.uint8), Truncated=z((T, E), torch.uint8),
            Valid=z((T, E), torch.uint8), Advantage=z((T, E), torch.float32), Return=z((T, E), torch.float32))
        b._obs_elems = 1
        for s in config.ObservationShape:
            b._obs_elems *= int(s)
        return b, OaStatus.Ok()

    def _dst(self) -> dict:
        B = self.Batch_
        return dict(obs=B.Observation.Tensor(), action=B.Action.Tensor(), reward=B.Reward.Tensor(), value=B.Value.Tensor(),
                    next_value=B.NextValue.Tensor(), logp=B.OldLogProbability.Tensor(), term=B.Terminated.Tensor(),
                    trunc=B.Truncated.Tensor(), valid=B.Valid.Tensor())

    def Append(self, tr: OaRlTransition) -> OaStatus:
        if not self.IsValid():
            return _err(OaStatusCode.FailedPrecondition, "rollout buffer was not created")
        if self.Finalized_ or self.Size_ >= self.Config_.Time:
            return _err(OaStatusCode.FailedPrecondition, "rollout buffer is full; Reset it before appending")
        E = self.Config_.Environments
        checks = ((tr.Observation, torch.float32, E * self._obs_elems), (tr.Action, torch.int32, E), (tr.Reward, torch.float32, E),
                  (tr.Value, torch.float32, E), (tr.NextValue, torch.float32, E), (tr.LogProbability, torch.float32, E),
                  (tr.Terminated, torch.uint8, E), (tr.Truncated, torch.uint8, E))
        for m, dt, n in checks:
            if m is None or m.IsEmpty() or m.Tensor().dtype != dt or m.Tensor().numel() != n:
                return _err(OaStatusCode.InvalidArgument, "transition field has the wrong dtype or element count")
        F._ctx_add("RlRolloutAppend")
        c = lambda m: F._c(m.Tensor().detach())
        src = dict(obs=c(tr.Observation), action=c(tr.Action), reward=c(tr.Reward), value=c(tr.Value), next_value=c(tr.NextValue),
                   logp=c(tr.LogProbability), term=c(tr.Terminated), trunc=c(tr.Truncated))
        R.rollout_append(src, self._dst(), self.Size_)
        self.Size_ += 1
        return OaStatus.Ok()

    def Finalize(self, config: Optional[OaGaeConfig] = None) -> OaStatus:
        if not self.IsFull():
            return _err(OaStatusCode.FailedPrecondition, "GAE needs a complete rollout")
        B = self.Batch_
        st = GaeInto(B.Reward, B.Value, B.NextValue, B.Terminated, B.Truncated, B.Advantage, B.Return, config)
        self.Finalized_ = bool(st)
        return st

    def Reset(self) -> None:
        """Starts a new collection cycle: clears Valid on the device, keeps every allocation."""
        if self.IsValid():
            F._ctx_add("RlRolloutReset")
            self.Batch_.Valid.Tensor().zero_()
        self.Size_ = 0
        self.Finalized_ = False

    def IsValid(self) -> bool: return self.Batch_.IsValid()
    def IsFull(self) -> bool: return self.Size_ == self.Config_.Time and self.Config_.Time > 0
    def IsFinalized(self) -> bool: return self.Finalized_
    def Size(self) -> int: return self.Size_
    def Capacity(self) -> int: return self.Config_.Time
    def Config(self) -> OaRlRolloutConfig: return self.Config_
    def Batch(self) -> OaRlRolloutBatch: return self.Batch_


# ---------------------------------------------------------------------------------------------------------- replay
@dataclass
class OaRlReplayConfig:
    Capacity: int = 0
    ObservationShape: tuple = ()
    ActionShape: tuple = ()
    ActionDtype: OaScalarType = OaScalarType.Int32


@dataclass
class OaRlReplayTransition:
    Observation: Optional[OaMatrix] = None
    Action: Optional[OaMatrix] = None
    NextObservation: Optional[OaMatrix] = None
    Reward: Optional[OaMatrix] = None
    Terminated: Optional[OaMatrix] = None
    Truncated: Optional[OaMatrix] = None


@dataclass
class OaRlReplayBatch:
    Observation: Optional[OaMatrix] = None
    Action: Optional[OaMatrix] = None
    NextObservation: Optional[OaMatrix] = None
    Reward: Optional[OaMatrix] = None
    Terminated: Optional[OaMatrix] = None
    Truncated: Optional[OaMatrix] = None
    Index: Optional[OaMatrix] = None

    def IsValid(self) -> bool:
        return all(getattr(self, k) is not None for k in ("Observation", "Action", "NextObservation", "Reward", "Terminated", "Truncated"))


def _prod(shape) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


class OaRlReplayBuffer:
    """Circular storage of (s, a, s', r, terminated, truncated); actions are Int32 (discrete) or fp32 (continuous)."""

    def __init__(self):
        self.Config_ = OaRlReplayConfig()
        self.Storage_ = OaRlReplayBatch()
        self.Size_ = 0
        self.Cursor_ = 0

    @staticmethod
    def Create(config: OaRlReplayConfig):
        if (config.Capacity <= 0 or not config.ObservationShape or any(int(s) <= 0 for s in config.ObservationShape)
                or any(int(s) <= 0 for s in config.ActionShape) or config.ActionDtype not in (OaScalarType.Int32, OaScalarType.Float32)):
            return None, _err(OaStatusCode.InvalidArgument, "replay needs positive capacity / extents and Int32 or Float32 actions")
        b = OaRlReplayBuffer()
        b.Config_ = config
        C, dev = config.Capacity, RT.get_engine().Device()
        z = lambda shape, dt: OaMatrix(torch.zeros(shape, dtype=dt, device=dev))
        adt = to_torch_dtype(config.ActionDtype)
        b.Storage_ = OaRlReplayBatch(
            Observation=z((C,) + tuple(config.ObservationShape), torch.float32), Action=z((C,) + tuple(config.ActionShape), adt),
            NextObservation=z((C,) + tuple(config.ObservationShape), torch.float32), Reward=z((C,), torch.float32),
            Terminated=z((C,), torch.uint8), Truncated=z((C,), torch.uint8))
        return b, OaStatus.Ok()

    @staticmethod
    def _dict(b: OaRlReplayBatch) -> dict:
        return dict(obs=b.Observation.Tensor(), action=b.Action.Tensor(), next_obs=b.NextObservation.Tensor(), reward=b.Reward.Tensor(),
                    term=b.Terminated.Tensor(), trunc=b.Truncated.Tensor())

    def Append(self, tr: OaRlReplayTransition) -> OaStatus:
        if not self.IsValid():
            return _err(OaStatusCode.FailedPrecondition, "replay buffer was not created")
        if tr.Reward is None or tr.Reward.IsEmpty():
            return _err(OaStatusCode.InvalidArgument, "empty transition")
        rows = tr.Reward.Tensor().numel()
        oe, ae = _prod(self.Config_.ObservationShape), _prod(self.Config_.ActionShape)
        adt = to_torch_dtype(self.Config_.ActionDtype)
        checks = ((tr.Observation, torch.float32, rows * oe), (tr.NextObservation, torch.float32, rows * oe), (tr.Action, adt, rows * ae),
                  (tr.Reward, torch.float32, rows), (tr.Terminated, torch.uint8, rows), (tr.Truncated, torch.uint8, rows))
        for m, dt, n in checks:
            if m is None or m.IsEmpty() or m.Tensor().dtype != dt or m.Tensor().numel() != n:
                return _err(OaStatusCode.InvalidArgument, "replay transition field has the wrong dtype or element count")
        if rows > self.Config_.Capacity:
            return _err(OaStatusCode.InvalidArgument, "more transitions than the replay capacity")
        F._ctx_add("RlReplayAppend")
        c = lambda m: F._c(m.Tensor().detach())
        src = dict(obs=c(tr.Observation), action=c(tr.Action), next_obs=c(tr.NextObservation), reward=c(tr.Reward), term=c(tr.Terminated),
                   trunc=c(tr.Truncated))
        R.replay_append(src, self._dict(self.Storage_), self.Cursor_, self.Config_.Capacity)
        self.Cursor_ = (self.Cursor_ + rows) % self.Config_.Capacity
        self.Size_ = min(self.Size_ + rows, self.Config_.Capacity)
        return OaStatus.Ok()

    def Sample(self, batch_size: int, seed: int):
        """Deterministic uniform sampling with replacement: returns (batch, status)."""
        if not self.IsValid() or batch_size <= 0:
            return None, _err(OaStatusCode.InvalidArgument, "invalid replay sample request")
        if self.Size_ == 0:
            return None, _err(OaStatusCode.FailedPrecondition, "replay buffer is empty")
        dev = self.Storage_.Reward.Tensor().device
        e = lambda like: OaMatrix(torch.empty((batch_size,) + tuple(like.Tensor().shape[1:]), dtype=like.Tensor().dtype, device=dev))
        S = self.Storage_
        out = OaRlReplayBatch(e(S.Observation), e(S.Action), e(S.NextObservation), e(S.Reward), e(S.Terminated), e(S.Truncated),
                              OaMatrix(torch.empty(batch_size, dtype=torch.int32, device=dev)))
        F._ctx_add("RlReplaySample")
        d = self._dict(out)
        d["index"] = out.Index.Tensor()
        R.replay_sample(self._dict(S), d, self.Size_, seed)
        return out, OaStatus.Ok()

    def Reset(self) -> None:
        self.Size_ = 0
        self.Cursor_ = 0

    def IsValid(self) -> bool: return self.Storage_.IsValid()
    def IsFull(self) -> bool: return self.Size_ == self.Config_.Capacity and self.Size_ > 0
    def Size(self) -> int: return self.Size_
    def Capacity(self) -> int: return self.Config_.Capacity
    def Cursor(self) -> int: return self.Cursor_
    def Config(self) -> OaRlReplayConfig: return self.Config_
