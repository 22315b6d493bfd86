"""Keyframes, curves, easing functions, time codes and the timeline.

Parity: Source/Public/Oa/Animation/Keyframe.h (keyframe records and tracks), Curve.h (float / vec3 / colour / quaternion
curves, derivative, the easing set), TimeCode.h / Time.h (frame-rate aware time), Timeline.h (time transform with offset,
scale and trim; play / pause / stop / seek, direction, looping).  Curves keep their keys as sorted tensors, so a whole
batch of sample times is evaluated with one `searchsorted` + gather on whichever device the times live on
(`EvaluateBatch`): sampling thousands of motion clips for a training batch costs one launch per curve, not one Python
call per sample.
"""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch


class OaKeyInterpolation(enum.IntEnum):
    Linear = 0
    Stepped = 1
    Cubic = 2          # Catmull-Rom through the neighbouring keys


@dataclass
class OaKeyframe:
    Time: float
    Value: Tuple[float, ...]
    Interpolation: OaKeyInterpolation = OaKeyInterpolation.Linear


class OaKeyframeTrack:
    """Keys kept sorted by time; a key added at an existing time replaces it."""

    def __init__(self, width: int):
        self.Width = width
        self._keys: List[OaKeyframe] = []

    def AddKeyframe(self, time: float, value, interpolation: OaKeyInterpolation = OaKeyInterpolation.Linear) -> None:
        v = tuple(float(x) for x in (value if isinstance(value, (tuple, list)) else (value,)))
        if len(v) != self.Width:
            raise ValueError(f"key has {len(v)} components, the track holds {self.Width}")
        k = OaKeyframe(float(time), v, interpolation)
        i = self.FindKeyframeAt(k.Time)
        if i >= 0 and self._keys[i].Time == k.Time:
            self._keys[i] = k
        else:
            self._keys.insert(i + 1, k)

    def RemoveKeyframe(self, index: int) -> None: del self._keys[index]
    def Clear(self) -> None: self._keys.clear()
    def GetKeyframeCount(self) -> int: return len(self._keys)
    def GetKeyframe(self, index: int) -> OaKeyframe: return self._keys[index]

    def FindKeyframeAt(self, time: float) -> int:
        """Index of the last key at or before `time`; -1 before the first key."""
        lo, hi = 0, len(self._keys)
        while lo < hi:
            mid = (lo + hi) // 2
            if self._keys[mid].Time <= time:
                lo = mid + 1
            else:
                hi = mid
        return lo - 1

    def Tensors(self, device="cpu"):
        t = torch.tensor([k.Time for k in self._keys], dtype=torch.float32, device=device)
        v = torch.tensor([k.Value for k in self._keys], dtype=torch.float32, device=device).reshape(len(self._keys), self.Width)
        m = torch.tensor([int(k.Interpolation) for k in self._keys], dtype=torch.int64, device=device)
        return t, v, m


class _Curve:
    WIDTH = 1

    def __init__(self):
        self.Track = OaKeyframeTrack(self.WIDTH)

    def AddKeyframe(self, time: float, value, interpolation: OaKeyInterpolation = OaKeyInterpolation.Linear) -> None:
        self.Track.AddKeyframe(time, value, interpolation)

    def Clear(self) -> None: self.Track.Clear()
    def GetKeyframeCount(self) -> int: return self.Track.GetKeyframeCount()

    def EvaluateBatch(self, times: torch.Tensor) -> torch.Tensor:
        """[N] times -> [N, width] values; clamps outside the key range."""
        n = self.Track.GetKeyframeCount()
        times = times.to(torch.float32)
        if n == 0:
            return torch.zeros(times.numel(), self.WIDTH, device=times.device)
        t, v, mode = self.Track.Tensors(times.device)
        if n == 1:
            return v[0].expand(times.numel(), self.WIDTH).clone()
        i = (torch.searchsorted(t, times.contiguous(), right=True) - 1).clamp(0, n - 2)
        t0, t1 = t[i], t[i + 1]
        u = ((times - t0) / (t1 - t0).clamp_min(1e-12)).clamp(0.0, 1.0)[:, None]
        p0, p1 = v[i], v[i + 1]
        pm, pn = v[(i - 1).clamp_min(0)], v[(i + 2).clamp_max(n - 1)]
        linear = self._mix(p0, p1, u)
        u2, u3 = u * u, u * u * u
        cubic = 0.5 * ((2 * p0) + (-pm + p1) * u + (2 * pm - 5 * p0 + 4 * p1 - pn) * u2 + (-pm + 3 * p0 - 3 * p1 + pn) * u3)
        m = mode[i][:, None]
        out = torch.where(m == int(OaKeyInterpolation.Stepped), torch.where(u >= 1.0, p1, p0),
                          torch.where(m == int(OaKeyInterpolation.Cubic), cubic, linear))
        return self._finish(out)

    @staticmethod
    def _mix(p0, p1, u):
        return p0 + (p1 - p0) * u

    @staticmethod
    def _finish(out):
        return out

    def _eval(self, time: float) -> Tuple[float, ...]:
        return tuple(self.EvaluateBatch(torch.tensor([time]))[0].tolist())

    def _deriv(self, time: float, h: float = 1e-3) -> Tuple[float, ...]:
        a, b = self.EvaluateBatch(torch.tensor([time - h, time + h]))
        return tuple(((b - a) / (2 * h)).tolist())


class OaCurveFloat(_Curve):
    WIDTH = 1
    def Evaluate(self, time: float) -> float: return self._eval(time)[0]
    def Derivative(self, time: float) -> float: return self._deriv(time)[0]


class OaCurveVec3(_Curve):
    WIDTH = 3
    def Evaluate(self, time: float): return self._eval(time)
    def Derivative(self, time: float): return self._deriv(time)


class OaCurveColor(_Curve):
    WIDTH = 4
    def Evaluate(self, time: float): return tuple(min(1.0, max(0.0, c)) for c in self._eval(time))


class OaCurveQuat(_Curve):
    """Unit quaternions (x, y, z, w): spherical interpolation along the shorter arc."""
    WIDTH = 4

    @staticmethod
    def _mix(p0, p1, u):
        d = (p0 * p1).sum(1, keepdim=True)
        p1 = torch.where(d < 0, -p1, p1)
        d = d.abs().clamp(max=1.0)
        theta = torch.acos(d)
        s = torch.sin(theta)
        near = s < 1e-5
        s = torch.where(near, torch.ones_like(s), s)
        w0, w1 = torch.sin((1 - u) * theta) / s, torch.sin(u * theta) / s
        return torch.where(near, p0 + (p1 - p0) * u, p0 * w0 + p1 * w1)

    @staticmethod
    def _finish(out):
        return out / out.norm(dim=1, keepdim=True).clamp_min(1e-12)

    def Evaluate(self, time: float): return self._eval(time)


class OaEasing:
    Linear = staticmethod(lambda t: t)
    EaseInQuad = staticmethod(lambda t: t * t)
    EaseOutQuad = staticmethod(lambda t: t * (2 - t))
    EaseInOutQuad = staticmethod(lambda t: 2 * t * t if t < 0.5 else -1 + (4 - 2 * t) * t)
    EaseInCubic = staticmethod(lambda t: t ** 3)
    EaseOutCubic = staticmethod(lambda t: (t - 1) ** 3 + 1)
    EaseInOutCubic = staticmethod(lambda t: 4 * t ** 3 if t < 0.5 else (t - 1) * (2 * t - 2) ** 2 + 1)
    EaseInQuart = staticmethod(lambda t: t ** 4)
    EaseOutQuart = staticmethod(lambda t: 1 - (t - 1) ** 4)
    EaseInOutQuart = staticmethod(lambda t: 8 * t ** 4 if t < 0.5 else 1 - 8 * (t - 1) ** 4)
    EaseInExpo = staticmethod(lambda t: 0.0 if t <= 0 else 2 ** (10 * (t - 1)))
    EaseOutExpo = staticmethod(lambda t: 1.0 if t >= 1 else 1 - 2 ** (-10 * t))
    EaseInOutExpo = staticmethod(lambda t: 0.0 if t <= 0 else 1.0 if t >= 1 else (2 ** (20 * t - 10) / 2 if t < 0.5 else (2 - 2 ** (-20 * t + 10)) / 2))
    EaseOutElastic = staticmethod(lambda t: 0.0 if t <= 0 else 1.0 if t >= 1 else 2 ** (-10 * t) * math.sin((t * 10 - 0.75) * (2 * math.pi / 3)) + 1)

    @staticmethod
    def EaseOutBounce(t: float) -> float:
        n, d = 7.5625, 2.75
        if t < 1 / d:
            return n * t * t
        if t < 2 / d:
            t -= 1.5 / d
            return n * t * t + 0.75
        if t < 2.5 / d:
            t -= 2.25 / d
            return n * t * t + 0.9375
        t -= 2.625 / d
        return n * t * t + 0.984375


@dataclass(frozen=True)
class OaFrameRate:
    Numerator: int = 30
    Denominator: int = 1

    def Fps(self) -> float: return self.Numerator / self.Denominator
    def FrameDuration(self) -> float: return self.Denominator / self.Numerator


@dataclass(frozen=True, order=True)
class OaTimeCode:
    """Time in seconds with frame conversion at a given rate."""
    Seconds: float = 0.0

    @staticmethod
    def FromFrames(frame: int, rate: OaFrameRate) -> "OaTimeCode": return OaTimeCode(frame * rate.Denominator / rate.Numerator)
    def ToFrames(self, rate: OaFrameRate) -> int: return int(math.floor(self.Seconds * rate.Numerator / rate.Denominator + 1e-9))
    def IsZero(self) -> bool: return self.Seconds == 0.0
    def __add__(self, o: "OaTimeCode") -> "OaTimeCode": return OaTimeCode(self.Seconds + o.Seconds)
    def __sub__(self, o: "OaTimeCode") -> "OaTimeCode": return OaTimeCode(self.Seconds - o.Seconds)
    def __mul__(self, s: float) -> "OaTimeCode": return OaTimeCode(self.Seconds * s)

    def ToSmpte(self, rate: OaFrameRate) -> str:
        f = self.ToFrames(rate)
        fps = int(round(rate.Fps()))
        return f"{f // (fps * 3600):02d}:{(f // (fps * 60)) % 60:02d}:{(f // fps) % 60:02d}:{f % fps:02d}"


@dataclass
class OaTimeTransform:
    Offset: OaTimeCode = OaTimeCode()
    Scale: float = 1.0
    TrimStart: OaTimeCode = OaTimeCode()
    TrimEnd: OaTimeCode = OaTimeCode()

    @staticmethod
    def Identity() -> "OaTimeTransform": return OaTimeTransform()
    @staticmethod
    def WithOffset(offset: OaTimeCode) -> "OaTimeTransform": return OaTimeTransform(Offset=offset)
    @staticmethod
    def WithScale(scale: float) -> "OaTimeTransform": return OaTimeTransform(Scale=scale)

    def ToLocal(self, parent: OaTimeCode) -> OaTimeCode: return (parent - self.Offset) * self.Scale
    def ToParent(self, local: OaTimeCode) -> OaTimeCode: return self.Offset if self.Scale == 0 else local * (1.0 / self.Scale) + self.Offset

    def ApplyTrim(self, local: OaTimeCode) -> OaTimeCode:
        if local < self.TrimStart:
            return self.TrimStart
        if not self.TrimEnd.IsZero() and local > self.TrimEnd:
            return self.TrimEnd
        return local

    def IsInTrim(self, local: OaTimeCode) -> bool:
        return not (local < self.TrimStart or (not self.TrimEnd.IsZero() and local > self.TrimEnd))


class OaTimeDirection(enum.IntEnum):
    Forward = 0
    Reverse = 1
    PingPong = 2


class OaTimelineState(enum.IntEnum):
    Stopped = 0
    Playing = 1
    Paused = 2


class OaTimeline:
    def __init__(self, duration: float = 0.0, rate: Optional[OaFrameRate] = None):
        self.FrameRate_ = rate or OaFrameRate()
        self.Duration_ = float(duration)
        self.Time_ = 0.0
        self.State_ = OaTimelineState.Stopped
        self.Direction_ = OaTimeDirection.Forward
        self.Loop_ = False
        self.Speed_ = 1.0
        self._sign = 1.0

    def SetFrameRate(self, rate: OaFrameRate) -> None: self.FrameRate_ = rate
    def GetFrameRate(self) -> OaFrameRate: return self.FrameRate_
    def SetDuration(self, seconds: float) -> None: self.Duration_ = float(seconds)
    def GetDuration(self) -> float: return self.Duration_
    def SetLooping(self, on: bool) -> None: self.Loop_ = on
    def SetSpeed(self, speed: float) -> None: self.Speed_ = float(speed)
    def SetDirection(self, d: OaTimeDirection) -> None:
        self.Direction_ = d
        self._sign = -1.0 if d == OaTimeDirection.Reverse else 1.0
    def GetState(self) -> OaTimelineState: return self.State_
    def GetTime(self) -> OaTimeCode: return OaTimeCode(self.Time_)
    def GetFrame(self) -> int: return OaTimeCode(self.Time_).ToFrames(self.FrameRate_)
    def Play(self) -> None: self.State_ = OaTimelineState.Playing
    def Pause(self) -> None:
        if self.State_ == OaTimelineState.Playing:
            self.State_ = OaTimelineState.Paused
    def Stop(self) -> None:
        self.State_, self.Time_ = OaTimelineState.Stopped, (self.Duration_ if self.Direction_ == OaTimeDirection.Reverse else 0.0)
    def Seek(self, time: OaTimeCode) -> None: self.Time_ = min(max(time.Seconds, 0.0), self.Duration_)
    def SeekFrame(self, frame: int) -> None: self.Seek(OaTimeCode.FromFrames(frame, self.FrameRate_))

    def Update(self, dt: float) -> None:
        """Advance a playing timeline by `dt` seconds of wall time."""
        if self.State_ != OaTimelineState.Playing or self.Duration_ <= 0:
            return
        t = self.Time_ + dt * self.Speed_ * self._sign
        if self.Direction_ == OaTimeDirection.PingPong:
            while t > self.Duration_ or t < 0:
                if t > self.Duration_:
                    t, self._sign = 2 * self.Duration_ - t, -1.0
                if t < 0:
                    if not self.Loop_:
                        t, self.State_ = 0.0, OaTimelineState.Stopped
                        break
                    t, self._sign = -t, 1.0
        elif self.Loop_:
            t = t % self.Duration_
        elif t >= self.Duration_ or t <= 0:
            t = min(max(t, 0.0), self.Duration_)
            self.State_ = OaTimelineState.Stopped
        self.Time_ = t
