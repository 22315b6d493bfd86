"""Environment schema, the stateful vector-environment session and the native CartPole environment.

Reference: Source/Public/Oa/Ml/Rl/Environment.h:18-167 (specs, transition, session life cycle) and the CartPole
environment of Tutorial/Ml/Rl/CartPole.{h,cpp} with its kernels Rl/Shader/Compute/Environment/RlCartPole{Reset,Step}.slang.

The session is a transaction on the engine's stream: Begin opens a recording, Reset / Step / ResetCompleted launch their
kernels, Submit closes the recording and returns a completion event; Cancel throws away host-side metadata authored since
Begin (device work is already ordered on the stream and is simply superseded by the next reset).
"""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass, field
from typing import Callable, Optional, Sequence

import torch

from ...core import fn_matrix as F
from ...core.matrix import OaMatrix
from ...core.types import OaScalarType, OaStatus, OaStatusCode, to_torch_dtype
from ...ops import rl as R
from ...runtime import engine as RT


class OaRlSpaceKind(enum.IntEnum):
    Box = 0
    Discrete = 1
    Binary = 2


def _invalid(msg: str) -> OaStatus:
    return OaStatus.Error(OaStatusCode.InvalidArgument, msg)


@dataclass
class OaRlFieldSpec:
    """One field of the schema; Shape excludes the leading environment axis (rank 0 = one scalar per environment)."""
    Name: str = ""
    Kind: OaRlSpaceKind = OaRlSpaceKind.Box
    Shape: tuple = ()
    Dtype: OaScalarType = OaScalarType.Float32
    Minimum: float = -math.inf
    Maximum: float = math.inf
    Cardinality: int = 0

    @staticmethod
    def Box(name: str, shape: Sequence[int], dtype=OaScalarType.Float32, minimum: float = -math.inf, maximum: float = math.inf):
        return OaRlFieldSpec(name, OaRlSpaceKind.Box, tuple(shape), dtype, minimum, maximum, 0)

    @staticmethod
    def Discrete(name: str, cardinality: int, dtype=OaScalarType.Int32):
        return OaRlFieldSpec(name, OaRlSpaceKind.Discrete, (), dtype, 0.0, float(cardinality - 1), int(cardinality))

    @staticmethod
    def Binary(name: str, shape: Sequence[int] = (), dtype=OaScalarType.UInt8):
        return OaRlFieldSpec(name, OaRlSpaceKind.Binary, tuple(shape), dtype, 0.0, 1.0, 2)

    def ValidateDefinition(self) -> OaStatus:
        if not self.Name:
            return _invalid("field has no name")
        if any(int(s) <= 0 for s in self.Shape):
            return _invalid(f"field {self.Name}: non-positive extent")
        if self.Kind == OaRlSpaceKind.Box:
            if math.isnan(self.Minimum) or math.isnan(self.Maximum) or self.Minimum > self.Maximum:
                return _invalid(f"field {self.Name}: invalid bounds")
            if self.Dtype not in (OaScalarType.Float32, OaScalarType.BFloat16, OaScalarType.Float16):
                return _invalid(f"field {self.Name}: box fields are floating point")
        elif self.Kind == OaRlSpaceKind.Discrete:
            if self.Cardinality < 2 or self.Dtype != OaScalarType.Int32 or self.Shape:
                return _invalid(f"field {self.Name}: discrete fields are Int32 scalars with cardinality >= 2")
        elif self.Dtype != OaScalarType.UInt8:
            return _invalid(f"field {self.Name}: binary fields are UInt8")
        return OaStatus.Ok()

    def ElementsPerEnvironment(self) -> int:
        n = 1
        for s in self.Shape:
            n *= int(s)
        return n

    def BatchedShape(self, environments: int) -> tuple:
        return (int(environments),) + tuple(int(s) for s in self.Shape)

    def ValidateMatrix(self, m: OaMatrix, environments: int) -> OaStatus:
        if m is None or m.IsEmpty():
            return _invalid(f"field {self.Name}: empty matrix")
        if tuple(m.Tensor().shape) != self.BatchedShape(environments):
            return OaStatus.Error(OaStatusCode.InvalidArgument, f"field {self.Name}: shape {tuple(m.Tensor().shape)} != {self.BatchedShape(environments)}")
        if m.Tensor().dtype != to_torch_dtype(self.Dtype):
            return _invalid(f"field {self.Name}: dtype mismatch")
        return OaStatus.Ok()


@dataclass
class OaRlEnvironmentSpec:
    Observation: OaRlFieldSpec = field(default_factory=OaRlFieldSpec)
    Action: OaRlFieldSpec = field(default_factory=OaRlFieldSpec)
    Reward: OaRlFieldSpec = field(default_factory=OaRlFieldSpec)
    Terminated: OaRlFieldSpec = field(default_factory=OaRlFieldSpec)
    Truncated: OaRlFieldSpec = field(default_factory=OaRlFieldSpec)

    def ValidateDefinition(self) -> OaStatus:
        for f in (self.Observation, self.Action, self.Reward, self.Terminated, self.Truncated):
            st = f.ValidateDefinition()
            if not st:
                return st
        if self.Reward.Kind != OaRlSpaceKind.Box or self.Reward.Shape:
            return _invalid("reward is one floating-point scalar per environment")
        if self.Terminated.Kind != OaRlSpaceKind.Binary or self.Truncated.Kind != OaRlSpaceKind.Binary:
            return _invalid("terminated / truncated are binary fields")
        return OaStatus.Ok()

    def ValidateReset(self, observation: OaMatrix, environments: int) -> OaStatus:
        return self.Observation.ValidateMatrix(observation, environments)

    def ValidateAction(self, action: OaMatrix, environments: int) -> OaStatus:
        return self.Action.ValidateMatrix(action, environments)

    def ValidateTransition(self, observation, action, next_observation, reward, terminated, truncated, environments: int) -> OaStatus:
        for f, m in ((self.Observation, observation), (self.Action, action), (self.Observation, next_observation),
                     (self.Reward, reward), (self.Terminated, terminated), (self.Truncated, truncated)):
            st = f.ValidateMatrix(m, environments)
            if not st:
                return st
        return OaStatus.Ok()


@dataclass
class OaRlEnvironmentTransition:
    Observation: Optional[OaMatrix] = None
    NextObservation: Optional[OaMatrix] = None
    Reward: Optional[OaMatrix] = None
    Terminated: Optional[OaMatrix] = None
    Truncated: Optional[OaMatrix] = None

    def IsValid(self) -> bool:
        return all(m is not None and not m.IsEmpty() for m in (self.Observation, self.NextObservation, self.Reward, self.Terminated, self.Truncated))


class OaRlEnvironment:
    """Stateful native environment session (Environment.h:96-167).  Subclasses implement the three Record* hooks."""

    def __init__(self, engine: Optional[RT.OaEngine] = None):
        self._engine = engine or RT.get_engine()
        self._open = True
        self._recording = False
        self._pending: Optional[RT.OaEvent] = None
        self._submissions = 0

    # ---- schema (subclass)
    def Spec(self) -> OaRlEnvironmentSpec: raise NotImplementedError
    def Environments(self) -> int: raise NotImplementedError
    def Observation(self) -> OaMatrix: raise NotImplementedError
    def RecordResetEnvironment_(self, seed: int) -> OaStatus: raise NotImplementedError
    def RecordStepEnvironment_(self, action: OaMatrix): raise NotImplementedError
    def RecordResetCompleted_(self) -> OaStatus: raise NotImplementedError
    def CommitRecordedState_(self) -> None: pass
    def RollbackRecordedState_(self) -> None: pass

    # ---- transaction
    def Begin(self) -> OaStatus:
        if not self._open:
            return OaStatus.Error(OaStatusCode.FailedPrecondition, "environment is closed")
        self._recording = True
        return OaStatus.Ok()

    def RecordCommands(self, commands: Callable[[], OaStatus]) -> OaStatus:
        st = self.Begin()
        if not st:
            return st
        try:
            st = commands()
        except Exception as e:  # a failing callback cancels the whole unsubmitted transaction
            self.Cancel()
            return OaStatus.Error(OaStatusCode.Aborted, str(e))
        if isinstance(st, OaStatus) and not st:
            self.Cancel()
            return st
        return OaStatus.Ok()

    def ResetEnvironment(self, seed: int) -> OaStatus:
        st = self.Begin()
        return self.RecordResetEnvironment_(int(seed)) if st else st

    def StepEnvironment(self, action: OaMatrix):
        """Returns (transition, status)."""
        st = self.Begin()
        if not st:
            return None, st
        st = self.Spec().ValidateAction(action, self.Environments())
        if not st:
            return None, st
        return self.RecordStepEnvironment_(action)

    def ResetCompleted(self) -> OaStatus:
        st = self.Begin()
        return self.RecordResetCompleted_() if st else st

    def Submit(self):
        """Returns (event, status): the completion of everything recorded since the previous Submit."""
        if not self._open:
            return None, OaStatus.Error(OaStatusCode.FailedPrecondition, "environment is closed")
        if not self._recording:
            return None, OaStatus.Error(OaStatusCode.FailedPrecondition, "nothing recorded")
        ev = RT.OaContext.GetDefault().Submit()
        self._recording = False
        self._pending = ev
        self._submissions += 1
        self.CommitRecordedState_()
        return ev, OaStatus.Ok()

    def Wait(self, event: RT.OaEvent) -> OaStatus:
        st = RT.OaContext.GetDefault().Wait(event)
        if event is self._pending:
            self._pending = None
        return st

    def Cancel(self) -> OaStatus:
        if self._recording:
            self._recording = False
            self.RollbackRecordedState_()
        return OaStatus.Ok()

    def Close(self) -> OaStatus:
        if not self._open:
            return OaStatus.Ok()
        st = OaStatus.Ok()
        if self._pending is not None:
            st = self.Wait(self._pending)
        self.Cancel()
        self._open = False
        return st

    def IsOpen(self) -> bool: return self._open
    def HasActiveRecording(self) -> bool: return self._recording
    def HasPendingEvent(self) -> bool: return self._pending is not None
    def SubmissionCount(self) -> int: return self._submissions


@dataclass
class OaCartPoleConfig:
    """Gymnasium CartPole-v1 constants (Tutorial/Ml/Rl/CartPole.h:7-24)."""
    DynamicsVersion = 1
    Environments: int = 1
    MaxEpisodeSteps: int = 500
    Seed: int = 1
    Gravity: float = 9.8
    CartMass: float = 1.0
    PoleMass: float = 0.1
    HalfPoleLength: float = 0.5
    ForceMagnitude: float = 10.0
    TimeStep: float = 0.02
    PositionThreshold: float = 2.4
    AngleThresholdRadians: float = 0.2094395102

    def Validate(self) -> OaStatus:
        vals = (self.Gravity, self.CartMass, self.PoleMass, self.HalfPoleLength, self.ForceMagnitude, self.TimeStep,
                self.PositionThreshold, self.AngleThresholdRadians)
        if not all(math.isfinite(v) for v in vals) or self.Environments <= 0 or self.MaxEpisodeSteps <= 0 or any(v <= 0 for v in vals[1:]):
            return _invalid("CartPole configuration must be finite and positive")
        return OaStatus.Ok()


class OaCartPoleEnvironment(OaRlEnvironment):
    """Vector CartPole-v1: observation [E, 4] fp32, action Int32 {0, 1}, reward 1 per live step, termination on
    |x| > 2.4 or |angle| > 12 degrees, truncation at MaxEpisodeSteps.  Done lanes idle (zero reward) until
    ResetCompleted re-seeds them with their next episode index."""

    def __init__(self, config: Optional[OaCartPoleConfig] = None, engine: Optional[RT.OaEngine] = None):
        super().__init__(engine)
        self.Config = config or OaCartPoleConfig()
        st = self.Config.Validate()
        if not st:
            raise ValueError(st.message)
        E = self.Config.Environments
        dev = self._engine.Device()
        self._state = torch.zeros(E, 4, dtype=torch.float32, device=dev)
        self._done = torch.zeros(E, dtype=torch.uint8, device=dev)
        self._steps = torch.zeros(E, dtype=torch.int32, device=dev)
        self._episode = torch.zeros(E, dtype=torch.int32, device=dev)
        self._obs = OaMatrix(self._state)
        self._seed = self.Config.Seed
        self._pending_seed = self._seed
        self._params = R.CartPoleParams(self.Config.Gravity, self.Config.CartMass, self.Config.PoleMass, self.Config.HalfPoleLength,
                                        self.Config.ForceMagnitude, self.Config.TimeStep, self.Config.PositionThreshold,
                                        self.Config.AngleThresholdRadians, self.Config.MaxEpisodeSteps)
        self._spec = OaRlEnvironmentSpec(
            Observation=OaRlFieldSpec.Box("observation", (4,)),
            Action=OaRlFieldSpec.Discrete("action", 2),
            Reward=OaRlFieldSpec.Box("reward", (), OaScalarType.Float32, 0.0, 1.0),
            Terminated=OaRlFieldSpec.Binary("terminated"),
            Truncated=OaRlFieldSpec.Binary("truncated"))

    @staticmethod
    def Create(config: Optional[OaCartPoleConfig] = None):
        cfg = config or OaCartPoleConfig()
        st = cfg.Validate()
        return (OaCartPoleEnvironment(cfg), st) if st else (None, st)

    def Spec(self) -> OaRlEnvironmentSpec: return self._spec
    def Environments(self) -> int: return self.Config.Environments
    def Observation(self) -> OaMatrix: return self._obs
    def Done(self) -> OaMatrix: return OaMatrix(self._done)
    def EpisodeSteps(self) -> OaMatrix: return OaMatrix(self._steps)

    def RecordResetEnvironment_(self, seed: int) -> OaStatus:
        self._pending_seed = seed if seed else self.Config.Seed
        F._ctx_add("RlCartPoleReset")
        R.cartpole_reset(self._state, self._done, self._steps, self._episode, self._pending_seed, False)
        return OaStatus.Ok()

    def RecordStepEnvironment_(self, action: OaMatrix):
        E, dev = self.Config.Environments, self._state.device
        F._ctx_add("RlCartPoleStep")
        t_obs = self._state.clone()                    # done lanes keep their last state as the transition observation
        reward = torch.empty(E, dtype=torch.float32, device=dev)
        term = torch.empty(E, dtype=torch.uint8, device=dev)
        trunc = torch.empty(E, dtype=torch.uint8, device=dev)
        R.cartpole_step(action.Tensor(), self._state, t_obs, reward, term, trunc, self._done, self._steps, self._params)
        tr = OaRlEnvironmentTransition(OaMatrix(t_obs), OaMatrix(self._state.clone()), OaMatrix(reward), OaMatrix(term), OaMatrix(trunc))
        return tr, OaStatus.Ok()

    def RecordResetCompleted_(self) -> OaStatus:
        F._ctx_add("RlCartPoleReset")
        R.cartpole_reset(self._state, self._done, self._steps, self._episode, self._pending_seed, True)
        return OaStatus.Ok()

    def CommitRecordedState_(self) -> None:
        self._seed = self._pending_seed

    def RollbackRecordedState_(self) -> None:
        self._pending_seed = self._seed


# ------------------------------------------------------------------------------------------ LunarLander3d
from ...ops import lunar as LL


@dataclass
class OaLunarLander3dConfig:
    """Vector LunarLander3d: lanes, seeds and the physics / reward / terrain constants (`ops.lunar.LunarParams`)."""
    Environments: int = 1
    Seed: int = 1
    TerrainSeed: int = 1
    Params: LL.LunarParams = field(default_factory=LL.LunarParams)
    Spawn: tuple = LL.SPAWN_DEFAULT

    def Validate(self) -> OaStatus:
        p = self.Params
        positive = (p.PolicyDt, p.Mass, *p.Inertia, p.MainThrust, p.AttitudeTorque, p.FuelCapacity, p.CellSize, p.PositionScale, p.VelocityScale,
                    p.AngularScale, p.TerrainClearanceScale, p.FootClearanceScale, p.MaxContactImpulse)
        if self.Environments <= 0 or p.Substeps <= 0 or p.ContactIterations <= 0 or p.CellsX <= 0 or p.CellsZ <= 0 or p.MaxEpisodeSteps <= 0 \
                or len(p.Supports) != 7 or len(self.Spawn) != 8 or not all(math.isfinite(v) and v > 0 for v in positive):
            return _invalid("LunarLander3d configuration must be finite and positive, with seven supports")
        if not 0 <= p.Restitution <= 1 or p.Friction < 0 or not 0 < p.RewardGamma <= 1 or p.TaskMaximumY <= p.TaskMinimumY:
            return _invalid("LunarLander3d restitution, friction, discount or altitude band out of range")
        return OaStatus.Ok()


class OaLunarLander3dEnvironment(OaRlEnvironment):
    """Observation [E, 33] fp32, action Int32 in {0 coast, 1 main engine, 2/3 pitch, 4/5 roll, 6/7 yaw}.  An episode ends
    (terminated) on a safe landing held for SafeDwellSteps, a hull impact, a hard foot impact, leaving the task volume, a
    numerical failure or an invalid action, and is truncated at MaxEpisodeSteps or by an external stop flag.  Finished
    lanes idle with zero reward until ResetCompleted re-spawns them."""

    def __init__(self, config: Optional[OaLunarLander3dConfig] = None, engine: Optional[RT.OaEngine] = None):
        super().__init__(engine)
        self.Config = config or OaLunarLander3dConfig()
        st = self.Config.Validate()
        if not st:
            raise ValueError(st.message)
        E, dev, p = self.Config.Environments, self._engine.Device(), self.Config.Params
        self._terrain = LL.make_terrain(p, self.Config.TerrainSeed).to(dev)
        self._sf = torch.zeros(E, LL.STATE_F32, dtype=torch.float32, device=dev)
        self._su = torch.zeros(E, LL.STATE_U32, dtype=torch.int32, device=dev)
        self._obs_t = torch.zeros(E, LL.OBS_WIDTH, dtype=torch.float32, device=dev)
        self._stop = torch.zeros(E, dtype=torch.uint8, device=dev)
        self._obs = OaMatrix(self._obs_t)
        self._seed = self._pending_seed = self.Config.Seed
        self._spec = OaRlEnvironmentSpec(
            Observation=OaRlFieldSpec.Box("observation", (LL.OBS_WIDTH,), OaScalarType.Float32, -1.0, 1.0),
            Action=OaRlFieldSpec.Discrete("action", 8),
            Reward=OaRlFieldSpec.Box("reward", ()),
            Terminated=OaRlFieldSpec.Binary("terminated"),
            Truncated=OaRlFieldSpec.Binary("truncated"))

    @staticmethod
    def Create(config: Optional[OaLunarLander3dConfig] = None):
        cfg = config or OaLunarLander3dConfig()
        st = cfg.Validate()
        return (OaLunarLander3dEnvironment(cfg), st) if st else (None, st)

    def Spec(self) -> OaRlEnvironmentSpec: return self._spec
    def Environments(self) -> int: return self.Config.Environments
    def Observation(self) -> OaMatrix: return self._obs
    def Terrain(self) -> OaMatrix: return OaMatrix(self._terrain)
    def StateF32(self) -> OaMatrix: return OaMatrix(self._sf)
    def StateU32(self) -> OaMatrix: return OaMatrix(self._su)
    def EndReason(self) -> OaMatrix: return OaMatrix(self._su[:, LL.U_REASON])
    def EpisodeReturn(self) -> OaMatrix: return OaMatrix(self._sf[:, LL.S_RETURN])
    def Done(self) -> OaMatrix: return OaMatrix(((self._su[:, LL.U_TERM] != 0) | (self._su[:, LL.U_TRUNC] != 0)).to(torch.uint8))

    def RequestStop(self, lanes: Optional[Sequence[int]] = None) -> None:
        """Truncate the given lanes (all by default) at their next step."""
        if lanes is None:
            self._stop.fill_(1)
        else:
            self._stop[torch.as_tensor(list(lanes), dtype=torch.long, device=self._stop.device)] = 1

    def RecordResetEnvironment_(self, seed: int) -> OaStatus:
        self._pending_seed = seed if seed else self.Config.Seed
        F._ctx_add("RlLunarLander3dReset")
        LL.reset(self.Config.Params, self._terrain, self._sf, self._su, self._obs_t, self._pending_seed, False, self.Config.Spawn)
        self._stop.zero_()
        return OaStatus.Ok()

    def RecordStepEnvironment_(self, action: OaMatrix):
        E, dev = self.Config.Environments, self._sf.device
        F._ctx_add("RlLunarLander3dStep")
        t_obs = torch.empty(E, LL.OBS_WIDTH, dtype=torch.float32, device=dev)
        reward = torch.empty(E, dtype=torch.float32, device=dev)
        term = torch.empty(E, dtype=torch.uint8, device=dev)
        trunc = torch.empty(E, dtype=torch.uint8, device=dev)
        reason = torch.empty(E, dtype=torch.int32, device=dev)
        LL.step(self.Config.Params, self._terrain, action.Tensor().to(torch.int32), self._stop, self._sf, self._su, t_obs, self._obs_t, reward,
                term, trunc, reason)
        tr = OaRlEnvironmentTransition(OaMatrix(t_obs), OaMatrix(self._obs_t.clone()), OaMatrix(reward), OaMatrix(term), OaMatrix(trunc))
        return tr, OaStatus.Ok()

    def RecordResetCompleted_(self) -> OaStatus:
        F._ctx_add("RlLunarLander3dReset")
        done = (self._su[:, LL.U_TERM] != 0) | (self._su[:, LL.U_TRUNC] != 0)
        LL.reset(self.Config.Params, self._terrain, self._sf, self._su, self._obs_t, self._pending_seed, True, self.Config.Spawn)
        self._stop[done] = 0
        return OaStatus.Ok()

    def CommitRecordedState_(self) -> None:
        self._seed = self._pending_seed

    def RollbackRecordedState_(self) -> None:
        self._pending_seed = self._seed
