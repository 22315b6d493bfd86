"""LunarLander3d dynamics: a batched rigid-body lander over a height-field terrain.

One lane = one lander: a rigid body (mass, diagonal inertia, unit quaternion stored scalar-first) with a main engine
along its up axis and three pairs of attitude thrusters (8 discrete actions), three body spheres and four foot spheres
that collide with a triangulated height field through sequential impulses (restitution, Coulomb friction, bounded
positional correction), potential-based reward shaping, and typed episode ends.  Layouts and semantics follow the
reference's kernels (Source/Private/Oa/Ml/Rl/Shader/Compute/Environment/RlLunarLander3dStep.slang: config indices
:3-58, state layout :60-82, end reasons :84-92, 33-wide observation :563-632, step :658-867) and the tutorial
constants (Tutorial/Ml/Rl/LunarLander3d/LunarLander3dPhysics.h:30-76, LunarTerrain.h:12-18).

On a CUDA engine `step` / `reset` launch `oa_rl_lunar_step` / `oa_rl_lunar_reset` (one thread per lane); the tensor
code below is the same arithmetic over all lanes at once and is both the CPU execution path and the oracle.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass, field
from typing import List, Tuple

import torch

from .. import _native as N
from . import kernels as K

OBS_WIDTH, STATE_F32, STATE_U32 = 33, 32, 16
END_NONE, END_SAFE_LANDING, END_BODY_IMPACT, END_HARD_FOOT_IMPACT, END_OUT_OF_BOUNDS, END_NUMERICAL_FAILURE, END_TIME_LIMIT, \
    END_EXTERNAL_STOP, END_INVALID_ACTION = range(9)
# float state columns
S_POS, S_VEL, S_QUAT, S_ANG, S_FUEL, S_THROTTLE, S_ATT, S_BODY_IMP, S_FOOT_IMP, S_RETURN = 0, 3, 6, 10, 13, 14, 15, 18, 21, 25
# integer state columns
U_ACTION, U_BODY, U_FOOT, U_PAD, U_REWARDED, U_STEP, U_DWELL, U_TERM, U_TRUNC, U_REASON = range(10)


@dataclass
class LunarParams:
    PolicyDt: float = 1.0 / 60.0
    Gravity: float = 1.62
    Mass: float = 1200.0
    Inertia: Tuple[float, float, float] = (900.0, 1100.0, 900.0)
    MainThrust: float = 4200.0
    AttitudeTorque: float = 900.0
    FuelCapacity: float = 100.0
    MainFuelRate: float = 2.0
    AttitudeFuelRate: float = 0.35
    Restitution: float = 0.05
    Friction: float = 0.65
    ContactSlop: float = 0.01
    CorrectionFraction: float = 0.6
    MaxPositionCorrection: float = 0.03
    MaxContactImpulse: float = 6000.0
    MaxBiasSpeed: float = 1.0
    TaskMinimumY: float = -2.0
    TaskMaximumY: float = 40.0
    SafeLinearSpeed: float = 0.55
    SafeAngularSpeed: float = 0.25
    SafeTilt: float = 0.18
    HardFootSpeed: float = 1.2
    PositionScale: float = 16.0
    VelocityScale: float = 4.0
    AngularScale: float = 2.0
    TerrainClearanceScale: float = 8.0
    FootClearanceScale: float = 2.0
    ProbeSpacing: float = 1.5
    RewardGamma: float = 0.99
    PositionPotentialWeight: float = 1.0
    VelocityPotentialWeight: float = 0.6
    TiltPotentialWeight: float = 0.5
    AngularPotentialWeight: float = 0.25
    MainFuelCostWeight: float = 0.04
    AttitudeFuelCostWeight: float = 0.02
    SoftFootReward: float = 0.02
    StableDwellReward: float = 0.05
    SuccessReward: float = 100.0
    FailurePenalty: float = -100.0
    CellSize: float = 1.0
    CellsX: int = 32
    CellsZ: int = 32
    PadHalfExtent: float = 3.0
    PadTransitionWidth: float = 3.0
    MaxAbsHeight: float = 1.5
    MaxSlope: float = 0.35
    Substeps: int = 4
    ContactIterations: int = 4
    SafeDwellSteps: int = 20
    MaxEpisodeSteps: int = 1200
    # (offset x, y, z, radius) in the body frame: three hull spheres, then the four feet
    Supports: Tuple[Tuple[float, float, float, float], ...] = (
        (0.0, 0.5, 0.0, 0.8), (0.0, 1.4, 0.0, 0.55), (0.0, -0.15, 0.0, 0.45),
        (1.4, -1.0, 1.4, 0.1), (-1.4, -1.0, 1.4, 0.1), (-1.4, -1.0, -1.4, 0.1), (1.4, -1.0, -1.4, 0.1))

    def TerrainMin(self) -> Tuple[float, float]:
        return -0.5 * self.CellsX * self.CellSize, -0.5 * self.CellsZ * self.CellSize

    def Floats(self) -> List[float]:
        """The 77-entry float table in the kernel's index order (47 scalars, 7 x 4 support entries, two bounds)."""
        mnx, mnz = self.TerrainMin()
        f = [self.PolicyDt, self.Gravity, self.Mass, *self.Inertia, self.MainThrust, self.AttitudeTorque, self.FuelCapacity,
             self.MainFuelRate, self.AttitudeFuelRate, self.Restitution, self.Friction, self.ContactSlop, self.CorrectionFraction,
             self.MaxPositionCorrection, self.MaxContactImpulse, self.MaxBiasSpeed, self.TaskMinimumY, self.TaskMaximumY,
             self.SafeLinearSpeed, self.SafeAngularSpeed, self.SafeTilt, self.HardFootSpeed, self.PositionScale, self.VelocityScale,
             self.AngularScale, self.TerrainClearanceScale, self.FootClearanceScale, self.ProbeSpacing, self.RewardGamma,
             self.PositionPotentialWeight, self.VelocityPotentialWeight, self.TiltPotentialWeight, self.AngularPotentialWeight,
             self.MainFuelCostWeight, self.AttitudeFuelCostWeight, self.SoftFootReward, self.StableDwellReward, self.SuccessReward,
             self.FailurePenalty, self.CellSize, mnx, -mnx, mnz, -mnz, self.PadHalfExtent]
        assert len(f) == 47
        for s in self.Supports:
            f.extend(s)
        # bounds that let a lane far above the ground skip its contact pass: the highest terrain vertex (terrain heights
        # must stay within +-MaxAbsHeight) and the largest distance of any support sphere's surface from the centre
        f.append(self.MaxAbsHeight)
        f.append(max(math.sqrt(s[0] ** 2 + s[1] ** 2 + s[2] ** 2) + s[3] for s in self.Supports))
        return [float(v) for v in f]

    def Ints(self) -> List[int]:
        return [self.Substeps, self.ContactIterations, self.SafeDwellSteps, self.MaxEpisodeSteps, self.CellsX, self.CellsZ]


def make_terrain(p: LunarParams, seed: int) -> torch.Tensor:
    """[(CellsZ + 1) * (CellsX + 1)] fp32 vertex heights: smooth value noise bounded by MaxAbsHeight and (per cell edge)
    MaxSlope, flat at height 0 on the landing pad and blended in over PadTransitionWidth."""
    g = torch.Generator().manual_seed(int(seed) & 0x7FFFFFFFFFFFFFFF)
    nx, nz = p.CellsX + 1, p.CellsZ + 1
    coarse = torch.rand(1, 1, nz // 4 + 2, nx // 4 + 2, generator=g) * 2 - 1
    h = torch.nn.functional.interpolate(coarse, size=(nz, nx), mode="bicubic", align_corners=True)[0, 0] * p.MaxAbsHeight
    mnx, mnz = p.TerrainMin()
    xs = mnx + torch.arange(nx, dtype=torch.float32) * p.CellSize
    zs = mnz + torch.arange(nz, dtype=torch.float32) * p.CellSize
    d = torch.maximum(xs.abs()[None, :].expand(nz, nx), zs.abs()[:, None].expand(nz, nx))
    t = ((d - p.PadHalfExtent) / max(p.PadTransitionWidth, 1e-6)).clamp(0, 1)
    h = h * (t * t * (3 - 2 * t))
    for _ in range(64):                                    # relax until every edge respects the slope bound
        lim = p.MaxSlope * p.CellSize
        dx, dz = h[:, 1:] - h[:, :-1], h[1:, :] - h[:-1, :]
        if float(dx.abs().max()) <= lim and float(dz.abs().max()) <= lim:
            break
        h = h * 0.9
    return h.clamp(-p.MaxAbsHeight, p.MaxAbsHeight).reshape(-1).contiguous().float()


# ------------------------------------------------------------------------------------------ tensor arithmetic
def _f(v: float) -> torch.Tensor:
    return torch.tensor(v, dtype=torch.float32)


def _cross(a, b):
    return torch.stack((a[:, 1] * b[:, 2] - a[:, 2] * b[:, 1], a[:, 2] * b[:, 0] - a[:, 0] * b[:, 2], a[:, 0] * b[:, 1] - a[:, 1] * b[:, 0]), 1)


def _dot(a, b):
    return a[:, 0] * b[:, 0] + a[:, 1] * b[:, 1] + a[:, 2] * b[:, 2]


def _len(a):
    return torch.sqrt(_dot(a, a))


def _rotate(q, v, inverse: bool = False):
    """q = (w, x, y, z); v' = v + w t + u x t with t = 2 u x v."""
    u = -q[:, 1:4] if inverse else q[:, 1:4]
    t = _cross(u, v) * 2.0
    return v + q[:, 0:1] * t + _cross(u, t)


def _quat_mul(a, b):
    aw, ax, ay, az = a.unbind(1)
    bw, bx, by, bz = b.unbind(1)
    return torch.stack((aw * bw - ax * bx - ay * by - az * bz, aw * bx + ax * bw + ay * bz - az * by,
                        aw * by - ax * bz + ay * bw + az * bx, aw * bz + ax * by - ay * bx + az * bw), 1)


def _finite_rows(*ts) -> torch.Tensor:
    ok = None
    for t in ts:
        r = torch.isfinite(t) if t.dim() == 1 else torch.isfinite(t).all(1)
        ok = r if ok is None else ok & r
    return ok


def _terrain(p: LunarParams, terrain: torch.Tensor, x: torch.Tensor, z: torch.Tensor):
    """(in bounds, height, normal [E, 3]) of the triangulated height field at (x, z)."""
    mnx, mnz = p.TerrainMin()
    inb = (x >= mnx) & (x <= -mnx) & (z >= mnz) & (z <= -mnz) & torch.isfinite(x) & torch.isfinite(z)
    cs = _f(p.CellSize)
    gx = torch.where(inb, (x - _f(mnx)) / cs, torch.zeros_like(x))
    gz = torch.where(inb, (z - _f(mnz)) / cs, torch.zeros_like(z))
    at_x, at_z = gx >= p.CellsX, gz >= p.CellsZ
    cx = torch.where(at_x, torch.full_like(gx, p.CellsX - 1), torch.floor(gx))
    cz = torch.where(at_z, torch.full_like(gz, p.CellsZ - 1), torch.floor(gz))
    lx = torch.where(at_x, torch.ones_like(gx), gx - cx)
    lz = torch.where(at_z, torch.ones_like(gz), gz - cz)
    row = p.CellsX + 1
    i00 = cz.long() * row + cx.long()
    h00, h10, h01, h11 = terrain[i00], terrain[i00 + 1], terrain[i00 + row], terrain[i00 + row + 1]
    lower = lz <= lx
    height = torch.where(lower, h00 + lx * (h10 - h00) + lz * (h11 - h10), h00 + lx * (h11 - h01) + lz * (h01 - h00))
    ddx = torch.where(lower, h10 - h00, h11 - h01) / cs
    ddz = torch.where(lower, h11 - h10, h01 - h00) / cs
    n = torch.stack((-ddx, torch.ones_like(ddx), -ddz), 1)
    n = n / _len(n)[:, None]
    up = torch.tensor([0.0, 1.0, 0.0]).expand_as(n)
    return inb, torch.where(inb, height, torch.zeros_like(height)), torch.where(inb[:, None], n, up)


class _Body:
    """Views of the float / integer state as named tensors (copies; `store` writes them back under a lane mask)."""

    def __init__(self, sf: torch.Tensor, su: torch.Tensor):
        self.pos, self.vel = sf[:, S_POS:S_POS + 3].clone(), sf[:, S_VEL:S_VEL + 3].clone()
        self.q, self.w = sf[:, S_QUAT:S_QUAT + 4].clone(), sf[:, S_ANG:S_ANG + 3].clone()
        self.fuel, self.throttle = sf[:, S_FUEL].clone(), sf[:, S_THROTTLE].clone()
        self.att = sf[:, S_ATT:S_ATT + 3].clone()
        self.body_imp, self.foot_imp = sf[:, S_BODY_IMP:S_BODY_IMP + 3].clone(), sf[:, S_FOOT_IMP:S_FOOT_IMP + 4].clone()
        self.ret = sf[:, S_RETURN].clone()
        self.u = su.clone()

    def finite(self) -> torch.Tensor:
        return _finite_rows(self.pos, self.vel, self.q, self.w, self.fuel)

    def store(self, sf: torch.Tensor, su: torch.Tensor, lanes: torch.Tensor) -> None:
        new = sf.clone()
        new[:, S_POS:S_POS + 3], new[:, S_VEL:S_VEL + 3], new[:, S_QUAT:S_QUAT + 4], new[:, S_ANG:S_ANG + 3] = self.pos, self.vel, self.q, self.w
        new[:, S_FUEL], new[:, S_THROTTLE], new[:, S_ATT:S_ATT + 3] = self.fuel, self.throttle, self.att
        new[:, S_BODY_IMP:S_BODY_IMP + 3], new[:, S_FOOT_IMP:S_FOOT_IMP + 4], new[:, S_RETURN] = self.body_imp, self.foot_imp, self.ret
        sf[lanes] = new[lanes]
        su[lanes] = self.u[lanes]


def _potential(p: LunarParams, b: _Body) -> torch.Tensor:
    one = torch.ones_like(b.fuel)
    up = _rotate(b.q, torch.tensor([0.0, 1.0, 0.0]).expand_as(b.pos))
    cost = (p.PositionPotentialWeight * torch.minimum(one, _len(b.pos) / p.PositionScale)
            + p.VelocityPotentialWeight * torch.minimum(one, _len(b.vel) / p.VelocityScale)
            + p.TiltPotentialWeight * ((1.0 - up[:, 1]) * 0.5).clamp(0.0, 1.0)
            + p.AngularPotentialWeight * torch.minimum(one, _len(b.w) / p.AngularScale))
    return torch.where(b.finite(), -cost, torch.zeros_like(cost))


def _inv_inertia(p: LunarParams) -> torch.Tensor:
    return torch.tensor([1.0 / p.Inertia[0], 1.0 / p.Inertia[1], 1.0 / p.Inertia[2]], dtype=torch.float32)


def _effective_inverse_mass(p, b, lever, direction):
    rb = _rotate(b.q, _cross(lever, direction), inverse=True)
    return 1.0 / p.Mass + _dot(rb, rb * _inv_inertia(p))


def _apply_impulse(p, b, lever, impulse, lanes):
    vel = b.vel + impulse / p.Mass
    w = b.w + _rotate(b.q, _cross(lever, impulse), inverse=True) * _inv_inertia(p)
    b.vel, b.w = torch.where(lanes[:, None], vel, b.vel), torch.where(lanes[:, None], w, b.w)


def _resolve_support(p, terrain, b: _Body, k: int, h: float, active: torch.Tensor, diag: dict) -> None:
    off = torch.tensor(p.Supports[k][:3], dtype=torch.float32).expand_as(b.pos)
    radius, is_foot = p.Supports[k][3], k >= 3
    center = b.pos + _rotate(b.q, off)
    inb, height, normal = _terrain(p, terrain, center[:, 0], center[:, 2])
    sep = center[:, 1] - radius - height
    m = active & inb & (sep < 0)
    if not bool(m.any()):
        return
    pen = -sep
    lever = center - b.pos
    pv = b.vel + _cross(_rotate(b.q, b.w), lever)
    vn = _dot(pv, normal)
    closing = (-vn).clamp_min(0.0)
    if is_foot:
        diag["foot_hit"] |= m
        diag["foot_speed"] = torch.where(m, torch.maximum(diag["foot_speed"], closing), diag["foot_speed"])
    bias = torch.minimum(torch.full_like(pen, p.MaxBiasSpeed), pen * p.CorrectionFraction / h)
    jn = ((-(1.0 + p.Restitution) * vn + bias).clamp_min(0.0) / _effective_inverse_mass(p, b, lever, normal)).clamp(0.0, p.MaxContactImpulse)
    _apply_impulse(p, b, lever, normal * jn[:, None], m)
    pv = b.vel + _cross(_rotate(b.q, b.w), lever)
    tv = pv - normal * _dot(pv, normal)[:, None]
    ts = _len(tv)
    slide = m & (ts > 1.0e-12)
    tdir = -tv / torch.where(ts > 1.0e-12, ts, torch.ones_like(ts))[:, None]
    jt = torch.minimum(ts / _effective_inverse_mass(p, b, lever, tdir), p.Friction * jn).clamp(0.0, p.MaxContactImpulse)
    _apply_impulse(p, b, lever, tdir * jt[:, None], slide)
    corr = torch.minimum(torch.full_like(pen, p.MaxPositionCorrection), pen * p.CorrectionFraction)
    b.pos = torch.where(m[:, None], b.pos + normal * corr[:, None], b.pos)
    if is_foot:
        foot = k - 3
        b.u[:, U_FOOT] = torch.where(m, b.u[:, U_FOOT] | (1 << foot), b.u[:, U_FOOT])
        b.foot_imp[:, foot] = torch.where(m, b.foot_imp[:, foot] + jn, b.foot_imp[:, foot])
    else:
        diag["body_hit"] |= m
        b.u[:, U_BODY] = torch.where(m, b.u[:, U_BODY] | (1 << k), b.u[:, U_BODY])
        b.body_imp[:, k] = torch.where(m, b.body_imp[:, k] + jn, b.body_imp[:, k])


def _refresh_contacts(p, terrain, b: _Body, lanes: torch.Tensor) -> None:
    body = torch.zeros_like(b.u[:, 0]); foot = torch.zeros_like(body); pad = torch.zeros_like(body)
    for k in range(7):
        center = b.pos + _rotate(b.q, torch.tensor(p.Supports[k][:3], dtype=torch.float32).expand_as(b.pos))
        inb, height, _ = _terrain(p, terrain, center[:, 0], center[:, 2])
        touch = inb & (center[:, 1] - p.Supports[k][3] - height <= p.ContactSlop)
        if k < 3:
            body = body | (touch.int() << k)
        else:
            foot = foot | (touch.int() << (k - 3))
            on_pad = inb & (torch.maximum(center[:, 0].abs(), center[:, 2].abs()) <= p.PadHalfExtent)
            pad = pad | (on_pad.int() << (k - 3))
    b.u[:, U_BODY] = torch.where(lanes, body, b.u[:, U_BODY])
    b.u[:, U_FOOT] = torch.where(lanes, foot, b.u[:, U_FOOT])
    b.u[:, U_PAD] = torch.where(lanes, pad, b.u[:, U_PAD])


def observe(p: LunarParams, terrain: torch.Tensor, sf: torch.Tensor, su: torch.Tensor) -> torch.Tensor:
    """[E, 33]: position, velocity, body up and forward axes, angular velocity (scaled and clamped to [-1, 1]), a 3 x 3
    grid of terrain clearances, four foot clearances, four foot contact flags, remaining fuel fraction."""
    b = _Body(sf, su)
    nv = lambda v, s: (v / s).clamp(-1.0, 1.0)
    cols = [nv(b.pos, p.PositionScale), nv(b.vel, p.VelocityScale),
            _rotate(b.q, torch.tensor([0.0, 1.0, 0.0]).expand_as(b.pos)).clamp(-1, 1),
            _rotate(b.q, torch.tensor([0.0, 0.0, -1.0]).expand_as(b.pos)).clamp(-1, 1), nv(b.w, p.AngularScale)]
    probes = []
    for pz in (-1, 0, 1):
        for px in (-1, 0, 1):
            inb, height, _ = _terrain(p, terrain, b.pos[:, 0] + px * p.ProbeSpacing, b.pos[:, 2] + pz * p.ProbeSpacing)
            probes.append(nv(torch.where(inb, b.pos[:, 1] - height, torch.full_like(height, p.TerrainClearanceScale)), p.TerrainClearanceScale))
    feet = []
    for k in range(3, 7):
        center = b.pos + _rotate(b.q, torch.tensor(p.Supports[k][:3], dtype=torch.float32).expand_as(b.pos))
        inb, height, _ = _terrain(p, terrain, center[:, 0], center[:, 2])
        feet.append(nv(torch.where(inb, center[:, 1] - p.Supports[k][3] - height, torch.full_like(height, p.FootClearanceScale)), p.FootClearanceScale))
    contacts = [((b.u[:, U_FOOT] >> f) & 1).float() for f in range(4)]
    obs = torch.cat(cols + [torch.stack(probes + feet + contacts + [(b.fuel / p.FuelCapacity).clamp(0.0, 1.0)], 1)], 1)
    return torch.where(b.finite()[:, None], obs, torch.zeros_like(obs))


def _step_cpu(p, terrain, action, external_stop, sf, su, trans_obs, obs, reward, terminated, truncated, end_reason) -> None:
    E = sf.shape[0]
    trans_obs.copy_(obs)
    done = (su[:, U_TERM] != 0) | (su[:, U_TRUNC] != 0)
    bad_action = ~done & ((action < 0) | (action >= 8))
    stopped = ~done & ~bad_action & (external_stop != 0)
    live = ~done & ~bad_action & ~stopped
    b = _Body(sf, su)
    act = torch.where(live, action, torch.zeros_like(action))
    pot_before = _potential(p, b)
    b.u[:, U_ACTION] = act
    b.throttle.zero_(); b.att.zero_(); b.body_imp.zero_(); b.foot_imp.zero_()
    b.u[:, U_BODY] = 0; b.u[:, U_FOOT] = 0; b.u[:, U_PAD] = 0
    diag = {"foot_hit": torch.zeros(E, dtype=torch.bool), "body_hit": torch.zeros(E, dtype=torch.bool), "foot_speed": torch.zeros(E)}
    main_used, att_used = torch.zeros(E), torch.zeros(E)
    valid = b.finite()
    h = float(torch.tensor(p.PolicyDt, dtype=torch.float32) / p.Substeps)
    axis = torch.zeros(8, 3)
    for a, (i, s) in {2: (0, 1.0), 3: (0, -1.0), 4: (2, 1.0), 5: (2, -1.0), 6: (1, 1.0), 7: (1, -1.0)}.items():
        axis[a, i] = s * p.AttitudeTorque
    inertia, inv_i = torch.tensor(p.Inertia, dtype=torch.float32), _inv_inertia(p)
    for _ in range(p.Substeps):
        is_main, is_att = act == 1, act >= 2
        want = torch.where(is_main, _f(p.MainFuelRate * h), torch.where(is_att, _f(p.AttitudeFuelRate * h), _f(0.0))).expand(E)
        frac = torch.where(want > 0, torch.minimum(torch.ones(E), b.fuel / torch.where(want > 0, want, torch.ones(E))), torch.ones(E))
        frac = torch.where(is_main | is_att, frac, torch.zeros(E))
        used = want * frac
        fuel = (b.fuel - used).clamp_min(0.0)
        main_used = torch.where(valid & is_main, main_used + used, main_used)
        att_used = torch.where(valid & is_att, att_used + used, att_used)
        throttle = torch.where(is_main, frac, torch.zeros(E))
        torque = axis[act.long()] * torch.where(is_att, frac, torch.zeros(E))[:, None]
        thrust = _rotate(b.q, torch.stack((torch.zeros(E), p.MainThrust * throttle, torch.zeros(E)), 1))
        vel = b.vel + (thrust / p.Mass + torch.tensor([0.0, -p.Gravity, 0.0])) * h
        pos = b.pos + vel * h
        w = b.w + (torque - _cross(b.w, inertia * b.w)) * inv_i * h
        dq = _quat_mul(b.q, torch.cat((torch.zeros(E, 1), w), 1)) * 0.5
        q = b.q + dq * h
        q = q / torch.sqrt((q * q).sum(1, keepdim=True))
        v1, v3 = valid, valid[:, None]
        b.fuel, b.throttle, b.att = torch.where(v1, fuel, b.fuel), torch.where(v1, throttle, b.throttle), torch.where(v3, torque, b.att)
        b.vel, b.pos, b.w, b.q = torch.where(v3, vel, b.vel), torch.where(v3, pos, b.pos), torch.where(v3, w, b.w), torch.where(v3, q, b.q)
        valid = valid & b.finite()
        for _ in range(p.ContactIterations):
            for k in range(7):
                _resolve_support(p, terrain, b, k, h, valid, diag)
            valid = valid & b.finite()
    _refresh_contacts(p, terrain, b, valid)
    b.u[:, U_STEP] += 1
    inb, _, _ = _terrain(p, terrain, b.pos[:, 0], b.pos[:, 2])
    reason = torch.zeros(E, dtype=torch.int32)
    numerical = ~valid | ~b.finite()
    oob = ~inb | (b.pos[:, 1] < p.TaskMinimumY) | (b.pos[:, 1] > p.TaskMaximumY)
    body = diag["body_hit"] | (b.u[:, U_BODY] != 0)
    hard = diag["foot_speed"] > p.HardFootSpeed
    up = _rotate(b.q, torch.tensor([0.0, 1.0, 0.0]).expand_as(b.pos))
    safe = ((b.u[:, U_FOOT] & 15) == 15) & ((b.u[:, U_PAD] & 15) == 15) & (b.u[:, U_BODY] == 0) & (_len(b.vel) <= p.SafeLinearSpeed) \
        & (_len(b.w) <= p.SafeAngularSpeed) & (torch.acos(up[:, 1].clamp(-1.0, 1.0)) <= p.SafeTilt)
    failed = numerical | oob | body | hard
    safe = safe & ~failed
    dwell = torch.where(safe, b.u[:, U_DWELL] + 1, torch.zeros_like(b.u[:, U_DWELL]))
    b.u[:, U_DWELL] = torch.where(failed, b.u[:, U_DWELL], dwell)
    landed = ~failed & (b.u[:, U_DWELL] >= p.SafeDwellSteps)
    for cond, code in ((landed, END_SAFE_LANDING), (hard, END_HARD_FOOT_IMPACT), (body, END_BODY_IMPACT), (oob, END_OUT_OF_BOUNDS),
                       (numerical, END_NUMERICAL_FAILURE)):            # later entries take precedence
        reason = torch.where(cond, torch.full_like(reason, code), reason)
    term = failed | landed
    trunc = ~term & (b.u[:, U_STEP] >= p.MaxEpisodeSteps)
    reason = torch.where(trunc, torch.full_like(reason, END_TIME_LIMIT), reason)
    pot_after = torch.where(term, torch.zeros(E), _potential(p, b))
    soft = torch.zeros(E)
    for f in range(4):
        fresh = ~hard & (((b.u[:, U_FOOT] >> f) & 1) != 0) & (((b.u[:, U_REWARDED] >> f) & 1) == 0)
        soft = soft + torch.where(fresh, _f(p.SoftFootReward), _f(0.0))
        b.u[:, U_REWARDED] = torch.where(fresh, b.u[:, U_REWARDED] | (1 << f), b.u[:, U_REWARDED])
    terminal = torch.where(landed, _f(p.SuccessReward), torch.where(term, _f(p.FailurePenalty), _f(0.0)))
    r = p.RewardGamma * pot_after - pot_before - p.MainFuelCostWeight * main_used - p.AttitudeFuelCostWeight * att_used + soft \
        + torch.where(safe, _f(p.StableDwellReward), _f(0.0)) + terminal
    broken = ~torch.isfinite(r) | ~torch.isfinite(b.ret + r)
    r = torch.where(broken, _f(p.FailurePenalty), r)
    term, trunc = term | broken, trunc & ~broken
    reason = torch.where(broken, torch.full_like(reason, END_NUMERICAL_FAILURE), reason)
    ret = b.ret + r
    b.ret = torch.where(torch.isfinite(ret), ret, torch.zeros(E))
    b.u[:, U_TERM], b.u[:, U_TRUNC], b.u[:, U_REASON] = term.int(), trunc.int(), reason
    b.store(sf, su, live)
    # lanes that did not simulate
    su[bad_action, U_STEP] += 1
    su[bad_action, U_TERM] = 1
    su[bad_action, U_REASON] = END_INVALID_ACTION
    sf[bad_action, S_RETURN] += p.FailurePenalty
    su[stopped, U_TRUNC] = 1
    su[stopped, U_REASON] = END_EXTERNAL_STOP
    reward.copy_(torch.where(live, r, torch.where(bad_action, _f(p.FailurePenalty), _f(0.0))))
    terminated.copy_((su[:, U_TERM] != 0).to(terminated.dtype))
    truncated.copy_((su[:, U_TRUNC] != 0).to(truncated.dtype))
    end_reason.copy_(su[:, U_REASON])
    fresh_obs = observe(p, terrain, sf, su)
    obs[~done] = fresh_obs[~done]


# ------------------------------------------------------------------------------------------ entry points
U_EPISODE = 10
SPAWN_DEFAULT = (6.0, 12.0, 20.0, 0.8, 1.5, 0.05, 0.5, 0.05)   # xz half extent, y range, planar / descent speed, tilt, yaw, spin
M32 = 0xFFFFFFFF


def _mix32(v: torch.Tensor) -> torch.Tensor:
    v = v & M32
    v = v ^ (v >> 16)
    v = (v * 0x7FEB352D) & M32
    v = v ^ (v >> 15)
    v = (v * 0x846CA68B) & M32
    return v ^ (v >> 16)


def _uniform(seed: int, env: torch.Tensor, episode: torch.Tensor, comp: int) -> torch.Tensor:
    seed = int(seed) & 0xFFFFFFFFFFFFFFFF
    lo, hi = seed & M32, seed >> 32
    v = _mix32(torch.tensor(lo, dtype=torch.int64) ^ _mix32(torch.tensor((hi + 0x9E3779B9) & M32, dtype=torch.int64)))
    v = _mix32(v ^ _mix32((env + 0x85EBCA6B) & M32))
    v = _mix32(v ^ _mix32((episode + 0xC2B2AE35) & M32))
    v = _mix32(v ^ _mix32(torch.tensor((comp + 0x27D4EB2F) & M32, dtype=torch.int64)))
    return (v >> 8).to(torch.float32) * (1.0 / 16777216.0)


_checked_terrains: set = set()


def _host_tables(p: LunarParams):
    f, n = p.Floats(), p.Ints()
    return (ctypes.c_float * len(f))(*f), (ctypes.c_int * len(n))(*n)


def _check(p: LunarParams, terrain, sf, su, obs) -> None:
    E = sf.shape[0]
    if terrain.numel() != (p.CellsX + 1) * (p.CellsZ + 1) or terrain.dtype != torch.float32:
        raise ValueError("terrain must hold (CellsZ + 1) x (CellsX + 1) fp32 heights")
    if sf.shape != (E, STATE_F32) or su.shape != (E, STATE_U32) or obs.shape != (E, OBS_WIDTH) or su.dtype != torch.int32:
        raise ValueError("state must be [E, 32] fp32 and [E, 16] int32, observation [E, 33] fp32")
    if len(p.Supports) != 7 or p.Substeps <= 0 or p.ContactIterations < 0:
        raise ValueError("seven supports and a positive substep count are required")
    key = (terrain.data_ptr(), terrain._version)
    if key not in _checked_terrains:                       # once per terrain: one device read
        if float(terrain.abs().max()) > p.MaxAbsHeight + 1e-6:
            raise ValueError("terrain heights must lie within +-MaxAbsHeight")
        if len(_checked_terrains) > 64:
            _checked_terrains.clear()
        _checked_terrains.add(key)


def reset(p: LunarParams, terrain, sf, su, obs, seed: int, only_done: bool, spawn=SPAWN_DEFAULT) -> None:
    """Re-spawn every lane (episode 0) or only the finished ones (their next episode index) in place."""
    _check(p, terrain, sf, su, obs)
    E = sf.shape[0]
    if sf.is_cuda:
        cf, cn = _host_tables(p)
        s = int(seed) & 0xFFFFFFFFFFFFFFFF
        K._launch(N.require().oa_rl_lunar_reset(cf, cn, (ctypes.c_float * 8)(*spawn), terrain.data_ptr(), sf.data_ptr(), su.data_ptr(),
                                                obs.data_ptr(), E, s & M32, s >> 32, int(only_done), N.stream()), "oa_rl_lunar_reset")
        return
    sel = ((su[:, U_TERM] != 0) | (su[:, U_TRUNC] != 0)) if only_done else torch.ones(E, dtype=torch.bool)
    episode = (su[:, U_EPISODE].to(torch.int64) + 1) if only_done else torch.zeros(E, dtype=torch.int64)
    env = torch.arange(E, dtype=torch.int64)
    u = [_uniform(seed, env, episode, c) for c in range(12)]
    sp = [_f(v) for v in spawn]
    new_f = torch.zeros(E, STATE_F32)
    new_f[:, S_POS + 0], new_f[:, S_POS + 1], new_f[:, S_POS + 2] = (u[0] * 2 - 1) * sp[0], sp[1] + u[2] * (sp[2] - sp[1]), (u[1] * 2 - 1) * sp[0]
    new_f[:, S_VEL + 0], new_f[:, S_VEL + 1], new_f[:, S_VEL + 2] = (u[3] * 2 - 1) * sp[3], -u[5] * sp[4], (u[4] * 2 - 1) * sp[3]
    q = torch.stack((torch.ones(E), (u[6] * 2 - 1) * sp[5], (u[8] * 2 - 1) * sp[6], (u[7] * 2 - 1) * sp[5]), 1)
    new_f[:, S_QUAT:S_QUAT + 4] = q / torch.sqrt((q * q).sum(1, keepdim=True))
    for i in range(3):
        new_f[:, S_ANG + i] = (u[9 + i] * 2 - 1) * sp[7]
    new_f[:, S_FUEL] = p.FuelCapacity
    new_u = torch.zeros(E, STATE_U32, dtype=torch.int32)
    new_u[:, U_EPISODE] = episode.to(torch.int32)
    b = _Body(new_f, new_u)
    _refresh_contacts(p, terrain, b, torch.ones(E, dtype=torch.bool))
    b.store(new_f, new_u, torch.ones(E, dtype=torch.bool))
    sf[sel], su[sel] = new_f[sel], new_u[sel]
    obs[sel] = observe(p, terrain, new_f, new_u)[sel]


def step(p: LunarParams, terrain, action, external_stop, sf, su, trans_obs, obs, reward, terminated, truncated, end_reason) -> None:
    """One policy step of every lane, in place.  action [E] int32 (0 coast, 1 main engine, 2..7 pitch / roll / yaw
    pairs), external_stop [E] uint8; outputs: trans_obs (the observation the action was chosen from), obs (the
    next one), reward [E] fp32, terminated / truncated [E] uint8, end_reason [E] int32."""
    _check(p, terrain, sf, su, obs)
    if sf.is_cuda:
        cf, cn = _host_tables(p)
        K._launch(N.require().oa_rl_lunar_step(cf, cn, terrain.data_ptr(), action.data_ptr(), external_stop.data_ptr(), sf.data_ptr(),
                                               su.data_ptr(), trans_obs.data_ptr(), obs.data_ptr(), reward.data_ptr(), terminated.data_ptr(),
                                               truncated.data_ptr(), end_reason.data_ptr(), sf.shape[0], N.stream()), "oa_rl_lunar_step")
        return
    _step_cpu(p, terrain, action, external_stop, sf, su, trans_obs, obs, reward, terminated, truncated, end_reason)
