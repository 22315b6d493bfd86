"""LunarLander3d: physical sanity of the tensor implementation on CPU; the CUDA kernels against it on a GPU."""
import math

import pytest
import torch

from oa_b200.core import fn_matrix as F
from oa_b200.ml.rl.environment import OaLunarLander3dConfig, OaLunarLander3dEnvironment
from oa_b200.ops import lunar as LL


def _buffers(E, device="cpu"):
    z = lambda *s, dt=torch.float32: torch.zeros(*s, dtype=dt, device=device)
    return dict(sf=z(E, 32), su=z(E, 16, dt=torch.int32), trans=z(E, 33), obs=z(E, 33), reward=z(E), term=z(E, dt=torch.uint8),
                trunc=z(E, dt=torch.uint8), reason=z(E, dt=torch.int32), stop=z(E, dt=torch.uint8))


def _step(p, terrain, action, b):
    LL.step(p, terrain, action, b["stop"], b["sf"], b["su"], b["trans"], b["obs"], b["reward"], b["term"], b["trunc"], b["reason"])


def _place(b, lane, pos, vel=(0, 0, 0), quat=(1, 0, 0, 0), fuel=100.0):
    b["sf"][lane] = 0
    b["sf"][lane, 0:3] = torch.tensor(pos, dtype=torch.float32)
    b["sf"][lane, 3:6] = torch.tensor(vel, dtype=torch.float32)
    b["sf"][lane, 6:10] = torch.tensor(quat, dtype=torch.float32)
    b["sf"][lane, 13] = fuel
    b["su"][lane] = 0


def test_terrain_is_bounded_and_flat_on_the_pad():
    p = LL.LunarParams()
    t = LL.make_terrain(p, 7).view(p.CellsZ + 1, p.CellsX + 1)
    assert torch.equal(t, LL.make_terrain(p, 7).view_as(t)) and not torch.equal(t, LL.make_terrain(p, 8).view_as(t))
    assert float(t.abs().max()) <= p.MaxAbsHeight and float(t.abs().max()) > 0.05
    lim = p.MaxSlope * p.CellSize + 1e-6
    assert float((t[:, 1:] - t[:, :-1]).abs().max()) <= lim and float((t[1:] - t[:-1]).abs().max()) <= lim
    c = p.CellsX // 2
    assert float(t[c - 3:c + 4, c - 3:c + 4].abs().max()) == 0.0
    inb, h, n = LL._terrain(p, t.reshape(-1), torch.tensor([0.0, 100.0, -16.0, 16.0]), torch.tensor([0.0, 0.0, 16.0, -16.0]))
    assert inb.tolist() == [True, False, True, True] and float(h[0]) == 0 and torch.allclose(n[0], torch.tensor([0.0, 1.0, 0.0]))
    # on a tilted plane the sampled height and normal are those of the plane
    plane = (0.2 * torch.arange(p.CellsX + 1, dtype=torch.float32))[None, :].expand(p.CellsZ + 1, -1).reshape(-1).contiguous()
    inb, h, n = LL._terrain(p, plane, torch.tensor([-3.3, 2.75]), torch.tensor([1.4, -7.9]))
    assert torch.allclose(h, 0.2 * (torch.tensor([-3.3, 2.75]) + 16.0), atol=1e-5)
    assert torch.allclose(n, torch.tensor([-0.2, 1.0, 0.0]).div(math.sqrt(1.04)).expand(2, 3), atol=1e-6)


def test_free_fall_main_engine_and_attitude():
    p = LL.LunarParams()
    terrain = torch.zeros((p.CellsX + 1) * (p.CellsZ + 1))
    b = _buffers(3)
    for lane in range(3):
        _place(b, lane, (0.0, 20.0, 0.0))
    b["obs"].copy_(LL.observe(p, terrain, b["sf"], b["su"]))
    first = b["obs"].clone()
    n = 30
    for _ in range(n):
        _step(p, terrain, torch.tensor([0, 1, 2], dtype=torch.int32), b)
    t = n * p.PolicyDt
    # coasting: v = -g t; semi-implicit Euler position = y0 - g h^2 k (k + 1) / 2 over k = n * substeps sub-steps
    k, h = n * p.Substeps, p.PolicyDt / p.Substeps
    assert float(b["sf"][0, 4]) == pytest.approx(-p.Gravity * t, rel=1e-4)
    assert float(b["sf"][0, 1]) == pytest.approx(20.0 - p.Gravity * h * h * k * (k + 1) / 2, rel=1e-5)
    assert float(b["sf"][0, 13]) == 100.0 and int(b["su"][0, 5]) == n
    # main engine: net acceleration thrust / mass - g upwards, fuel burnt at the main rate
    assert float(b["sf"][1, 4]) == pytest.approx((p.MainThrust / p.Mass - p.Gravity) * t, rel=1e-4)
    assert float(b["sf"][1, 13]) == pytest.approx(100.0 - p.MainFuelRate * t, rel=1e-4) and float(b["sf"][1, 14]) == 1.0
    # pitch thruster: angular velocity torque / Ix about body x, orientation stays a unit quaternion, fuel at the attitude rate
    assert float(b["sf"][2, 10]) == pytest.approx(p.AttitudeTorque / p.Inertia[0] * t, rel=1e-4)
    assert float(b["sf"][2, 6:10].norm()) == pytest.approx(1.0, abs=1e-6) and float(b["sf"][2, 7]) > 0
    assert float(b["sf"][2, 13]) == pytest.approx(100.0 - p.AttitudeFuelRate * t, rel=1e-4)
    assert float(b["trans"][0, 4]) > float(b["obs"][0, 4]) and float(b["obs"].abs().max()) <= 1.0     # the transition keeps the earlier velocity
    assert torch.allclose(first[0, 15:24], torch.full((9,), 1.0)) and float(first[0, 32]) == 1.0     # 20 m above: clearances saturate
    assert bool((b["term"] == 0).all()) and bool((b["reason"] == 0).all())
    # shaping of the coasting lane: gamma * phi(after) - phi(before) with phi = -(position + velocity costs) here
    y1, v1 = float(b["sf"][0, 1]), float(b["sf"][0, 4])
    v0 = v1 + p.Gravity * p.PolicyDt
    phi = lambda y, v: -(p.PositionPotentialWeight * min(1.0, abs(y) / p.PositionScale) + p.VelocityPotentialWeight * min(1.0, abs(v) / p.VelocityScale))
    y0 = y1 - sum((v0 - p.Gravity * h * (i + 1)) * h for i in range(p.Substeps))
    assert float(b["reward"][0]) == pytest.approx(p.RewardGamma * phi(y1, v1) - phi(y0, v0), abs=2e-5)


def test_touchdown_outcomes():
    p = LL.LunarParams(SafeDwellSteps=5)
    terrain = torch.zeros((p.CellsX + 1) * (p.CellsZ + 1))
    rest_y = 1.0 + 0.1                      # feet 1.0 below the centre, radius 0.1
    b = _buffers(5)
    _place(b, 0, (0.0, rest_y + 0.02, 0.0))                              # gentle touchdown on the pad
    _place(b, 1, (0.0, rest_y + 0.5, 0.0), vel=(0.0, -3.0, 0.0))         # too fast: hard foot impact
    _place(b, 2, (0.0, 1.0, 0.0), quat=(0.0, 1.0, 0.0, 0.0))             # upside down: hull hits the ground
    _place(b, 3, (15.9, 5.0, 0.0), vel=(5.0, 0.0, 0.0))                  # drifts out of the terrain
    _place(b, 4, (8.0, rest_y + 0.02, 8.0))                              # gentle touchdown away from the pad
    b["obs"].copy_(LL.observe(p, terrain, b["sf"], b["su"]))
    total = torch.zeros(5)
    for i in range(40):
        act = torch.zeros(5, dtype=torch.int32)
        _step(p, terrain, act, b)
        total += b["reward"]
    assert b["reason"].tolist() == [LL.END_SAFE_LANDING, LL.END_HARD_FOOT_IMPACT, LL.END_BODY_IMPACT, LL.END_OUT_OF_BOUNDS, LL.END_NONE]
    assert b["term"].tolist() == [1, 1, 1, 1, 0] and b["trunc"].tolist() == [0, 0, 0, 0, 0]
    assert int(b["su"][0, 2]) == 15 and int(b["su"][0, 3]) == 15 and int(b["su"][4, 2]) == 15 and int(b["su"][4, 3]) == 0
    assert float(b["sf"][0, 1]) == pytest.approx(rest_y, abs=0.03) and float(b["sf"][0, 3:6].norm()) < 0.05
    assert float(total[0]) > 90 and float(total[1]) < -90 and float(total[2]) < -90 and float(total[3]) < -90
    assert float(b["sf"][0, 25]) == pytest.approx(float(total[0]), rel=1e-4)
    assert b["obs"][0, 28:32].tolist() == [1.0, 1.0, 1.0, 1.0] and float(b["obs"][0, 24:28].abs().max()) < 0.02
    steps_done = int(b["su"][0, 5])
    _step(p, terrain, torch.zeros(5, dtype=torch.int32), b)              # finished lanes idle
    assert int(b["su"][0, 5]) == steps_done and float(b["reward"][0]) == 0.0 and int(b["term"][0]) == 1


def test_invalid_action_external_stop_and_time_limit():
    p = LL.LunarParams(MaxEpisodeSteps=3)
    terrain = torch.zeros((p.CellsX + 1) * (p.CellsZ + 1))
    b = _buffers(3)
    for lane in range(3):
        _place(b, lane, (0.0, 20.0, 0.0))
    b["stop"][1] = 1
    _step(p, terrain, torch.tensor([9, 0, 0], dtype=torch.int32), b)
    assert b["reason"].tolist() == [LL.END_INVALID_ACTION, LL.END_EXTERNAL_STOP, LL.END_NONE]
    assert b["term"].tolist() == [1, 0, 0] and b["trunc"].tolist() == [0, 1, 0] and b["reward"].tolist()[:2] == [p.FailurePenalty, 0.0]
    assert float(b["sf"][1, 1]) == 20.0                                   # the stopped lane did not move
    for _ in range(2):
        _step(p, terrain, torch.zeros(3, dtype=torch.int32), b)
    assert int(b["reason"][2]) == LL.END_TIME_LIMIT and int(b["trunc"][2]) == 1 and int(b["term"][2]) == 0


def test_environment_session_on_cpu():
    env, st = OaLunarLander3dEnvironment.Create(OaLunarLander3dConfig(Environments=6, Seed=11, TerrainSeed=3))
    assert st.IsOk() and env.Spec().Observation.ElementsPerEnvironment() == 33
    assert env.Begin().IsOk() and env.ResetEnvironment(0).IsOk()
    first = env.Observation().Tensor().clone()
    sf = env.StateF32().Tensor()
    assert first.shape == (6, 33) and float(first.abs().max()) <= 1.0 and float(sf[:, 1].min()) >= 12.0 and float(sf[:, 1].max()) <= 20.0
    assert torch.allclose(sf[:, 6:10].norm(dim=1), torch.ones(6), atol=1e-6) and len({round(float(v), 4) for v in sf[:, 0]}) == 6
    assert env.Begin().IsOk()
    tr, st = env.StepEnvironment(F.FromInt32([0, 1, 2, 3, 4, 9], [6]))
    assert st.IsOk() and tr.IsValid() and torch.equal(tr.Observation.Tensor(), first)
    assert tr.Terminated.Tensor().tolist() == [0, 0, 0, 0, 0, 1] and int(env.EndReason().Tensor()[5]) == LL.END_INVALID_ACTION
    before = env.StateF32().Tensor().clone()
    assert env.ResetCompleted().IsOk()
    after = env.StateF32().Tensor()
    assert torch.equal(before[:5], after[:5]) and not torch.equal(before[5], after[5]) and int(env.StateU32().Tensor()[5, 10]) == 1
    again, _ = OaLunarLander3dEnvironment.Create(OaLunarLander3dConfig(Environments=6, Seed=11, TerrainSeed=3))
    again.Begin(); again.ResetEnvironment(0)
    assert torch.equal(again.Observation().Tensor(), first)
    assert not OaLunarLander3dConfig(Environments=0).Validate().IsOk()


@pytest.mark.gpu
def test_cuda_kernels_match_the_tensor_implementation():
    """Step by step from identical states (the CPU trajectory drives both), so that a contact that starts one ulp apart
    cannot compound; lanes start low so that touchdowns, impacts and exits all occur within the run."""
    p = LL.LunarParams(SafeDwellSteps=5, MaxEpisodeSteps=80)
    terrain = LL.make_terrain(p, 5)
    E = 64
    c, g = _buffers(E), _buffers(E, "cuda")
    spawn = (12.0, 1.2, 4.0, 1.5, 1.5, 0.2, 0.5, 0.2)
    LL.reset(p, terrain, c["sf"], c["su"], c["obs"], 123, False, spawn)
    LL.reset(p, terrain.cuda(), g["sf"], g["su"], g["obs"], 123, False, spawn)
    assert torch.allclose(g["sf"].cpu(), c["sf"], atol=1e-6) and torch.equal(g["su"].cpu(), c["su"]) and torch.allclose(g["obs"].cpu(), c["obs"], atol=1e-5)
    gen = torch.Generator().manual_seed(0)
    checked = matched = 0
    reasons = set()
    for step in range(60):
        action = torch.randint(0, 8, (E,), generator=gen, dtype=torch.int32)
        action[step % E] = 11 if step % 17 == 0 else action[step % E]
        for k in ("sf", "su", "obs"):
            g[k].copy_(c[k])
        _step(p, terrain, action, c)
        _step(p, terrain.cuda(), action.cuda(), g)
        same_flags = (g["term"].cpu() == c["term"]) & (g["trunc"].cpu() == c["trunc"]) & (g["reason"].cpu() == c["reason"]) \
            & (g["su"].cpu() == c["su"]).all(1)
        close = (g["sf"].cpu() - c["sf"]).abs().amax(1) <= 2e-3 * (1 + c["sf"].abs().amax(1))
        close &= (g["obs"].cpu() - c["obs"]).abs().amax(1) <= 2e-3
        close &= (g["reward"].cpu() - c["reward"]).abs() <= 2e-3 * (1 + c["reward"].abs())
        close &= torch.allclose(g["trans"].cpu(), c["trans"], atol=1e-6)
        checked += E
        matched += int((same_flags & close).sum())
        reasons |= set(c["reason"].tolist())
        if step % 10 == 9:
            LL.reset(p, terrain, c["sf"], c["su"], c["obs"], 123, True, spawn)
    assert matched >= 0.98 * checked, (matched, checked)
    assert {LL.END_NONE, LL.END_INVALID_ACTION} <= reasons and len(reasons) >= 3, reasons
    g["su"].copy_(c["su"]); g["sf"].copy_(c["sf"]); g["obs"].copy_(c["obs"])
    LL.reset(p, terrain, c["sf"], c["su"], c["obs"], 77, True, spawn)
    LL.reset(p, terrain.cuda(), g["sf"], g["su"], g["obs"], 77, True, spawn)
    assert torch.allclose(g["sf"].cpu(), c["sf"], atol=1e-6) and torch.equal(g["su"].cpu(), c["su"])
