"""Reinforcement-learning stack on the CPU engine: environment dynamics, GAE, policies, losses, storage and trainers.

Test strategy of the reference: Test/Ml/Rl/*.cpp (closed-form oracles for GAE / losses, deterministic environment
replays, short end-to-end trainer runs).
"""
import math

import pytest
import torch

from oa_b200.core import fn_matrix as F
from oa_b200.core.matrix import OaMatrix
from oa_b200.ml import autograd as AG
from oa_b200.ml import optim as O
from oa_b200.ml import rl as RL
from oa_b200.ml.module import OaModule
from oa_b200.ml.nn.layers import OaLinear
from oa_b200.ml.rl import fn_rl as FR

M = lambda t: OaMatrix(t)


def _u8(x):
    return torch.tensor(x, dtype=torch.uint8)


# ------------------------------------------------------------------------------------------------------ environment
def test_field_and_environment_specs_validate():
    box = RL.OaRlFieldSpec.Box("observation", (4,))
    assert box.ValidateDefinition() and box.ElementsPerEnvironment() == 4 and box.BatchedShape(3) == (3, 4)
    assert not RL.OaRlFieldSpec.Box("", (4,)).ValidateDefinition()
    assert not RL.OaRlFieldSpec.Box("x", (0,)).ValidateDefinition()
    assert not RL.OaRlFieldSpec.Discrete("a", 1).ValidateDefinition()
    assert box.ValidateMatrix(M(torch.zeros(3, 4)), 3)
    assert not box.ValidateMatrix(M(torch.zeros(3, 5)), 3)
    assert not box.ValidateMatrix(M(torch.zeros(3, 4, dtype=torch.int32)), 3)
    env = RL.OaCartPoleEnvironment(RL.OaCartPoleConfig(Environments=3))
    spec = env.Spec()
    assert spec.ValidateDefinition()
    assert spec.ValidateAction(M(torch.zeros(3, dtype=torch.int32)), 3)
    assert not spec.ValidateAction(M(torch.zeros(3)), 3)


def test_cartpole_matches_gymnasium_dynamics_and_lifecycle():
    E = 5
    env = RL.OaCartPoleEnvironment(RL.OaCartPoleConfig(Environments=E, MaxEpisodeSteps=7, Seed=11))
    assert env.ResetEnvironment(11)
    s0 = env.Observation().Tensor().clone()
    assert s0.shape == (E, 4) and s0.abs().max() < 0.05 + 1e-7 and s0.std() > 0
    env2 = RL.OaCartPoleEnvironment(RL.OaCartPoleConfig(Environments=E, MaxEpisodeSteps=7, Seed=11))
    env2.ResetEnvironment(11)
    assert torch.equal(env2.Observation().Tensor(), s0)                   # deterministic in (seed, lane, episode)
    action = torch.tensor([0, 1, 0, 1, 1], dtype=torch.int32)
    tr, st = env.StepEnvironment(M(action))
    assert st and tr.IsValid() and torch.equal(tr.Observation.Tensor(), s0)
    # explicit Euler step of CartPole-v1 in float64
    x, xv, th, thv = s0.double().unbind(1)
    force = torch.where(action == 1, 10.0, -10.0).double()
    tmp = (force + 0.05 * thv ** 2 * torch.sin(th)) / 1.1
    tha = (9.8 * torch.sin(th) - torch.cos(th) * tmp) / (0.5 * (4.0 / 3.0 - 0.1 * torch.cos(th) ** 2 / 1.1))
    xa = tmp - 0.05 * tha * torch.cos(th) / 1.1
    want = torch.stack((x + 0.02 * xv, xv + 0.02 * xa, th + 0.02 * thv, thv + 0.02 * tha), 1)
    assert (tr.NextObservation.Tensor().double() - want).abs().max() < 1e-6
    assert torch.equal(tr.Reward.Tensor(), torch.ones(E)) and tr.Terminated.Tensor().sum() == 0
    # run to the step limit: truncation, then idle lanes with zero reward until ResetCompleted
    for _ in range(6):
        alt = (env.EpisodeSteps().Tensor() % 2).to(torch.int32)
        tr, st = env.StepEnvironment(M(alt))
    assert (tr.Truncated.Tensor() | tr.Terminated.Tensor()).all()
    tr, _ = env.StepEnvironment(M(action))
    assert tr.Reward.Tensor().abs().sum() == 0 and tr.Truncated.Tensor().sum() == 0
    assert env.ResetCompleted()
    assert env.Done().Tensor().sum() == 0 and env.EpisodeSteps().Tensor().sum() == 0
    assert not torch.equal(env.Observation().Tensor(), s0)                # next episode index -> new initial state
    ev, st = env.Submit()
    assert st and env.Wait(ev) and env.SubmissionCount() == 1 and not env.HasActiveRecording()
    # invalid action terminates with zero reward
    bad = torch.tensor([2, 0, 0, 0, 0], dtype=torch.int32)
    tr, _ = env.StepEnvironment(M(bad))
    assert tr.Terminated.Tensor()[0] == 1 and tr.Reward.Tensor()[0] == 0
    assert env.Cancel() and env.Close() and not env.IsOpen()
    assert not env.Begin()


# ---------------------------------------------------------------------------------------------------------- GAE
def test_gae_matches_closed_form_with_masks():
    T, E = 6, 3
    g = torch.Generator().manual_seed(0)
    r, v, nv = torch.randn(T, E, generator=g), torch.randn(T, E, generator=g), torch.randn(T, E, generator=g)
    term, trunc = torch.zeros(T, E, dtype=torch.uint8), torch.zeros(T, E, dtype=torch.uint8)
    term[2, 0] = 1
    trunc[3, 1] = 1
    res = FR.Gae(M(r), M(v), M(nv), M(term), M(trunc), FR.OaGaeConfig(0.9, 0.8))
    assert res.IsValid()
    adv = torch.zeros(T, E)
    for e in range(E):
        nxt = 0.0
        for t in range(T - 1, -1, -1):
            boot = 0.0 if term[t, e] else 1.0
            trace = 0.0 if (term[t, e] or trunc[t, e]) else 1.0
            a = r[t, e] + 0.9 * boot * nv[t, e] - v[t, e] + 0.9 * 0.8 * trace * nxt
            adv[t, e] = a
            nxt = a
    assert (res.Advantage.Tensor() - adv).abs().max() < 1e-5
    assert (res.Return.Tensor() - (adv + v)).abs().max() < 1e-5
    assert not FR.Gae(M(r), M(v), M(nv[:, :2]), M(term), M(trunc)).IsValid()
    n = FR.NormalizeAdvantages(res.Advantage).Tensor()
    assert abs(n.mean().item()) < 1e-6 and abs(n.std(unbiased=False).item() - 1.0) < 1e-4


# ------------------------------------------------------------------------------------------------------- policies
def test_categorical_policy_gradients_match_torch():
    E, A = 6, 4
    g = torch.Generator().manual_seed(1)
    logits_t = torch.randn(E, A, generator=g)
    action = torch.randint(0, A, (E,), generator=g, dtype=torch.int32)
    value = torch.randn(E, generator=g)
    logits = M(logits_t.clone())
    logits.SetRequiresGrad(True)
    tape = AG.OaGradientTape()
    pol = FR.EvaluateCategoricalPolicy(logits, M(action), M(value))
    loss = F.Sub(F.Mean(pol.LogProbability), F.Scale(F.Mean(pol.Entropy), 0.3))
    tape.Backward(loss)
    tape.Close()
    lt = logits_t.clone().requires_grad_(True)
    dist = torch.distributions.Categorical(logits=lt)
    ref = dist.log_prob(action.long()).mean() - 0.3 * dist.entropy().mean()
    ref.backward()
    assert (pol.LogProbability.Tensor() - dist.log_prob(action.long()).detach()).abs().max() < 1e-5
    assert (pol.Entropy.Tensor() - dist.entropy().detach()).abs().max() < 1e-5
    assert (logits.GradTensor() - lt.grad).abs().max() < 1e-5
    # sampling: deterministic per seed, distribution follows softmax
    big = torch.log(torch.tensor([[0.1, 0.2, 0.3, 0.4]])).repeat(20000, 1).contiguous()
    s1 = FR.SampleLogits(M(big), 1.0, 0, 1.0, 7).Tensor()
    s2 = FR.SampleLogits(M(big), 1.0, 0, 1.0, 7).Tensor()
    assert torch.equal(s1, s2) and s1.dtype == torch.int32
    freq = torch.bincount(s1.long(), minlength=4).float() / s1.numel()
    assert (freq - torch.tensor([0.1, 0.2, 0.3, 0.4])).abs().max() < 0.02
    assert torch.equal(FR.SampleLogits(M(logits_t), 0.0, 0, 1.0, 3).Tensor().long(), logits_t.argmax(1))
    topk = FR.SampleLogits(M(big), 1.0, 2, 1.0, 9).Tensor()
    assert set(topk.tolist()) <= {2, 3}


def test_tanh_normal_policy_matches_formula_and_differentiates():
    E, A = 5, 3
    g = torch.Generator().manual_seed(2)
    mean_t, ls_t, raw_t = torch.randn(E, A, generator=g), 0.3 * torch.randn(E, A, generator=g), torch.randn(E, A, generator=g)
    value = torch.zeros(E)
    mean, ls = M(mean_t.clone()), M(ls_t.clone())
    mean.SetRequiresGrad(True)
    ls.SetRequiresGrad(True)
    tape = AG.OaGradientTape()
    pol = FR.EvaluateTanhNormalPolicy(mean, ls, M(raw_t), M(value), -2.0, 2.0)
    tape.Backward(F.Mean(pol.LogProbability))
    tape.Close()
    mt, lt = mean_t.clone().requires_grad_(True), ls_t.clone().requires_grad_(True)
    base = torch.distributions.Normal(mt, lt.exp()).log_prob(raw_t)
    jac = torch.log(2.0 * (1 - torch.tanh(raw_t) ** 2 + 1e-6))
    want = (base - jac).sum(1)
    want.mean().backward()
    assert (pol.LogProbability.Tensor() - want.detach()).abs().max() < 1e-4
    assert (pol.Action.Tensor() - 2.0 * torch.tanh(raw_t)).abs().max() < 1e-6
    assert (pol.Entropy.Tensor() - torch.distributions.Normal(mt, lt.exp()).entropy().sum(1).detach()).abs().max() < 1e-5
    assert (mean.GradTensor() - mt.grad).abs().max() < 1e-5 and (ls.GradTensor() - lt.grad).abs().max() < 1e-5
    a = FR.SampleTanhNormalPolicy(M(mean_t), M(ls_t), M(value), -2.0, 2.0, seed=5)
    b = FR.SampleTanhNormalPolicy(M(mean_t), M(ls_t), M(value), -2.0, 2.0, seed=5)
    assert a.IsValid() and torch.equal(a.Action.Tensor(), b.Action.Tensor()) and a.Action.Tensor().abs().max() <= 2.0
    assert not FR.EvaluateTanhNormalPolicy(M(mean_t), M(ls_t), M(raw_t), M(value), 1.0, -1.0).IsValid()


def test_transforms():
    obs = M(torch.tensor([[1.0, 100.0]]))
    out = FR.NormalizeObservation(obs, M(torch.tensor([[0.0, 0.0]])), M(torch.tensor([[2.0, 1.0]])), 0.0, 10.0).Tensor()
    assert torch.allclose(out, torch.tensor([[0.5, 10.0]]))
    assert torch.allclose(FR.ScaleAction(M(torch.tensor([-1.0, 0.0, 3.0])), -1, 1, 0, 10).Tensor(), torch.tensor([0.0, 5.0, 10.0]))
    assert torch.allclose(FR.ClipReward(M(torch.tensor([-5.0, 0.5, 7.0]))).Tensor(), torch.tensor([-1.0, 0.5, 1.0]))


# ----------------------------------------------------------------------------------------------------------- losses
def test_ppo_loss_and_gradient_match_autograd():
    n = 64
    g = torch.Generator().manual_seed(3)
    new_t, old_t, adv_t = 0.5 * torch.randn(n, generator=g), 0.5 * torch.randn(n, generator=g), torch.randn(n, generator=g)
    val_t, ret_t, ent_t = torch.randn(n, generator=g), torch.randn(n, generator=g), torch.rand(n, generator=g)
    new, val, ent = M(new_t.clone()), M(val_t.clone()), M(ent_t.clone())
    for m in (new, val, ent):
        m.SetRequiresGrad(True)
    tape = AG.OaGradientTape()
    res = FR.Ppo(new, M(old_t), M(adv_t), val, M(ret_t), ent, FR.OaPpoLossConfig(0.2, 0.5, 0.01))
    assert res.IsValid()
    tape.Backward(res.TotalLoss)
    tape.Close()
    nt, vt, et = (t.clone().requires_grad_(True) for t in (new_t, val_t, ent_t))
    ratio = torch.exp(nt - old_t)
    pl = -torch.minimum(ratio * adv_t, ratio.clamp(0.8, 1.2) * adv_t).mean()
    vl = ((vt - ret_t) ** 2).mean()
    total = pl + 0.5 * vl - 0.01 * et.mean()
    total.backward()
    assert abs(res.PolicyLoss.Item() - pl.item()) < 1e-5 and abs(res.ValueLoss.Item() - vl.item()) < 1e-5
    assert abs(res.TotalLoss.Item() - total.item()) < 1e-5
    assert (new.GradTensor() - nt.grad).abs().max() < 1e-6
    assert (val.GradTensor() - vt.grad).abs().max() < 1e-6 and (ent.GradTensor() - et.grad).abs().max() < 1e-6
    assert (FR.PpoClippedPolicyBwd(M(new_t), M(old_t), M(adv_t), 0.2).Tensor() - nt.grad).abs().max() < 1e-6
    assert FR.PpoClippedPolicy(M(new_t), M(old_t), M(adv_t), 1.5) is None
    assert not FR.Ppo(new, M(old_t), M(adv_t), val, M(ret_t[:10]), ent).IsValid()


def test_dqn_and_sac_losses():
    B, A = 8, 3
    g = torch.Generator().manual_seed(4)
    q_t, nq_t = torch.randn(B, A, generator=g), torch.randn(B, A, generator=g)
    act = torch.randint(0, A, (B,), generator=g, dtype=torch.int32)
    r = torch.randn(B, generator=g)
    term, trunc = _u8([1, 0, 0, 0, 1, 0, 0, 0]), _u8([0, 1, 0, 0, 0, 0, 0, 0])
    q = M(q_t.clone())
    q.SetRequiresGrad(True)
    tape = AG.OaGradientTape()
    res = FR.Dqn(q, M(act), M(r), M(nq_t), M(term), M(trunc), FR.OaDqnLossConfig(0.9))
    assert res.IsValid()
    tape.Backward(res.Loss)
    tape.Close()
    target = r + torch.where(term.bool(), torch.zeros(B), 0.9 * nq_t.max(1).values)     # truncation keeps the bootstrap
    qt = q_t.clone().requires_grad_(True)
    sel = qt.gather(1, act.long()[:, None])[:, 0]
    ref = torch.nn.functional.smooth_l1_loss(sel, target)
    ref.backward()
    assert (res.TargetQ.Tensor() - target).abs().max() < 1e-6 and abs(res.Loss.Item() - ref.item()) < 1e-6
    assert (q.GradTensor() - qt.grad).abs().max() < 1e-6
    # SAC
    q1_t, q2_t, n1, n2, lp = (torch.randn(B, generator=g) for _ in range(5))
    q1, q2 = M(q1_t.clone()), M(q2_t.clone())
    q1.SetRequiresGrad(True)
    q2.SetRequiresGrad(True)
    tape = AG.OaGradientTape()
    cr = FR.SacCritic(q1, q2, M(r), M(n1), M(n2), M(lp), M(term), M(trunc), FR.OaSacLossConfig(0.95, 0.2))
    assert cr.IsValid()
    tape.Backward(cr.TotalLoss)
    tape.Close()
    tq = r + torch.where(term.bool(), torch.zeros(B), 0.95 * (torch.minimum(n1, n2) - 0.2 * lp))
    assert (cr.TargetQ.Tensor() - tq).abs().max() < 1e-6
    assert abs(cr.TotalLoss.Item() - (((q1_t - tq) ** 2).mean() + ((q2_t - tq) ** 2).mean()).item()) < 1e-5
    assert (q1.GradTensor() - 2 * (q1_t - tq) / B).abs().max() < 1e-6
    lpm = M(lp.clone())
    lpm.SetRequiresGrad(True)
    q1b = M(q1_t.clone())
    q1b.SetRequiresGrad(True)
    tape = AG.OaGradientTape()
    al = FR.SacActor(q1b, M(q2_t), lpm, 0.2)
    tape.Backward(al)
    tape.Close()
    assert abs(al.Item() - (0.2 * lp - torch.minimum(q1_t, q2_t)).mean().item()) < 1e-6
    assert (lpm.GradTensor() - torch.full((B,), 0.2 / B)).abs().max() < 1e-7
    assert (q1b.GradTensor() - torch.where(q1_t <= q2_t, -1.0 / B, 0.0)).abs().max() < 1e-7


# ---------------------------------------------------------------------------------------------------------- storage
def test_rollout_buffer_appends_and_finalizes():
    T, E = 3, 2
    buf, st = RL.OaRlRolloutBuffer.Create(RL.OaRlRolloutConfig(T, E, (4,)))
    assert st and buf.IsValid() and buf.Capacity() == T and not buf.IsFull()
    assert not buf.Finalize()
    for t in range(T):
        tr = RL.OaRlTransition(M(torch.full((E, 4), float(t))), M(torch.tensor([t, t + 1], dtype=torch.int32)), M(torch.ones(E)),
                               M(torch.zeros(E)), M(torch.zeros(E)), M(torch.full((E,), -0.5)), M(_u8([0, 0])), M(_u8([0, 0])))
        assert buf.Append(tr)
    assert buf.IsFull() and not buf.Append(tr)
    B = buf.Batch()
    assert B.Observation.Tensor()[2, 1, 0] == 2.0 and B.Action.Tensor()[1].tolist() == [1, 2] and B.Valid.Tensor().all()
    assert buf.Finalize(FR.OaGaeConfig(1.0, 1.0)) and buf.IsFinalized()
    assert torch.allclose(B.Advantage.Tensor()[:, 0], torch.tensor([3.0, 2.0, 1.0]))
    buf.Reset()
    assert buf.Size() == 0 and B.Valid.Tensor().sum() == 0 and not buf.IsFinalized()
    bad = RL.OaRlTransition(M(torch.zeros(E, 3)), M(torch.zeros(E, dtype=torch.int32)), M(torch.ones(E)), M(torch.zeros(E)), M(torch.zeros(E)),
                            M(torch.zeros(E)), M(_u8([0, 0])), M(_u8([0, 0])))
    assert not buf.Append(bad)
    assert not RL.OaRlRolloutBuffer.Create(RL.OaRlRolloutConfig(0, 2, (4,)))[1]


def test_replay_buffer_wraps_and_samples_deterministically():
    from oa_b200.core.types import OaScalarType
    buf, st = RL.OaRlReplayBuffer.Create(RL.OaRlReplayConfig(5, (2,), (), OaScalarType.Int32))
    assert st

    def tr(base, rows):
        ids = torch.arange(base, base + rows)
        return RL.OaRlReplayTransition(M(ids.float()[:, None].repeat(1, 2)), M(ids.to(torch.int32)), M(ids.float()[:, None].repeat(1, 2) + 0.5),
                                       M(ids.float()), M(torch.zeros(rows, dtype=torch.uint8)), M((ids % 2).to(torch.uint8)))

    assert buf.Append(tr(0, 3)) and buf.Size() == 3 and buf.Cursor() == 3
    assert buf.Append(tr(3, 4)) and buf.Size() == 5 and buf.Cursor() == 2 and buf.IsFull()
    stored = buf.Storage_.Reward.Tensor().tolist()
    assert stored == [5.0, 6.0, 2.0, 3.0, 4.0]                                # rows 5, 6 wrapped over 0, 1
    a, st = buf.Sample(64, 42)
    b, _ = buf.Sample(64, 42)
    c, _ = buf.Sample(64, 43)
    assert st and torch.equal(a.Index.Tensor(), b.Index.Tensor()) and not torch.equal(a.Index.Tensor(), c.Index.Tensor())
    idx = a.Index.Tensor().long()
    assert idx.min() >= 0 and idx.max() < 5 and len(set(idx.tolist())) == 5
    assert torch.equal(a.Reward.Tensor(), buf.Storage_.Reward.Tensor()[idx])
    assert torch.equal(a.Observation.Tensor(), buf.Storage_.Observation.Tensor()[idx])
    assert torch.equal(a.NextObservation.Tensor(), a.Observation.Tensor() + 0.5)
    assert torch.equal(a.Action.Tensor().float(), a.Reward.Tensor())
    assert not buf.Append(tr(0, 6))
    buf.Reset()
    assert buf.Size() == 0 and not buf.Sample(4, 1)[1]


# --------------------------------------------------------------------------------------------------------- trainers
def _ppo_setup(E=32, horizon=32, rollouts=12, epochs=4, seed=3):
    F.SetRngSeed(seed)
    torch.manual_seed(seed)
    env = RL.OaCartPoleEnvironment(RL.OaCartPoleConfig(Environments=E, Seed=seed))
    model, st = RL.OaCategoricalActorCritic.Create(RL.OaCategoricalActorCriticConfig(4, 2, 32))
    assert st
    opt = O.OaAdam(model.AllParameterPtrs(), lr=3e-3)
    trainer, st = RL.OaPpoTrainer.Create(model, opt, RL.OaPpoTrainerConfig(rollouts, horizon, E, epochs, (4,), seed))
    assert st and trainer.IsValid()
    return env, model, trainer


def test_ppo_trainer_improves_cartpole_return():
    env, model, trainer = _ppo_setup()
    before, st = RL.OaFnRl.EvaluateCategorical(env, model, RL.OaRlEvaluationConfig(200, 5))
    assert st and before.CompletedEpisodes > 0
    assert env.ResetEnvironment(3)
    cycles = 0
    while not trainer.IsDone():
        assert trainer.NeedsCollection() and trainer.BeginCollection()
        assert not trainer.Update()                                           # wrong phase
        for _ in range(trainer.Config().Horizon):
            obs = OaMatrix(env.Observation().Tensor().clone())
            pol = trainer.Act(obs)
            assert pol.IsValid()
            tr, st = env.StepEnvironment(pol.Action)
            assert st and trainer.Observe(tr.Observation, tr.NextObservation, tr.Reward, tr.Terminated, tr.Truncated, pol)
            assert env.ResetCompleted()
        assert trainer.EndCollection() and trainer.Phase() == RL.OaRlTrainingPhase.Update
        while trainer.Phase() == RL.OaRlTrainingPhase.Update and not trainer.IsDone():
            assert trainer.Update()
        cycles += 1
    assert cycles == 12 and trainer.TrainingLoop().StepCount() == 48
    m = trainer.Metrics()
    assert math.isfinite(m.TotalLoss) and m.Entropy > 0 and m.Rollout == 12
    after, st = RL.OaFnRl.EvaluateCategorical(env, model, RL.OaRlEvaluationConfig(200, 5))
    assert st and after.MeanCompletedReturn > 1.5 * before.MeanCompletedReturn, (before, after)


def test_collector_records_a_full_rollout():
    env, model, _ = _ppo_setup(E=8, horizon=16)
    col, st = RL.OaRlCollector.Create(env, model, RL.OaRlCollectorConfig(16, 9))
    assert st
    buf, _ = RL.OaRlRolloutBuffer.Create(RL.OaRlRolloutConfig(16, 8, (4,)))
    env.ResetEnvironment(9)
    ev, st = col.Collect(buf)
    assert st and env.Wait(ev)
    assert buf.IsFull() and buf.IsFinalized() and col.Metrics().Transitions == 128 and col.Metrics().Collections == 1
    B = buf.Batch()
    assert B.Valid.Tensor().all() and B.Reward.Tensor().sum() > 0 and torch.isfinite(B.Advantage.Tensor()).all()
    wrong, _ = RL.OaRlRolloutBuffer.Create(RL.OaRlRolloutConfig(8, 8, (4,)))
    assert not col.Collect(wrong)[1]


class _Mlp(OaModule):
    def __init__(self, i, h, o):
        super().__init__()
        self.A = self.RegisterModule("0", OaLinear(i, h))
        self.B = self.RegisterModule("1", OaLinear(h, o))

    def Forward(self, x):
        return self.B.Forward(F.Relu(self.A.Forward(x)))


def test_dqn_trainer_updates_and_syncs_target(tmp_path):
    from oa_b200.core.types import OaScalarType
    F.SetRngSeed(5)
    online, target = _Mlp(4, 16, 2), _Mlp(4, 16, 2)
    opt = O.OaAdam(online.AllParameterPtrs(), lr=1e-2)
    replay, _ = RL.OaRlReplayBuffer.Create(RL.OaRlReplayConfig(256, (4,), (), OaScalarType.Int32))
    trainer, st = RL.OaDqnTrainer.Create(online, target, opt, replay, RL.OaDqnTrainerConfig(6, 32, 3, (4,), 1))
    assert st
    assert all(torch.equal(a.Data.Tensor(), b.Data.Tensor()) for a, b in zip(online.AllParameterPtrs(), target.AllParameterPtrs()))
    assert not trainer.Update()                                               # replay still empty
    env = RL.OaCartPoleEnvironment(RL.OaCartPoleConfig(Environments=64, Seed=2))
    env.ResetEnvironment(2)
    for i in range(4):
        act = M(torch.randint(0, 2, (64,), dtype=torch.int32))
        tr, _ = env.StepEnvironment(act)
        assert replay.Append(RL.OaRlReplayTransition(tr.Observation, act, tr.NextObservation, tr.Reward, tr.Terminated, tr.Truncated))
        env.ResetCompleted()
    losses = []
    while not trainer.IsDone():
        assert trainer.Update()
        losses.append(trainer.Metrics().Loss)
        same = all(torch.equal(a.Data.Tensor(), b.Data.Tensor()) for a, b in zip(online.AllParameterPtrs(), target.AllParameterPtrs()))
        assert same == (trainer.Metrics().Update % 3 == 0)
    assert len(losses) == 6 and all(math.isfinite(l) for l in losses) and trainer.TrainingLoop().StepCount() == 6
    path = str(tmp_path / "dqn.oam")
    assert trainer.Save(path) and trainer.Load(path)
    bad_replay, _ = RL.OaRlReplayBuffer.Create(RL.OaRlReplayConfig(16, (4,), (1,), OaScalarType.Float32))
    assert not RL.OaDqnTrainer.Create(online, target, opt, bad_replay, RL.OaDqnTrainerConfig(6, 4, 3, (4,), 1))[1]


def test_sac_trainer_runs_both_optimizer_units():
    from oa_b200.core.types import OaScalarType
    F.SetRngSeed(6)
    O_, A_ = 3, 2
    actor = _Mlp(O_, 16, 2 * A_)
    c1, c2, t1, t2 = (_Mlp(O_ + A_, 16, 1) for _ in range(4))
    aopt = O.OaAdam(actor.AllParameterPtrs(), lr=1e-3)
    copt = O.OaAdam(c1.AllParameterPtrs() + c2.AllParameterPtrs(), lr=1e-3)
    replay, _ = RL.OaRlReplayBuffer.Create(RL.OaRlReplayConfig(128, (O_,), (A_,), OaScalarType.Float32))
    g = torch.Generator().manual_seed(0)
    n = 96
    replay.Append(RL.OaRlReplayTransition(M(torch.randn(n, O_, generator=g)), M(torch.rand(n, A_, generator=g) * 2 - 1), M(torch.randn(n, O_, generator=g)),
                                          M(torch.randn(n, generator=g)), M((torch.rand(n, generator=g) < 0.1).to(torch.uint8)),
                                          M(torch.zeros(n, dtype=torch.uint8))))
    trainer, st = RL.OaSacTrainer.Create(actor, c1, c2, t1, t2, aopt, copt, replay, RL.OaSacTrainerConfig(4, 32, A_, 2, (O_,), -1.0, 1.0, 7))
    assert st
    a0 = [p.Data.Tensor().clone() for p in actor.AllParameterPtrs()]
    c0 = [p.Data.Tensor().clone() for p in c1.AllParameterPtrs()]
    while not trainer.IsDone():
        assert trainer.Update()
    m = trainer.Metrics()
    assert m.Update == 4 and math.isfinite(m.ActorLoss) and math.isfinite(m.CriticLoss)
    assert trainer.TrainingLoop().StepCount() == 4 and trainer.ActorTrainingLoop().StepCount() == 4
    assert any(not torch.equal(a, p.Data.Tensor()) for a, p in zip(a0, actor.AllParameterPtrs()))
    assert any(not torch.equal(a, p.Data.Tensor()) for a, p in zip(c0, c1.AllParameterPtrs()))
    assert all(torch.equal(a.Data.Tensor(), b.Data.Tensor()) for a, b in zip(c1.AllParameterPtrs(), t1.AllParameterPtrs()))   # synced at update 4
    wrong, _ = RL.OaRlReplayBuffer.Create(RL.OaRlReplayConfig(128, (O_,), (), OaScalarType.Int32))
    assert not RL.OaSacTrainer.Create(actor, c1, c2, t1, t2, aopt, copt, wrong, RL.OaSacTrainerConfig(4, 32, A_, 2, (O_,)))[1]


def test_public_surface_exposes_rl():
    import oa
    assert oa.OaFnRl.Gae is FR.Gae and oa.OaFnLoss.Ppo is FR.Ppo and oa.OaPpoTrainer is RL.OaPpoTrainer
    assert "OaFnRl" not in oa.UNAVAILABLE and oa.OaRlSpaceKind.Discrete == 1
