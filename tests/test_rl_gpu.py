"""RL kernels on the GPU against the CPU (PyTorch) statement of the same ops, and a short PPO run on the device."""
import pytest
import torch

from oa_b200.ops import rl as R

pytestmark = pytest.mark.gpu


def _both(fn, tensors):
    """Runs fn on CPU clones and on CUDA clones of the tensors; returns both tensor lists after the call."""
    cpu = [t.clone() for t in tensors]
    gpu = [t.cuda() for t in tensors]
    fn(*cpu)
    fn(*gpu)
    torch.cuda.synchronize()
    return cpu, [t.cpu() for t in gpu]


def test_cartpole_kernels_match_cpu_path():
    from oa_b200.ops import kernels as K
    E = 1000
    state, done = torch.zeros(E, 4), torch.zeros(E, dtype=torch.uint8)
    steps, episode = torch.zeros(E, dtype=torch.int32), torch.zeros(E, dtype=torch.int32)
    p = R.CartPoleParams(max_steps=9)
    g = torch.Generator().manual_seed(0)
    actions = [torch.randint(0, 2, (E,), generator=g, dtype=torch.int32) for _ in range(30)]

    def run(state, done, steps, episode):
        dev = state.device
        R.cartpole_reset(state, done, steps, episode, 0x1234567890, False)
        obs, rew = torch.zeros(E, 4, device=dev), torch.zeros(E, device=dev)
        term, trunc = torch.zeros(E, dtype=torch.uint8, device=dev), torch.zeros(E, dtype=torch.uint8, device=dev)
        total = torch.zeros(E, device=dev)
        for i, a in enumerate(actions):
            R.cartpole_step(a.to(dev), state, obs, rew, term, trunc, done, steps, p)
            total += rew
            if i % 3 == 2:
                R.cartpole_reset(state, done, steps, episode, 0x1234567890, True)
        steps.copy_(steps + total.to(torch.int32) * 1000)        # fold the reward trace into a compared tensor

    cpu, gpu = _both(run, [state, done, steps, episode])
    assert (cpu[0] - gpu[0]).abs().max() < 1e-4
    for a, b in zip(cpu[1:], gpu[1:]):
        assert torch.equal(a, b)
    assert cpu[3].max() > 0                                      # some lanes went through several episodes
    K.check_status()


def test_gae_replay_rollout_and_loss_kernels_match_cpu_path():
    T, E = 33, 257
    g = torch.Generator().manual_seed(1)
    r, v, nv = (torch.randn(T, E, generator=g) for _ in range(3))
    term, trunc = (torch.rand(T, E, generator=g) < 0.1).to(torch.uint8), (torch.rand(T, E, generator=g) < 0.05).to(torch.uint8)
    cpu, gpu = _both(lambda *a: R.gae(*a, 0.99, 0.95), [r, v, nv, term, trunc, torch.zeros(T, E), torch.zeros(T, E)])
    assert (cpu[5] - gpu[5]).abs().max() < 1e-4 and (cpu[6] - gpu[6]).abs().max() < 1e-4
    # losses
    n = 5000
    a, b, c = 0.5 * torch.randn(n, generator=g), 0.5 * torch.randn(n, generator=g), torch.randn(n, generator=g)
    for bw in (False, True):
        assert (R.ppo_clip(a, b, c, 0.2, bw) - R.ppo_clip(a.cuda(), b.cuda(), c.cuda(), 0.2, bw).cpu()).abs().max() < 1e-5
    nq = torch.randn(n, 6, generator=g)
    tm = (torch.rand(n, generator=g) < 0.2).to(torch.uint8)
    assert (R.dqn_target(a, nq, tm, 0.9) - R.dqn_target(a.cuda(), nq.cuda(), tm.cuda(), 0.9).cpu()).abs().max() < 1e-6
    assert (R.sac_target(a, b, c, a, tm, 0.9, 0.2) - R.sac_target(a.cuda(), b.cuda(), c.cuda(), a.cuda(), tm.cuda(), 0.9, 0.2).cpu()).abs().max() < 1e-6
    # categorical sampling draws the same classes on both paths (ties in the running sum aside)
    logits = torch.randn(4096, 5, generator=g)
    sc, sg = R.sample_categorical(logits, 99), R.sample_categorical(logits.cuda(), 99).cpu()
    assert (sc != sg).float().mean() < 1e-3
    assert torch.equal(R.sample_categorical(logits, 1, greedy=True), R.sample_categorical(logits.cuda(), 1, greedy=True).cpu())
    # replay ring + sampling
    cap, rows, oe, ae = 50, 20, 3, 2
    mk = lambda dev: dict(obs=torch.zeros(cap, oe, device=dev), action=torch.zeros(cap, ae, device=dev), next_obs=torch.zeros(cap, oe, device=dev),
                          reward=torch.zeros(cap, device=dev), term=torch.zeros(cap, dtype=torch.uint8, device=dev),
                          trunc=torch.zeros(cap, dtype=torch.uint8, device=dev))
    sc_, sg_ = mk("cpu"), mk("cuda")
    cursor = 0
    for i in range(4):
        src = dict(obs=torch.randn(rows, oe, generator=g), action=torch.randn(rows, ae, generator=g), next_obs=torch.randn(rows, oe, generator=g),
                   reward=torch.randn(rows, generator=g), term=(torch.rand(rows, generator=g) < 0.3).to(torch.uint8),
                   trunc=(torch.rand(rows, generator=g) < 0.3).to(torch.uint8))
        R.replay_append(src, sc_, cursor, cap)
        R.replay_append({k: t.cuda() for k, t in src.items()}, sg_, cursor, cap)
        cursor = (cursor + rows) % cap
    for k in sc_:
        assert torch.equal(sc_[k], sg_[k].cpu()), k
    B = 64
    mo = lambda dev: dict(obs=torch.zeros(B, oe, device=dev), action=torch.zeros(B, ae, device=dev), next_obs=torch.zeros(B, oe, device=dev),
                          reward=torch.zeros(B, device=dev), term=torch.zeros(B, dtype=torch.uint8, device=dev),
                          trunc=torch.zeros(B, dtype=torch.uint8, device=dev), index=torch.zeros(B, dtype=torch.int32, device=dev))
    oc, og = mo("cpu"), mo("cuda")
    R.replay_sample(sc_, oc, cap, 77)
    R.replay_sample(sg_, og, cap, 77)
    for k in oc:
        assert torch.equal(oc[k], og[k].cpu()), k
    # rollout append
    Tn = 4
    md = lambda dev: dict(obs=torch.zeros(Tn, E, 4, device=dev), action=torch.zeros(Tn, E, dtype=torch.int32, device=dev),
                          reward=torch.zeros(Tn, E, device=dev), value=torch.zeros(Tn, E, device=dev), next_value=torch.zeros(Tn, E, device=dev),
                          logp=torch.zeros(Tn, E, device=dev), term=torch.zeros(Tn, E, dtype=torch.uint8, device=dev),
                          trunc=torch.zeros(Tn, E, dtype=torch.uint8, device=dev), valid=torch.zeros(Tn, E, dtype=torch.uint8, device=dev))
    dc, dg = md("cpu"), md("cuda")
    for slot in (2, 0):
        src = dict(obs=torch.randn(E, 4, generator=g), action=torch.randint(0, 2, (E,), generator=g, dtype=torch.int32),
                   reward=torch.randn(E, generator=g), value=torch.randn(E, generator=g), next_value=torch.randn(E, generator=g),
                   logp=torch.randn(E, generator=g), term=(torch.rand(E, generator=g) < 0.3).to(torch.uint8),
                   trunc=(torch.rand(E, generator=g) < 0.3).to(torch.uint8))
        R.rollout_append(src, dc, slot)
        R.rollout_append({k: t.cuda() for k, t in src.items()}, dg, slot)
    for k in dc:
        assert torch.equal(dc[k], dg[k].cpu()), k


def test_ppo_learns_cartpole_on_device():
    from oa_b200.core import fn_matrix as F
    from oa_b200.core.matrix import OaMatrix
    from oa_b200.ml import optim as O
    from oa_b200.ml import rl as RL
    from oa_b200.ops import kernels as K
    F.SetRngSeed(3)
    E, H = 256, 32
    env = RL.OaCartPoleEnvironment(RL.OaCartPoleConfig(Environments=E, Seed=3))
    assert env.Observation().Tensor().is_cuda
    model, _ = RL.OaCategoricalActorCritic.Create(RL.OaCategoricalActorCriticConfig(4, 2, 64))
    opt = O.OaAdam(model.AllParameterPtrs(), lr=3e-3)
    trainer, st = RL.OaPpoTrainer.Create(model, opt, RL.OaPpoTrainerConfig(20, H, E, 4, (4,), 3))
    assert st
    before, _ = RL.OaFnRl.EvaluateCategorical(env, model, RL.OaRlEvaluationConfig(200, 5))
    env.ResetEnvironment(3)
    while not trainer.IsDone():
        assert trainer.BeginCollection()
        for _ in range(H):
            pol = trainer.Act(OaMatrix(env.Observation().Tensor().clone()))
            tr, st = env.StepEnvironment(pol.Action)
            assert st and trainer.Observe(tr.Observation, tr.NextObservation, tr.Reward, tr.Terminated, tr.Truncated, pol)
            env.ResetCompleted()
        assert trainer.EndCollection()
        while trainer.Phase() == RL.OaRlTrainingPhase.Update and not trainer.IsDone():
            assert trainer.Update()
    after, _ = RL.OaFnRl.EvaluateCategorical(env, model, RL.OaRlEvaluationConfig(200, 5))
    assert after.MeanCompletedReturn > 2.0 * before.MeanCompletedReturn or after.CompletedEpisodes < before.CompletedEpisodes // 4, (before, after)
    K.check_status()
