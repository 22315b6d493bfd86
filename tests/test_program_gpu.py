"""A captured training program must be the step it replaces: five steps of a small model with dropout give the same
losses and weights whether every step runs eagerly or steps 2.. replay the captured graph (fresh dropout masks on every
replay, the ones the eager run draws); steps that freeze host scalars are refused; a step whose recorded structure changed
is not replayed.  Reference: Test/Ml/Nn/TestMoeSystems.cpp:14-92 (replay equals eager), TrainingProgram.cpp:167-324."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(seed=11):
    from oa_b200.core import fn_matrix as F
    from oa_b200.core.types import OaPrecision
    from oa_b200.ml.module import OaModule
    from oa_b200.ml.nn.layers import OaLinear
    from oa_b200.runtime.engine import OaEngineConfig, OaInitComputeEngine
    assert OaInitComputeEngine(OaEngineConfig(Precision=OaPrecision.FP32, DeviceIndex=0))
    F.SetRngSeed(seed)

    class Net(OaModule):
        def __init__(self):
            super().__init__()
            self.A = self.RegisterModule("a", OaLinear(32, 64))
            self.B = self.RegisterModule("b", OaLinear(64, 8))
            self.Extra = False

        def Forward(self, x):
            h = F.Dropout(F.Relu(self.A.Forward(x)), 0.1, True)
            if self.Extra:
                h = F.Scale(h, 1.0)
            return self.B.Forward(h)

    return F, Net()


def _run(program: bool, steps: int = 5, optimizer: str = "adamw", validate_every: int = 0, change_at: int = -1):
    from oa_b200.ml import fn_loss as L
    from oa_b200.ml.autograd import OaGradientTape
    from oa_b200.ml.optim import OaAdamW, OaSGD
    from oa_b200.ml.training import OaItTraining, OaItTrainingConfig
    F, net = _setup()
    opt = OaAdamW(net.AllParameterPtrs(), 1e-2) if optimizer == "adamw" else OaSGD(net.AllParameterPtrs(), 1e-2)
    g = torch.Generator().manual_seed(3)
    xs = [torch.randn(16, 32, generator=g) for _ in range(steps)]
    ys = [torch.randn(16, 8, generator=g) for _ in range(steps)]
    x = F.FromTensor(torch.zeros(16, 32, device="cuda"))
    y = F.FromTensor(torch.zeros(16, 8, device="cuda"))
    k = {"i": 0}

    def prepare():
        x.Tensor().copy_(xs[k["i"]])
        y.Tensor().copy_(ys[k["i"]])
        if k["i"] == change_at:
            net.Extra = True
        k["i"] += 1

    def record():
        opt.ZeroGrad()
        with OaGradientTape() as tape:
            loss = L.Mse(net.Forward(x), y)
            tape.Backward(loss)
        return loss

    tr = OaItTraining(opt, OaItTrainingConfig(TotalSteps=steps, Program=program, ValidateEvery=validate_every))
    losses = []
    while not tr.IsDone():
        losses.append(tr.Step(prepare, record))
    weights = torch.cat([p.Tensor().float().reshape(-1) for p in net.AllParameterPtrs()]).cpu()
    return losses, weights, tr


def test_replayed_steps_equal_eager_steps_with_dropout():
    eager_losses, eager_w, _ = _run(False)
    replay_losses, replay_w, tr = _run(True)
    prog = tr.Program()
    assert prog.IsCaptured() and prog.Replays >= 3
    assert prog.RngCountersPerStep > 0 and "rng-rewrite" in [s for s, _ in prog.StageLog]
    assert prog.StructureHash != 0 and prog.Levels > 0
    assert len(set(round(l, 9) for l in replay_losses)) == len(replay_losses), "every step must see its own batch and mask"
    for a, b in zip(eager_losses, replay_losses):
        assert abs(a - b) <= 1e-6 * max(1.0, abs(a)), (eager_losses, replay_losses)
    assert (eager_w - replay_w).abs().max().item() <= 1e-6


def test_capture_refuses_host_stepped_optimizer():
    losses, _, tr = _run(True, steps=3, optimizer="sgd")
    assert not tr.IsValid()
    assert "launch arguments" in tr.LastStatus.message
    assert not tr.Program().IsCaptured()


def test_changed_step_is_not_replayed():
    losses, _, tr = _run(True, steps=8, validate_every=4, change_at=4)
    # step index 4 was run eagerly, found different from the captured structure, and the program was dropped and re-captured
    assert hasattr(tr, "LastVerify") and not tr.LastVerify
    assert "changed" in tr.LastVerify.message
    assert tr.Program().IsCaptured() and tr.Program().Replays >= 1
    assert all(l == l for l in losses)


def test_accumulated_step_replays_the_micro_step():
    """Four micro-steps per optimizer step, the micro-step captured once and replayed: losses and weights equal the eager
    run (gradient accumulation into the arenas is recorded in its accumulating form; ZeroGrad and the optimizer stay outside)."""
    from oa_b200.ml import fn_loss as L
    from oa_b200.ml.autograd import OaGradientTape
    from oa_b200.ml.optim import OaAdamW
    from oa_b200.ml.training import OaAccumulatedStep

    def run(program: bool):
        F, net = _setup(seed=23)
        opt = OaAdamW(net.AllParameterPtrs(), 1e-2)
        opt.SetGradScale(0.25)
        g = torch.Generator().manual_seed(5)
        xs = [torch.randn(16, 32, generator=g) for _ in range(20)]
        ys = [torch.randn(16, 8, generator=g) for _ in range(20)]
        x = F.FromTensor(torch.zeros(16, 32, device="cuda"))
        y = F.FromTensor(torch.zeros(16, 8, device="cuda"))
        k = {"i": 0}

        def feed():
            x.Tensor().copy_(xs[k["i"]])
            y.Tensor().copy_(ys[k["i"]])
            k["i"] += 1

        def micro():
            with OaGradientTape() as tape:
                loss = L.Mse(net.Forward(x), y)
                tape.Backward(loss)
            return loss

        step = OaAccumulatedStep([opt], micro, accum=4, program=program)
        losses = [step.Run(feed).Item() for _ in range(5)]
        w = torch.cat([p.Tensor().float().reshape(-1) for p in net.AllParameterPtrs()]).cpu()
        return losses, w, step

    eager_l, eager_w, _ = run(False)
    prog_l, prog_w, step = run(True)
    assert step.IsReplaying() and step.Program().Replays >= 4 * 3, step.LastStatus.message
    for a, b in zip(eager_l, prog_l):
        assert abs(a - b) <= 1e-6 * max(1.0, abs(a)), (eager_l, prog_l)
    assert (eager_w - prog_w).abs().max().item() <= 1e-6
