"""Learning-rate schedules, callbacks and the checkpoint manager on the CPU engine."""
import math
import os

import pytest
import torch

from oa_b200.core import fn_matrix as F
from oa_b200.core.matrix import OaMatrix
from oa_b200.ml import autograd as AG
from oa_b200.ml import fn_loss as L
from oa_b200.ml import lr_scheduler as S
from oa_b200.ml.callbacks import (OaCbCheckpoint, OaCbCsvLogger, OaCbEarlyStop, OaCbLrScheduler, OaCbPhase, OaCbProgressBar, OaCbSummary,
                                  OaCbValidation, OaValidationResult)
from oa_b200.ml.checkpoint import OaCheckpointManager, OaCheckpointManagerConfig
from oa_b200.ml.nn.layers import OaLinear
from oa_b200.ml.optim import OaAdam
from oa_b200.ml.training import OaItTraining, OaItTrainingConfig


def test_schedules_match_their_definitions():
    cos = S.OaCosineScheduler(1.0, 0.1, 100)
    assert cos.GetLr(0) == pytest.approx(1.0) and cos.GetLr(50) == pytest.approx(0.55) and cos.GetLr(100) == pytest.approx(0.1)
    warm = S.OaWarmupScheduler(1.0, 10, cos)
    assert warm.GetLr(0) == pytest.approx(0.1) and warm.GetLr(9) == pytest.approx(1.0) and warm.GetLr(10) == pytest.approx(1.0)
    one = S.OaOneCycleScheduler(1.0, 100)
    ref = torch.optim.lr_scheduler.OneCycleLR(torch.optim.SGD([torch.zeros(1, requires_grad=True)], 1.0), 1.0, total_steps=100)
    assert one.GetLr(30) == pytest.approx(1.0) and one.GetLr(0) == pytest.approx(1.0 / 25 / 1e4, rel=1e-3)
    del ref
    cyc = S.OaCyclicScheduler(0.1, 1.0, 10)
    assert cyc.GetLr(0) == pytest.approx(0.1) and cyc.GetLr(10) == pytest.approx(1.0) and cyc.GetLr(20) == pytest.approx(0.1)
    cyc2 = S.OaCyclicScheduler(0.1, 1.0, 10, S.OaCyclicMode.Triangular2)
    assert cyc2.GetLr(30) == pytest.approx(0.1 + 0.9 * 0.5)
    wr = S.OaCosineWarmRestartsScheduler(1.0, 10, 2)
    assert wr.GetLr(0) == pytest.approx(1.0) and wr.GetLr(10) == pytest.approx(1.0) and wr.GetLr(20) == pytest.approx(0.5)
    pl = S.OaReduceOnPlateauScheduler(1.0, 0.5, patience=1)
    for m in (1.0, 1.0, 1.0):
        pl.Step(m)
    assert pl.GetLr(0) == pytest.approx(0.5)
    seq = S.OaSequentialScheduler([S.OaWarmupScheduler(1.0, 5), S.OaCosineScheduler(1.0, 0.0, 10)], [5])
    assert seq.GetLr(4) == pytest.approx(1.0) and seq.GetLr(10) == pytest.approx(0.5)
    lw = S.OaLinearWarmupCosineScheduler(4, 104, 1.0, 0.0)
    assert lw.GetLr(0) == lw.GetLr(1) == pytest.approx(0.25) and lw.GetLr(4) == pytest.approx(1.0) and lw.GetLr(54) == pytest.approx(0.5, abs=0.02)


def _loop(tmp_path, steps=12, spe=4, callbacks=()):
    F.SetRngSeed(0)
    torch.manual_seed(0)
    net = OaLinear(4, 2)
    opt = OaAdam(net.AllParameterPtrs(), 5e-2)
    x, y = torch.randn(8, 4), torch.randn(8, 2)
    tr = OaItTraining(opt, OaItTrainingConfig(TotalSteps=steps, BatchSize=8, StepsPerEpoch=spe))
    for cb in callbacks(net, opt) if callable(callbacks) else callbacks:
        tr.AddCallback(cb)
    while not tr.IsDone():
        opt.ZeroGrad()
        with AG.OaGradientTape() as tape:
            loss = L.Mse(net.Forward(OaMatrix(x)), OaMatrix(y))
            tape.Backward(loss)
        tr.Next(loss)
    tr.Finish()
    return net, opt, tr


def test_callbacks_drive_a_run(tmp_path, capsys):
    csv = str(tmp_path / "log.csv")
    seen = {"val": 0, "phase": []}

    def make(net, opt):
        ph = OaCbPhase()
        ph.AddPhase("warm", 1, 4)
        ph.AddPhase("main", 2, 8)
        ph.SetOnPhaseBegin(lambda i, p: seen["phase"].append(p.Id))

        def ev(tr):
            seen["val"] += 1
            return OaValidationResult(Loss=tr.LastLoss(), Samples=8)

        mgr = OaCheckpointManager(OaCheckpointManagerConfig(Dir=str(tmp_path / "ck"), ModelName="lin", MaxKeep=2))
        seen["mgr"] = mgr
        return [OaCbProgressBar(), OaCbValidation(ev), OaCbCheckpoint(mgr, net, opt, save_every=3, verbose=False),
                OaCbLrScheduler(S.OaCosineScheduler(5e-2, 5e-3, 12), opt), OaCbCsvLogger(csv), OaCbSummary(), ph]

    net, opt, tr = _loop(tmp_path, callbacks=make)
    assert tr.StepCount() == 12 and tr.Epoch() == 3
    assert seen["val"] == 3 and seen["phase"] == ["warm", "main"]
    lines = open(csv).read().strip().split("\n")
    assert len(lines) == 13 and lines[0].startswith("epoch,step,batch_size")
    mgr = seen["mgr"]
    assert os.path.isfile(mgr.GetMasterPath())
    inc = os.listdir(mgr.GetIncrementalDir())
    assert len(inc) == 2 and all(f.startswith("lin_step") for f in inc)            # steps 3, 6, 9 saved, oldest rotated out
    assert opt.Lr() == pytest.approx(S.OaCosineScheduler(5e-2, 5e-3, 12).GetLr(13))
    out = capsys.readouterr().out
    assert "steps 12" in out and "Phase 2/2" in out


def test_early_stop_and_resume(tmp_path):
    stop = OaCbEarlyStop(patience=1, min_delta=10.0)         # nothing improves by 10: stops after the second epoch
    net, opt, tr = _loop(tmp_path, steps=40, spe=4, callbacks=[stop])
    assert stop.ShouldStop() and tr.StepCount() == 8
    mgr = OaCheckpointManager(OaCheckpointManagerConfig(Dir=str(tmp_path / "ck2"), ModelName="lin"))
    assert mgr.SaveIncremental(net, opt, 8, tr.LastLoss())
    F.SetRngSeed(3)
    net2 = OaLinear(4, 2)
    opt2 = OaAdam(net2.AllParameterPtrs(), 1e-3)
    fresh = OaCheckpointManager(OaCheckpointManagerConfig(Dir=str(tmp_path / "ck2"), ModelName="lin"))   # scans the directory
    assert fresh.LoadLatestInto(net2, opt2)
    assert torch.equal(net2.Weight.Tensor(), net.Weight.Tensor()) and opt2.StepCount() == opt.StepCount()
    assert not OaCheckpointManager(OaCheckpointManagerConfig(Dir=str(tmp_path / "none"))).LoadLatestInto(net2, opt2)


def test_training_session_commands_apply_at_step_boundaries():
    import threading
    from oa_b200.ml import training_session as TS
    F.SetRngSeed(0)
    net = OaLinear(4, 2)
    opt = OaAdam(net.AllParameterPtrs(), 1e-2)
    tr = OaItTraining(opt, OaItTrainingConfig(TotalSteps=1000, BatchSize=8))
    done = {"ckpt": 0}
    cfg = TS.OaTrainingSessionConfig(CommandCapacity=4)
    cfg.Handlers.Checkpoint = lambda: (done.__setitem__("ckpt", done["ckpt"] + 1), OaStatus_ok())[1]
    ses = TS.OaTrainingSession(tr, cfg)
    V = TS.OaTrainingValue
    assert ses.RegisterParameter(TS.OaTrainingParameterDesc("lr", TS.OaTrainingParameterClass.Hot, TS.OaTrainingValueKind.Float, 0.0, 1.0,
                                                            lambda: V.FromFloat(opt.Lr()), lambda v: (opt.SetLr(v.Float), OaStatus_ok())[1]))
    assert ses.RegisterParameter(TS.OaTrainingParameterDesc("width", TS.OaTrainingParameterClass.Immutable, TS.OaTrainingValueKind.Integer))
    x, y = torch.randn(8, 4), torch.randn(8, 2)

    def one_step():
        tr.IsDone()
        opt.ZeroGrad()
        with AG.OaGradientTape() as tape:
            loss = L.Mse(net.Forward(OaMatrix(x)), OaMatrix(y))
            tape.Backward(loss)
        tr.Next(loss)
        ses.OnStepCompleted()

    s1, st = ses.SetParameter("lr", V.FromFloat(0.5))
    assert st and opt.Lr() == pytest.approx(1e-2)                 # queued, not applied yet
    ses.SetParameter("lr", V.FromFloat(7.0))                       # out of range
    ses.SetParameter("width", V.FromInteger(3))                    # immutable
    ses.Checkpoint()
    _, full = ses.Pause()
    assert not full and full.code.name == "ResourceExhausted"      # capacity 4
    assert ses.TryBeginStep()
    assert opt.Lr() == pytest.approx(0.5) and done["ckpt"] == 1 and ses.Revision() == 2
    res = ses.TakeResults()
    assert [r.Disposition.name for r in res] == ["Applied", "Rejected", "Rejected", "Applied"]
    assert res[1].Status.code.name == "OutOfRange" and res[2].Status.code.name == "PermissionDenied"
    one_step()
    snap = ses.LatestSnapshot()
    assert snap.Step == 1 and snap.LearningRate == pytest.approx(0.5) and snap.Revision == 2
    # stale expected revision is rejected
    ses.Pause(expected_revision=1)
    assert ses.TryBeginStep() and ses.TakeResults()[0].Status.code.name == "Aborted"
    # pause from another thread, resume later: the loop blocks in WaitBeginStep meanwhile
    ses.Pause()
    assert not ses.TryBeginStep() and ses.State() == TS.OaTrainingState.Paused
    t = threading.Timer(0.1, lambda: ses.Resume())
    t.start()
    assert ses.WaitBeginStep() and ses.State() == TS.OaTrainingState.Running
    ses.Stop()
    assert not ses.WaitBeginStep() and tr.IsDone()
    ses.OnFinished(tr.LastStatus)
    assert ses.State() == TS.OaTrainingState.Completed and not ses.Pause()[1]


def OaStatus_ok():
    from oa_b200.core.types import OaStatus
    return OaStatus.Ok()


def test_context_collects_nodes_and_compiles_them():
    """The nodes of a recorded step go through the native compute graph: the structure hash follows the kernel sequence,
    replay-unsafe marks are collected only while a step is being collected, and a recording context compiles every
    executed interval."""
    from oa_b200.core import fn_matrix as F
    from oa_b200.runtime import engine as RT
    ctx = RT.OaContext.GetDefault()
    ctx.MarkReplayUnsafe("ignored outside a collection")
    ctx.BeginCollect()
    a = F.Ones([4, 4])
    b = F.Add(F.Scale(a, 2.0), a)
    ctx.MarkReplayUnsafe("host scalar")
    nodes, unsafe = ctx.EndCollect()
    assert unsafe == ["host scalar"] and len(nodes) >= 2
    g1, h1 = RT.OaContext.Compile(nodes)
    g2, h2 = RT.OaContext.Compile(nodes)
    g3, h3 = RT.OaContext.Compile(nodes + [("Extra", (), ())])
    assert h1 == h2 != h3 and g1.NumNodes() == len(nodes) and g3.NumNodes() == len(nodes) + 1
    assert not ctx.IsCollecting()
    ctx.SetRecording(True)
    try:
        ctx.Execute()
        F.Add(b, a)
        assert ctx.Execute()
        rep = ctx.LastCompiled()
        assert rep["nodes"] >= 1 and rep["levels"] >= 1 and rep["structure_hash"] != 0
    finally:
        ctx.SetRecording(False)


def test_program_rng_bookkeeping_on_cpu():
    """Without CUDA there is no device state: BeginProgramRng answers None and the host offset is untouched."""
    from oa_b200.core import fn_matrix as F
    F.SetRngSeed(5)
    assert F.BeginProgramRng() is None
    F.AdvanceHostRng(12)
    assert F._rng["offset"] == 12
