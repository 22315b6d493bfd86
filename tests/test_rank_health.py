"""Heartbeats, failure detection between steps and host-side fault injection: unit checks on a dictionary store with a
manual clock, then three CPU processes over a TCP store where one rank exits / raises / goes silent at a chosen step."""
import os
import subprocess
import sys

import pytest

from oa_b200.core.types import OaStatusCode
from oa_b200.parallel.health import OaFault, OaFaultInjector, OaFaultKind, OaRankFailure, OaRankMonitor

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class DictStore:
    def __init__(self): self.d = {}
    def set(self, k, v): self.d[k] = bytes(v)
    def get(self, k): return self.d[k]
    def check(self, keys): return all(k in self.d for k in keys)


def test_monitor_on_a_manual_clock():
    store, now = DictStore(), [100.0]
    clock = lambda: now[0]
    m0, m1, m2 = (OaRankMonitor(store, r, 3, timeout_s=5.0, clock=clock) for r in range(3))
    assert m0.Check().IsOk()                                  # nobody has published yet, but the timeout has not run out
    for m in (m0, m1, m2):
        m.Beat(0)
    now[0] += 3; m0.Beat(1); m1.Beat(1)
    assert m0.Check().IsOk() and m0.SlowestPeer().Rank == 2
    now[0] += 3                                               # rank 2 silent for 6 s
    st = m0.Check()
    assert st.code == OaStatusCode.Unavailable and "[2]" in st.message and m1.Check().code == OaStatusCode.Unavailable
    with pytest.raises(OaRankFailure) as e:
        m0.Guard(2)
    assert e.value.Ranks == [2]
    m2.Leave(1)                                               # a rank that says goodbye is not a failure
    m1.Beat(2)
    assert m0.Check().IsOk()
    m1.ReportFailure(2)                                       # a rank that reports its own failure is one at once
    assert m0.Check().code == OaStatusCode.Unavailable and "[1]" in m0.Check().message
    late = OaRankMonitor(DictStore(), 0, 2, timeout_s=1.0, clock=clock)
    now[0] += 2
    assert late.Check().code == OaStatusCode.Unavailable      # a peer that never showed up within the timeout
    with pytest.raises(OaRankFailure) as e:                   # Guard names exactly the ranks Check found, also a never-seen one
        late.Guard(0)
    assert e.value.Ranks == [1] and "[1]" in str(e.value)


@pytest.mark.parametrize("bad", ["1", "a:2", "1:2:explode", "1:2:delay:-1", "1:2:raise:0:9"])
def test_fault_injector_rejects_malformed_items(monkeypatch, bad):
    monkeypatch.setenv("OA_FAULT", "0:1:raise," + bad)
    with pytest.raises(ValueError) as e:
        OaFaultInjector.FromEnv()
    assert "OA_FAULT" in str(e.value) and bad in str(e.value)


def test_fault_injector_schedule(monkeypatch):
    monkeypatch.setenv("OA_FAULT", "1:3:raise,2:5:delay:0.01,0:2:silence")
    inj = OaFaultInjector.FromEnv()
    assert [(f.Rank, f.Step, f.Kind) for f in inj.Faults] == [(1, 3, "raise"), (2, 5, "delay"), (0, 2, "silence")] and inj.Faults[1].Seconds == 0.01
    store = DictStore()
    m = OaRankMonitor(store, 1, 2)
    inj.AtStep(1, 2, m)                                       # nothing scheduled
    with pytest.raises(RuntimeError):
        inj.AtStep(1, 3, m)
    assert OaRankMonitor(store, 0, 2).Check().code == OaStatusCode.Unavailable     # the raise was reported first
    inj.AtStep(2, 5)
    m0 = OaRankMonitor(store, 0, 2)
    inj.AtStep(0, 2)
    inj.Beat(m0, 2)
    assert inj.Silenced and "oa/health/0" not in store.d


_WORKER = """
import os, sys, time, datetime
sys.path.insert(0, {root!r})
import torch.distributed as dist
from oa_b200.parallel.health import OaFault, OaFaultInjector, OaRankFailure, OaRankMonitor
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
store = dist.TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]), world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=20))
monitor = OaRankMonitor(store, rank, world, timeout_s=1.5)
assert monitor.WaitForPeers(30.0).IsOk()
inj = OaFaultInjector([OaFault(2, 3, {kind!r})])
done = 0
try:
    for step in range(40):
        inj.AtStep(rank, step, monitor)       # between steps: nothing in flight
        inj.Beat(monitor, step)
        st = monitor.Check()
        if not st.IsOk():
            print(f"rank {{rank}} stops before step {{step}}: {{st.message}}", flush=True)
            break
        time.sleep(0.1)                       # the step itself
        done += 1
    else:
        print(f"rank {{rank}} finished all steps", flush=True)
except RuntimeError as e:
    print(f"rank {{rank}} raised: {{e}}", flush=True)
print(f"rank {{rank}} done {{done}}", flush=True)
if rank == 0:
    time.sleep(1.5)                           # the store lives in rank 0: let the others read it to the end
"""


@pytest.mark.parametrize("kind", ["exit", "raise", "silence"])
def test_survivors_stop_between_steps(kind, tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(_WORKER.format(root=ROOT, kind=kind))
    port = 29700 + (os.getpid() + {"exit": 0, "raise": 1, "silence": 2}[kind]) % 200
    procs = []
    for r in range(3):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="3", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=60)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outs.append(out)
    for r in (0, 1):                                         # the survivors notice within a few steps and leave cleanly
        assert procs[r].returncode == 0, outs[r]
        assert f"rank {r} stops before step" in outs[r] and "[2]" in outs[r], outs[r]
        done = int(outs[r].split(f"rank {r} done ")[1].split()[0])
        assert 3 <= done <= 25, outs[r]
    if kind == "exit":
        assert procs[2].returncode == 17
    elif kind == "raise":
        assert "rank 2 raised: injected failure" in outs[2] and "rank 2 done 3" in outs[2]
    else:
        assert procs[2].returncode == 0 and "rank 2" in outs[2]


def test_training_loop_stops_when_a_peer_falls_silent():
    import torch
    from oa_b200.core import fn_matrix as F
    from oa_b200.core.matrix import OaMatrix
    from oa_b200.ml import autograd as AG
    from oa_b200.ml import fn_loss as L
    from oa_b200.ml.nn.layers import OaLinear
    from oa_b200.ml.optim import OaAdamW
    from oa_b200.ml.training import OaItTraining, OaItTrainingConfig
    store, now = DictStore(), [0.0]
    clock = lambda: now[0]
    me, peer = OaRankMonitor(store, 0, 2, timeout_s=2.0, clock=clock), OaRankMonitor(store, 1, 2, timeout_s=2.0, clock=clock)
    model = OaLinear(4, 3)
    opt = OaAdamW(model.AllParameterPtrs(), 1e-2)
    training = OaItTraining(opt, OaItTrainingConfig(TotalSteps=10, BatchSize=5, SequenceLength=1, Program=False))
    training.SetRankMonitor(me)
    x, y = OaMatrix(torch.randn(5, 4)), OaMatrix(torch.randint(0, 3, (5,), dtype=torch.int32))

    def record():
        opt.ZeroGrad()
        with AG.OaGradientTape() as tape:
            loss = L.CrossEntropy(model.Forward(x), y)
        tape.Backward(loss)
        return loss

    steps = 0
    while not training.IsDone():
        if steps < 3:
            peer.Beat(steps)                    # the peer is alive for three steps, then falls silent
        now[0] += 1.0
        training.Step(None, record)
        steps += 1
    training.Finish()
    assert training.StepCount() == 4 and not training.LastStatus.IsOk() and "[1]" in training.LastStatus.message
    assert training.LastStatus.code == OaStatusCode.Unavailable
