"""Framework behaviour on the CPU engine: optimizers against torch.optim, module save/load (.oam) with integrity
rejection, sparse MoE against its dense statement, recurrent scans against per-step cells, the training loop
(char LM overfit, save -> reload -> same logits -> same greedy text) and metrics."""
import os
import struct

import pytest
import torch

from oa_b200.core import fn_matrix as F
from oa_b200.core.matrix import OaMatrix
from oa_b200.io.oam import OamHash, OamModel
from oa_b200.ml import autograd as AG
from oa_b200.ml import fn_loss as L
from oa_b200.ml.module import OaModule
from oa_b200.ml.nn.layers import OaLinear, OaSequential, OaRelu
from oa_b200.ml.optim import OaAdam, OaAdamW, OaSGD
from oa_b200.models import OaGptConfig, OaGptModel


# ------------------------------------------------------------------------------------------------------- optimizers
def _problem(seed=0):
    torch.manual_seed(seed)
    F.SetRngSeed(seed)
    net = OaSequential(OaLinear(6, 8), OaRelu(), OaLinear(8, 3))
    x, y = torch.randn(16, 6), torch.randn(16, 3)
    ref = torch.nn.Sequential(torch.nn.Linear(6, 8), torch.nn.ReLU(), torch.nn.Linear(8, 3))
    ps = net.AllParameterPtrs()
    with torch.no_grad():
        for p, r in zip(ps, ref.parameters()):
            r.copy_(p.Tensor())
    return net, ref, x, y


@pytest.mark.parametrize("kind", ["adam", "adamw", "sgd", "sgd_momentum"])
def test_optimizer_matches_torch(kind):
    net, ref, x, y = _problem()
    ps = net.AllParameterPtrs()
    if kind == "adam":
        opt, topt = OaAdam(ps, 1e-2), torch.optim.Adam(ref.parameters(), 1e-2)
    elif kind == "adamw":
        opt, topt = OaAdamW(ps, 1e-2, weight_decay=0.1), torch.optim.AdamW(ref.parameters(), 1e-2, weight_decay=0.1)
    elif kind == "sgd":
        opt, topt = OaSGD(ps, 0.05), torch.optim.SGD(ref.parameters(), 0.05)
    else:
        opt, topt = OaSGD(ps, 0.05, momentum=0.9), torch.optim.SGD(ref.parameters(), 0.05, momentum=0.9)
    for _ in range(5):
        opt.ZeroGrad()
        with AG.OaGradientTape() as tape:
            loss = L.Mse(net.Forward(OaMatrix(x)), OaMatrix(y))
            tape.Backward(loss)
        opt.Step()
        topt.zero_grad()
        tl = torch.nn.functional.mse_loss(ref(x), y)
        tl.backward()
        topt.step()
        assert abs(loss.Item() - tl.item()) < 1e-4
    for p, r in zip(net.AllParameterPtrs(), ref.parameters()):
        assert (p.Tensor() - r).abs().max().item() < 1e-4


def test_optimizer_state_round_trip(tmp_path):
    net, _, x, y = _problem()
    opt = OaAdamW(net.AllParameterPtrs(), 1e-2)

    def step(n, o):
        o.ZeroGrad()
        with AG.OaGradientTape() as tape:
            loss = L.Mse(n.Forward(OaMatrix(x)), OaMatrix(y))
            tape.Backward(loss)
        o.Step()
        return loss.Item()

    for _ in range(3):
        step(net, opt)
    path = str(tmp_path / "ck.oam")
    assert net.Save(path, opt)
    net2, _, _, _ = _problem(seed=5)
    opt2 = OaAdamW(net2.AllParameterPtrs(), 1e-2)
    assert net2.Load(path, opt2)
    a, b = step(net, opt), step(net2, opt2)
    assert abs(a - b) < 1e-6
    for p, q in zip(net.AllParameterPtrs(), net2.AllParameterPtrs()):
        assert torch.equal(p.Tensor(), q.Tensor())


# ------------------------------------------------------------------------------------------------------- .oam files
def _save_small(tmp_path):
    F.SetRngSeed(3)
    net = OaSequential(OaLinear(4, 5), OaRelu(), OaLinear(5, 2))
    path = str(tmp_path / "m.oam")
    assert net.Save(path)
    return net, path


def test_oam_header_and_hash(tmp_path):
    net, path = _save_small(tmp_path)
    raw = open(path, "rb").read()
    assert raw[:4] == b"OAM\x00" or raw[:3] == b"OAM"
    assert OamHash(b"") == 0xCBF29CE484222325                     # FNV-1a offset basis
    assert OamHash(b"a") == 0xAF63DC4C8601EC8C
    m, st = OamModel.Load(path)
    assert st and m is not None
    names = [w.Name for w in m.Weights()]
    named = net.AllNamedParameterPtrs()
    assert names == [n.Name for n in named]
    for w, n in zip(m.Weights(), named):
        assert torch.equal(w.ToTorch().reshape(n.Param.Tensor().shape), n.Param.Tensor().cpu())


def test_oam_rejects_corruption(tmp_path):
    _, path = _save_small(tmp_path)
    raw = bytearray(open(path, "rb").read())
    # a flipped payload bit, a truncated file and a wrong magic must all fail to load
    flipped = bytearray(raw)
    flipped[-5] ^= 0x10
    cases = {"flip": bytes(flipped), "trunc": bytes(raw[: len(raw) - 7]), "magic": b"XXXX" + bytes(raw[4:]), "empty": b""}
    for name, blob in cases.items():
        p = str(tmp_path / f"{name}.oam")
        open(p, "wb").write(blob)
        m, st = OamModel.Load(p)
        assert m is None and not st, name


def test_load_validates_before_mutating(tmp_path):
    _, path = _save_small(tmp_path)
    F.SetRngSeed(9)
    other = OaSequential(OaLinear(4, 6), OaRelu(), OaLinear(6, 2))       # different hidden width
    before = [p.Tensor().clone() for p in other.AllParameterPtrs()]
    st = other.Load(path)
    assert not st
    for p, b in zip(other.AllParameterPtrs(), before):
        assert torch.equal(p.Tensor(), b)                                    # nothing was overwritten


def test_save_is_atomic(tmp_path):
    net, path = _save_small(tmp_path)
    assert net.Save(path)                                                    # overwrite in place
    assert [f for f in os.listdir(tmp_path) if f.endswith(".tmp")] == []
    assert OamModel.Load(path)[0].HasWeights()


# ------------------------------------------------------------------------------------------------------------- MoE
def test_moe_sparse_matches_dense_statement():
    from oa_b200.ml.nn.moe import OaMoE
    F.SetRngSeed(1)
    layer = OaMoE(16, 24, 4, 2, num_shared_experts=1)
    layer.SetAuxLossAlpha(0.01)
    x = torch.randn(10, 16)
    xm = OaMatrix(x.clone()).SetRequiresGrad(True)
    with AG.OaGradientTape() as tape:
        y = layer.Forward(xm)
        tape.Backward(F.Add(F.Sum(F.Mul(y, y)), layer.AuxLoss()))
    sparse_y, sparse_dx = y.Tensor().clone(), xm.GradTensor().clone()
    grads = [p.Grad().Tensor().clone() for p in layer.AllParameterPtrs()]
    for p in layer.AllParameterPtrs():
        p.Data.ZeroGrad()
    xd = OaMatrix(x.clone()).SetRequiresGrad(True)
    layer.SparseExecution = False                 # every expert on every token, gated by the masked probabilities
    with AG.OaGradientTape() as tape:
        yd = layer.Forward(xd)
        tape.Backward(F.Add(F.Sum(F.Mul(yd, yd)), layer.AuxLoss()))
    assert (sparse_y - yd.Tensor()).abs().max().item() < 1e-4
    assert (sparse_dx - xd.GradTensor()).abs().max().item() < 1e-3
    for g, p in zip(grads, layer.AllParameterPtrs()):
        assert (g - p.Grad().Tensor()).abs().max().item() < 1e-3 * max(1.0, g.abs().max().item()), p.Name


# ------------------------------------------------------------------------------------------------------- recurrent
@pytest.mark.parametrize("kind", ["gru", "rnn"])
def test_recurrent_scan_matches_cell_steps(kind, monkeypatch):
    from oa_b200.ml.nn.recurrent import OaGru, OaRnn
    cls = OaGru if kind == "gru" else OaRnn
    flag = "OA_DISABLE_GRU_SCAN" if kind == "gru" else "OA_DISABLE_RNN_SCAN"
    F.SetRngSeed(2)
    net = cls(5, 7, num_layers=2)
    x = torch.randn(3, 6, 5)

    def run():
        for p in net.AllParameterPtrs():
            p.Data.ZeroGrad()
        xm = OaMatrix(x.clone()).SetRequiresGrad(True)
        with AG.OaGradientTape() as tape:
            out = net.Forward(xm)
            tape.Backward(F.Sum(F.Mul(out, out)))
        return out.Tensor().clone(), xm.GradTensor().clone(), [p.Grad().Tensor().clone() for p in net.AllParameterPtrs()]

    o1, dx1, g1 = run()
    monkeypatch.setenv(flag, "1")
    o2, dx2, g2 = run()
    assert (o1 - o2).abs().max().item() < 1e-5
    assert (dx1 - dx2).abs().max().item() < 1e-4
    for a, b in zip(g1, g2):
        assert (a - b).abs().max().item() < 1e-4


# ---------------------------------------------------------------------------------------------------- training loop
CORPUS = (b"to be, or not to be, that is the question: whether 'tis nobler in the mind to suffer the slings and arrows of "
          b"outrageous fortune, or to take arms against a sea of troubles and by opposing end them. ")


def _greedy(model, prompt: bytes, n: int, window: int) -> bytes:
    out = bytearray(prompt)
    with AG.OaGradNo():
        for _ in range(n):
            ctx = bytes(out[-window:])
            ids = OaMatrix(torch.tensor([list(ctx)], dtype=torch.int32))
            logits = model.Forward(ids).Tensor()
            out.append(int(logits[len(ctx) - 1].argmax()))
    return bytes(out)


def test_char_lm_overfits_and_round_trips(tmp_path):
    from oa_b200.ml.training import OaItTraining, OaItTrainingConfig
    F.SetRngSeed(20260714)
    cfg = OaGptConfig(256, 32, 1, 2, 64, 16, "layer", "gelu", 0.0, True, 1e-5, 0.02)
    model = OaGptModel(cfg)
    opt = OaAdam(model.AllParameterPtrs(), 3e-3)
    data = torch.tensor(list(CORPUS), dtype=torch.int32)
    B, S = 8, cfg.SeqLen
    gen = torch.Generator().manual_seed(0)
    training = OaItTraining(opt, OaItTrainingConfig(TotalSteps=150, BatchSize=B, SequenceLength=S, Program=False))
    first = last = None
    while not training.IsDone():
        starts = torch.randint(0, len(data) - S - 1, (B,), generator=gen)
        ids = torch.stack([data[s:s + S] for s in starts])
        tg = torch.stack([data[s + 1:s + S + 1] for s in starts])
        opt.ZeroGrad()
        with AG.OaGradientTape() as tape:
            loss = model.Loss(OaMatrix(ids), OaMatrix(tg))
            tape.Backward(loss)
        last = training.Next(loss)
        first = first if first is not None else last
    training.Finish()
    assert last < 0.6 * first, (first, last)
    path = str(tmp_path / "lm.oam")
    assert model.Save(path, opt)
    F.SetRngSeed(1)
    again = OaGptModel(cfg)
    assert again.Load(path)
    ids = OaMatrix(torch.tensor([list(CORPUS[:S])], dtype=torch.int32))
    with AG.OaGradNo():
        a, b = model.Forward(ids).Tensor(), again.Forward(ids).Tensor()
    assert torch.equal(a, b)
    assert _greedy(model, b"to be", 12, S) == _greedy(again, b"to be", 12, S)


def test_metrics():
    from oa_b200.ml.metric import OaFnMetric, OaMetricAccuracy, OaMetricLoss
    logits = OaMatrix(torch.tensor([[2.0, 1.0], [0.0, 3.0], [5.0, 1.0]]))
    tg = OaMatrix(torch.tensor([0, 1, 1], dtype=torch.int32))
    assert abs(OaFnMetric.Accuracy(logits, tg) - 2.0 / 3.0) < 1e-6
    m = OaMetricAccuracy()
    m.UpdateFrom(logits, tg)
    assert abs(m.Value() - 2.0 / 3.0) < 1e-6
    ml = OaMetricLoss()
    ml.Update(1.0)
    ml.Update(3.0)
    assert abs(ml.Value() - 2.0) < 1e-6 and ml.Count() == 2 and ml.Last() == 3.0
