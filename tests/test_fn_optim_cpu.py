"""OaFnOptim against the reference's CPU statements of the optimizer kernels (Test/Ml/Optim/TestOptimKernels.cpp:19-75:
CpuAdam / CpuAdamW with bias correction and decoupled decay) and the SgdMomentum / ClipGradNorm contracts."""
import math

import torch

import oa
from oa_b200.core import fn_matrix as F
from oa_b200.ml import fn_optim as O


def _cpu_adamw(w, g, m, v, lr, b1, b2, eps, wd, step):
    w = w - lr * wd * w
    m = b1 * m + (1 - b1) * g
    v = b2 * v + (1 - b2) * g * g
    mh, vh = m / (1 - b1 ** step), v / (1 - b2 ** step)
    return w - lr * mh / (vh.sqrt() + eps), m, v


def test_adamw_step_matches_cpu_reference_over_steps():
    torch.manual_seed(0)
    n = 1000
    w0, m0, v0 = torch.randn(n), torch.zeros(n), torch.zeros(n)
    w, m, v = F.FromTensor(w0.clone()), F.FromTensor(m0.clone()), F.FromTensor(v0.clone())
    wr, mr, vr = w0.clone(), m0.clone(), v0.clone()
    for step in range(1, 6):
        g = torch.randn(n)
        O.AdamWStep(w, m, v, F.FromTensor(g), 1e-2, 0.9, 0.999, 1e-8, 0.1, step)
        wr, mr, vr = _cpu_adamw(wr, g, mr, vr, 1e-2, 0.9, 0.999, 1e-8, 0.1, step)
    assert torch.allclose(w.Tensor(), wr, atol=1e-6) and torch.allclose(m.Tensor(), mr, atol=1e-7) and torch.allclose(v.Tensor(), vr, atol=1e-7)


def test_graph_variants_follow_the_device_state():
    torch.manual_seed(1)
    n = 64
    w0 = torch.randn(n)
    state = O.MakeAdamWState(0, 1e-2, 0.9, 0.999, 1e-8, 0.0)
    sets = [O.OaAdamWParamSet(F.FromTensor(w0.clone()), F.Zeros([n]), F.Zeros([n]), F.FromTensor(torch.ones(n))) for _ in range(3)]
    wr, mr, vr = w0.clone(), torch.zeros(n), torch.zeros(n)
    for step in range(1, 4):
        O.AdamWAdvanceGraphState(state)
        O.AdamWStepManyGraph(sets, state)
        wr, mr, vr = _cpu_adamw(wr, torch.ones(n), mr, vr, 1e-2, 0.9, 0.999, 1e-8, 0.0, step)
    assert float(state.Tensor()[0]) == 3.0
    for s in sets:
        assert torch.allclose(s.Param.Tensor(), wr, atol=1e-6)
    # a learning rate written into the state is what the next step uses (no launch argument involved)
    state.Tensor()[1] = 0.0
    before = sets[0].Param.Tensor().clone()
    O.AdamWAdvanceGraphState(state)
    O.AdamWStepGraph(sets[0].Param, sets[0].M, sets[0].V, sets[0].Grad, state)
    assert torch.equal(sets[0].Param.Tensor(), before)


def test_sgd_momentum_contract():
    w, mom, g = F.FromTensor(torch.tensor([1.0, -2.0])), F.Zeros([2]), F.FromTensor(torch.tensor([0.5, 0.5]))
    O.SgdStep(w, mom, g, 0.1, 0.9, 0.01)          # m = 0.9*0 + g; w -= lr*m + wd*w
    assert torch.allclose(w.Tensor(), torch.tensor([1.0 - 0.05 - 0.01, -2.0 - 0.05 + 0.02]), atol=1e-6)
    O.SgdStep(w, None, g, 0.1, 0.0, 0.0)
    assert torch.allclose(w.Tensor(), torch.tensor([0.94 - 0.05, -2.03 - 0.05]), atol=1e-6)


def test_clip_grad_norm_scales_all_gradients_by_one_coefficient():
    a, b = F.FromTensor(torch.full((10,), 3.0)), F.FromTensor(torch.full((6,), 4.0))
    total = math.sqrt(10 * 9 + 6 * 16)
    coef = O.ClipGradNorm([a, None, b], 1.0, None, F.Zeros([16]))
    assert abs(float(coef.Tensor()[0]) - 1.0 / total) < 1e-5
    assert abs(math.sqrt(float((a.Tensor() ** 2).sum() + (b.Tensor() ** 2).sum())) - 1.0) < 1e-4
    c = F.FromTensor(torch.full((4,), 0.1))
    assert float(O.ClipGradNorm([c], 1.0).Tensor()[0]) == 1.0 and torch.allclose(c.Tensor(), torch.full((4,), 0.1))


def test_muon_step_orthogonalises_matrix_updates():
    torch.manual_seed(2)
    w, mom = F.FromTensor(torch.zeros(8, 16)), F.Zeros([8 * 16])
    O.MuonStep(w, mom, F.FromTensor(torch.randn(8, 16)), 0.1, 0.95, 0.0)
    u = w.Tensor() / w.Tensor().norm() * math.sqrt(8)
    sv = torch.linalg.svdvals(u)
    assert sv.max() / sv.min() < 2.5, "the update must be close to a scaled orthogonal matrix"
    v, mv = F.FromTensor(torch.ones(5)), F.Zeros([5])
    O.MuonStep(v, mv, F.FromTensor(torch.ones(5)), 0.1, 0.5, 0.0)
    assert torch.allclose(v.Tensor(), torch.full((5,), 1.0 - 0.1 * (0.5 + 0.5 * 0.5)), atol=1e-6)


def test_surface_exports_the_namespace():
    assert set(oa.OaFnOptim.__all__) >= {"AdamWStep", "AdamWAdvanceGraphState", "AdamWStepGraph", "AdamWStepMany", "AdamWStepManyGraph",
                                         "SgdStep", "MuonStep", "ClipGradNorm"}
