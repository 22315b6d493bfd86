"""Mamba-3 variants composed from the SISO core, against plain torch statements differentiated by torch.autograd:
MIMO (R independent SISO states, Source/Private/Oa/Ml/Nn/Mamba3/Mamba3.cpp:193-219), one B / C projection per head
(ngroups == n_heads, Mamba3.cpp:314-317), and the benchmark options (causal depthwise convolution, learned A_log)."""
import pytest
import torch

from oa_b200.core import fn_matrix as F
from oa_b200.core.matrix import OaMatrix
from oa_b200.ml.autograd import OaGradientTape
from oa_b200.ml.nn.mamba3 import OaMamba3Module
from oa_b200.ops import mamba3 as M3


def _make(**kw):
    F.SetRngSeed(3)
    m = OaMamba3Module(16, d_state=8, expand=2, headdim=8, **kw)        # d_inner 32, 4 heads
    g = torch.Generator().manual_seed(5)
    for p in m.AllParameterPtrs():                                      # move every parameter off its symmetric init
        t = p.Tensor()
        t.add_(0.1 * torch.randn(t.shape, generator=g))
    return m


def _oracle(m, x, w):
    """x [B, L, d_model] -> y; `w` maps parameter name -> torch tensor (requires_grad)."""
    B, L, _ = x.shape
    H, P, N, DI, A = m.NHeads, m.HeadDim, m.DState, m.DInner, m.NumRopeAngles
    proj = x.reshape(B * L, -1) @ w["in_proj"].t()
    c = m._columns()
    col = lambda n: proj[:, c[n][0]:c[n][1]]
    if m.ConvWidth > 0:
        lo, hi = c["x"][0], c["C"][1]
        xbc = proj[:, lo:hi].reshape(B, L, hi - lo)
        acc = 0
        for k in range(m.ConvWidth):
            sh = torch.cat((torch.zeros(B, k, hi - lo), xbc[:, :L - k]), 1) if k else xbc
            acc = acc + sh * w["conv_weight"][k]
        proj = torch.cat((proj[:, :lo], torch.nn.functional.silu(acc).reshape(B * L, -1), proj[:, hi:]), 1)
    if m.HasALog:
        lo, hi = c["dd_A"]
        proj = torch.cat((proj[:, :lo], (torch.exp(w["A_log"]) - 1.0).expand(B * L, H), proj[:, hi:]), 1)
    col = lambda n: proj[:, c[n][0]:c[n][1]]
    tail = proj[:, c["dd_dt"][0]:]
    if m.IsMimo:
        d = M3.Mamba3Dims(DI, H, P, N, A, has_z=m.Dims.has_z)
        y = 0
        for r in range(m.MimoRank):
            pr = torch.cat((col("z") * w["mimo_z"][:, r].reshape(-1), col("x") * w["mimo_x"][:, r].reshape(-1),
                            col("B")[:, r * N:(r + 1) * N], col("C")[:, r * N:(r + 1) * N], tail), 1)
            yr = M3.reference_core(pr, w["dt_bias"], w["B_bias"][:, r], w["C_bias"][:, r], w["D"], d, B, L)
            y = y + yr * w["mimo_o"][:, r].reshape(-1)
        z = col("z")
    elif m.NGroups == H:
        d = M3.Mamba3Dims(P, 1, P, N, A, has_z=m.Dims.has_z)
        ys = []
        for h in range(H):
            ph = torch.cat((col("z")[:, h * P:(h + 1) * P], col("x")[:, h * P:(h + 1) * P], col("B")[:, h * N:(h + 1) * N],
                            col("C")[:, h * N:(h + 1) * N], col("dd_dt")[:, h:h + 1], col("dd_A")[:, h:h + 1], col("trap")[:, h:h + 1],
                            col("angle")), 1)
            ys.append(M3.reference_core(ph, w["dt_bias"][:, h:h + 1], w["B_bias"][h:h + 1], w["C_bias"][h:h + 1], w["D"][h:h + 1], d, B, L))
        y = torch.cat(ys, 1)
        z = col("z")
    else:
        y = M3.reference_core(proj, w["dt_bias"], w["B_bias"], w["C_bias"], w["D"], m.Dims, B, L)
        z = col("z")
    if m.IsOutprojNorm:
        yr = y.reshape(-1, P)
        n = yr * torch.rsqrt((yr * yr).mean(-1, keepdim=True) + 1e-5) * torch.nn.functional.silu(z.reshape(-1, P))
        y = n.reshape(B * L, DI) * w["norm_weight"].reshape(-1)
    return (y @ w["out_proj"].t()).reshape(B, L, -1)


CASES = [dict(is_mimo=True, mimo_rank=2), dict(is_mimo=True, mimo_rank=3, is_outproj_norm=True), dict(ngroups=4),
         dict(ngroups=4, is_outproj_norm=True), dict(conv_width=4), dict(a_log=True), dict(conv_width=4, a_log=True, is_outproj_norm=True)]


@pytest.mark.parametrize("kw", CASES, ids=lambda k: ",".join(f"{a}={b}" for a, b in k.items()))
def test_variant_forward_and_gradients_match_torch(kw):
    m = _make(**kw)
    named = m.AllNamedParameterPtrs()
    names, params = [n.Name for n in named], [n.Param for n in named]
    w = {n: p.Tensor().detach().clone().requires_grad_(True) for n, p in zip(names, params)}
    torch.manual_seed(1)
    B, L = 2, 11
    xt = torch.randn(B, L, 16)
    gt = torch.randn(B, L, 16)
    x = OaMatrix(xt.clone()).SetRequiresGrad(True)
    with OaGradientTape() as tape:
        y = m.Forward(x)
        tape.Backward(y, grad=gt.clone())
    xr = xt.clone().requires_grad_(True)
    yr = _oracle(m, xr, w)
    yr.backward(gt)
    assert torch.allclose(y.Tensor(), yr, atol=2e-4, rtol=1e-4), (y.Tensor() - yr).abs().max()
    assert torch.allclose(x.GradTensor(), xr.grad, atol=5e-4, rtol=1e-3), (x.GradTensor() - xr.grad).abs().max()
    for n, p in zip(names, params):
        g, gr = p.Data.GradTensor(), w[n].grad
        assert gr is not None and g is not None, n
        assert torch.allclose(g.reshape(gr.shape), gr, atol=5e-4, rtol=2e-3), (n, (g.reshape(gr.shape) - gr).abs().max())


def test_parameter_shapes_follow_the_reference():
    m = _make(is_mimo=True, mimo_rank=3)
    shapes = {n.Name: tuple(n.Param.Tensor().shape) for n in m.AllNamedParameterPtrs()}
    H, N, P = 4, 8, 8
    assert shapes["in_proj"] == (2 * 32 + 2 * N * 3 + 3 * H + m.NumRopeAngles, 16)
    assert shapes["B_bias"] == (H, 3, N) and shapes["mimo_x"] == (H, 3, P) and shapes["mimo_o"] == (H, 3, P)
    assert list(shapes)[:7] == ["in_proj", "dt_bias", "B_bias", "C_bias", "mimo_x", "mimo_z", "mimo_o"]
    g = _make(ngroups=4)
    assert tuple(g.InProj.Tensor().shape)[0] == 2 * 32 + 2 * N * 4 + 3 * H + g.NumRopeAngles
    with pytest.raises(ValueError):
        OaMamba3Module(16, 8, 2, 8, ngroups=2)
    with pytest.raises(ValueError):
        OaMamba3Module(16, 8, 2, 8, ngroups=4, is_mimo=True)


def test_variant_decode_step_matches_forward():
    m = _make(is_mimo=True, mimo_rank=2)
    torch.manual_seed(2)
    x = torch.randn(2, 6, 16)
    full = m.Forward(OaMatrix(x.clone())).Tensor()
    m.ResetState()
    m.Prefill(OaMatrix(x[:, :4].contiguous()))
    y4 = m.Step(OaMatrix(x[:, 4].contiguous())).Tensor()
    y5 = m.Step(OaMatrix(x[:, 5].contiguous())).Tensor()
    assert torch.allclose(y4, full[:, 4], atol=1e-5) and torch.allclose(y5, full[:, 5], atol=1e-5)
