"""Vector quantisation and the flow-matching backbone on the CPU engine."""
import math

import pytest
import torch

from oa_b200.core import fn_matrix as F
from oa_b200.core.matrix import OaMatrix
from oa_b200.ml import autograd as AG
from oa_b200.ml.nn import flow as FL
from oa_b200.ml.nn import vq as VQ

M = lambda t: OaMatrix(t)


def test_vq_assign_is_nearest_code_with_lowest_index_on_ties():
    g = torch.Generator().manual_seed(0)
    z, e = torch.randn(50, 8, generator=g), torch.randn(12, 8, generator=g)
    e[7] = e[3]                                                           # a duplicated code: ties go to the lower index
    r = VQ.VqAssign(M(z), M(e))
    d = ((z[:, None, :] - e[None]) ** 2).sum(-1)
    assert torch.equal(r.Idx.Tensor().long(), d.argmin(1)) and 7 not in r.Idx.Tensor().tolist()
    assert torch.equal(r.Zq.Tensor(), e[d.argmin(1)])


def test_vq_ema_update_matches_definition_and_revives_dead_codes():
    g = torch.Generator().manual_seed(1)
    n, d, k = 40, 4, 6
    z = torch.randn(n, d, generator=g)
    idx = torch.randint(0, 4, (n,), generator=g, dtype=torch.int32)        # codes 4 and 5 receive nothing
    es, cs, cb = torch.randn(k, d, generator=g), torch.full((k,), 2.0), torch.zeros(k, d)
    cs[5] = 0.5                                                           # decays below the dead threshold
    es0, cs0 = es.clone(), cs.clone()
    VQ.VqEmaUpdate(M(z), M(idx), M(es), M(cs), M(cb), 0.9, 1e-5, 0.5, 3, False)
    for c in range(5):
        sel = idx == c
        nk = 0.9 * cs0[c] + 0.1 * sel.sum()
        mk = 0.9 * es0[c] + 0.1 * z[sel].sum(0)
        assert abs(cs[c] - nk) < 1e-6 and (es[c] - mk).abs().max() < 1e-6 and (cb[c] - mk / nk).abs().max() < 1e-6
    row = z[VQ._revival_row(5, 3, n)]
    assert cs[5] == 1.0 and torch.equal(cb[5], row) and torch.equal(es[5], row)
    cb2 = torch.zeros(k, d)
    VQ.VqEmaUpdate(M(z), M(idx), M(es0.clone()), M(cs0.clone()), M(cb2), 0.9, 1e-5, 0.0, 3, True)
    assert (cb2.square().mean(1).sqrt() - 1.0).abs().max() < 1e-5          # unit-RMS rows


def test_vector_quantizer_straight_through_and_checkpoint(tmp_path):
    F.SetRngSeed(4)
    vq = VQ.OaVectorQuantizer(VQ.OaVectorQuantizerConfig(NumCodes=16, CodeDim=8, CommitBeta=0.25))
    g = torch.Generator().manual_seed(2)
    lat = torch.randn(64, 8, generator=g)
    vq.Seed(M(lat))
    top = lat.square().sum(1).argsort(descending=True, stable=True)[:16]
    assert torch.equal(vq.Codebook().Tensor(), lat[top])
    ze = M(lat[:32].clone())
    ze.SetRequiresGrad(True)
    tape = AG.OaGradientTape()
    r = vq.Quantize(ze)
    loss = F.Add(F.Sum(F.Mul(r.Quantized, r.Quantized)), r.CommitLoss)
    tape.Backward(loss)
    tape.Close()
    zq = vq.Codebook().Tensor()[r.Idx.Tensor().long()]
    assert torch.allclose(r.Quantized.Tensor(), zq, atol=1e-6)                      # forward value is the code
    want = 2 * zq + 0.25 * 2 * (lat[:32] - zq) / zq.numel()                         # gradient passes straight to z_e
    assert (ze.GradTensor() - want).abs().max() < 1e-5
    assert abs(r.CommitLoss.Item() - 0.25 * ((lat[:32] - zq) ** 2).mean().item()) < 1e-6
    assert torch.equal(vq.Lookup(r.Idx).Tensor(), zq)
    before = vq.Codebook().Tensor().clone()
    vq.EmaUpdate(ze, r.Idx)
    assert not torch.equal(before, vq.Codebook().Tensor()) and vq.EmaStep_ == 1
    path = str(tmp_path / "vq.oam")
    assert vq.Save(path)
    other = VQ.OaVectorQuantizer(VQ.OaVectorQuantizerConfig(NumCodes=16, CodeDim=8))
    assert other.Load(path) and torch.equal(other.Codebook().Tensor(), vq.Codebook().Tensor())
    assert torch.equal(other.ClusterSize_.Tensor(), vq.ClusterSize_.Tensor())


def test_residual_vq_reduces_error_with_depth():
    F.SetRngSeed(5)
    g = torch.Generator().manual_seed(3)
    lat = torch.randn(256, 8, generator=g)
    rvq = VQ.OaResidualVectorQuantizer(VQ.OaVectorQuantizerConfig(NumCodes=32, CodeDim=8, EmaDecay=0.5), 3)
    rvq.Seed(M(lat))
    for _ in range(12):                       # EMA steps act as k-means iterations on each level's residual
        rvq.EmaUpdate(rvq.Quantize(M(lat)))
    r = rvq.Quantize(M(lat))
    assert len(r.Idx) == 3 and len(r.Residuals) == 3 and rvq.NumLevels() == 3
    errs = [(lat - rvq.Lookup(r.Idx[:q + 1]).Tensor()).square().mean().item() for q in range(3)]
    assert errs[0] > errs[1] > errs[2]
    assert torch.allclose(rvq.Lookup(r.Idx).Tensor(), r.Quantized.Tensor(), atol=1e-5)
    rvq.EmaUpdate(r)
    assert all(rvq.Level(q).EmaStep_ == 13 for q in range(3))
    with pytest.raises(ValueError):
        rvq.Lookup([])


def test_time_embedding_formula():
    emb = FL.OaFlowTimeEmbedding(8, 100.0, 10.0)
    t = torch.tensor([0.0, 0.25, 1.0])
    out = emb.Forward(M(t)).Tensor()
    f = torch.tensor([10.0 * math.exp(-math.log(100.0) * i / 4) for i in range(4)])
    want = torch.cat((torch.sin(t[:, None] * f), torch.cos(t[:, None] * f)), 1)
    assert out.shape == (3, 8) and (out - want).abs().max() < 1e-5
    with pytest.raises(ValueError):
        FL.OaFlowTimeEmbedding(7)
    with pytest.raises(ValueError):
        emb.Forward(M(torch.zeros(3, 2)))


def _ref_block(x, blk, cond, mask, B, S, H):
    """Plain PyTorch statement of the conditioned bidirectional block."""
    D = x.shape[1]
    lin = lambda l, t: t @ l.Weight.Tensor().t() + (l.Bias.Tensor() if l.Bias else 0)
    mod = lin(blk.AdaptiveModulation, cond).repeat_interleave(S, 0)
    sh_a, sc_a, g_a, sh_f, sc_f, g_f = mod.split(D, 1)
    ln = lambda n, t: torch.nn.functional.layer_norm(t, (D,), n.Weight.Tensor(), n.Bias.Tensor(), 1e-5)
    h = ln(blk.LnAttn, x) * (1 + sc_a) + sh_a
    a = blk.Attention
    q, k, v = (lin(l, h).reshape(B, S, H, D // H).transpose(1, 2) for l in (a.QProj, a.KProj, a.VProj))
    sc = q @ k.transpose(-1, -2) / math.sqrt(D // H)
    if mask is not None:
        sc = sc + ((mask.reshape(B, 1, 1, S) - 1.0) * 1e4)
    o = (torch.softmax(sc, -1) @ v).transpose(1, 2).reshape(B * S, D)
    x = x + lin(a.OutProj, o) * g_a
    h = ln(blk.LnFfn, x) * (1 + sc_f) + sh_f
    return x + lin(blk.Ffn2, torch.nn.functional.gelu(lin(blk.Ffn1, h), approximate="tanh")) * g_f


def test_flow_transformer_conditioned_masked_matches_reference_math():
    F.SetRngSeed(7)
    B, S, D, H = 2, 6, 16, 4
    net = FL.OaFlowTransformer(FL.OaFlowTransformerConfig(D, 32, S, 2, H))
    g = torch.Generator().manual_seed(4)
    for i in range(2):          # AdaLN-Zero starts as the identity: give the modulation real weights for the comparison
        net.Block(i).AdaptiveModulation.Weight.Data.Tensor().copy_(0.2 * torch.randn(6 * D, D, generator=g))
        net.Block(i).AdaptiveModulation.Bias.Data.Tensor().copy_(0.2 * torch.randn(6 * D, generator=g))
    x, cond = torch.randn(B, S, D, generator=g), torch.randn(B, D, generator=g)
    mask = torch.ones(B, S)
    mask[1, 4:] = 0
    out = net.ForwardConditioned(M(x), M(cond), M(mask)).Tensor()
    ref = x.reshape(B * S, D)
    for i in range(2):
        ref = _ref_block(ref, net.Block(i), cond, mask, B, S, H)
    on = net.OutputNorm_
    ref = torch.nn.functional.layer_norm(ref, (D,), on.Weight.Tensor(), on.Bias.Tensor(), 1e-5).reshape(B, S, D)
    assert out.shape == (B, S, D) and (out - ref).abs().max() < 2e-4
    # masked keys do not influence kept positions
    x2 = x.clone()
    x2[1, 4:] += 5.0
    out2 = net.ForwardConditioned(M(x2), M(cond), M(mask)).Tensor()
    assert (out2[1, :4] - out[1, :4]).abs().max() < 1e-3 and (out2[0] - out[0]).abs().max() < 1e-6
    # attention is bidirectional: a late token changes early outputs
    x3 = x.clone()
    x3[0, 5, 0] += 3.0
    assert (net.Forward(M(x3)).Tensor()[0, 0] - net.Forward(M(x)).Tensor()[0, 0]).abs().max() > 1e-5
    with pytest.raises(ValueError):
        net.ForwardConditioned(M(x), M(torch.randn(B, D + 1)))
    with pytest.raises(ValueError):
        FL.OaFlowTransformer(FL.OaFlowTransformerConfig(10, 32, S, 2, 4))


def test_flow_denoiser_trains_and_guides():
    from oa_b200.ml import optim as O
    F.SetRngSeed(8)
    B, S, I, C, D = 4, 5, 3, 6, 16
    net = FL.OaFlowDenoiser(FL.OaFlowDenoiserConfig(I, C, FL.OaFlowTransformerConfig(D, 32, S, 2, 4), ConditionDropoutP=0.25))
    g = torch.Generator().manual_seed(5)
    x, t, c = torch.randn(B, S, I, generator=g), torch.rand(B, generator=g), torch.randn(B, C, generator=g)
    target = torch.randn(B, S, I, generator=g)
    opt = O.OaAdam(net.AllParameterPtrs(), lr=3e-3)
    losses = []
    from oa_b200.ml import fn_loss as L
    for _ in range(30):
        opt.ZeroGrad()
        tape = AG.OaGradientTape()
        out = net.ForwardConditioned(M(x), M(t), M(c))
        loss = L.Mse(out, M(target))
        tape.Backward(loss)
        tape.Close()
        opt.Step()
        losses.append(loss.Item())
    assert losses[-1] < 0.7 * losses[0]
    assert net.Backbone().Block(0).AdaptiveModulation.Weight.Data.Tensor().abs().max() > 0      # the zero-init modulation learned
    net.Eval()
    cond = net.ForwardConditioned(M(x), M(t), M(c)).Tensor()
    unc = net.ForwardConditioned(M(x), M(t)).Tensor()
    gd = net.ForwardGuided(M(x), M(t), M(c), 2.5).Tensor()
    assert (gd - (unc + 2.5 * (cond - unc))).abs().max() < 1e-5
    assert net.Forward(M(x)).Tensor().shape == (B, S, I) and not net.IsMoe()
