"""Row compaction / scatter, accuracy counters, stochastic rounding, int8 product and the composite functions: CPU
definitions against plain PyTorch; the CUDA kernels against the CPU definitions."""
import pytest
import torch

from oa_b200.core import fn_matrix as F
from oa_b200.core.matrix import OaMatrix
from oa_b200.ml import autograd as AG


def _m(t, device="cpu"):
    return OaMatrix(t.to(device))


def _compact_suite(device):
    g = torch.Generator().manual_seed(0)
    x = torch.randn(37, 5, generator=g)
    mask = (torch.rand(37, generator=g) > 0.6).float()
    sel = torch.nonzero(mask).reshape(-1)
    r = F.CompactRows(_m(x, device), _m(mask, device))
    n = int(r.Count.Tensor()[0])
    assert n == sel.numel() and torch.equal(r.RowMap.Tensor()[:n].cpu().long(), sel)
    assert torch.equal(r.Values.Tensor()[:n].cpu(), x[sel]) and float(r.Values.Tensor()[n:].abs().sum()) == 0
    assert r.DispatchArgs.Tensor().cpu().tolist() == [(n * 5 + 255) // 256, 1, 1]
    back = F.CompactRowsBwd(r.Values, r.RowMap, r.Count, [37, 5]).Tensor().cpu()
    assert torch.equal(back, x * mask[:, None])
    base = torch.full((37, 5), 7.0)
    sc = F.ScatterRows(_m(base, device), r.Values, r).Tensor().cpu()
    assert torch.equal(sc, torch.where(mask[:, None] != 0, x, base))
    gsrc = F.ScatterRowsBwdSource(_m(x, device), r.RowMap, r.Count).Tensor().cpu()
    assert torch.equal(gsrc[:n], x[sel]) and float(gsrc[n:].abs().sum()) == 0
    idx = torch.randint(0, 6, (37,), generator=g, dtype=torch.int32)
    add = F.ScatterAddRows(_m(x, device), _m(idx, device), 6).Tensor().cpu()
    assert torch.allclose(add, torch.zeros(6, 5).index_add_(0, idx.long(), x), atol=1e-5)
    # nothing selected / everything selected, and a bf16 matrix wider than one warp
    empty = F.CompactRows(_m(x, device), _m(torch.zeros(37), device))
    assert int(empty.Count.Tensor()[0]) == 0 and float(empty.Values.Tensor().abs().sum()) == 0
    xb = torch.randn(2100, 70, generator=g).bfloat16()
    mb = (torch.rand(2100, generator=g) > 0.3).float()
    rb = F.CompactRows(_m(xb, device), _m(mb, device))
    nb = int(rb.Count.Tensor()[0])
    assert nb == int(mb.sum()) and torch.equal(rb.Values.Tensor()[:nb].cpu(), xb[torch.nonzero(mb).reshape(-1)])
    # rows whose byte width is a multiple of 16 take the 16-byte vector path on the GPU
    for shape, dt in (((300, 64), torch.bfloat16), ((50, 8), torch.float32), ((129, 4), torch.float32), ((40000, 8), torch.float32)):   # the last spans three scan blocks
        xv = torch.randn(*shape, generator=g).to(dt)
        mv = (torch.rand(shape[0], generator=g) > 0.4).float()
        sv = torch.nonzero(mv).reshape(-1)
        rv = F.CompactRows(_m(xv, device), _m(mv, device))
        nv = int(rv.Count.Tensor()[0])
        assert nv == sv.numel() and torch.equal(rv.Values.Tensor()[:nv].cpu(), xv[sv]) and float(rv.Values.Tensor()[nv:].float().abs().sum()) == 0
        basev = torch.ones(*shape).to(dt)
        scv = F.ScatterRows(_m(basev, device), rv.Values, rv).Tensor().cpu()
        assert torch.equal(scv, torch.where(mv[:, None] != 0, xv, basev))
        gv = F.ScatterRowsBwdSource(_m(xv, device), rv.RowMap, rv.Count).Tensor().cpu()
        assert torch.equal(gv[:nv], xv[sv]) and float(gv[nv:].float().abs().sum()) == 0
    # gradients through the tape: d/dx sum(w * compact(x)) and through ScatterRows
    xm = _m(x.clone(), device); xm.SetRequiresGrad(True)
    w = torch.randn(37, 5, generator=g)
    with AG.OaGradientTape() as tape:
        loss = F.Sum(F.Mul(F.CompactRows(xm, _m(mask, device)).Values, _m(w, device)))
    tape.Backward(loss)
    want = torch.zeros(37, 5); want[sel] = w[:n]
    assert torch.allclose(xm.GradMatrix().Tensor().cpu(), want)
    sm, bm = _m(x.clone(), device), _m(base.clone(), device)
    sm.SetRequiresGrad(True); bm.SetRequiresGrad(True)
    with AG.OaGradientTape() as tape:
        loss = F.Sum(F.Mul(F.ScatterRows(bm, sm, r.RowMap, r.Count), _m(w, device)))
    tape.Backward(loss)
    assert torch.allclose(bm.GradMatrix().Tensor().cpu(), w * (1 - mask[:, None]))
    gs = sm.GradMatrix().Tensor().cpu()
    assert torch.allclose(gs[:n], w[sel]) and float(gs[n:].abs().sum()) == 0


def _accuracy_suite(device):
    g = torch.Generator().manual_seed(1)
    logits = torch.randn(300, 33, generator=g)
    logits[5, 7] = logits[5, 20] = 9.0                       # tie: the lower index wins
    labels = logits.argmax(-1).to(torch.int32)
    labels[::3] = (labels[::3] + 1) % 33
    labels[5] = 7
    want = int((logits.argmax(-1).to(torch.int32) == labels).sum())
    assert int(F.CategoricalAccuracyCount(_m(logits, device), _m(labels, device)).Tensor()[0]) == want
    mask = (torch.rand(300, generator=g) > 0.5).float()
    wantm = int(((logits.argmax(-1).to(torch.int32) == labels) & (mask != 0)).sum())
    assert int(F.MaskedCategoricalAccuracyCount(_m(logits, device), _m(labels, device), _m(mask, device)).Tensor()[0]) == wantm
    lb = logits.bfloat16()
    assert int(F.CategoricalAccuracyCount(_m(lb, device), _m(labels, device)).Tensor()[0]) == int((lb.float().argmax(-1).to(torch.int32) == labels).sum())


def _sr_suite(device):
    x = torch.tensor([1.0, 1.0 + 2 ** -9, -3.14159, 0.0, float("inf"), 1e-30, 65504.0])
    lo = x.view(torch.int32).bitwise_and(-65536).view(torch.float32)                      # truncation towards zero
    hi = torch.nextafter(lo.bfloat16(), torch.where(x >= 0, torch.tensor(float("inf")), torch.tensor(-float("inf"))).bfloat16()).float()
    acc = torch.zeros_like(x, dtype=torch.float64)
    trials = 400
    for s in range(trials):
        r = F.SrRoundBf16(_m(x, device), seed=s).Tensor().float().cpu()
        assert r.dtype == torch.float32 and bool(((r == lo) | (r == hi) | torch.isinf(x)).all())
        acc += torch.nan_to_num(r.double(), posinf=0.0)
    mean = acc / trials
    exact = lo == x
    assert torch.equal(mean[exact & ~torch.isinf(x)].float(), x[exact & ~torch.isinf(x)])   # representable values never move
    frac = ((x - lo) / (hi - lo))[1].item()                                               # 1 + 2^-9 sits 1/4 of the way up
    up = ((mean[1] - lo[1]) / (hi[1] - lo[1])).item()
    assert frac == pytest.approx(0.25) and abs(up - 0.25) < 0.08
    a = F.SrRoundBf16(_m(torch.randn(1000, generator=torch.Generator().manual_seed(2)), device), seed=5).Tensor().cpu()
    b = F.SrRoundBf16(_m(torch.randn(1000, generator=torch.Generator().manual_seed(2)), "cpu"), seed=5).Tensor()
    assert torch.equal(a, b)                                                               # same bits on both paths


def _int8_suite(device):
    g = torch.Generator().manual_seed(3)
    for M, Nn, Kd in ((17, 9, 64), (5, 33, 31), (40, 40, 4)):
        a = torch.randint(-128, 128, (M, Kd), generator=g, dtype=torch.int8)
        b = torch.randint(-128, 128, (Nn, Kd), generator=g, dtype=torch.int8)
        ref = a.to(torch.int64) @ b.to(torch.int64).T
        out = F.GemmInt8(_m(a, device), _m(b, device)).Tensor().cpu()
        assert out.dtype == torch.int32 and torch.equal(out.to(torch.int64), ref)
        rs, cs = torch.rand(M, generator=g), torch.rand(Nn, generator=g)
        sc = F.GemmInt8(_m(a, device), _m(b, device), _m(rs, device), _m(cs, device)).Tensor().cpu()
        assert torch.allclose(sc, ref.float() * rs[:, None] * cs[None, :], rtol=1e-5)
    with pytest.raises(ValueError):
        F.GemmInt8(_m(torch.zeros(2, 3), device), _m(torch.zeros(2, 3, dtype=torch.int8), device))


def test_compact_scatter_cpu(): _compact_suite("cpu")
def test_accuracy_counters_cpu(): _accuracy_suite("cpu")
def test_stochastic_rounding_cpu(): _sr_suite("cpu")
def test_int8_product_cpu(): _int8_suite("cpu")


@pytest.mark.gpu
def test_compact_scatter_cuda(): _compact_suite("cuda")


@pytest.mark.gpu
def test_accuracy_counters_cuda(): _accuracy_suite("cuda")


@pytest.mark.gpu
def test_stochastic_rounding_cuda(): _sr_suite("cuda")


@pytest.mark.gpu
def test_int8_product_cuda(): _int8_suite("cuda")


def test_composite_functions():
    g = torch.Generator().manual_seed(4)
    x, w = torch.randn(6, 4, generator=g), torch.randn(5, 4, generator=g)
    dy = torch.randn(6, 5, generator=g)
    y = torch.relu(x @ w.T)
    assert torch.allclose(F.LinearReluBwdData(OaMatrix(dy), OaMatrix(y), OaMatrix(w)).Tensor(), (dy * (y > 0)) @ w, atol=1e-5)
    pre = torch.randn(6, 4, generator=g)
    assert torch.allclose(F.LinearDataReluBwd(OaMatrix(dy), OaMatrix(w), OaMatrix(pre)).Tensor(), (dy @ w) * (pre > 0), atol=1e-5)
    assert torch.allclose(F.SumDim(OaMatrix(x), 1).Tensor().reshape(-1), x.sum(1), atol=1e-5)
    assert torch.allclose(F.ReduceCols(OaMatrix(x)).Tensor().reshape(-1), x.sum(0), atol=1e-5)
    assert torch.allclose(F.MeanBwd(OaMatrix(torch.tensor([2.4])), [3, 4]).Tensor(), torch.full((3, 4), 0.2))
    mx = x.max(-1).values
    gm = F.MaxBwd(OaMatrix(x), OaMatrix(mx), OaMatrix(torch.arange(6.0))).Tensor()
    assert torch.equal(gm.sum(-1), torch.arange(6.0)) and torch.equal(gm.ne(0).sum(-1)[1:], torch.ones(5, dtype=torch.long)) and bool((gm[x != mx[:, None]] == 0).all())
    xl = x.clone().requires_grad_(True)
    torch.log_softmax(xl, -1).backward(dy[:, :4])
    assert torch.allclose(F.LogSoftmaxBwd(OaMatrix(torch.log_softmax(x, -1)), OaMatrix(dy[:, :4].contiguous())).Tensor(), xl.grad, atol=1e-5)
    d = OaMatrix(torch.zeros(3, 4))
    F.CopyAtOffset(d, OaMatrix(torch.tensor([1.0, 2.0, 3.0])), 5)
    assert d.Tensor().reshape(-1).tolist()[4:9] == [0.0, 1.0, 2.0, 3.0, 0.0]
    F.MatrixCopyRegion(d, OaMatrix(x), 1, 2, src_row=4, src_col=1, rows=2, cols=2)
    assert torch.equal(d.Tensor()[1:3, 2:4], x[4:6, 1:3])
    with pytest.raises(ValueError):
        F.MatrixCopyRegion(d, OaMatrix(x), 2, 2, rows=2, cols=2)
    b3 = torch.randn(2, 3, 5, generator=g)
    assert torch.equal(F.TransposeBatched(OaMatrix(b3)).Tensor(), b3.transpose(1, 2))
    a3 = torch.randn(2, 5, 3, generator=g).transpose(1, 2)                 # strided view [2, 3, 5]
    assert torch.allclose(F.GemmStrided(OaMatrix(a3), OaMatrix(b3.transpose(1, 2))).Tensor(), a3 @ b3.transpose(1, 2), atol=1e-5)
    p, t = torch.randn(8, 3, generator=g), torch.randn(8, 3, generator=g)
    m = torch.tensor([1, 0, 1, 1, 0, 0, 1, 1.0])
    assert float(F.MaskedMse(OaMatrix(p), OaMatrix(t), OaMatrix(m)).Tensor()) == pytest.approx(float((((p - t) ** 2) * m[:, None]).sum() / (m.sum() * 3)), rel=1e-5)
    assert float(F.SmoothL1Mean(OaMatrix(p), OaMatrix(t), 0.5).Tensor()) == pytest.approx(float(torch.nn.functional.smooth_l1_loss(p, t, beta=0.5)), rel=1e-5)
    vp, vt = p.view(2, 4, 3), t.view(2, 4, 3)
    want = torch.nn.functional.smooth_l1_loss(vp[:, 1:] - vp[:, :-1], vt[:, 1:] - vt[:, :-1])
    assert float(F.VelSmoothL1(OaMatrix(p), OaMatrix(t), 2, 4).Tensor()) == pytest.approx(float(want), rel=1e-5)
