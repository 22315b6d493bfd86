"""Differentiable OaFnMatrix / OaFnLoss operations against torch.autograd on the CPU engine (forward values and every
input gradient), plus tape mechanics: fan-out accumulation, view-shaped upstream gradients, no-grad scopes."""
import pytest
import torch

from oa_b200.core import fn_matrix as F
from oa_b200.core.matrix import OaMatrix
from oa_b200.ml import autograd as AG
from oa_b200.ml import fn_loss as L


def _check(oa_fn, torch_fn, shapes, tol=1e-4, positive=False, seed=0, int_inputs=()):
    g = torch.Generator().manual_seed(seed)
    raw = []
    for s in shapes:
        t = torch.randn(*s, generator=g)
        if positive:
            t = t.abs() + 0.5
        raw.append(t)
    mats = [OaMatrix(t.clone()).SetRequiresGrad(True) for t in raw]
    leaves = [t.clone().requires_grad_(True) for t in raw]
    with AG.OaGradientTape() as tape:
        out = oa_fn(*mats, *[OaMatrix(i) for i in int_inputs])
        up = torch.randn(out.Tensor().shape, generator=g)
        tape.Backward(out, grad=up.clone())
    ref = torch_fn(*leaves, *int_inputs)
    if ref.dim() == 0:
        ref = ref.reshape(1)                      # full reductions and losses are [1] matrices
    assert out.Tensor().shape == ref.shape, (out.Tensor().shape, ref.shape)
    assert (out.Tensor().float() - ref).abs().max().item() <= tol * max(1.0, ref.abs().max().item())
    ref.backward(up)
    for i, (m, l) in enumerate(zip(mats, leaves)):
        got = m.GradTensor()
        want = l.grad if l.grad is not None else torch.zeros_like(l)
        assert got is not None, f"input {i} got no gradient"
        assert (got.float() - want).abs().max().item() <= tol * max(1.0, want.abs().max().item()), f"gradient of input {i}"


UNARY = [
    ("Neg", F.Neg, torch.neg, False), ("Abs", F.Abs, torch.abs, False), ("Log", F.Log, torch.log, True),
    ("Exp", F.Exp, torch.exp, False), ("Sqrt", F.Sqrt, torch.sqrt, True), ("Sin", F.Sin, torch.sin, False),
    ("Cos", F.Cos, torch.cos, False), ("Reciprocal", F.Reciprocal, torch.reciprocal, True),
    ("Square", F.Square, torch.square, False), ("Relu", F.Relu, torch.relu, False),
    ("Gelu", F.Gelu, lambda x: torch.nn.functional.gelu(x, approximate="tanh"), False),
    ("Silu", F.Silu, torch.nn.functional.silu, False), ("Tanh", F.Tanh, torch.tanh, False),
    ("Sigmoid", F.Sigmoid, torch.sigmoid, False), ("Softplus", F.Softplus, torch.nn.functional.softplus, False),
    ("LeakyRelu", lambda m: F.LeakyRelu(m, 0.1), lambda x: torch.nn.functional.leaky_relu(x, 0.1), False),
    ("Elu", F.Elu, torch.nn.functional.elu, False), ("Mish", F.Mish, torch.nn.functional.mish, False),
    ("Scale", lambda m: F.Scale(m, 2.5), lambda x: x * 2.5, False),
    ("AddScalar", lambda m: F.AddScalar(m, 1.5), lambda x: x + 1.5, False),
    ("SubScalar", lambda m: F.SubScalar(m, 1.5), lambda x: x - 1.5, False),
    ("DivScalar", lambda m: F.DivScalar(m, 4.0), lambda x: x / 4.0, False),
    ("Pow", lambda m: F.Pow(m, 3.0), lambda x: x ** 3.0, True),
    ("ClampMax", lambda m: F.ClampMax(m, 0.3), lambda x: torch.clamp(x, max=0.3), False),
    ("ClampMin", lambda m: F.ClampMin(m, -0.3), lambda x: torch.clamp(x, min=-0.3), False),
]


@pytest.mark.parametrize("name,oa_fn,torch_fn,positive", UNARY, ids=[u[0] for u in UNARY])
def test_unary(name, oa_fn, torch_fn, positive):
    _check(oa_fn, torch_fn, [(5, 7)], positive=positive)


BINARY = [("Add", F.Add, torch.add), ("Sub", F.Sub, torch.sub), ("Mul", F.Mul, torch.mul), ("Div", F.Div, torch.div)]


@pytest.mark.parametrize("name,oa_fn,torch_fn", BINARY, ids=[b[0] for b in BINARY])
@pytest.mark.parametrize("shapes", [[(4, 6), (4, 6)], [(4, 6), (6,)], [(3, 4, 6), (1, 4, 1)]])
def test_binary_broadcast(name, oa_fn, torch_fn, shapes):
    _check(oa_fn, torch_fn, shapes, positive=(name == "Div"))


def test_matrix_operators():
    _check(lambda a, b: (a + b) * a - b / 2.0 + 1.0, lambda a, b: (a + b) * a - b / 2.0 + 1.0, [(3, 5), (3, 5)])


def test_shape_ops():
    _check(lambda m: F.Reshape(m, [6, 4]), lambda x: x.reshape(6, 4), [(2, 3, 4)])
    _check(lambda m: F.Transpose(m, 0, 1), lambda x: x.transpose(0, 1), [(3, 5)])
    _check(lambda m: F.Permute(m, [2, 0, 1]), lambda x: x.permute(2, 0, 1), [(2, 3, 4)])
    _check(lambda m: F.Slice(m, 1, 1, 3), lambda x: x[:, 1:3], [(4, 5)])
    _check(lambda a, b: F.Concat([a, b], 1), lambda a, b: torch.cat([a, b], 1), [(3, 2), (3, 4)])
    _check(lambda m: F.Split(m, [2, 3], -1)[1], lambda x: x.split([2, 3], -1)[1], [(4, 5)])
    _check(lambda m: F.RepeatInterleave(m, 3, 0), lambda x: x.repeat_interleave(3, 0), [(2, 5)])


def test_reductions():
    _check(lambda m: F.Sum(m), lambda x: x.sum(), [(4, 5)])
    _check(lambda m: F.Sum(m, 1), lambda x: x.sum(1), [(4, 5)])
    _check(lambda m: F.Mean(m), lambda x: x.mean(), [(4, 5)])
    _check(lambda m: F.Mean(m, 0), lambda x: x.mean(0), [(4, 5)])
    _check(lambda m: F.Max(m, -1), lambda x: x.max(-1).values, [(4, 5)])
    _check(lambda m: F.Softmax(m), lambda x: torch.softmax(x, -1), [(4, 9)])
    _check(lambda m: F.LogSoftmax(m), lambda x: torch.log_softmax(x, -1), [(4, 9)])


def test_softmax_scaled_masked():
    mask = F.CausalMask(6)
    tm = mask.Tensor().float()
    _check(lambda s: F.SoftmaxScaledMasked(s, 0.5, mask), lambda s: torch.softmax(s * 0.5 + tm, -1), [(3, 6, 6)])


def test_indexing():
    ids = torch.tensor([[1, 0, 3], [2, 2, 1]], dtype=torch.int32)
    _check(lambda t, i: F.Gather(t, i), lambda t, i: t[i.long().reshape(-1)], [(5, 4)], int_inputs=(ids,))
    idx = torch.tensor([2, 0, 1, 2], dtype=torch.int32)
    _check(lambda m, i: F.GatherLastDim(m, i), lambda m, i: m.gather(-1, i.long().unsqueeze(-1)), [(4, 3)],
           int_inputs=(idx,))
    pos = torch.tensor([[0, 1, 2], [0, 1, 2]], dtype=torch.int32)
    _check(lambda t, p, i: F.Embedding(t, i, p, 3), lambda t, p, i: (t[i.long()] + p[:3].unsqueeze(0)).reshape(6, 4), [(5, 4), (8, 4)],
           int_inputs=(ids,))
    del pos


def test_linear_family():
    _check(lambda a, b: F.MatMulNt(a, b), lambda a, b: a @ b.t(), [(6, 5), (4, 5)])
    _check(lambda x, w, b: F.Linear(x, w, b), lambda x, w, b: x @ w.t() + b, [(6, 5), (4, 5), (4,)])
    _check(lambda x, w, b: F.LinearGelu(x, w, b), lambda x, w, b: torch.nn.functional.gelu(x @ w.t() + b, approximate="tanh"),
           [(6, 5), (4, 5), (4,)])
    _check(lambda x, w, b: F.LinearRelu(x, w, b), lambda x, w, b: torch.relu(x @ w.t() + b), [(6, 5), (4, 5), (4,)])
    _check(lambda x, w0, w1: F.PackedLinear2(x, w0, w1), lambda x, w0, w1: torch.cat([x @ w0.t(), x @ w1.t()], -1),
           [(6, 5), (4, 5), (3, 5)])
    _check(lambda a, b: F.Bmm(a, b), lambda a, b: a @ b, [(3, 4, 5), (3, 5, 2)])


def test_norms_and_gates():
    rms = lambda x, w, eps: x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w
    _check(lambda x, w: F.RmsNorm(x, w, 1e-6), lambda x, w: rms(x, w, 1e-6), [(5, 8), (8,)])
    _check(lambda x, w, b: F.LayerNorm(x, w, b, 1e-5), lambda x, w, b: torch.nn.functional.layer_norm(x, (8,), w, b, 1e-5),
           [(5, 8), (8,), (8,)])
    silu = torch.nn.functional.silu
    _check(lambda x, w, b, z: F.RmsNormGated(x, w, b, z, 1e-6), lambda x, w, b, z: (rms(x, w, 1e-6) + b) * silu(z),
           [(5, 8), (8,), (8,), (5, 8)])
    _check(lambda x, w, b, z: F.RmsNormGated(x, w, b, z, 1e-6, False), lambda x, w, b, z: rms(x * silu(z), w, 1e-6) + b,
           [(5, 8), (8,), (8,), (5, 8)])
    _check(lambda gu: F.Swiglu(gu), lambda gu: torch.nn.functional.silu(gu[:, :4]) * gu[:, 4:], [(5, 8)])
    _check(lambda a, b: F.SiluMul(a, b), lambda a, b: torch.nn.functional.silu(a) * b, [(5, 4), (5, 4)])


def test_norm_backward_folds_the_residual_stream_gradient(monkeypatch):
    """x feeds a residual add and an RmsNorm (and through a second block again): the gradient that x has collected through
    the residual stream is handed to the norm's backward, which returns the sum, and no separate add is launched."""
    from oa_b200.ops import kernels as K
    rms = lambda x, w, eps: x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w
    adds = []
    real = K.binary
    monkeypatch.setattr(K, "binary", lambda op, *a, **k: (adds.append(op), real(op, *a, **k))[1])

    def block(h, c, w0, w1):                   # two pre-norm residual blocks on an intermediate (non-leaf) stream
        h = F.Mul(h, c)
        h = F.Add(h, F.Mul(F.RmsNorm(h, w0, 1e-6), F.RmsNorm(h, w0, 1e-6)))
        return F.Add(h, F.RmsNorm(h, w1, 1e-6))

    def ref(h, c, w0, w1):
        h = h * c
        h = h + rms(h, w0, 1e-6) * rms(h, w0, 1e-6)
        return h + rms(h, w1, 1e-6)

    _check(block, ref, [(5, 8), (5, 8), (8,), (8,)])
    # "add" appears for the two forward Adds only, none for the gradient fan-in of the stream
    assert adds.count("add") == 2, adds


def _rope_ref(x, heads, hd, seq, theta=10000.0):
    rows = x.shape[0]
    xv = x.reshape(rows // seq, seq, heads, hd)
    half = hd // 2
    inv = theta ** (-torch.arange(half, dtype=torch.float32) * 2.0 / hd)
    ang = torch.arange(seq, dtype=torch.float32)[:, None] * inv[None, :]
    c, s = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]
    x1, x2 = xv[..., :half], xv[..., half:]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1).reshape(rows, heads * hd)


def test_rope_and_attention():
    B, S, H, hd = 2, 5, 2, 8
    _check(lambda x: F.RoPE(x, H, hd, S), lambda x: _rope_ref(x, H, hd, S), [(B * S, H * hd)])

    def ref(q, k, v):
        sh = lambda t: t.reshape(B, S, H, hd).transpose(1, 2)
        o = torch.nn.functional.scaled_dot_product_attention(sh(q), sh(k), sh(v), is_causal=True)
        return o.transpose(1, 2).reshape(B * S, H * hd)

    _check(lambda q, k, v: F.FlashAttentionCausal(q, k, v, B, S, H), ref, [(B * S, H * hd)] * 3)


def test_losses():
    tg = torch.tensor([1, 0, 3, 2, 2], dtype=torch.int32)
    _check(lambda lg, t: L.CrossEntropy(lg, t), lambda lg, t: torch.nn.functional.cross_entropy(lg, t.long()), [(5, 4)], int_inputs=(tg,))
    tgi = torch.tensor([1, -100, 3, 2, -100], dtype=torch.int32)
    _check(lambda lg, t: L.CrossEntropy(lg, t),
           lambda lg, t: torch.nn.functional.cross_entropy(lg, t.long(), ignore_index=-100, reduction="sum") / 5, [(5, 4)], int_inputs=(tgi,))
    mk = torch.tensor([1, 0, 1, 1, 0], dtype=torch.int32)
    _check(lambda lg, t, m: L.MaskedCrossEntropy(lg, t, m),
           lambda lg, t, m: torch.nn.functional.cross_entropy(lg[m.bool()], t[m.bool()].long()), [(5, 4)], int_inputs=(tg, mk))
    t = torch.randn(5, 4)
    _check(lambda p: L.Mse(p, OaMatrix(t)), lambda p: torch.nn.functional.mse_loss(p, t), [(5, 4)])
    _check(lambda p: L.L1(p, OaMatrix(t)), lambda p: torch.nn.functional.l1_loss(p, t), [(5, 4)])
    _check(lambda p: L.SmoothL1(p, OaMatrix(t), 0.7), lambda p: torch.nn.functional.smooth_l1_loss(p, t, beta=0.7), [(5, 4)])
    y = (torch.rand(5, 4) > 0.5).float()
    _check(lambda p: L.Bce(F.Sigmoid(p), OaMatrix(y)), lambda p: torch.nn.functional.binary_cross_entropy(torch.sigmoid(p), y), [(5, 4)])


def test_fan_out_and_no_grad():
    a = OaMatrix(torch.randn(3, 4)).SetRequiresGrad(True)
    with AG.OaGradientTape() as tape:
        b = F.Exp(a)
        c = F.Add(F.Mul(b, b), F.Sum(b, 1).Reshape([3, 1]))      # b is used three times
        tape.Backward(F.Sum(c))
    t = a.Tensor().clone().requires_grad_(True)
    tb = t.exp()
    (tb * tb + tb.sum(1, keepdim=True)).sum().backward()
    assert (a.GradTensor() - t.grad).abs().max().item() < 1e-4
    with AG.OaGradNo():
        d = F.Exp(a)
    assert not d.HasGradFn()
    assert not AG.IsEnabled()


def test_gradient_accumulates_across_backward_calls_until_zeroed():
    a = OaMatrix(torch.ones(2, 2)).SetRequiresGrad(True)
    for _ in range(2):
        with AG.OaGradientTape() as tape:
            tape.Backward(F.Sum(F.Scale(a, 3.0)))
    assert torch.allclose(a.GradTensor(), torch.full((2, 2), 6.0))
    a.ZeroGrad()
    assert a.GradTensor() is None or float(a.GradTensor().abs().sum()) == 0.0


def test_backward_root_must_be_scalar():
    a = OaMatrix(torch.ones(2, 2)).SetRequiresGrad(True)
    with AG.OaGradientTape() as tape:
        with pytest.raises(ValueError):
            tape.Backward(F.Exp(a))
