"""Convolution / pooling / up-sampling / batch-norm layers against torch.nn.functional (CPU autograd parity), and the
CUDA support kernels against their PyTorch statement (GPU)."""
import pytest
import torch
import torch.nn.functional as TF

from oa_b200.core import fn_matrix as F
from oa_b200.core.matrix import OaMatrix
from oa_b200.ml import autograd as AG
from oa_b200.ml.nn import conv as NN
from oa_b200.ops import conv as C


def _grad_check(module_fn, torch_fn, x, params):
    xm = OaMatrix(x.clone()).SetRequiresGrad(True)
    with AG.OaGradientTape() as tape:
        y = module_fn(xm)
        up = torch.randn(y.Tensor().shape, generator=torch.Generator().manual_seed(3))
        tape.Backward(y, grad=up.clone())
    xt = x.clone().requires_grad_(True)
    leaves = [p.Tensor().detach().clone().requires_grad_(True) for p in params]
    ref = torch_fn(xt, *leaves)
    assert y.Tensor().shape == ref.shape
    assert (y.Tensor() - ref).abs().max().item() < 1e-4
    ref.backward(up)
    assert (xm.GradTensor() - xt.grad).abs().max().item() < 1e-4
    for p, l in zip(params, leaves):
        assert (p.Grad().Tensor() - l.grad).abs().max().item() < 1e-4 * max(1.0, l.grad.abs().max().item())


def test_conv2d_and_transpose():
    F.SetRngSeed(0)
    torch.manual_seed(0)
    x = torch.randn(2, 3, 9, 8)
    m = NN.OaConv2d(3, 5, (3, 2), stride=(2, 1), padding=(1, 0), dilation=(1, 2))
    _grad_check(m.Forward, lambda t, w, b: TF.conv2d(t, w, b, (2, 1), (1, 0), (1, 2)), x, [m.Weight, m.Bias])
    t = NN.OaConvTranspose2d(3, 4, 3, stride=2, padding=1, output_padding=1)
    _grad_check(t.Forward, lambda u, w, b: TF.conv_transpose2d(u, w, b, 2, 1, 1), x, [t.Weight, t.Bias])


def test_conv1d_and_transpose():
    F.SetRngSeed(1)
    x = torch.randn(2, 4, 17)
    m = NN.OaConv1d(4, 6, 5, stride=2, padding=2)
    _grad_check(m.Forward, lambda t, w, b: TF.conv1d(t, w, b, 2, 2), x, [m.Weight, m.Bias])
    t = NN.OaConvTranspose1d(4, 3, 4, stride=2, padding=1)
    _grad_check(t.Forward, lambda u, w, b: TF.conv_transpose1d(u, w, b, 2, 1), x, [t.Weight, t.Bias])


def test_pools_upsample_batchnorm():
    torch.manual_seed(2)
    x = torch.randn(2, 3, 8, 8)
    _grad_check(NN.OaMaxPool2d(3, 2, 1).Forward, lambda t: TF.max_pool2d(t, 3, 2, 1), x, [])
    _grad_check(NN.OaAvgPool2d(2).Forward, lambda t: TF.avg_pool2d(t, 2), x, [])
    _grad_check(NN.OaAdaptiveAvgPool2d(2).Forward, lambda t: TF.adaptive_avg_pool2d(t, 2), x, [])
    _grad_check(NN.OaUpsample(2).Forward, lambda t: TF.interpolate(t, scale_factor=2, mode="nearest"), x, [])
    bn = NN.OaBatchNorm2d(3)
    ref = torch.nn.BatchNorm2d(3)
    _grad_check(bn.Forward, lambda t, w, b: TF.batch_norm(t, None, None, w, b, True, 0.1, 1e-5), x, [bn.Weight, bn.Bias])
    ref.train()
    ref(x)
    assert (bn.RunningMean.Data.Tensor() - ref.running_mean).abs().max().item() < 1e-5
    assert (bn.RunningVar.Data.Tensor() - ref.running_var).abs().max().item() < 1e-5
    bn.Eval()
    ref.eval()
    with AG.OaGradNo():
        assert (bn.Forward(OaMatrix(x)).Tensor() - ref(x)).abs().max().item() < 1e-5


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-6), (torch.bfloat16, 2e-2)])
def test_conv_kernels_match_reference(dtype, tol):
    torch.manual_seed(0)
    x = torch.randn(2, 3, 11, 9).to(dtype)
    args = dict(kernel=(3, 2), stride=(2, 1), padding=(1, 1), dilation=(1, 2))
    cols = C.im2col(x.cuda(), **args)
    ref = C.im2col(x, **args)
    assert (cols.cpu().float() - ref.float()).abs().max().item() <= tol
    back = C.col2im(cols, x.shape, **args)
    refb = C.col2im(ref, x.shape, **args)
    assert (back.cpu().float() - refb.float()).abs().max().item() <= tol * 8
    for mode in ("max", "avg"):
        y, idx = C.pool2d_fwd(x.cuda(), mode, 3, 2, 1)
        yr, idxr = C.pool2d_fwd(x, mode, 3, 2, 1)
        assert (y.cpu().float() - yr.float()).abs().max().item() <= tol
        dy = torch.randn(y.shape).to(dtype)
        dx = C.pool2d_bwd(dy.cuda(), idx, x.shape, mode, 3, 2, 1)
        dxr = C.pool2d_bwd(dy, idxr, x.shape, mode, 3, 2, 1)
        assert (dx.cpu().float() - dxr.float()).abs().max().item() <= tol * 8
    up = C.upsample_nearest(x.cuda(), 2, 3)
    assert torch.equal(up.cpu(), C.upsample_nearest(x, 2, 3))
    assert (C.upsample_nearest(up, 2, 3, backward=True).cpu().float() - 6 * x.float()).abs().max().item() <= tol * 8
