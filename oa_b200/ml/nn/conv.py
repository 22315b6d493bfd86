"""Convolution, pooling, up-sampling and batch-norm layers (the generated layer set of the reference:
Source/Public/Oa/Ml/Nn/Layers.h:7-28 - Conv1d, ConvTranspose1d, Conv2d, ConvTranspose2d, MaxPool2d, AvgPool2d,
AdaptiveAvgPool2d, Upsample, BatchNorm2d; convolution lowering as in Ml/FnMatrix Conv1dGemm / Im2Col1d / Col2Im1d).

A convolution is im2col -> one tensor-core GEMM (+ bias) -> layout permute; its transpose is GEMM -> col2im.  Im2Col and
Col2Im are each other's adjoint, so each is the other's backward.  Layout NCHW (NCL for the 1-d layers); weights
[C_out, C_in, kh, kw] (ConvTranspose: [C_in, C_out, kh, kw]), as in the reference checkpoints.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ...core import fn_matrix as F
from ...core.matrix import OaMatrix
from ...ops import conv as C
from .. import autograd as AG
from ..module import OaModule


# ------------------------------------------------------------------------------------------------ differentiable ops
def Im2Col(x: OaMatrix, kernel, stride=1, padding=0, dilation=1) -> OaMatrix:
    F._ctx_add("Im2Col")
    tx = F._c(x.Tensor())
    out = OaMatrix(C.im2col(tx, kernel, stride, padding, dilation))
    return AG.attach("Im2Col", out, [x], lambda g: (C.col2im(F._c(g), tx.shape, kernel, stride, padding, dilation),))


def Col2Im(cols: OaMatrix, shape, kernel, stride=1, padding=0, dilation=1) -> OaMatrix:
    F._ctx_add("Col2Im")
    out = OaMatrix(C.col2im(F._c(cols.Tensor()), shape, kernel, stride, padding, dilation))
    return AG.attach("Col2Im", out, [cols], lambda g: (C.im2col(F._c(g), kernel, stride, padding, dilation),))


def Conv2d(x: OaMatrix, w: OaMatrix, b: Optional[OaMatrix], stride=1, padding=0, dilation=1) -> OaMatrix:
    """x [N, C, H, W], w [O, C, kh, kw] -> [N, O, Ho, Wo]."""
    n, c, h, wd = x.Tensor().shape
    o, _, kh, kw = w.Tensor().shape
    (sh, sw), (ph, pw), (dh, dw) = C._pair(stride), C._pair(padding), C._pair(dilation)
    ho, wo = C.out_size(h, kh, sh, ph, dh), C.out_size(wd, kw, sw, pw, dw)
    cols = Im2Col(x, (kh, kw), stride, padding, dilation)
    y = F.Linear(cols, w.Reshape([o, c * kh * kw]), b, name="Conv2dGemm")
    return F.Permute(y.Reshape([n, ho, wo, o]), [0, 3, 1, 2])


def ConvTranspose2d(x: OaMatrix, w: OaMatrix, b: Optional[OaMatrix], stride=1, padding=0, output_padding=0) -> OaMatrix:
    """x [N, C, H, W], w [C, O, kh, kw] -> [N, O, (H-1)*s - 2p + kh + op, ...]."""
    n, c, h, wd = x.Tensor().shape
    _, o, kh, kw = w.Tensor().shape
    (sh, sw), (ph, pw), (oph, opw) = C._pair(stride), C._pair(padding), C._pair(output_padding)
    ho, wo = (h - 1) * sh - 2 * ph + kh + oph, (wd - 1) * sw - 2 * pw + kw + opw
    x2 = F.Permute(x, [0, 2, 3, 1]).Reshape([n * h * wd, c])
    cols = F.MatMulNt(x2, F.Transpose(w.Reshape([c, o * kh * kw]), 0, 1))         # [N*H*W, O*kh*kw]
    y = Col2Im(cols, (n, o, ho, wo), (kh, kw), stride, padding)
    return F.Add(y, b.Reshape([1, o, 1, 1])) if b is not None else y


def _pool(x: OaMatrix, mode: str, kernel, stride, padding) -> OaMatrix:
    name = "MaxPool2d" if mode == "max" else "AvgPool2d"
    F._ctx_add(name)
    tx = F._c(x.Tensor())
    y, idx = C.pool2d_fwd(tx, mode, kernel, stride, padding)
    return AG.attach(name, OaMatrix(y), [x], lambda g: (C.pool2d_bwd(F._c(g), idx, tx.shape, mode, kernel, stride, padding),))


def MaxPool2dFn(x, kernel, stride=None, padding=0): return _pool(x, "max", kernel, stride, padding)
def AvgPool2dFn(x, kernel, stride=None, padding=0): return _pool(x, "avg", kernel, stride, padding)


def UpsampleNearest(x: OaMatrix, fy: int, fx: int) -> OaMatrix:
    F._ctx_add("Upsample")
    out = OaMatrix(C.upsample_nearest(F._c(x.Tensor()), fy, fx))
    return AG.attach("Upsample", out, [x], lambda g: (C.upsample_nearest(F._c(g), fy, fx, backward=True),))


# ----------------------------------------------------------------------------------------------------------- modules
def _kaiming(shape, fan_in: int) -> OaMatrix:
    bound = 1.0 / math.sqrt(fan_in)
    return F.AddScalar(F.Scale(F.Rand(list(shape)), 2.0 * bound), -bound)


class OaConv2d(OaModule):
    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride=1, padding=0, dilation=1, bias: bool = True):
        super().__init__()
        kh, kw = C._pair(kernel_size)
        self.Stride, self.Padding, self.Dilation = stride, padding, dilation
        fan_in = in_channels * kh * kw
        self.Weight = self.RegisterParameter("weight", _kaiming((out_channels, in_channels, kh, kw), fan_in))
        self.Bias = self.RegisterParameter("bias", _kaiming((out_channels,), fan_in)) if bias else None

    def Forward(self, x: OaMatrix) -> OaMatrix:
        return Conv2d(x, self.Weight.Data, self.Bias.Data if self.Bias else None, self.Stride, self.Padding, self.Dilation)


class OaConvTranspose2d(OaModule):
    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride=1, padding=0, output_padding=0, bias: bool = True):
        super().__init__()
        kh, kw = C._pair(kernel_size)
        self.Stride, self.Padding, self.OutputPadding = stride, padding, output_padding
        fan_in = out_channels * kh * kw
        self.Weight = self.RegisterParameter("weight", _kaiming((in_channels, out_channels, kh, kw), fan_in))
        self.Bias = self.RegisterParameter("bias", _kaiming((out_channels,), fan_in)) if bias else None

    def Forward(self, x: OaMatrix) -> OaMatrix:
        return ConvTranspose2d(x, self.Weight.Data, self.Bias.Data if self.Bias else None, self.Stride, self.Padding, self.OutputPadding)


class OaConv1d(OaModule):
    """x [N, C, L] -> [N, O, Lo]; weight [O, C, k]."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size: int, stride: int = 1, padding: int = 0, dilation: int = 1, bias: bool = True):
        super().__init__()
        self.K, self.Stride, self.Padding, self.Dilation = kernel_size, stride, padding, dilation
        fan_in = in_channels * kernel_size
        self.Weight = self.RegisterParameter("weight", _kaiming((out_channels, in_channels, kernel_size), fan_in))
        self.Bias = self.RegisterParameter("bias", _kaiming((out_channels,), fan_in)) if bias else None

    def Forward(self, x: OaMatrix) -> OaMatrix:
        n, c, l = x.Tensor().shape
        o = self.Weight.Tensor().shape[0]
        y = Conv2d(x.Reshape([n, c, 1, l]), self.Weight.Data.Reshape([o, c, 1, self.K]), self.Bias.Data if self.Bias else None,
                   (1, self.Stride), (0, self.Padding), (1, self.Dilation))
        return y.Reshape([n, o, y.Size(3)])


class OaConvTranspose1d(OaModule):
    """x [N, C, L] -> [N, O, (L-1)*s - 2p + k + op]; weight [C, O, k]."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size: int, stride: int = 1, padding: int = 0, output_padding: int = 0,
                 bias: bool = True):
        super().__init__()
        self.K, self.Stride, self.Padding, self.OutputPadding = kernel_size, stride, padding, output_padding
        fan_in = out_channels * kernel_size
        self.Weight = self.RegisterParameter("weight", _kaiming((in_channels, out_channels, kernel_size), fan_in))
        self.Bias = self.RegisterParameter("bias", _kaiming((out_channels,), fan_in)) if bias else None

    def Forward(self, x: OaMatrix) -> OaMatrix:
        n, c, l = x.Tensor().shape
        o = self.Weight.Tensor().shape[1]
        y = ConvTranspose2d(x.Reshape([n, c, 1, l]), self.Weight.Data.Reshape([c, o, 1, self.K]), self.Bias.Data if self.Bias else None,
                            (1, self.Stride), (0, self.Padding), (0, self.OutputPadding))
        return y.Reshape([n, o, y.Size(3)])


class OaMaxPool2d(OaModule):
    def __init__(self, kernel_size, stride=None, padding=0):
        super().__init__()
        self.K, self.Stride, self.Padding = kernel_size, stride, padding

    def Forward(self, x): return MaxPool2dFn(x, self.K, self.Stride, self.Padding)


class OaAvgPool2d(OaModule):
    def __init__(self, kernel_size, stride=None, padding=0):
        super().__init__()
        self.K, self.Stride, self.Padding = kernel_size, stride, padding

    def Forward(self, x): return AvgPool2dFn(x, self.K, self.Stride, self.Padding)


class OaAdaptiveAvgPool2d(OaModule):
    """Output size (oh, ow); the input size must be a multiple of it (uniform windows)."""

    def __init__(self, output_size):
        super().__init__()
        self.Out = C._pair(output_size)

    def Forward(self, x):
        h, w = x.Size(2), x.Size(3)
        if h % self.Out[0] or w % self.Out[1]:
            raise ValueError(f"OaAdaptiveAvgPool2d: input {h}x{w} is not a multiple of the output {self.Out}")
        k = (h // self.Out[0], w // self.Out[1])
        return AvgPool2dFn(x, k, k, 0)


class OaUpsample(OaModule):
    def __init__(self, scale_factor=2):
        super().__init__()
        self.Fy, self.Fx = C._pair(scale_factor)

    def Forward(self, x): return UpsampleNearest(x, self.Fy, self.Fx)


class OaBatchNorm2d(OaModule):
    """Per-channel normalisation over (N, H, W) with running statistics (buffers `running_mean`, `running_var`)."""

    def __init__(self, num_features: int, eps: float = 1e-5, momentum: float = 0.1):
        super().__init__()
        self.C_, self.Eps, self.Momentum = num_features, eps, momentum
        self.Weight = self.RegisterParameter("weight", F.Ones([num_features]))
        self.Bias = self.RegisterParameter("bias", F.Zeros([num_features]))
        self.RunningMean = self.RegisterBuffer("running_mean", F.Zeros([num_features], torch.float32))
        self.RunningVar = self.RegisterBuffer("running_var", F.Ones([num_features], torch.float32))

    def Forward(self, x: OaMatrix) -> OaMatrix:
        n, c, h, w = x.Tensor().shape
        shape = [1, c, 1, 1]
        if self.IsTraining():
            rows = F.Permute(x, [1, 0, 2, 3]).Reshape([c, n * h * w])
            mean = F.Mean(rows, 1)
            centred = F.Sub(rows, mean.Reshape([c, 1]))
            var = F.Mean(F.Mul(centred, centred), 1)
            with AG.OaGradNo():
                m = self.Momentum
                unbiased = n * h * w / max(1, n * h * w - 1)
                rm, rv = self.RunningMean.Data.Tensor(), self.RunningVar.Data.Tensor()
                rm.mul_(1 - m).add_(mean.Tensor().float().reshape(-1), alpha=m)
                rv.mul_(1 - m).add_(var.Tensor().float().reshape(-1), alpha=m * unbiased)
        else:
            mean = OaMatrix(self.RunningMean.Data.Tensor().to(x.Tensor().dtype))
            var = OaMatrix(self.RunningVar.Data.Tensor().to(x.Tensor().dtype))
        inv = F.Reciprocal(F.Sqrt(F.AddScalar(var, self.Eps)))
        scale = F.Mul(inv, self.Weight.Data)
        return F.Add(F.Mul(F.Sub(x, mean.Reshape(shape)), scale.Reshape(shape)), self.Bias.Data.Reshape(shape))
