"""Raw-tensor convolution / pooling support ops: im2col, col2im, pooling, nearest up-sampling (CUDA kernels in
csrc/kernels/conv.cu; the CPU branch is the plain PyTorch statement and the oracle of the GPU tests)."""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.nn.functional as TF

from .. import _native as N
from . import kernels as K


def _pair(v) -> tuple:
    return (int(v), int(v)) if isinstance(v, int) else (int(v[0]), int(v[1]))


def out_size(H: int, k: int, s: int, p: int, d: int = 1) -> int:
    return (H + 2 * p - d * (k - 1) - 1) // s + 1


def im2col(x: torch.Tensor, kernel, stride=1, padding=0, dilation=1) -> torch.Tensor:
    """x [N, C, H, W] -> columns [N*Ho*Wo, C*kh*kw]."""
    (kh, kw), (sh, sw), (ph, pw), (dh, dw) = _pair(kernel), _pair(stride), _pair(padding), _pair(dilation)
    n, c, h, w = x.shape
    ho, wo = out_size(h, kh, sh, ph, dh), out_size(w, kw, sw, pw, dw)
    if not x.is_cuda:
        u = TF.unfold(x.float(), (kh, kw), dilation=(dh, dw), padding=(ph, pw), stride=(sh, sw))        # [N, C*kh*kw, Ho*Wo]
        return u.transpose(1, 2).reshape(n * ho * wo, c * kh * kw).to(x.dtype).contiguous()
    x = x.contiguous()
    cols = torch.empty((n * ho * wo, c * kh * kw), dtype=x.dtype, device=x.device)
    K._launch(N.require().oa_im2col(K.dt(x), x.data_ptr(), cols.data_ptr(), n, c, h, w, kh, kw, sh, sw, ph, pw, dh, dw, N.stream()), "oa_im2col")
    return cols


def col2im(cols: torch.Tensor, shape: Sequence[int], kernel, stride=1, padding=0, dilation=1) -> torch.Tensor:
    """columns [N*Ho*Wo, C*kh*kw] -> overlap-added [N, C, H, W] (the adjoint of im2col)."""
    (kh, kw), (sh, sw), (ph, pw), (dh, dw) = _pair(kernel), _pair(stride), _pair(padding), _pair(dilation)
    n, c, h, w = shape
    ho, wo = out_size(h, kh, sh, ph, dh), out_size(w, kw, sw, pw, dw)
    if not cols.is_cuda:
        u = cols.float().reshape(n, ho * wo, c * kh * kw).transpose(1, 2)
        return TF.fold(u, (h, w), (kh, kw), dilation=(dh, dw), padding=(ph, pw), stride=(sh, sw)).to(cols.dtype)
    cols = cols.contiguous()
    x = torch.empty((n, c, h, w), dtype=cols.dtype, device=cols.device)
    K._launch(N.require().oa_col2im(K.dt(cols), cols.data_ptr(), x.data_ptr(), n, c, h, w, kh, kw, sh, sw, ph, pw, dh, dw, N.stream()), "oa_col2im")
    return x


def pool2d_fwd(x: torch.Tensor, mode: str, kernel, stride=None, padding=0):
    """mode 'max' -> (y, idx int32 plane offsets), 'avg' -> (y, None); the average excludes padding."""
    (kh, kw), (ph, pw) = _pair(kernel), _pair(padding)
    sh, sw = _pair(stride if stride is not None else kernel)
    n, c, h, w = x.shape
    ho, wo = out_size(h, kh, sh, ph), out_size(w, kw, sw, pw)
    if not x.is_cuda:
        if mode == "max":
            y, idx = TF.max_pool2d(x.float(), (kh, kw), (sh, sw), (ph, pw), return_indices=True)
            return y.to(x.dtype), idx.to(torch.int32)
        return TF.avg_pool2d(x.float(), (kh, kw), (sh, sw), (ph, pw), count_include_pad=False).to(x.dtype), None
    x = x.contiguous()
    y = torch.empty((n, c, ho, wo), dtype=x.dtype, device=x.device)
    idx = torch.empty((n, c, ho, wo), dtype=torch.int32, device=x.device) if mode == "max" else None
    K._launch(N.require().oa_pool2d_fwd(K.dt(x), 0 if mode == "max" else 1, x.data_ptr(), y.data_ptr(), N.ptr(idx), n, c, h, w, kh, kw, sh, sw,
                                        ph, pw, N.stream()), "oa_pool2d_fwd")
    return y, idx


def pool2d_bwd(dy: torch.Tensor, idx: Optional[torch.Tensor], shape, mode: str, kernel, stride=None, padding=0) -> torch.Tensor:
    (kh, kw), (ph, pw) = _pair(kernel), _pair(padding)
    sh, sw = _pair(stride if stride is not None else kernel)
    n, c, h, w = shape
    if not dy.is_cuda:
        dx = torch.zeros((n, c, h * w), dtype=torch.float32)
        if mode == "max":
            dx.scatter_add_(2, idx.long().reshape(n, c, -1), dy.float().reshape(n, c, -1))
            return dx.reshape(n, c, h, w).to(dy.dtype)
        xr = torch.zeros((n, c, h, w), dtype=torch.float32, requires_grad=True)
        y = TF.avg_pool2d(xr, (kh, kw), (sh, sw), (ph, pw), count_include_pad=False)
        return torch.autograd.grad(y, xr, dy.float())[0].to(dy.dtype)
    dy = dy.contiguous()
    dx = torch.empty((n, c, h, w), dtype=dy.dtype, device=dy.device)
    K._launch(N.require().oa_pool2d_bwd(K.dt(dy), 0 if mode == "max" else 1, dy.data_ptr(), N.ptr(idx), dx.data_ptr(), n, c, h, w, kh, kw, sh, sw,
                                        ph, pw, N.stream()), "oa_pool2d_bwd")
    return dx


def upsample_nearest(x: torch.Tensor, fy: int, fx: int, backward: bool = False) -> torch.Tensor:
    """Forward: [N, C, H, W] -> [N, C, H*fy, W*fx].  Backward: the gradient [N, C, H*fy, W*fx] -> [N, C, H, W] (block sums)."""
    n, c, hh, ww = x.shape
    h, w = (hh // fy, ww // fx) if backward else (hh, ww)
    if not x.is_cuda:
        if backward:
            return x.float().reshape(n, c, h, fy, w, fx).sum((3, 5)).to(x.dtype)
        return x.repeat_interleave(fy, 2).repeat_interleave(fx, 3)
    x = x.contiguous()
    out = torch.empty((n, c, h, w) if backward else (n, c, h * fy, w * fx), dtype=x.dtype, device=x.device)
    K._launch(N.require().oa_upsample_nearest(K.dt(x), x.data_ptr(), out.data_ptr(), n * c, h, w, fy, fx, int(backward), N.stream()),
              "oa_upsample_nearest")
    return out
