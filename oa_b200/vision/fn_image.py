"""OaFnImage: the tensor-native image operations on planar fp32 NCHW tensors.

Reference: Source/Public/Oa/Vision/FnImage.h:30-105 with the operation inventory in
Tools/FnAutogen/Schema/Vision/VisionFnImage{Pixel,Filter,Geometric,Color,Resize}.toml (50 operations) and the kernels under
Source/Private/Oa/Vision/Shader/Compute/{Color,Filter,Geometric}.  Every operation runs one of nine kernels of `image.cu`
on the GPU; on a CPU tensor the same function is evaluated with tensor expressions (that path is also the oracle the GPU
tests compare against).  As in the reference, an operation whose arguments are invalid returns its input unchanged.
"""
from __future__ import annotations

import ctypes
import enum
import math
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

from .. import _native as N
from ..core.matrix import OaMatrix
from ..ops import kernels as K


class OaInterpolationMode(enum.IntEnum):
    Nearest = 0
    Bilinear = 1
    Bicubic = 2


class OaBorderMode(enum.IntEnum):
    Constant = 0
    Replicate = 1
    Reflect = 2
    Reflect101 = 3
    Wrap = 4


class OaImageLayout(enum.IntEnum):
    Nchw = 0
    Nhwc = 1
    Chw = 2
    Hwc = 3
    Hw = 4


class OaImageFormat(enum.IntEnum):
    Gray = 0
    GrayAlpha = 1
    Rgb = 2
    Rgba = 3
    Bgr = 4
    Bgra = 5


def OaImageFormatChannels(fmt: OaImageFormat) -> int:
    return {OaImageFormat.Gray: 1, OaImageFormat.GrayAlpha: 2, OaImageFormat.Rgb: 3, OaImageFormat.Rgba: 4, OaImageFormat.Bgr: 3,
            OaImageFormat.Bgra: 4}[OaImageFormat(fmt)]


@dataclass
class OaNormalizationParams:
    Mean: Tuple[float, float, float] = (0.485, 0.456, 0.406)
    Std: Tuple[float, float, float] = (0.229, 0.224, 0.225)


class OaImage:
    """A tensor with its layout and channel meaning (Source/Public/Oa/Core/Image.h:63-112)."""

    def __init__(self, data: Optional[OaMatrix] = None, layout: OaImageLayout = OaImageLayout.Nchw, fmt: OaImageFormat = OaImageFormat.Rgb):
        self.Data_, self.Layout_, self.Format_ = data, OaImageLayout(layout), OaImageFormat(fmt)

    def AsMatrix(self) -> Optional[OaMatrix]: return self.Data_
    def Layout(self) -> OaImageLayout: return self.Layout_
    def Format(self) -> OaImageFormat: return self.Format_
    def IsEmpty(self) -> bool: return self.Data_ is None or self.Data_.Tensor().dim() == 0

    def _axes(self):
        # (batch, channel, height, width) axis numbers, None where the layout has no such axis
        return {OaImageLayout.Nchw: (0, 1, 2, 3), OaImageLayout.Nhwc: (0, 3, 1, 2), OaImageLayout.Chw: (None, 0, 1, 2),
                OaImageLayout.Hwc: (None, 2, 0, 1), OaImageLayout.Hw: (None, None, 0, 1)}[self.Layout_]

    def _dim(self, k: int, default: int) -> int:
        ax = self._axes()[k]
        return default if self.IsEmpty() or ax is None else int(self.Data_.Tensor().shape[ax])

    def BatchSize(self) -> int: return self._dim(0, 1)
    def Channels(self) -> int: return self._dim(1, OaImageFormatChannels(self.Format_))
    def Height(self) -> int: return self._dim(2, 0)
    def Width(self) -> int: return self._dim(3, 0)

    def Validate(self) -> bool:
        if self.IsEmpty():
            return True
        rank = {OaImageLayout.Nchw: 4, OaImageLayout.Nhwc: 4, OaImageLayout.Chw: 3, OaImageLayout.Hwc: 3, OaImageLayout.Hw: 2}[self.Layout_]
        if self.Data_.Tensor().dim() != rank:
            return False
        if self.Layout_ == OaImageLayout.Hw:
            return OaImageFormatChannels(self.Format_) == 1
        return self.Channels() == OaImageFormatChannels(self.Format_)

    def ToNchw(self) -> torch.Tensor:
        t = self.Data_.Tensor()
        if self.Layout_ == OaImageLayout.Nchw:
            return t
        if self.Layout_ == OaImageLayout.Nhwc:
            return t.permute(0, 3, 1, 2).contiguous()
        if self.Layout_ == OaImageLayout.Chw:
            return t.unsqueeze(0)
        if self.Layout_ == OaImageLayout.Hwc:
            return t.permute(2, 0, 1).unsqueeze(0).contiguous()
        return t.reshape(1, 1, *t.shape)

    def FromNchw(self, t: torch.Tensor, fmt: Optional[OaImageFormat] = None) -> "OaImage":
        if self.Layout_ == OaImageLayout.Nhwc:
            t = t.permute(0, 2, 3, 1).contiguous()
        elif self.Layout_ == OaImageLayout.Chw:
            t = t[0]
        elif self.Layout_ == OaImageLayout.Hwc:
            t = t[0].permute(1, 2, 0).contiguous()
        elif self.Layout_ == OaImageLayout.Hw:
            t = t[0, 0]
        return OaImage(OaMatrix(t), self.Layout_, self.Format_ if fmt is None else fmt)


# ------------------------------------------------------------------------------------------------ helpers
PW = {"binary": 0, "binary_inv": 1, "truncate": 2, "tozero": 3, "tozero_inv": 4, "inrange": 5, "clamp": 6, "invert": 7, "contrast": 8,
      "gamma": 9, "solarize": 10, "posterize": 11}
TF_CONV2D, TF_SEPARABLE, TF_MIN, TF_MAX, TF_MEDIAN, TF_BILATERAL, TF_ADAPTIVE_MEAN, TF_ADAPTIVE_GAUSS = range(8)


def _t(m) -> torch.Tensor:
    return m.Tensor() if isinstance(m, OaMatrix) else m


def _is_image(m) -> bool:
    if not isinstance(m, OaMatrix):
        return False
    t = m.Tensor()
    return t.dim() == 4 and t.dtype == torch.float32 and t.numel() > 0


def _finite(*vals: float) -> bool:
    return all(math.isfinite(float(v)) for v in vals)


def _valid_border(b) -> bool:
    try:
        OaBorderMode(int(b))
        return True
    except ValueError:
        return False


def _border_index(idx: torch.Tensor, n: int, mode: int):
    """Source index and validity for coordinates `idx` on an axis of length n (same rules as `border_index` in image.cu)."""
    inside = (idx >= 0) & (idx < n)
    if mode == OaBorderMode.Replicate:
        return idx.clamp(0, n - 1), torch.ones_like(inside)
    if mode == OaBorderMode.Reflect:
        p = 2 * n
        m = idx % p
        return torch.where(m < n, m, p - 1 - m), torch.ones_like(inside)
    if mode == OaBorderMode.Reflect101:
        if n == 1:
            return torch.zeros_like(idx), torch.ones_like(inside)
        p = 2 * n - 2
        m = idx % p
        return torch.where(m < n, m, p - m), torch.ones_like(inside)
    if mode == OaBorderMode.Wrap:
        return idx % n, torch.ones_like(inside)
    return idx.clamp(0, n - 1), inside


def _sample_border(t: torch.Tensor, ys: torch.Tensor, xs: torch.Tensor, mode: int, value: float) -> torch.Tensor:
    """t [N,C,H,W]; ys, xs integer coordinates broadcastable to [N,1,Ho,Wo] (or [Ho,Wo]); returns t at those coordinates."""
    H, W = t.shape[2], t.shape[3]
    sy, vy = _border_index(ys, H, mode)
    sx, vx = _border_index(xs, W, mode)
    flat = t.reshape(t.shape[0], t.shape[1], H * W)
    lin = (sy * W + sx)
    if lin.dim() == 2:
        out = flat[:, :, lin.reshape(-1)].reshape(t.shape[0], t.shape[1], *lin.shape)
        ok = (vy & vx)[None, None]
    else:
        lin4 = lin.expand(t.shape[0], 1, *lin.shape[-2:]).expand(t.shape[0], t.shape[1], *lin.shape[-2:])
        out = torch.gather(flat, 2, lin4.reshape(t.shape[0], t.shape[1], -1)).reshape(lin4.shape)
        ok = (vy & vx).expand(t.shape[0], 1, *lin.shape[-2:])
    return torch.where(ok, out, torch.full_like(out, value))


def _pad_cpu(t: torch.Tensor, left: int, right: int, top: int, bottom: int, mode: int, value: float) -> torch.Tensor:
    H, W = t.shape[2], t.shape[3]
    ys = torch.arange(-top, H + bottom)[:, None].expand(H + top + bottom, W + left + right)
    xs = torch.arange(-left, W + right)[None, :].expand(H + top + bottom, W + left + right)
    return _sample_border(t, ys, xs, mode, value)


def _windows(t: torch.Tensor, kw: int, kh: int, mode: int, value: float) -> torch.Tensor:
    """[N,C,H,W,kh,kw] neighbourhoods with the border rule applied."""
    p = _pad_cpu(t, kw // 2, kw // 2, kh // 2, kh // 2, mode, value)
    return p.unfold(2, kh, 1).unfold(3, kw, 1)


def _tile_filter(img: OaMatrix, kw: int, kh: int, mode: int, border: int, border_value: float = 0.0, k0: Optional[torch.Tensor] = None,
                 k1: Optional[torch.Tensor] = None, p0: float = 0.0, p1: float = 0.0, p2: float = 0.0) -> OaMatrix:
    t = _t(img).contiguous()
    Nn, C, H, W = t.shape
    if t.is_cuda:
        out = torch.empty_like(t)
        k0c = k0.to(device=t.device, dtype=torch.float32).contiguous() if k0 is not None else None
        k1c = k1.to(device=t.device, dtype=torch.float32).contiguous() if k1 is not None else None
        K._launch(N.require().oa_image_tile_filter(t.data_ptr(), out.data_ptr(), Nn * C, H, W, kw, kh, mode, int(border), float(border_value),
                                                   N.ptr(k0c), N.ptr(k1c), float(p0), float(p1), float(p2), N.stream()), "oa_image_tile_filter")
        return OaMatrix(out)
    win = _windows(t, kw, kh, int(border), float(border_value))
    if mode == TF_CONV2D:
        out = (win * k0.float().reshape(kh, kw)).sum((-1, -2))
    elif mode == TF_SEPARABLE:
        out = (win * (k1.float().reshape(kh, 1) * k0.float().reshape(1, kw))).sum((-1, -2))
    elif mode == TF_MIN:
        out = win.amin((-1, -2))
    elif mode == TF_MAX:
        out = win.amax((-1, -2))
    elif mode == TF_MEDIAN:
        out = win.reshape(*win.shape[:4], -1).sort(-1).values[..., (kw * kh) // 2]
    else:
        dy = torch.arange(kh).float()[:, None] - kh // 2
        dx = torch.arange(kw).float()[None, :] - kw // 2
        ss, sc = max(p0, 1e-6), max(p1, 1e-6)
        spatial = torch.exp(-(dx * dx + dy * dy) / (2 * ss * ss))
        center = t[..., None, None]
        if mode == TF_BILATERAL:
            w = torch.exp(-(dx * dx + dy * dy) / (2 * ss * ss) - (win - center) ** 2 / (2 * sc * sc))
        elif mode == TF_ADAPTIVE_GAUSS:
            w = spatial.expand_as(win)
        else:
            w = torch.ones_like(win)
        filtered = (win * w).sum((-1, -2)) / w.sum((-1, -2)).clamp_min(1e-20)
        out = filtered if mode == TF_BILATERAL else torch.where(t > filtered - p1, torch.full_like(t, p2), torch.zeros_like(t))
    return OaMatrix(out.contiguous())


def _pointwise(img: OaMatrix, name: str, p0: float = 0.0, p1: float = 0.0, p2: float = 0.0) -> OaMatrix:
    t = _t(img).contiguous()
    op = PW[name]
    if t.is_cuda:
        out = torch.empty_like(t)
        K._launch(N.require().oa_image_pointwise(t.data_ptr(), out.data_ptr(), t.numel(), op, float(p0), float(p1), float(p2), N.stream()),
                  "oa_image_pointwise")
        return OaMatrix(out)
    z = torch.zeros_like(t)
    if name == "binary":
        out = torch.where(t > p0, torch.full_like(t, p1), z)
    elif name == "binary_inv":
        out = torch.where(t > p0, z, torch.full_like(t, p1))
    elif name == "truncate":
        out = t.clamp_max(p0)
    elif name == "tozero":
        out = torch.where(t > p0, t, z)
    elif name == "tozero_inv":
        out = torch.where(t > p0, z, t)
    elif name == "inrange":
        out = torch.where((t >= p0) & (t <= p1), torch.full_like(t, p2), z)
    elif name == "clamp":
        out = t.clamp(p0, p1)
    elif name == "invert":
        out = p0 - t
    elif name == "contrast":
        out = t * p0 + p1
    elif name == "gamma":
        out = t.clamp_min(0).pow(p0) * p1
    elif name == "solarize":
        out = torch.where(t >= p0, p1 - t, t)
    else:
        levels = max(float(p0), 2.0)
        nrm = ((t - p1) / (p2 - p1)).clamp(0, 1)
        out = torch.floor(nrm * (levels - 1) + 0.5) / (levels - 1) * (p2 - p1) + p1
    return OaMatrix(out)


def _channels(img: OaMatrix, cout: int, matrix: Optional[Sequence[Sequence[float]]] = None, sel: Optional[Sequence[int]] = None,
              twist: Optional[torch.Tensor] = None) -> OaMatrix:
    t = _t(img).contiguous()
    Nn, C, H, W = t.shape
    mode = 1 if sel is not None else (2 if twist is not None else 0)
    if t.is_cuda:
        out = torch.empty((Nn, cout, H, W), dtype=torch.float32, device=t.device)
        m20 = (ctypes.c_float * 20)(*([0.0] * 20))
        if matrix is not None:
            for c, row in enumerate(matrix):
                for j, v in enumerate(row):
                    m20[c * 5 + j] = float(v)
        s4 = (ctypes.c_int * 4)(*((list(sel) + [0, 0, 0, 0])[:4] if sel is not None else [0, 0, 0, 0]))
        tw = twist.to(device=t.device, dtype=torch.float32).contiguous() if twist is not None else None
        K._launch(N.require().oa_image_channels(t.data_ptr(), out.data_ptr(), Nn, C, cout, H * W, m20, s4, N.ptr(tw), mode, N.stream()),
                  "oa_image_channels")
        return OaMatrix(out)
    if mode == 1:
        return OaMatrix(t[:, list(sel)[:cout]].contiguous())
    if mode == 2:
        T = twist.float().reshape(3, 4)
        rgb = torch.einsum("cj,njhw->nchw", T[:, :3], t[:, :3]) + T[:, 3].reshape(1, 3, 1, 1)
        return OaMatrix(torch.cat([rgb, t[:, 3:]], 1).contiguous())
    M = torch.tensor([list(r)[:C + 1] for r in matrix], dtype=torch.float32)
    return OaMatrix((torch.einsum("cj,njhw->nchw", M[:, :C], t) + M[:, C].reshape(1, cout, 1, 1)).contiguous())


def _blend(a: OaMatrix, b: Optional[OaMatrix], mask: Optional[OaMatrix], op: int, alpha: float = 0.0, rect=(0, 0, 0, 0),
           value: float = 0.0) -> OaMatrix:
    ta = _t(a).contiguous()
    Nn, C, H, W = ta.shape
    tb = _t(b).contiguous() if b is not None else None
    tm = _t(mask).contiguous() if mask is not None else None
    if ta.is_cuda:
        out = torch.empty_like(ta)
        K._launch(N.require().oa_image_blend(ta.data_ptr(), N.ptr(tb), N.ptr(tm), out.data_ptr(), Nn, C, H, W, op, float(alpha),
                                             tm.shape[1] if tm is not None else 1, *[int(v) for v in rect], float(value), N.stream()),
                  "oa_image_blend")
        return OaMatrix(out)
    if op == 0:
        return OaMatrix(ta * (1 - alpha) + tb * alpha)
    if op == 1:
        m = tm.clamp(0, 1)
        return OaMatrix(ta * (1 - m) + tb * m)
    out = ta.clone()
    x, y, w, h = rect
    out[:, :, y:y + h, x:x + w] = value
    return OaMatrix(out)


def _index_map(img: OaMatrix, Ho: int, Wo: int, op: int, a0: int, a1: int, border: int = 0, value: float = 0.0) -> OaMatrix:
    t = _t(img).contiguous()
    Nn, C, H, W = t.shape
    if t.is_cuda:
        out = torch.empty((Nn, C, Ho, Wo), dtype=torch.float32, device=t.device)
        K._launch(N.require().oa_image_index_map(t.data_ptr(), out.data_ptr(), Nn * C, H, W, Ho, Wo, op, int(a0), int(a1), int(border),
                                                 float(value), N.stream()), "oa_image_index_map")
        return OaMatrix(out)
    if op == 0:
        return OaMatrix(t[:, :, a1:a1 + Ho, a0:a0 + Wo].contiguous())
    if op == 1:
        dims = ([3] if a0 else []) + ([2] if a1 else [])
        return OaMatrix(t.flip(dims).contiguous() if dims else t.clone())
    if op == 2:
        k = {90: -1, 180: 2, 270: 1}[a0]                    # clockwise quarter turns
        return OaMatrix(torch.rot90(t, k, (2, 3)).contiguous())
    return OaMatrix(_pad_cpu(t, a0, Wo - W - a0, a1, Ho - H - a1, int(border), float(value)).contiguous())


def _bilinear_cpu(t: torch.Tensor, sy: torch.Tensor, sx: torch.Tensor, border: int, value: float) -> torch.Tensor:
    y0, x0 = torch.floor(sy).long(), torch.floor(sx).long()
    wy, wx = sy - y0, sx - x0                              # [Ho,Wo] or [N,1,Ho,Wo]: both broadcast over [N,C,Ho,Wo]
    v00 = _sample_border(t, y0, x0, border, value)
    v01 = _sample_border(t, y0, x0 + 1, border, value)
    v10 = _sample_border(t, y0 + 1, x0, border, value)
    v11 = _sample_border(t, y0 + 1, x0 + 1, border, value)
    top = v00 + (v01 - v00) * wx
    bot = v10 + (v11 - v10) * wx
    return top + (bot - top) * wy


def _warp(img: OaMatrix, mp: torch.Tensor, Ho: int, Wo: int, op: int, interp: int, border: int, value: float) -> OaMatrix:
    t = _t(img).contiguous()
    Nn, C, H, W = t.shape
    if t.is_cuda:
        out = torch.empty((Nn, C, Ho, Wo), dtype=torch.float32, device=t.device)
        mpc = mp.to(device=t.device, dtype=torch.float32).contiguous()
        K._launch(N.require().oa_image_warp(t.data_ptr(), mpc.data_ptr(), out.data_ptr(), Nn, C, H, W, Ho, Wo, op, mpc.shape[0] if op == 0 else 1,
                                            int(interp), int(border), float(value), N.stream()), "oa_image_warp")
        return OaMatrix(out)
    ys = torch.arange(Ho, dtype=torch.float32)[:, None].expand(Ho, Wo)
    xs = torch.arange(Wo, dtype=torch.float32)[None, :].expand(Ho, Wo)
    m = mp.float()
    valid = torch.ones(Ho, Wo, dtype=torch.bool)
    if op == 0:
        sx, sy = m[:, 0:1], m[:, 1:2]                       # [Nm,1,Ho,Wo]
        sx, sy = sx.expand(Nn, 1, Ho, Wo), sy.expand(Nn, 1, Ho, Wo)
        valid = valid.expand(Nn, 1, Ho, Wo)
    else:
        f = m.reshape(-1)
        if op == 1:
            sx = f[0] * xs + f[1] * ys + f[2]
            sy = f[3] * xs + f[4] * ys + f[5]
        else:
            den = f[6] * xs + f[7] * ys + f[8]
            valid = den.abs() > 1e-12
            safe = torch.where(valid, den, torch.ones_like(den))
            sx = (f[0] * xs + f[1] * ys + f[2]) / safe
            sy = (f[3] * xs + f[4] * ys + f[5]) / safe
    valid = valid & torch.isfinite(sx) & torch.isfinite(sy) & (sx.abs() <= 1e9) & (sy.abs() <= 1e9)
    sx = torch.where(valid, sx, torch.zeros_like(sx))
    sy = torch.where(valid, sy, torch.zeros_like(sy))
    if interp == 0:
        out = _sample_border(t, torch.floor(sy + 0.5).long(), torch.floor(sx + 0.5).long(), border, value)
    else:
        out = _bilinear_cpu(t, sy, sx, border, value)
    return OaMatrix(torch.where(valid if valid.dim() == 4 else valid[None, None], out, torch.full_like(out, value)).contiguous())


# ------------------------------------------------------------------------------------------------ pointwise operations
def ThresholdBinary(Image: OaMatrix, Threshold: float, MaxValue: float = 1.0) -> OaMatrix:
    return _pointwise(Image, "binary", Threshold, MaxValue) if _is_image(Image) and _finite(Threshold, MaxValue) else Image


def ThresholdBinaryInv(Image: OaMatrix, Threshold: float, MaxValue: float = 1.0) -> OaMatrix:
    return _pointwise(Image, "binary_inv", Threshold, MaxValue) if _is_image(Image) and _finite(Threshold, MaxValue) else Image


def ThresholdTruncate(Image: OaMatrix, Threshold: float) -> OaMatrix:
    return _pointwise(Image, "truncate", Threshold) if _is_image(Image) and _finite(Threshold) else Image


def ThresholdToZero(Image: OaMatrix, Threshold: float) -> OaMatrix:
    return _pointwise(Image, "tozero", Threshold) if _is_image(Image) and _finite(Threshold) else Image


def ThresholdToZeroInv(Image: OaMatrix, Threshold: float) -> OaMatrix:
    return _pointwise(Image, "tozero_inv", Threshold) if _is_image(Image) and _finite(Threshold) else Image


def InRange(Image: OaMatrix, Low: float, High: float, TrueValue: float = 1.0) -> OaMatrix:
    return _pointwise(Image, "inrange", Low, High, TrueValue) if _is_image(Image) and _finite(Low, High, TrueValue) and Low <= High else Image


def Clamp(Image: OaMatrix, Low: float, High: float) -> OaMatrix:
    return _pointwise(Image, "clamp", Low, High) if _is_image(Image) and _finite(Low, High) and Low <= High else Image


def Invert(Image: OaMatrix, MaxValue: float = 1.0) -> OaMatrix:
    return _pointwise(Image, "invert", MaxValue) if _is_image(Image) and _finite(MaxValue) else Image


def BrightnessContrast(Image, Brightness: float = 0.0, Contrast: float = 1.0):
    if isinstance(Image, OaImage):
        return _on_image(Image, lambda m: BrightnessContrast(m, Brightness, Contrast))
    return _pointwise(Image, "contrast", Contrast, Brightness) if _is_image(Image) and _finite(Brightness, Contrast) else Image


def GammaContrast(Image: OaMatrix, Gamma: float, Gain: float = 1.0) -> OaMatrix:
    return _pointwise(Image, "gamma", Gamma, Gain) if _is_image(Image) and _finite(Gamma, Gain) and Gamma > 0 else Image


def Solarize(Image: OaMatrix, Threshold: float = 0.5, MaxValue: float = 1.0) -> OaMatrix:
    return _pointwise(Image, "solarize", Threshold, MaxValue) if _is_image(Image) and _finite(Threshold, MaxValue) else Image


def Posterize(Image: OaMatrix, Levels: int, Low: float = 0.0, High: float = 1.0) -> OaMatrix:
    return _pointwise(Image, "posterize", float(Levels), Low, High) if _is_image(Image) and Levels >= 2 and _finite(Low, High) and High > Low else Image


# ------------------------------------------------------------------------------------------------ channel operations
REC709 = (0.2126, 0.7152, 0.0722)


def Grayscale(Image: OaMatrix) -> OaMatrix:
    """Rec.709 luma of the first three channels -> [N,1,H,W]."""
    if not _is_image(Image) or _t(Image).shape[1] not in (3, 4):
        return Image
    C = _t(Image).shape[1]
    row = list(REC709) + [0.0] * (C - 3) + [0.0]
    return _channels(Image, 1, matrix=[row])


def ChannelReorder(Image: OaMatrix, Channel0: int, Channel1: int = 1, Channel2: int = 2, Channel3: int = 3) -> OaMatrix:
    if not _is_image(Image):
        return Image
    C = _t(Image).shape[1]
    sel = [Channel0, Channel1, Channel2, Channel3][:C]
    if C > 4 or any(s < 0 or s >= C for s in sel):
        return Image
    return _channels(Image, C, sel=sel)


def ColorTwist(Image: OaMatrix, Transform: OaMatrix) -> OaMatrix:
    """rgb' = T[:, :3] rgb + T[:, 3] with a shared 3x4 matrix; a fourth channel passes through."""
    if not _is_image(Image) or _t(Image).shape[1] not in (3, 4) or _t(Transform).numel() != 12:
        return Image
    return _channels(Image, _t(Image).shape[1], twist=_t(Transform))


def Normalize(Image, Params: OaNormalizationParams):
    if isinstance(Image, OaImage):
        return _on_image(Image, lambda m: Normalize(m, Params))
    if not _is_image(Image) or _t(Image).shape[1] > 4 or any(s == 0 or not math.isfinite(s) for s in Params.Std):
        return Image
    C = _t(Image).shape[1]
    rows = []
    for c in range(C):
        row = [0.0] * (C + 1)
        if c < 3:
            row[c], row[C] = 1.0 / Params.Std[c], -Params.Mean[c] / Params.Std[c]
        else:
            row[c] = 1.0
        rows.append(row)
    return _channels(Image, C, matrix=rows)


def AlphaBlend(A: OaMatrix, B: OaMatrix, Alpha: float) -> OaMatrix:
    if not (_is_image(A) and _is_image(B)) or _t(A).shape != _t(B).shape or not _finite(Alpha):
        return A
    return _blend(A, B, None, 0, alpha=Alpha)


def Composite(A: OaMatrix, B: OaMatrix, Mask: OaMatrix) -> OaMatrix:
    """A where the mask is 0, B where it is 1 (mask [N,1,H,W] or [N,C,H,W], clamped to [0,1])."""
    if not (_is_image(A) and _is_image(B) and _is_image(Mask)) or _t(A).shape != _t(B).shape:
        return A
    ta, tm = _t(A), _t(Mask)
    if tm.shape[0] != ta.shape[0] or tm.shape[2:] != ta.shape[2:] or tm.shape[1] not in (1, ta.shape[1]):
        return A
    return _blend(A, B, Mask, 1)


def Erase(Image: OaMatrix, X: int, Y: int, Width: int, Height: int, Value: float = 0.0) -> OaMatrix:
    if not _is_image(Image) or min(X, Y) < 0 or Width <= 0 or Height <= 0 or not _finite(Value):
        return Image
    return _blend(Image, None, None, 2, rect=(X, Y, Width, Height), value=Value)


def SegmentationOverlay(Image: OaMatrix, Mask: OaMatrix, Palette: OaMatrix, Alpha: float = 0.5) -> OaMatrix:
    """Blends palette[label] over the colour channels; labels outside [0, K) leave the pixel unchanged."""
    if not _is_image(Image) or _t(Image).shape[1] not in (3, 4) or not _finite(Alpha):
        return Image
    t, lab, pal = _t(Image).contiguous(), _t(Mask), _t(Palette)
    Nn, C, H, W = t.shape
    if lab.dtype != torch.int32 or lab.numel() != Nn * H * W or pal.dim() != 2 or pal.shape[1] != 3 or pal.dtype != torch.float32:
        return Image
    lab = lab.reshape(Nn, H, W).contiguous()
    a = min(max(float(Alpha), 0.0), 1.0)
    if t.is_cuda:
        out = torch.empty_like(t)
        K._launch(N.require().oa_image_overlay(t.data_ptr(), lab.data_ptr(), pal.contiguous().data_ptr(), out.data_ptr(), Nn, C, H * W,
                                               pal.shape[0], a, N.stream()), "oa_image_overlay")
        return OaMatrix(out)
    ok = (lab >= 0) & (lab < pal.shape[0])
    colour = pal[lab.clamp(0, pal.shape[0] - 1).long()].permute(0, 3, 1, 2)
    out = t.clone()
    out[:, :3] = torch.where(ok[:, None], t[:, :3] * (1 - a) + colour * a, t[:, :3])
    return OaMatrix(out)


# ------------------------------------------------------------------------------------------------ noise
_M32 = 0xFFFFFFFF


def _mix32(v: torch.Tensor) -> torch.Tensor:
    v = v ^ (v >> 16)
    v = (v * 0x85EBCA6B) & _M32
    v = v ^ (v >> 13)
    v = (v * 0xC2B2AE35) & _M32
    return v ^ (v >> 16)


def _uniform_cpu(seed: int, n: int, stream: int) -> torch.Tensor:
    """The counter-based generator of `image_uniform` in image.cu, evaluated with 64-bit integer tensors."""
    lo, hi = seed & _M32, (seed >> 32) & _M32
    i = torch.arange(n, dtype=torch.int64)
    s = lambda x: torch.tensor([x & _M32], dtype=torch.int64)
    v = _mix32(s(lo) ^ _mix32(s(hi + 0x9E3779B9)))
    v = _mix32(v ^ _mix32(((i & _M32) + 0x85EBCA6B) & _M32))
    v = _mix32(v ^ _mix32(((i >> 32) + 0xC2B2AE35) & _M32))
    v = _mix32(v ^ _mix32(s(stream + 0x27D4EB2F)))
    return (v >> 8).float() * (1.0 / 16777216.0)


def _noise(Image: OaMatrix, op: int, p0: float, p1: float, p2: float, seed: int) -> OaMatrix:
    t = _t(Image).contiguous()
    if t.is_cuda:
        out = torch.empty_like(t)
        K._launch(N.require().oa_image_noise(t.data_ptr(), out.data_ptr(), t.numel(), op, float(p0), float(p1), float(p2),
                                             ctypes.c_ulonglong(int(seed) & 0xFFFFFFFFFFFFFFFF), N.stream()), "oa_image_noise")
        return OaMatrix(out)
    u0 = _uniform_cpu(int(seed), t.numel(), 0).reshape(t.shape)
    if op == 0:
        u1 = _uniform_cpu(int(seed), t.numel(), 1).reshape(t.shape)
        return OaMatrix(t + p0 + p1 * torch.sqrt(-2.0 * torch.log(1.0 - u0)) * torch.cos(2 * math.pi * u1))
    half = p0 * 0.5
    out = torch.where(u0 < half, torch.full_like(t, p2), torch.where(u0 >= 1 - half, torch.full_like(t, p1), t))
    return OaMatrix(out)


def GaussianNoise(Image: OaMatrix, Mean: float = 0.0, Stddev: float = 0.01, Seed: int = 0) -> OaMatrix:
    """Image + N(Mean, Stddev) from a counter-based generator keyed by (Seed, element): the same on every device."""
    if not _is_image(Image) or not _finite(Mean, Stddev) or Stddev < 0:
        return Image
    return _noise(Image, 0, Mean, Stddev, 0.0, Seed)


def SaltPepperNoise(Image: OaMatrix, Probability: float = 0.01, SaltValue: float = 1.0, PepperValue: float = 0.0, Seed: int = 0) -> OaMatrix:
    if not _is_image(Image) or not _finite(Probability, SaltValue, PepperValue) or not 0 <= Probability <= 1:
        return Image
    return _noise(Image, 1, Probability, SaltValue, PepperValue, Seed)


# ------------------------------------------------------------------------------------------------ filters
def _odd(k: int, cap: int) -> bool:
    return 0 < k <= cap and (k & 1) == 1


def Convolve2d(Image: OaMatrix, Kernel: OaMatrix, Border: OaBorderMode = OaBorderMode.Reflect101, BorderValue: float = 0.0) -> OaMatrix:
    """Same-shape cross-correlation of every plane with one odd [kh, kw] kernel."""
    if not _is_image(Image) or not _valid_border(Border) or not _finite(BorderValue):
        return Image
    k = _t(Kernel)
    if k.dim() != 2 or not _odd(k.shape[0], 31) or not _odd(k.shape[1], 31) or k.dtype != torch.float32:
        return Image
    return _tile_filter(Image, k.shape[1], k.shape[0], TF_CONV2D, Border, BorderValue, k0=k)


def SeparableConvolve2d(Image: OaMatrix, KernelX: OaMatrix, KernelY: OaMatrix, Border: OaBorderMode = OaBorderMode.Reflect101,
                        BorderValue: float = 0.0) -> OaMatrix:
    if not _is_image(Image) or not _valid_border(Border) or not _finite(BorderValue):
        return Image
    kx, ky = _t(KernelX).reshape(-1), _t(KernelY).reshape(-1)
    if not _odd(kx.numel(), 31) or not _odd(ky.numel(), 31):
        return Image
    return _tile_filter(Image, kx.numel(), ky.numel(), TF_SEPARABLE, Border, BorderValue, k0=kx, k1=ky)


def _const_kernel(vals: Sequence[Sequence[float]]) -> OaMatrix:
    return OaMatrix(torch.tensor(vals, dtype=torch.float32))


def AverageBlur(Image: OaMatrix, KernelWidth: int = 3, KernelHeight: int = 3, Border: OaBorderMode = OaBorderMode.Reflect101) -> OaMatrix:
    if not _is_image(Image) or not _odd(KernelWidth, 31) or not _odd(KernelHeight, 31) or not _valid_border(Border):
        return Image
    kx = torch.full((KernelWidth,), 1.0 / KernelWidth)
    ky = torch.full((KernelHeight,), 1.0 / KernelHeight)
    return _tile_filter(Image, KernelWidth, KernelHeight, TF_SEPARABLE, Border, 0.0, k0=kx, k1=ky)


def _derivative(Image: OaMatrix, Dx: int, Dy: int, Border, smooth: Sequence[float]) -> OaMatrix:
    if not _is_image(Image) or not _valid_border(Border) or (Dx, Dy) not in ((1, 0), (0, 1)):
        return Image
    d, s = torch.tensor([-1.0, 0.0, 1.0]), torch.tensor(list(smooth))
    kx, ky = (d, s) if Dx == 1 else (s, d)
    return _tile_filter(Image, 3, 3, TF_SEPARABLE, Border, 0.0, k0=kx, k1=ky)


def Sobel(Image: OaMatrix, Dx: int = 1, Dy: int = 0, Border: OaBorderMode = OaBorderMode.Reflect101) -> OaMatrix:
    """Signed 3x3 Sobel derivative along x (Dx=1, Dy=0) or y (Dx=0, Dy=1): derivative [-1,0,1] times smoothing [1,2,1]."""
    return _derivative(Image, Dx, Dy, Border, (1.0, 2.0, 1.0))


def Scharr(Image: OaMatrix, Dx: int = 1, Dy: int = 0, Border: OaBorderMode = OaBorderMode.Reflect101) -> OaMatrix:
    return _derivative(Image, Dx, Dy, Border, (3.0, 10.0, 3.0))


def Laplacian(Image: OaMatrix, Border: OaBorderMode = OaBorderMode.Reflect101) -> OaMatrix:
    return Convolve2d(Image, _const_kernel([[0, 1, 0], [1, -4, 1], [0, 1, 0]]), Border)


def Sharpen(Image: OaMatrix, Amount: float = 1.0, Border: OaBorderMode = OaBorderMode.Reflect101) -> OaMatrix:
    if not _finite(Amount) or Amount < 0:
        return Image
    a = float(Amount)
    return Convolve2d(Image, _const_kernel([[0, -a, 0], [-a, 1 + 4 * a, -a], [0, -a, 0]]), Border)


def _gaussian_taps(sigma: float, kernel_size: int) -> torch.Tensor:
    radius = min(int(math.ceil(3.0 * sigma)) if kernel_size == 0 else kernel_size // 2, 15)
    x = torch.arange(-radius, radius + 1, dtype=torch.float64)
    g = torch.exp(-(x * x) / (2.0 * sigma * sigma))
    return (g / g.sum()).float()


def GaussianBlur(Image: OaMatrix, Sigma: float, KernelSize: int = 0) -> OaMatrix:
    """Separable Gaussian, replicated edges; KernelSize 0 picks radius ceil(3 sigma) (at most 15)."""
    if not _is_image(Image) or not _finite(Sigma) or Sigma <= 0 or (KernelSize != 0 and not _odd(KernelSize, 31)):
        return Image
    g = _gaussian_taps(float(Sigma), int(KernelSize))
    return _tile_filter(Image, g.numel(), g.numel(), TF_SEPARABLE, OaBorderMode.Replicate, 0.0, k0=g, k1=g)


def UnsharpMask(Image: OaMatrix, Sigma: float = 1.0, Amount: float = 1.0, KernelSize: int = 0) -> OaMatrix:
    """Image + Amount * (Image - blur): the detail is added back by the blend kernel with alpha = -Amount."""
    if not _is_image(Image) or not _finite(Sigma, Amount) or Sigma <= 0:
        return Image
    blurred = GaussianBlur(Image, Sigma, KernelSize)
    if blurred is Image:
        return Image
    return _blend(Image, blurred, None, 0, alpha=-float(Amount))


def _morph(Image: OaMatrix, kw: int, kh: int, mode: int, Border, BorderValue: float) -> Optional[OaMatrix]:
    if not _is_image(Image) or not _odd(kw, 31) or not _odd(kh, 31) or not _valid_border(Border) or not _finite(BorderValue):
        return None
    return _tile_filter(Image, kw, kh, mode, Border, BorderValue)


def Erode(Image, KernelWidth=3, KernelHeight=3, Border=OaBorderMode.Reflect101, BorderValue=0.0):
    r = _morph(Image, KernelWidth, KernelHeight, TF_MIN, Border, BorderValue)
    return Image if r is None else r


def Dilate(Image, KernelWidth=3, KernelHeight=3, Border=OaBorderMode.Reflect101, BorderValue=0.0):
    r = _morph(Image, KernelWidth, KernelHeight, TF_MAX, Border, BorderValue)
    return Image if r is None else r


def MorphologyOpen(Image, KernelWidth=3, KernelHeight=3, Border=OaBorderMode.Reflect101, BorderValue=0.0):
    e = _morph(Image, KernelWidth, KernelHeight, TF_MIN, Border, BorderValue)
    return Image if e is None else _morph(e, KernelWidth, KernelHeight, TF_MAX, Border, BorderValue)


def MorphologyClose(Image, KernelWidth=3, KernelHeight=3, Border=OaBorderMode.Reflect101, BorderValue=0.0):
    d = _morph(Image, KernelWidth, KernelHeight, TF_MAX, Border, BorderValue)
    return Image if d is None else _morph(d, KernelWidth, KernelHeight, TF_MIN, Border, BorderValue)


def _difference(a: OaMatrix, b: OaMatrix) -> OaMatrix:
    return OaMatrix(K.binary("sub", _t(a), _t(b)))


def MorphologyGradient(Image, KernelWidth=3, KernelHeight=3, Border=OaBorderMode.Reflect101, BorderValue=0.0):
    d = _morph(Image, KernelWidth, KernelHeight, TF_MAX, Border, BorderValue)
    return Image if d is None else _difference(d, _morph(Image, KernelWidth, KernelHeight, TF_MIN, Border, BorderValue))


def MorphologyTopHat(Image, KernelWidth=3, KernelHeight=3, Border=OaBorderMode.Reflect101, BorderValue=0.0):
    o = MorphologyOpen(Image, KernelWidth, KernelHeight, Border, BorderValue)
    return Image if o is Image else _difference(Image, o)


def MorphologyBlackHat(Image, KernelWidth=3, KernelHeight=3, Border=OaBorderMode.Reflect101, BorderValue=0.0):
    c = MorphologyClose(Image, KernelWidth, KernelHeight, Border, BorderValue)
    return Image if c is Image else _difference(c, Image)


def MedianBlur(Image: OaMatrix, KernelSize: int = 3, Border: OaBorderMode = OaBorderMode.Reflect101) -> OaMatrix:
    if not _is_image(Image) or not _odd(KernelSize, 15) or not _valid_border(Border):
        return Image
    return _tile_filter(Image, KernelSize, KernelSize, TF_MEDIAN, Border)


def BilateralFilter(Image: OaMatrix, KernelSize: int = 5, SigmaColor: float = 0.1, SigmaSpace: float = 1.0,
                    Border: OaBorderMode = OaBorderMode.Reflect101) -> OaMatrix:
    if not _is_image(Image) or not _odd(KernelSize, 15) or not _valid_border(Border) or not _finite(SigmaColor, SigmaSpace) \
            or SigmaColor <= 0 or SigmaSpace <= 0:
        return Image
    return _tile_filter(Image, KernelSize, KernelSize, TF_BILATERAL, Border, p0=SigmaSpace, p1=SigmaColor)


def AdaptiveThresholdMean(Image: OaMatrix, KernelSize: int = 11, C: float = 0.0, MaxValue: float = 1.0,
                          Border: OaBorderMode = OaBorderMode.Reflect101) -> OaMatrix:
    """MaxValue where the pixel exceeds (local mean - C), else 0."""
    if not _is_image(Image) or not _odd(KernelSize, 15) or not _valid_border(Border) or not _finite(C, MaxValue):
        return Image
    return _tile_filter(Image, KernelSize, KernelSize, TF_ADAPTIVE_MEAN, Border, p0=1.0, p1=C, p2=MaxValue)


def AdaptiveThresholdGaussian(Image: OaMatrix, KernelSize: int = 11, C: float = 0.0, MaxValue: float = 1.0, Sigma: float = 0.0,
                              Border: OaBorderMode = OaBorderMode.Reflect101) -> OaMatrix:
    if not _is_image(Image) or not _odd(KernelSize, 15) or not _valid_border(Border) or not _finite(C, MaxValue, Sigma) or Sigma < 0:
        return Image
    sigma = Sigma if Sigma > 0 else 0.3 * ((KernelSize - 1.0) * 0.5 - 1.0) + 0.8
    return _tile_filter(Image, KernelSize, KernelSize, TF_ADAPTIVE_GAUSS, Border, p0=sigma, p1=C, p2=MaxValue)


# ------------------------------------------------------------------------------------------------ geometry
def Crop(Image: OaMatrix, X: int, Y: int, Width: int, Height: int) -> OaMatrix:
    if not _is_image(Image):
        return Image
    H, W = _t(Image).shape[2:]
    if min(X, Y) < 0 or Width <= 0 or Height <= 0 or X + Width > W or Y + Height > H:
        return Image
    return _index_map(Image, Height, Width, 0, X, Y)


def CenterCrop(Image: OaMatrix, Width: int, Height: int) -> OaMatrix:
    if not _is_image(Image):
        return Image
    H, W = _t(Image).shape[2:]
    if Width <= 0 or Height <= 0 or Width > W or Height > H:
        return Image
    return Crop(Image, (W - Width) // 2, (H - Height) // 2, Width, Height)


def Flip(Image: OaMatrix, Horizontal: bool = True, Vertical: bool = False) -> OaMatrix:
    if not _is_image(Image):
        return Image
    H, W = _t(Image).shape[2:]
    return _index_map(Image, H, W, 1, int(bool(Horizontal)), int(bool(Vertical)))


def Rotate(Image: OaMatrix, Degrees: int) -> OaMatrix:
    """Clockwise rotation by 90, 180 or 270 degrees."""
    if not _is_image(Image) or Degrees not in (90, 180, 270):
        return Image
    H, W = _t(Image).shape[2:]
    Ho, Wo = (H, W) if Degrees == 180 else (W, H)
    return _index_map(Image, Ho, Wo, 2, Degrees, 0)


def Pad(Image: OaMatrix, Left: int, Right: int, Top: int, Bottom: int, Border: OaBorderMode = OaBorderMode.Constant,
        BorderValue: float = 0.0) -> OaMatrix:
    if not _is_image(Image) or min(Left, Right, Top, Bottom) < 0 or not _valid_border(Border) or not _finite(BorderValue):
        return Image
    H, W = _t(Image).shape[2:]
    return _index_map(Image, H + Top + Bottom, W + Left + Right, 3, Left, Top, Border, BorderValue)


def _resize(t: torch.Tensor, Wo: int, Ho: int, mode: int, norm: Optional[OaNormalizationParams] = None) -> torch.Tensor:
    t = t.contiguous()
    Nn, C, H, W = t.shape
    if t.is_cuda:
        out = torch.empty((Nn, C, Ho, Wo), dtype=torch.float32, device=t.device)
        mean = (ctypes.c_float * 3)(*norm.Mean) if norm else None
        std = (ctypes.c_float * 3)(*norm.Std) if norm else None
        K._launch(N.require().oa_image_resize(t.data_ptr(), out.data_ptr(), Nn * C, C, H, W, Ho, Wo, mode, mean, std, N.stream()),
                  "oa_image_resize")
        return out
    sy_, sx_ = torch.tensor(H / Ho, dtype=torch.float32), torch.tensor(W / Wo, dtype=torch.float32)
    ys, xs = torch.arange(Ho, dtype=torch.float32), torch.arange(Wo, dtype=torch.float32)
    if mode == 0:
        iy = torch.floor(ys * sy_).long().clamp_max(H - 1)
        ix = torch.floor(xs * sx_).long().clamp_max(W - 1)
        out = t[:, :, iy][:, :, :, ix]
    else:
        fy = ((ys + 0.5) * sy_ - 0.5).clamp(0, H - 1)[:, None].expand(Ho, Wo)
        fx = ((xs + 0.5) * sx_ - 0.5).clamp(0, W - 1)[None, :].expand(Ho, Wo)
        out = _bilinear_cpu(t, fy, fx, OaBorderMode.Replicate, 0.0)
    if norm:
        mean = torch.tensor(list(norm.Mean)[:min(C, 3)]).reshape(1, -1, 1, 1)
        std = torch.tensor(list(norm.Std)[:min(C, 3)]).reshape(1, -1, 1, 1)
        out = torch.cat([(out[:, :3] - mean) / std, out[:, 3:]], 1)
    return out.contiguous()


def _resize_axis_matrix(n_in: int, n_out: int, mode: int) -> torch.Tensor:
    """[n_out, n_in] fp32 matrix of the resize along one axis (the forward pass is Wy @ x @ Wx^T)."""
    o = torch.arange(n_out, dtype=torch.float32)
    scale = torch.tensor(n_in / n_out, dtype=torch.float32)
    m = torch.zeros(n_out, n_in, dtype=torch.float32)
    rows = torch.arange(n_out)
    if mode == 0:
        m[rows, torch.floor(o * scale).long().clamp_max(n_in - 1)] = 1.0
        return m
    f = ((o + 0.5) * scale - 0.5).clamp(0, n_in - 1)
    i0 = torch.floor(f).long()
    i1 = (i0 + 1).clamp_max(n_in - 1)
    w = f - i0.float()
    m.index_put_((rows, i0), 1.0 - w, accumulate=True)
    m.index_put_((rows, i1), w, accumulate=True)
    return m


def _resize_bwd(grad: torch.Tensor, H: int, W: int, mode: int) -> torch.Tensor:
    g = grad.contiguous().float()
    Nn, C, Ho, Wo = g.shape
    if g.is_cuda:
        dx = torch.empty((Nn, C, H, W), dtype=torch.float32, device=g.device)
        K._launch(N.require().oa_image_resize_bwd(g.data_ptr(), dx.data_ptr(), Nn * C, H, W, Ho, Wo, mode, N.stream()), "oa_image_resize_bwd")
        return dx
    wy, wx = _resize_axis_matrix(H, Ho, mode), _resize_axis_matrix(W, Wo, mode)
    return torch.einsum("oh,ncow,wv->nchv", wy, g, wx).contiguous()


def ResizeBilinearBwd(GradOutput: OaMatrix, InputHeight: int, InputWidth: int) -> OaMatrix:
    """Gradient of the bilinear `Resize` with respect to its [N, C, InputHeight, InputWidth] input."""
    return OaMatrix(_resize_bwd(_t(GradOutput), int(InputHeight), int(InputWidth), 1))


def ResizeNearestBwd(GradOutput: OaMatrix, InputHeight: int, InputWidth: int) -> OaMatrix:
    """Gradient of the nearest-neighbour `Resize`: every input pixel collects the outputs that copied it."""
    return OaMatrix(_resize_bwd(_t(GradOutput), int(InputHeight), int(InputWidth), 0))


def Resize(Image, Width: int, Height: int, Interpolation: OaInterpolationMode = OaInterpolationMode.Bilinear):
    """Nearest (floor of the scaled coordinate) or bilinear (half-pixel centres, clamped edges) resize.  Records on the
    gradient tape when the input requires a gradient."""
    if isinstance(Image, OaImage):
        return _on_image(Image, lambda m: Resize(m, Width, Height, Interpolation))
    if not _is_image(Image) or Width <= 0 or Height <= 0 or int(Interpolation) not in (0, 1):
        return Image
    t = _t(Image)
    out = OaMatrix(_resize(t, int(Width), int(Height), int(Interpolation)))
    if isinstance(Image, OaMatrix) and Image.RequiresGrad():
        from ..ml import autograd as AG
        H, W, mode = t.shape[-2], t.shape[-1], int(Interpolation)
        return AG.attach("Resize", out, [Image], lambda g: (_resize_bwd(g.reshape(out.Tensor().shape), H, W, mode).reshape(Image.Tensor().shape),))
    return out


def ResizeBatch(Images: Sequence[OaMatrix], TargetWidth: int, TargetHeight: int,
                Mode: OaInterpolationMode = OaInterpolationMode.Bilinear) -> List[OaMatrix]:
    return [Resize(m, TargetWidth, TargetHeight, Mode) for m in Images]


def ResizeNormalize(Image, Width: int, Height: int, Params: OaNormalizationParams):
    """Bilinear resize with the per-channel normalisation applied in the same kernel."""
    if isinstance(Image, OaImage):
        return _on_image(Image, lambda m: ResizeNormalize(m, Width, Height, Params))
    if not _is_image(Image) or Width <= 0 or Height <= 0 or any(s == 0 for s in Params.Std):
        return Image
    return OaMatrix(_resize(_t(Image), int(Width), int(Height), 1, Params))


def Remap(Image: OaMatrix, Map: OaMatrix, Interpolation: OaInterpolationMode = OaInterpolationMode.Bilinear,
          Border: OaBorderMode = OaBorderMode.Constant, BorderValue: float = 0.0) -> OaMatrix:
    """out[n,c,y,x] = Image[n,c] sampled at (Map[n,0,y,x], Map[n,1,y,x]) in absolute pixel coordinates; Map is [N or 1, 2, Ho, Wo]."""
    if not _is_image(Image) or not _valid_border(Border) or not _finite(BorderValue) or int(Interpolation) not in (0, 1):
        return Image
    m = _t(Map)
    if m.dim() != 4 or m.shape[1] != 2 or m.shape[0] not in (1, _t(Image).shape[0]) or m.dtype != torch.float32:
        return Image
    return _warp(Image, m.contiguous(), m.shape[2], m.shape[3], 0, int(Interpolation), int(Border), float(BorderValue))


def WarpAffine(Image: OaMatrix, Transform: OaMatrix, Width: int, Height: int, Interpolation: OaInterpolationMode = OaInterpolationMode.Bilinear,
               Border: OaBorderMode = OaBorderMode.Constant, BorderValue: float = 0.0) -> OaMatrix:
    """Inverse map: the 2x3 transform takes output pixel (x, y) to the source position."""
    if not _is_image(Image) or _t(Transform).numel() != 6 or Width <= 0 or Height <= 0 or not _valid_border(Border) \
            or not _finite(BorderValue) or int(Interpolation) not in (0, 1):
        return Image
    return _warp(Image, _t(Transform).reshape(1, 6), Height, Width, 1, int(Interpolation), int(Border), float(BorderValue))


def WarpPerspective(Image: OaMatrix, Transform: OaMatrix, Width: int, Height: int,
                    Interpolation: OaInterpolationMode = OaInterpolationMode.Bilinear, Border: OaBorderMode = OaBorderMode.Constant,
                    BorderValue: float = 0.0) -> OaMatrix:
    if not _is_image(Image) or _t(Transform).numel() != 9 or Width <= 0 or Height <= 0 or not _valid_border(Border) \
            or not _finite(BorderValue) or int(Interpolation) not in (0, 1):
        return Image
    return _warp(Image, _t(Transform).reshape(1, 9), Height, Width, 2, int(Interpolation), int(Border), float(BorderValue))


# ------------------------------------------------------------------------------------------------ semantic image overloads
def _on_image(image: OaImage, fn, fmt: Optional[OaImageFormat] = None) -> OaImage:
    if image.IsEmpty() or not image.Validate():
        return image
    src = OaMatrix(image.ToNchw().contiguous())
    out = fn(src)
    return image if out is src else image.FromNchw(_t(out), fmt)


_SWAP = {OaImageFormat.Rgb: OaImageFormat.Bgr, OaImageFormat.Bgr: OaImageFormat.Rgb, OaImageFormat.Rgba: OaImageFormat.Bgra,
         OaImageFormat.Bgra: OaImageFormat.Rgba}


def ConvertColor(Image: OaImage, Destination: OaImageFormat) -> OaImage:
    """Conversions among Gray / GrayAlpha / Rgb / Rgba / Bgr / Bgra: one channel-transform launch each (Rec.709 luma toward
    gray, replication away from it, alpha 1 where it is created)."""
    src, dst = Image.Format(), OaImageFormat(Destination)
    if Image.IsEmpty() or not Image.Validate() or Image.Layout() == OaImageLayout.Hw and OaImageFormatChannels(dst) != 1:
        return Image
    if src == dst:
        return Image
    cs, cd = OaImageFormatChannels(src), OaImageFormatChannels(dst)
    colour_s, colour_d = cs >= 3, cd >= 3
    bgr_s, bgr_d = src in (OaImageFormat.Bgr, OaImageFormat.Bgra), dst in (OaImageFormat.Bgr, OaImageFormat.Bgra)
    alpha_s, alpha_d = cs in (2, 4), cd in (2, 4)
    rows = []
    for c in range(cd):
        row = [0.0] * (cs + 1)
        if alpha_d and c == cd - 1:
            if alpha_s:
                row[cs - 1] = 1.0
            else:
                row[cs] = 1.0
        elif colour_d:
            k = 2 - c if bgr_d else c                       # 0 = red, 1 = green, 2 = blue
            if colour_s:
                row[2 - k if bgr_s else k] = 1.0
            else:
                row[0] = 1.0
        else:
            if colour_s:
                for k in range(3):
                    row[2 - k if bgr_s else k] = REC709[k]
            else:
                row[0] = 1.0
        rows.append(row)
    exact = all(sum(1 for v in r[:cs] if v == 1.0) == 1 and all(v in (0.0, 1.0) for v in r) and r[cs] == 0.0 for r in rows)
    if exact:
        sel = [r[:cs].index(1.0) for r in rows]
        return _on_image(Image, lambda m: _channels(m, cd, sel=sel), dst)
    return _on_image(Image, lambda m: _channels(m, cd, matrix=rows), dst)
