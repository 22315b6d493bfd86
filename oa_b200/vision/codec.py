"""Still-image codecs: PNG, BMP, TGA, PPM / PGM and baseline JPEG, decode and encode, to and from uint8 HWC tensors.

The reference's image codec layer (Source/Private/Oa/Vision: JPEG / PNG / BMP / TGA / WebP through bundled decoders)
feeds `OaImage`; here the lossless formats are implemented directly (PNG inflate / deflate through zlib, all five scanline
filters, 8-bit grey / grey-alpha / RGB / RGBA / palette, 16-bit reduced to 8) and baseline JPEG is written out from the
standard in `jpeg.py` (sequential and progressive frames).  Lossless WebP (VP8L) is decoded and encoded by `webp.py`; lossy WebP
(VP8) is rejected with Unimplemented; video codecs need the vendor's decode engine through a graphics API and are unavailable here.
"""
from __future__ import annotations

import enum
import struct
import zlib
from typing import Optional, Tuple

import numpy as np
import torch

from ..core.matrix import OaMatrix
from ..core.types import OaStatus, OaStatusCode
from .fn_image import OaImage, OaImageFormat, OaImageLayout

_PNG_SIG = b"\x89PNG\r\n\x1a\n"


def _fmt(channels: int) -> OaImageFormat:
    return {1: OaImageFormat.Gray, 3: OaImageFormat.Rgb, 4: OaImageFormat.Rgba}.get(channels, OaImageFormat.Rgb)


def _unfilter(raw: np.ndarray, height: int, stride: int, bpp: int) -> np.ndarray:
    out = np.zeros((height, stride), dtype=np.uint8)
    prev = np.zeros(stride, dtype=np.int32)
    pos = 0
    for y in range(height):
        ft = int(raw[pos]); line = raw[pos + 1:pos + 1 + stride].astype(np.int32); pos += 1 + stride
        if ft == 0:
            cur = line
        elif ft == 2:
            cur = (line + prev) & 255
        elif ft == 1:
            cur = line.copy()
            for i in range(bpp, stride):
                cur[i] = (cur[i] + cur[i - bpp]) & 255
        elif ft == 3:
            cur = line.copy()
            for i in range(stride):
                left = cur[i - bpp] if i >= bpp else 0
                cur[i] = (cur[i] + ((left + prev[i]) >> 1)) & 255
        elif ft == 4:
            cur = line.copy()
            for i in range(stride):
                a = cur[i - bpp] if i >= bpp else 0
                b = prev[i]
                c = prev[i - bpp] if i >= bpp else 0
                p = a + b - c
                pa, pb, pc = abs(p - a), abs(p - b), abs(p - c)
                pred = a if (pa <= pb and pa <= pc) else (b if pb <= pc else c)
                cur[i] = (cur[i] + pred) & 255
        else:
            raise ValueError(f"unknown PNG filter {ft}")
        out[y] = cur
        prev = cur
    return out


def DecodePng(data: bytes) -> np.ndarray:
    if data[:8] != _PNG_SIG:
        raise ValueError("not a PNG stream")
    pos, idat, palette, trns, ihdr = 8, [], None, None, None
    while pos + 8 <= len(data):
        n, tag = struct.unpack(">I4s", data[pos:pos + 8])
        body = data[pos + 8:pos + 8 + n]
        crc = struct.unpack(">I", data[pos + 8 + n:pos + 12 + n])[0]
        if zlib.crc32(tag + body) != crc:
            raise ValueError(f"PNG chunk {tag!r} fails its checksum")
        if tag == b"IHDR":
            ihdr = struct.unpack(">IIBBBBB", body)
        elif tag == b"PLTE":
            palette = np.frombuffer(body, dtype=np.uint8).reshape(-1, 3)
        elif tag == b"tRNS":
            trns = np.frombuffer(body, dtype=np.uint8)
        elif tag == b"IDAT":
            idat.append(body)
        elif tag == b"IEND":
            break
        pos += 12 + n
    if ihdr is None:
        raise ValueError("PNG stream has no header")
    w, h, depth, ctype, _, _, interlace = ihdr
    if interlace:
        raise NotImplementedError("interlaced PNG")
    channels = {0: 1, 2: 3, 3: 1, 4: 2, 6: 4}[ctype]
    if depth not in (8, 16) and not (ctype in (0, 3) and depth in (1, 2, 4)):
        raise ValueError("unsupported PNG bit depth")
    bits = channels * depth
    stride, bpp = (w * bits + 7) // 8, max(1, bits // 8)
    px = _unfilter(np.frombuffer(zlib.decompress(b"".join(idat)), dtype=np.uint8), h, stride, bpp)
    if depth == 16:
        px = px.reshape(h, w * channels, 2)[:, :, 0]                     # keep the high byte
    elif depth < 8:
        per = 8 // depth
        shifts = np.arange(per - 1, -1, -1, dtype=np.uint8) * depth
        px = ((px[:, :, None] >> shifts) & ((1 << depth) - 1)).reshape(h, -1)[:, :w]
        if ctype == 0:
            px = (px.astype(np.uint16) * 255 // ((1 << depth) - 1)).astype(np.uint8)
    img = px.reshape(h, w, channels)
    if ctype == 3:
        if palette is None:
            raise ValueError("palette PNG without a palette")
        rgb = palette[img[:, :, 0]]
        if trns is not None:
            alpha = np.full(256, 255, dtype=np.uint8); alpha[:len(trns)] = trns
            rgb = np.concatenate([rgb, alpha[img[:, :, 0]][:, :, None]], axis=2)
        img = rgb
    elif ctype == 4:
        img = np.concatenate([np.repeat(img[:, :, :1], 3, axis=2), img[:, :, 1:]], axis=2)
    return np.ascontiguousarray(img)


def EncodePng(img: np.ndarray, level: int = 6) -> bytes:
    h, w, c = img.shape
    ctype = {1: 0, 3: 2, 4: 6}[c]
    raw = np.concatenate([np.zeros((h, 1), dtype=np.uint8), img.reshape(h, w * c)], axis=1).tobytes()     # filter 0 on every line

    def chunk(tag: bytes, body: bytes) -> bytes:
        return struct.pack(">I", len(body)) + tag + body + struct.pack(">I", zlib.crc32(tag + body))

    return _PNG_SIG + chunk(b"IHDR", struct.pack(">IIBBBBB", w, h, 8, ctype, 0, 0, 0)) + chunk(b"IDAT", zlib.compress(raw, level)) + chunk(b"IEND", b"")


def DecodeBmp(data: bytes) -> np.ndarray:
    if data[:2] != b"BM" or len(data) < 54:
        raise ValueError("not a BMP stream")
    offset = struct.unpack("<I", data[10:14])[0]
    w, h, _, bits, comp = struct.unpack("<iiHHI", data[18:34])
    if comp not in (0, 3) or bits not in (8, 24, 32):
        raise NotImplementedError("compressed or low-depth BMP")
    flip = h > 0
    h = abs(h)
    stride = ((w * bits + 31) // 32) * 4
    rows = np.frombuffer(data, dtype=np.uint8, count=stride * h, offset=offset).reshape(h, stride)
    if bits == 8:
        pal = np.frombuffer(data, dtype=np.uint8, count=256 * 4, offset=54).reshape(256, 4)[:, [2, 1, 0]]
        img = pal[rows[:, :w]]
    else:
        n = bits // 8
        px = rows[:, :w * n].reshape(h, w, n)
        img = px[:, :, [2, 1, 0]] if n == 3 else px[:, :, [2, 1, 0, 3]]
    return np.ascontiguousarray(img[::-1] if flip else img)


def EncodeBmp(img: np.ndarray) -> bytes:
    h, w, c = img.shape
    if c == 1:
        img = np.repeat(img, 3, axis=2)
    n = img.shape[2]
    bgr = img[:, :, [2, 1, 0]] if n == 3 else img[:, :, [2, 1, 0, 3]]
    stride = ((w * n * 8 + 31) // 32) * 4
    rows = np.zeros((h, stride), dtype=np.uint8)
    rows[:, :w * n] = bgr[::-1].reshape(h, w * n)
    head = b"BM" + struct.pack("<IHHI", 54 + stride * h, 0, 0, 54) + struct.pack("<IiiHHIIiiII", 40, w, h, 1, n * 8, 0, stride * h, 2835, 2835, 0, 0)
    return head + rows.tobytes()


def DecodeTga(data: bytes) -> np.ndarray:
    idlen, cmap, kind = data[0], data[1], data[2]
    w, h, bits, desc = struct.unpack("<HHBB", data[12:18])
    if cmap or kind not in (2, 3, 10, 11) or bits not in (8, 24, 32):
        raise NotImplementedError("colour-mapped or low-depth TGA")
    n, pos = bits // 8, 18 + idlen
    if kind in (2, 3):
        px = np.frombuffer(data, dtype=np.uint8, count=w * h * n, offset=pos).reshape(h * w, n)
    else:                                                           # run-length packets
        out = np.empty((w * h, n), dtype=np.uint8); i = 0
        while i < w * h:
            head = data[pos]; pos += 1
            count = (head & 127) + 1
            if head & 128:
                out[i:i + count] = np.frombuffer(data, dtype=np.uint8, count=n, offset=pos); pos += n
            else:
                out[i:i + count] = np.frombuffer(data, dtype=np.uint8, count=n * count, offset=pos).reshape(count, n); pos += n * count
            i += count
        px = out
    img = px.reshape(h, w, n)
    if n >= 3:
        img = img[:, :, [2, 1, 0] + ([3] if n == 4 else [])]
    return np.ascontiguousarray(img if desc & 0x20 else img[::-1])


def EncodeTga(img: np.ndarray) -> bytes:
    h, w, c = img.shape
    px = img if c == 1 else img[:, :, [2, 1, 0] + ([3] if c == 4 else [])]
    head = struct.pack("<BBBHHBHHHHBB", 0, 0, 3 if c == 1 else 2, 0, 0, 0, 0, 0, w, h, c * 8, 0x20 | (8 if c == 4 else 0))
    return head + np.ascontiguousarray(px).tobytes()


def DecodePnm(data: bytes) -> np.ndarray:
    parts, pos = [], 0
    while len(parts) < 4:
        while data[pos:pos + 1].isspace():
            pos += 1
        if data[pos:pos + 1] == b"#":
            pos = data.index(b"\n", pos) + 1
            continue
        end = pos
        while not data[end:end + 1].isspace():
            end += 1
        parts.append(data[pos:end]); pos = end
    magic, w, h, mx = parts[0], int(parts[1]), int(parts[2]), int(parts[3])
    if magic not in (b"P5", b"P6") or mx != 255:
        raise NotImplementedError("only binary 8-bit PGM / PPM")
    c = 1 if magic == b"P5" else 3
    return np.frombuffer(data, dtype=np.uint8, count=w * h * c, offset=pos + 1).reshape(h, w, c).copy()


def EncodePnm(img: np.ndarray) -> bytes:
    h, w, c = img.shape
    if c not in (1, 3):
        raise ValueError("PGM / PPM hold 1 or 3 channels")
    return (b"P5" if c == 1 else b"P6") + f"\n{w} {h}\n255\n".encode() + np.ascontiguousarray(img).tobytes()


class OaImageIo:
    """Decode to / encode from `OaImage` (uint8 HWC on the host; `ToFloat` gives the planar fp32 NCHW form the image
    operations work on)."""

    @staticmethod
    def Detect(data: bytes) -> str:
        if data[:8] == _PNG_SIG: return "png"
        if data[:2] == b"BM": return "bmp"
        if data[:2] in (b"P5", b"P6"): return "pnm"
        if data[:3] == b"\xff\xd8\xff": return "jpeg"
        if data[:4] == b"RIFF" and data[8:12] == b"WEBP": return "webp"
        return "tga" if len(data) >= 18 and data[2] in (2, 3, 10, 11) and data[16] in (8, 24, 32) else "unknown"

    @staticmethod
    def DecodeMemory(data: bytes) -> Tuple[Optional[OaImage], OaStatus]:
        kind = OaImageIo.Detect(data)
        from .jpeg import DecodeJpeg
        from .webp import DecodeWebp
        fn = {"png": DecodePng, "bmp": DecodeBmp, "tga": DecodeTga, "pnm": DecodePnm, "jpeg": DecodeJpeg, "webp": DecodeWebp}.get(kind)
        if fn is None:
            return None, OaStatus(OaStatusCode.InvalidArgument, "unrecognised image stream")
        try:
            px = fn(data)
        except NotImplementedError as e:
            return None, OaStatus(OaStatusCode.Unimplemented, str(e))
        except (ValueError, KeyError, IndexError, struct.error, zlib.error) as e:
            return None, OaStatus(OaStatusCode.DataLoss, f"corrupt {kind} stream: {e}")
        return OaImage(OaMatrix(torch.from_numpy(np.array(px))), OaImageLayout.Hwc, _fmt(px.shape[2])), OaStatus.Ok()

    @staticmethod
    def DecodeFile(path: str) -> Tuple[Optional[OaImage], OaStatus]:
        try:
            with open(path, "rb") as f:
                return OaImageIo.DecodeMemory(f.read())
        except OSError as e:
            return None, OaStatus(OaStatusCode.NotFound, str(e))

    @staticmethod
    def _pixels(image) -> np.ndarray:
        t = (image.AsMatrix() if isinstance(image, OaImage) else image).Tensor().detach().cpu()
        if isinstance(image, OaImage):
            layout = image.Layout()
        elif t.dim() == 4:
            layout = OaImageLayout.Nchw                       # bare matrices are planar, as the image operations produce them
        else:
            layout = OaImageLayout.Hwc if t.dim() == 3 and t.shape[2] <= 4 else OaImageLayout.Chw
        if t.dim() == 4:
            if t.shape[0] != 1:
                raise ValueError("one image per file")
            t = t[0]
            layout = OaImageLayout.Chw if layout == OaImageLayout.Nchw else OaImageLayout.Hwc
        if t.dim() == 2:
            t = t[:, :, None]
        elif layout == OaImageLayout.Chw:
            t = t.permute(1, 2, 0)
        if t.is_floating_point():
            t = (t.clamp(0, 1) * 255.0 + 0.5).floor()
        return np.ascontiguousarray(t.to(torch.uint8).numpy())

    @staticmethod
    def EncodeMemory(image, kind: str = "png") -> Tuple[Optional[bytes], OaStatus]:
        from .jpeg import EncodeJpeg
        from .webp import EncodeWebp
        fn = {"png": EncodePng, "bmp": EncodeBmp, "tga": EncodeTga, "pnm": EncodePnm, "ppm": EncodePnm, "pgm": EncodePnm, "jpg": EncodeJpeg,
              "jpeg": EncodeJpeg, "webp": EncodeWebp}.get(kind.lower())
        if fn is None:
            return None, OaStatus(OaStatusCode.Unimplemented, f"no encoder for '{kind}'")
        try:
            return fn(OaImageIo._pixels(image)), OaStatus.Ok()
        except (ValueError, KeyError) as e:
            return None, OaStatus(OaStatusCode.InvalidArgument, str(e))

    @staticmethod
    def EncodeFile(image, path: str) -> OaStatus:
        blob, st = OaImageIo.EncodeMemory(image, path.rsplit(".", 1)[-1])
        if blob is None:
            return st
        with open(path, "wb") as f:
            f.write(blob)
        return OaStatus.Ok()

    @staticmethod
    def ToFloat(image: OaImage) -> OaMatrix:
        """uint8 HWC -> fp32 [1, C, H, W] in [0, 1]."""
        t = image.AsMatrix().Tensor()
        return OaMatrix((t.permute(2, 0, 1).float() / 255.0).unsqueeze(0).contiguous())


# ------------------------------------------------------------------------------------------ the reference's codec surface
class OaImageCodec(enum.IntEnum):
    Auto = 0
    Jpeg = 1
    Png = 2
    Webp = 3
    Bmp = 4
    Tga = 5


class OaPixelFormat(enum.IntEnum):
    """Storage formats of image tensors (distinct from OaImageFormat, which names the meaning of the channels)."""
    NV12 = 0
    RGB8 = 1
    RGBA8 = 2
    BF16 = 3
    F32 = 4


class OaFilter(enum.IntEnum):
    Nearest = 0
    Linear = 1


_KIND = {OaImageCodec.Png: "png", OaImageCodec.Bmp: "bmp", OaImageCodec.Tga: "tga", OaImageCodec.Jpeg: "jpeg", OaImageCodec.Webp: "webp"}


def _convert(image: OaImage, fmt: OaImageFormat) -> OaImage:
    """Decoded pixels brought to the requested channel meaning (grey <-> colour, alpha added or dropped)."""
    t = image.AsMatrix().Tensor()
    want = {OaImageFormat.Gray: 1, OaImageFormat.Rgb: 3, OaImageFormat.Rgba: 4}.get(fmt)
    c = t.shape[2]
    if want is None or want == c:
        return image
    if c == 1:
        t = t.expand(-1, -1, 3)
        c = 3
    if want == 1:
        w = torch.tensor([0.299, 0.587, 0.114])
        t = (t[:, :, :3].float() * w).sum(2, keepdim=True).round().clamp(0, 255).to(torch.uint8)
    elif want == 3:
        t = t[:, :, :3]
    elif want == 4 and c == 3:
        t = torch.cat([t, torch.full_like(t[:, :, :1], 255)], 2)
    return OaImage(OaMatrix(t.contiguous()), OaImageLayout.Hwc, fmt)


class OaImageDecoder:
    @staticmethod
    def Supports(codec: OaImageCodec) -> bool:
        return OaImageCodec(codec) in (OaImageCodec.Auto, OaImageCodec.Png, OaImageCodec.Bmp, OaImageCodec.Tga, OaImageCodec.Jpeg, OaImageCodec.Webp)

    @staticmethod
    def LoadMemory(Data: bytes, Format: OaImageFormat = OaImageFormat.Rgb) -> OaImage:
        img, st = OaImageIo.DecodeMemory(bytes(Data))
        if img is None:
            raise RuntimeError(st.message)
        return _convert(img, Format)

    @staticmethod
    def LoadFile(Path, Format: OaImageFormat = OaImageFormat.Rgb) -> OaImage:
        img, st = OaImageIo.DecodeFile(str(Path))
        if img is None:
            raise RuntimeError(st.message)
        return _convert(img, Format)


class OaImageEncoder:
    @staticmethod
    def Supports(codec: OaImageCodec) -> bool:
        return OaImageCodec(codec) in _KIND

    @staticmethod
    def Encode(Image: OaImage, Codec: OaImageCodec, Quality: int = 90) -> bytes:
        """`Quality` applies to lossy codecs only (baseline JPEG here; WebP is written lossless)."""
        if not OaImageEncoder.Supports(Codec):
            raise RuntimeError(f"no encoder for {OaImageCodec(Codec).name} in this build")
        blob, st = OaImageIo.EncodeMemory(Image, _KIND[OaImageCodec(Codec)])
        if blob is None:
            raise RuntimeError(st.message)
        return blob

    @staticmethod
    def SaveFile(Path, Image: OaImage, Quality: int = 90) -> None:
        st = OaImageIo.EncodeFile(Image, str(Path))
        if not st.IsOk():
            raise RuntimeError(st.message)


class OaImageBatch(OaImage):
    """An OaImage that must carry a batch axis (NCHW or NHWC)."""

    def Validate(self) -> bool:
        return self.Layout() in (OaImageLayout.Nchw, OaImageLayout.Nhwc) and super().Validate()

    def Dtype(self):
        return None if self.IsEmpty() else self.AsMatrix().Tensor().dtype
