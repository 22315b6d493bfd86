"""Baseline JPEG decoder / encoder against the standard's behaviour and, when Pillow is present, against libjpeg (oracle only):
every chroma sampling mode, optimised Huffman tables, restart intervals, greyscale; progressive streams are refused."""
import io

import numpy as np
import pytest

from oa_b200.core.types import OaStatusCode
from oa_b200.vision import jpeg as J
from oa_b200.vision.codec import OaImageIo


def _image(h=70, w=93):
    y, x = np.mgrid[0:h, 0:w]
    return np.stack([127 + 100 * np.sin(x / 9.0), 127 + 100 * np.cos(y / 7.0), ((x * 2 + y) % 256) * 0.5 + 60], -1).clip(0, 255).astype(np.uint8)


def _psnr(a, b):
    return 10 * np.log10(255.0 ** 2 / np.mean((a.astype(float) - b.astype(float)) ** 2))


@pytest.mark.parametrize("subsample", [False, True])
@pytest.mark.parametrize("restart", [0, 3])
def test_encode_decode_round_trip(subsample, restart):
    img = _image()
    blob = J.EncodeJpeg(img, 90, subsample, restart)
    assert blob[:3] == b"\xff\xd8\xff" and blob[-2:] == b"\xff\xd9"
    assert (b"\xff\xdd" in blob) == bool(restart)
    out = J.DecodeJpeg(blob)
    assert out.shape == img.shape and _psnr(out, img) > (42 if subsample else 45)
    assert len(J.EncodeJpeg(img, 30, subsample)) < len(J.EncodeJpeg(img, 95, subsample))


def test_greyscale_odd_sizes_and_alpha():
    g = _image(17, 9)[:, :, 0]
    out = J.DecodeJpeg(J.EncodeJpeg(g, 95))
    assert out.shape == (17, 9, 1) and _psnr(out[:, :, 0], g) > 40
    rgba = np.concatenate([_image(8, 8), np.full((8, 8, 1), 200, np.uint8)], -1)
    assert J.DecodeJpeg(J.EncodeJpeg(rgba)).shape == (8, 8, 3)
    with pytest.raises(ValueError):
        J.EncodeJpeg(np.zeros((4, 4, 2), np.uint8))
    with pytest.raises(ValueError):
        J.DecodeJpeg(b"not a jpeg")


def test_image_io_routes_jpeg(tmp_path):
    img = _image(32, 40)
    blob, st = OaImageIo.EncodeMemory(__import__("oa_b200.core.matrix", fromlist=["OaMatrix"]).OaMatrix(__import__("torch").from_numpy(img)), "jpg")
    assert st.IsOk() and OaImageIo.Detect(blob) == "jpeg"
    dec, st = OaImageIo.DecodeMemory(blob)
    assert st.IsOk() and tuple(dec.AsMatrix().Tensor().shape) == (32, 40, 3)
    cut, st = OaImageIo.DecodeMemory(blob[:200])
    assert cut is None and st.code == OaStatusCode.DataLoss


def test_against_libjpeg():
    Image = pytest.importorskip("PIL.Image")
    img = _image()
    for kw in (dict(quality=85, subsampling=0), dict(quality=75, subsampling=2), dict(quality=75, subsampling=1), dict(quality=60, subsampling=2, optimize=True)):
        b = io.BytesIO()
        Image.fromarray(img).save(b, "JPEG", **kw)
        ours = J.DecodeJpeg(b.getvalue())
        ref = np.array(Image.open(io.BytesIO(b.getvalue())).convert("RGB"))
        d = np.abs(ours.astype(int) - ref)
        assert d.max() <= 3 and d.mean() < 0.7, kw                     # integer vs floating-point inverse DCT and colour conversion
    for sub in (False, True):                                          # libjpeg reads what the encoder writes
        blob = J.EncodeJpeg(img, 90, sub, restart_interval=5)
        ref = np.array(Image.open(io.BytesIO(blob)).convert("RGB"))
        assert _psnr(ref, img) > 42 and np.abs(ref.astype(int) - J.DecodeJpeg(blob)).max() <= 3


def test_progressive_against_libjpeg():
    """Progressive frames (spectral selection + successive approximation, as libjpeg's default scan script writes them) decode to
    libjpeg's pixels within the rounding of the inverse DCT: every sampling, greyscale, restart markers, optimised tables."""
    Image = pytest.importorskip("PIL.Image")
    img = _image(70, 101)
    cases = [dict(quality=90), dict(quality=50, subsampling=0), dict(quality=75, subsampling=2), dict(quality=95, subsampling=1),
             dict(quality=80, restart_marker_blocks=3), dict(quality=80, restart_marker_rows=1), dict(quality=70, optimize=True)]
    for kw in cases:
        for mode in ("RGB", "L"):
            b = io.BytesIO()
            try:
                Image.fromarray(img).convert(mode).save(b, "JPEG", progressive=True, **kw)
            except TypeError:                                           # an older Pillow without the restart options
                continue
            assert b"\xff\xc2" in b.getvalue()
            ref = np.array(Image.open(io.BytesIO(b.getvalue())).convert(mode))
            ref = ref if ref.ndim == 3 else ref[:, :, None]
            ours = J.DecodeJpeg(b.getvalue())
            d = np.abs(ours.astype(int) - ref)
            assert ours.shape == ref.shape and d.max() <= 8 and d.mean() < 0.7, (kw, mode)     # chroma upsampling differs at sharp edges
            base = io.BytesIO()                                         # the sequential file of the same image has the same coefficients
            Image.fromarray(img).convert(mode).save(base, "JPEG", progressive=False, **kw)
            assert np.array_equal(ours, J.DecodeJpeg(base.getvalue())), (kw, mode)
    b = io.BytesIO()
    Image.fromarray(img).save(b, "JPEG", progressive=True)
    dec, st = OaImageIo.DecodeMemory(b.getvalue())
    assert st.IsOk() and tuple(dec.AsMatrix().Tensor().shape) == (70, 101, 3)
    cut, st = OaImageIo.DecodeMemory(b.getvalue()[:len(b.getvalue()) // 3])          # the first scans only: still an image, coarser
    assert cut is not None or st.code == OaStatusCode.DataLoss
