"""Lossless WebP (VP8L): files written by libwebp (through Pillow) decode to the pixels libwebp itself decodes, over every feature
its encoder uses (predictor / cross-colour / subtract-green / palette transforms with pixel bundling, LZ77 with the distance map,
colour cache, meta prefix codes, alpha); files written here decode in libwebp and in the own decoder; damaged streams are refused."""
import io

import numpy as np
import pytest
import torch

from oa_b200.core.matrix import OaMatrix
from oa_b200.core.types import OaStatusCode
from oa_b200.vision.codec import OaImageIo
from oa_b200.vision.webp import DecodeWebp, EncodeWebp

PIL = pytest.importorskip("PIL.Image")
from PIL import features  # noqa: E402

HAS_WEBP = bool(features.check("webp"))


def _images():
    rng = np.random.default_rng(7)
    yy, xx = np.mgrid[0:64, 0:96]
    grad = np.stack([(xx * 2) % 256, (yy * 3) % 256, (xx + yy) % 256], -1).astype(np.uint8)
    tile = (rng.random((20, 30, 3)) * 255).astype(np.uint8)
    tiled = np.tile(tile, (5, 4, 1))
    tiled[30:60, 40:90] = 255 - tiled[30:60, 40:90]
    pal4 = rng.integers(0, 255, (4, 3)).astype(np.uint8)[rng.integers(0, 4, (40, 50))]
    pal13 = rng.integers(0, 255, (13, 3)).astype(np.uint8)[rng.integers(0, 13, (33, 47))]
    photo = np.clip(128 + 60 * np.sin(xx / 7.0)[..., None] + 40 * np.cos(yy / 5.0)[..., None] + rng.normal(0, 6, (64, 96, 3)), 0, 255).astype(np.uint8)
    rgba = np.concatenate([grad, ((xx * 5) % 256)[..., None].astype(np.uint8)], -1)
    return {"noise": (rng.random((31, 45, 3)) * 255).astype(np.uint8), "gradient": grad, "tiled": tiled, "palette4": pal4, "palette13": pal13,
            "photo": photo, "rgba": rgba, "flat": np.full((20, 30, 3), 77, np.uint8), "pixel": np.array([[[1, 2, 3]]], np.uint8),
            "column": (rng.random((50, 1, 3)) * 255).astype(np.uint8)}


@pytest.mark.skipif(not HAS_WEBP, reason="Pillow without WebP")
@pytest.mark.parametrize("method", [0, 4, 6])
def test_decodes_what_libwebp_writes(method):
    for name, im in _images().items():
        b = io.BytesIO()
        PIL.fromarray(im).save(b, "WEBP", lossless=True, method=method, quality=100 if method else 50, exact=True)
        want = np.array(PIL.open(io.BytesIO(b.getvalue())).convert("RGBA" if im.shape[2] == 4 else "RGB"))
        got = DecodeWebp(b.getvalue())
        assert got.shape == want.shape and np.array_equal(got, want), (name, method)
        assert np.array_equal(want, im), name                      # lossless: libwebp's own round trip is exact too


def test_own_files_round_trip_and_open_in_libwebp():
    for name, im in _images().items():
        blob = EncodeWebp(im)
        assert blob[:4] == b"RIFF" and blob[8:16] == b"WEBPVP8L" and len(blob) % 2 == 0
        assert np.array_equal(DecodeWebp(blob), im), name
        if HAS_WEBP:
            ref = np.array(PIL.open(io.BytesIO(blob)).convert("RGBA" if im.shape[2] == 4 else "RGB"))
            assert np.array_equal(ref, im), name
    grey = (np.arange(48).reshape(6, 8) * 5).astype(np.uint8)
    assert np.array_equal(DecodeWebp(EncodeWebp(grey))[:, :, 1], grey)                   # grey is written as R = G = B
    flat, runs = EncodeWebp(np.full((64, 64, 3), 9, np.uint8)), EncodeWebp(_images()["noise"])
    assert len(flat) < 400 < len(runs)                                                   # 64 x 64 equal pixels: back references, not 4096 literals


def test_codec_layer_and_refusals(tmp_path):
    im = _images()["gradient"]
    blob, st = OaImageIo.EncodeMemory(OaMatrix(torch.from_numpy(im)), "webp")
    assert st.IsOk() and OaImageIo.Detect(blob) == "webp"
    img, st = OaImageIo.DecodeMemory(blob)
    assert st.IsOk() and np.array_equal(img.AsMatrix().Tensor().numpy(), im)
    assert OaImageIo.EncodeFile(OaMatrix(torch.from_numpy(im)), str(tmp_path / "a.webp")).IsOk()
    assert np.array_equal(OaImageIo.DecodeFile(str(tmp_path / "a.webp"))[0].AsMatrix().Tensor().numpy(), im)
    assert OaImageIo.DecodeMemory(b"RIFF\x10\0\0\0WEBPVP8 \0\0\0\0")[1].code == OaStatusCode.Unimplemented     # lossy stream
    cut = blob[:len(blob) // 2]
    assert OaImageIo.DecodeMemory(cut)[1].code == OaStatusCode.DataLoss
    bad = bytearray(blob)
    bad[20] = 0x00                                                                           # signature byte of the VP8L payload
    assert OaImageIo.DecodeMemory(bytes(bad))[1].code == OaStatusCode.DataLoss
    with pytest.raises(ValueError):
        EncodeWebp(np.zeros((2, 2, 2), np.uint8))
