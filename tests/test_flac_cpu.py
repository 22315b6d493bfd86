"""FLAC decoder (and the compact encoder that feeds it): bit-exact round trips over every subframe type, stereo decorrelation,
bit depths and block sizes; CRC and MD5 checks; a stream written by the reference FLAC encoder when one is at hand."""
import hashlib
import os

import numpy as np
import pytest

from oa_b200.audio import flac as F
from oa_b200.audio.codec import OaAudioDecoder
from oa_b200.core.types import OaStatusCode


def _signal(n=9000, seed=0):
    rng = np.random.default_rng(seed)
    t = np.arange(n)
    left = (8000 * np.sin(t * 0.03) + 3000 * np.sin(t * 0.11 + 1) + rng.normal(0, 40, n)).astype(np.int64)
    right = (7000 * np.sin(t * 0.03 + 0.2) + rng.normal(0, 40, n)).astype(np.int64)
    return left, right


def test_crcs():
    assert F.crc8(b"") == 0 and F.crc8(b"123456789") == 0xF4           # CRC-8 (poly 0x07)
    assert F.crc16(b"123456789") == 0xFEE8                             # CRC-16/UMTS (poly 0x8005, MSB first, init 0)


@pytest.mark.parametrize("case", ["stereo16", "mono16", "stereo24", "noise8", "constant", "short_block", "three_channels"])
def test_lossless_round_trip(case):
    left, right = _signal()
    rng = np.random.default_rng(1)
    x, bps, block = {"stereo16": (np.stack([left, right]), 16, 1152), "mono16": (left[None], 16, 4096), "stereo24": (np.stack([left, right]) * 200, 24, 1152),
                     "noise8": (rng.integers(-128, 128, (1, 5000)), 8, 576), "constant": (np.full((2, 3000), -7), 16, 1000),
                     "short_block": (np.stack([left, right])[:, :37], 16, 16), "three_channels": (np.stack([left, right, left // 2]), 16, 2000)}[case]
    blob = F.EncodeFlac(x, 44100, bps, block)
    y, rate, b = F.DecodeFlac(blob)
    assert np.array_equal(x, y) and (rate, b) == (44100, bps)
    if case in ("stereo16", "mono16", "stereo24"):
        assert len(blob) < 0.7 * x.size * bps / 8                        # the predictors and Rice coding do compress
    if case == "noise8":
        assert len(blob) < 1.05 * x.size                                # incompressible data falls back to VERBATIM


def test_subframe_types_are_all_exercised():
    """One block per subframe type: a constant, noise (VERBATIM), a cubic (FIXED order 4: zero residual), a resonant signal (LPC)."""
    n = 2048
    t = np.arange(n)
    rng = np.random.default_rng(2)
    cubic = (t ** 3 // 4000 - 3 * t ** 2 // 7 + 11 * t).astype(np.int64) % 30000 - 15000
    poly = ((t - 1000) ** 3 // 200000).astype(np.int64)
    reson = np.zeros(n)
    e = rng.normal(0, 50, n)
    for i in range(2, n):                                                # a two-pole resonator: an order-2+ LPC predictor wins clearly
        reson[i] = 1.8 * reson[i - 1] - 0.95 * reson[i - 2] + e[i]
    kinds = {}
    for name, sig in (("const", np.full(n, 5)), ("noise", rng.integers(-30000, 30000, n)), ("poly", poly), ("reson", np.rint(reson).astype(np.int64))):
        w = F._Writer()
        F._encode_subframe(w, sig.astype(np.int64), 16)
        kinds[name] = w.out[0] >> 1
        assert np.array_equal(F.DecodeFlac(F.EncodeFlac(sig[None], 8000, 16, n))[0][0], sig)
    assert kinds["const"] == 0 and kinds["noise"] == 1 and 8 <= kinds["poly"] <= 12 and kinds["reson"] >= 32, kinds


def test_corruption_is_detected():
    left, right = _signal(3000)
    blob = bytearray(F.EncodeFlac(np.stack([left, right]), 8000, 16, 1000))
    bad = bytes(blob[:200]) + bytes([blob[200] ^ 0x10]) + bytes(blob[201:])
    with pytest.raises(ValueError, match="CRC|Huffman|sync|reserved|ends|MD5|partition"):
        F.DecodeFlac(bad)
    md5_off = 4 + 4 + 18
    wrong = bytes(blob[:md5_off]) + bytes(16 * [0xAA]) + bytes(blob[md5_off + 16:])
    with pytest.raises(ValueError, match="MD5"):
        F.DecodeFlac(wrong)
    assert np.array_equal(F.DecodeFlac(wrong, verify_md5=False)[0][0], left)
    with pytest.raises(ValueError):
        F.DecodeFlac(bytes(blob[:-7]))
    with pytest.raises(ValueError):
        F.EncodeFlac(np.array([[40000]]), 8000, 16)


def test_audio_decoder_reads_flac():
    left, right = _signal(2000)
    a, st = OaAudioDecoder.LoadMemory(F.EncodeFlac(np.stack([left, right]), 22050, 16, 500))
    assert st.IsOk() and a.Channels() == 2 and a.SampleRate() == 22050
    assert np.allclose(a.AsMatrix().Tensor().numpy(), np.stack([left, right]) / 32768.0)
    assert OaAudioDecoder.LoadMemory(b"fLaC" + bytes(50))[1].code == OaStatusCode.DataLoss


def test_stream_of_the_reference_encoder():
    """A file written by libFLAC: decoding must reproduce the MD5 signature its encoder stored."""
    path = os.environ.get("OA_FLAC_SAMPLE", "")
    if not path or not os.path.exists(path):
        pytest.skip("OA_FLAC_SAMPLE does not name a FLAC file written by another encoder")
    data = open(path, "rb").read()
    x, rate, bps = F.DecodeFlac(data)                                    # raises on an MD5 mismatch
    assert x.shape[0] >= 1 and x.shape[1] > 1000 and rate > 0
    assert hashlib.md5(F.PcmBytes(x, bps)).digest() == data[26:42]
