"""Image and audio codecs (round trips, a hand-built filtered PNG, corrupt input) and the framed TCP transport."""
import struct
import threading
import zlib

import numpy as np
import pytest
import torch

from oa_b200.audio.codec import OaAudioDecoder, OaAudioEncoder
from oa_b200.audio.fn_audio import OaAudio, OaChannelLayout
from oa_b200.core.matrix import OaMatrix
from oa_b200.core.types import OaStatusCode
from oa_b200.network import OaTcpFramed, OaTcpListener, OaTcpStream
from oa_b200.vision.codec import DecodePng, OaImageIo as OaImageCodec, _PNG_SIG
from oa_b200.vision.fn_image import OaImage, OaImageFormat, OaImageLayout


@pytest.mark.parametrize("kind,channels", [("png", 1), ("png", 3), ("png", 4), ("bmp", 3), ("bmp", 4), ("tga", 1), ("tga", 3), ("tga", 4),
                                           ("ppm", 3), ("pgm", 1)])
def test_image_round_trips(kind, channels, tmp_path):
    px = np.random.default_rng(channels).integers(0, 256, size=(13, 7, channels), dtype=np.uint8)
    img = OaImage(OaMatrix(torch.from_numpy(px)), OaImageLayout.Hwc, {1: OaImageFormat.Gray, 3: OaImageFormat.Rgb, 4: OaImageFormat.Rgba}[channels])
    path = str(tmp_path / f"x.{kind}")
    assert OaImageCodec.EncodeFile(img, path).IsOk()
    back, st = OaImageCodec.DecodeFile(path)
    assert st.IsOk() and back.Layout() == OaImageLayout.Hwc and back.Height() == 13 and back.Width() == 7
    got = back.AsMatrix().Tensor().numpy()
    want = np.repeat(px, 3, axis=2) if (kind == "bmp" and channels == 1) else px
    assert np.array_equal(got, want)
    f = OaImageCodec.ToFloat(back).Tensor()
    assert f.shape == (1, channels, 13, 7) and float(f.max()) <= 1.0
    blob, st = OaImageCodec.EncodeMemory(OaMatrix(f), "png")                 # planar fp32 in, same pixels out
    assert st.IsOk() and np.array_equal(DecodePng(blob), px)


def _png(w, h, ctype, depth, lines, extra=b""):
    chunk = lambda tag, body: struct.pack(">I", len(body)) + tag + body + struct.pack(">I", zlib.crc32(tag + body))
    return _PNG_SIG + chunk(b"IHDR", struct.pack(">IIBBBBB", w, h, depth, ctype, 0, 0, 0)) + extra + chunk(b"IDAT", zlib.compress(b"".join(lines))) \
        + chunk(b"IEND", b"")


def test_png_filters_palette_and_depths():
    # 3 x 5 RGB image stored with filters Sub, Up, Average, Paeth and None
    px = np.random.default_rng(0).integers(0, 256, size=(5, 3, 3), dtype=np.int32)
    flat, lines, prev = px.reshape(5, 9), [], np.zeros(9, dtype=np.int32)
    for y, ft in enumerate([1, 2, 3, 4, 0]):
        cur, enc = flat[y], np.zeros(9, dtype=np.int32)
        for i in range(9):
            a = cur[i - 3] if i >= 3 else 0
            b, c = prev[i], (prev[i - 3] if i >= 3 else 0)
            p = a + b - c
            paeth = a if (abs(p - a) <= abs(p - b) and abs(p - a) <= abs(p - c)) else (b if abs(p - b) <= abs(p - c) else c)
            pred = [0, a, b, (a + b) >> 1, paeth][ft]
            enc[i] = (cur[i] - pred) & 255
        lines.append(bytes([ft]) + enc.astype(np.uint8).tobytes())
        prev = cur
    assert np.array_equal(DecodePng(_png(3, 5, 2, 8, lines)), px.astype(np.uint8))
    chunk = lambda tag, body: struct.pack(">I", len(body)) + tag + body + struct.pack(">I", zlib.crc32(tag + body))
    pal = bytes([255, 0, 0, 0, 255, 0, 0, 0, 255, 9, 9, 9])
    out = DecodePng(_png(4, 1, 3, 2, [bytes([0, 0b00011011])], chunk(b"PLTE", pal) + chunk(b"tRNS", bytes([255, 128]))))
    assert out.shape == (1, 4, 4) and out[0, :, :3].tolist() == [[255, 0, 0], [0, 255, 0], [0, 0, 255], [9, 9, 9]] and out[0, :, 3].tolist() == [255, 128, 255, 255]
    assert DecodePng(_png(2, 1, 0, 16, [bytes([0, 0x12, 0x34, 0xAB, 0xCD])]))[0, :, 0].tolist() == [0x12, 0xAB]
    assert DecodePng(_png(8, 1, 0, 1, [bytes([0, 0b10100000])]))[0, :, 0].tolist() == [255, 0, 255, 0, 0, 0, 0, 0]
    good = _png(1, 1, 0, 8, [bytes([0, 7])])
    bad = bytearray(good); bad[-20] ^= 0xFF
    img, st = OaImageCodec.DecodeMemory(bytes(bad))
    assert img is None and st.code == OaStatusCode.DataLoss
    assert OaImageCodec.DecodeMemory(b"\xff\xd8\xff\xe0rest")[1].code == OaStatusCode.DataLoss          # JPEG signature, no image behind it
    assert OaImageCodec.DecodeMemory(b"RIFF\0\0\0\0WEBPVP8 ")[1].code == OaStatusCode.Unimplemented
    assert OaImageCodec.DecodeMemory(b"garbage")[1].code == OaStatusCode.InvalidArgument


def test_tga_run_length():
    body = bytes([0x82, 10, 20, 30]) + bytes([0x01, 1, 2, 3, 4, 5, 6])          # 3 x (10,20,30) BGR, then two raw pixels
    head = struct.pack("<BBBHHBHHHHBB", 0, 0, 10, 0, 0, 0, 0, 0, 5, 1, 24, 0x20)
    img, st = OaImageCodec.DecodeMemory(head + body)
    assert st.IsOk() and img.AsMatrix().Tensor()[0].tolist() == [[30, 20, 10]] * 3 + [[3, 2, 1], [6, 5, 4]]


def test_wav_round_trip_and_integer_formats(tmp_path):
    x = torch.stack([torch.sin(torch.linspace(0, 20, 500)), torch.linspace(-1, 1, 500)])
    clip = OaAudio(OaMatrix(x), 16000, OaChannelLayout.Stereo)
    path = str(tmp_path / "a.wav")
    assert OaAudioEncoder.SaveWavF32(clip, path).IsOk()
    back, st = OaAudioDecoder.LoadFile(path)
    assert st.IsOk() and back.SampleRate() == 16000 and back.Channels() == 2 and torch.equal(back.AsMatrix().Tensor(), x) and back.Validate()

    def wav(kind, bits, pcm, channels=1):
        fmt = struct.pack("<HHIIHH", kind, channels, 8000, 8000 * channels * bits // 8, channels * bits // 8, bits)
        body = b"WAVE" + b"fmt " + struct.pack("<I", 16) + fmt + b"LIST" + struct.pack("<I", 3) + b"abc\0" + b"data" + struct.pack("<I", len(pcm)) + pcm
        return b"RIFF" + struct.pack("<I", len(body)) + body

    a16, _ = OaAudioDecoder.LoadMemory(wav(1, 16, struct.pack("<4h", 0, 16384, -32768, 32767)))
    assert a16.AsMatrix().Tensor()[0].tolist() == [0.0, 0.5, -1.0, 32767 / 32768]
    a8, _ = OaAudioDecoder.LoadMemory(wav(1, 8, bytes([128, 255, 0])))
    assert a8.AsMatrix().Tensor()[0].tolist() == [0.0, 127 / 128, -1.0]
    a24, _ = OaAudioDecoder.LoadMemory(wav(1, 24, bytes([0, 0, 0x40, 0, 0, 0x80]), 2))
    assert a24.Channels() == 2 and a24.AsMatrix().Tensor()[:, 0].tolist() == [0.5, -1.0]
    assert OaAudioDecoder.LoadMemory(b"fLaC....")[1].code == OaStatusCode.DataLoss                  # FLAC marker, nothing behind it
    assert OaAudioDecoder.LoadMemory(b"ID3\x04rest")[1].code == OaStatusCode.Unimplemented
    assert OaAudioDecoder.LoadMemory(b"nope")[1].code == OaStatusCode.InvalidArgument
    assert OaAudioDecoder.LoadMemory(wav(7, 8, b"\0"))[1].code == OaStatusCode.Unimplemented
    assert OaAudioEncoder.EncodeWavF32(OaAudio())[0] is None


def test_framed_tcp_echo():
    listener, st = OaTcpListener.Bind(0)
    assert st.IsOk() and listener.Port() > 0
    got = []

    def serve():
        peer, st = listener.Accept(timeout=10)
        while True:
            msg, st = OaTcpFramed.ReadMessage(peer)
            if msg is None:
                break
            got.append(msg)
            OaTcpFramed.WriteMessage(peer, msg[::-1])
        peer.Close()

    th = threading.Thread(target=serve)
    th.start()
    c, st = OaTcpStream.Connect("127.0.0.1", listener.Port())
    assert st.IsOk() and c.IsOpen() and c.RemotePort() == listener.Port()
    big = bytes(range(256)) * 4000
    for payload in (b"hello", b"", big):
        assert OaTcpFramed.WriteMessage(c, payload).IsOk()
        back, st = OaTcpFramed.ReadMessage(c)
        assert st.IsOk() and back == payload[::-1]
    c.Close()
    th.join(10)
    assert got == [b"hello", b"", big] and not c.IsOpen() and c.Write(b"x") == -1
    assert OaTcpFramed.ReadU32Le(OaTcpFramed.WriteU32Le(0xDEADBEEF)) == 0xDEADBEEF and OaTcpFramed.ReadU32Le(b"ab") is None
    assert listener.Accept(timeout=0.05)[1].code == OaStatusCode.DeadlineExceeded
    listener.Close()
    assert OaTcpStream.Connect("127.0.0.1", 1, timeout=1.0)[0] is None


def test_reference_codec_surface_and_hash_types(tmp_path):
    import oa
    px = np.random.default_rng(9).integers(0, 256, size=(6, 5, 3), dtype=np.uint8)
    img = OaImage(OaMatrix(torch.from_numpy(px)), OaImageLayout.Hwc, OaImageFormat.Rgb)
    blob = oa.OaImageEncoder.Encode(img, oa.OaImageCodec.Png)
    assert oa.OaImageDecoder.Supports(oa.OaImageCodec.Png) and oa.OaImageDecoder.Supports(oa.OaImageCodec.Jpeg)
    assert oa.OaImageEncoder.Supports(oa.OaImageCodec.Tga) and oa.OaImageEncoder.Supports(oa.OaImageCodec.Webp)
    webp = oa.OaImageEncoder.Encode(img, oa.OaImageCodec.Webp)
    assert webp[:4] == b"RIFF" and np.array_equal(oa.OaImageDecoder.LoadMemory(webp).AsMatrix().Tensor().numpy(), px)
    back = oa.OaImageDecoder.LoadMemory(blob)
    assert np.array_equal(back.AsMatrix().Tensor().numpy(), px) and back.Format() == OaImageFormat.Rgb
    grey = oa.OaImageDecoder.LoadMemory(blob, OaImageFormat.Gray).AsMatrix().Tensor()
    want = np.round(px[:, :, 0] * 0.299 + px[:, :, 1] * 0.587 + px[:, :, 2] * 0.114)
    assert grey.shape == (6, 5, 1) and np.abs(grey[:, :, 0].numpy().astype(np.int32) - want).max() <= 1
    rgba = oa.OaImageDecoder.LoadMemory(blob, OaImageFormat.Rgba).AsMatrix().Tensor()
    assert rgba.shape == (6, 5, 4) and bool((rgba[:, :, 3] == 255).all())
    oa.OaImageEncoder.SaveFile(tmp_path / "x.bmp", img)
    assert np.array_equal(oa.OaImageDecoder.LoadFile(tmp_path / "x.bmp").AsMatrix().Tensor().numpy(), px)
    jpg = oa.OaImageDecoder.LoadMemory(oa.OaImageEncoder.Encode(img, oa.OaImageCodec.Jpeg)).AsMatrix().Tensor()
    assert jpg.shape == (6, 5, 3)
    with pytest.raises(RuntimeError):
        oa.OaImageDecoder.LoadMemory(b"\xff\xd8\xff\xe0....")
    batch = oa.OaImageBatch(OaMatrix(torch.rand(2, 3, 4, 4)), OaImageLayout.Nchw, OaImageFormat.Rgb)
    assert batch.Validate() and batch.BatchSize() == 2 and batch.Dtype() == torch.float32
    assert not oa.OaImageBatch(OaMatrix(torch.rand(3, 4, 4)), OaImageLayout.Chw, OaImageFormat.Rgb).Validate()
    assert oa.OaPixelFormat.NV12 == 0 and oa.OaFilter.Linear == 1
    import hashlib
    h = oa.OaHasher().Update(b"ab").Update(b"c").Finalize()
    assert h.Bytes() == hashlib.shake_256(b"abc").digest(32) and h == oa.OaHash.FromHex(h.ToHex()) and len(h.ToShortHex()) == 8
    assert oa.OaHash.Zero().IsZero() and not h.IsZero() and repr(h).startswith("OaHash(") and oa.OaHash.Of(b"abc") == h
    with pytest.raises(ValueError):
        oa.OaHash(b"short")
    hs = oa.OaHasher(); hs.Update(b"x"); hs.Reset()
    assert hs.Finalize() == oa.OaHash.Of(b"")
    assert oa.OaLinearWeightBiasBwdResult is not None
    for name in ("OaVideoStream", "OaVideoRecorder", "OaScreenCapture"):
        with pytest.raises(AttributeError):
            getattr(oa, name)
