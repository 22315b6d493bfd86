"""WAV decoding and encoding (Source/Public/Oa/Audio/AudioDecoder.h: LoadFile / LoadMemory; AudioEncoder.h: EncodeWavF32 /
SaveWavF32).  Decodes RIFF/WAVE PCM 8 / 16 / 24 / 32-bit integer and 32 / 64-bit IEEE float (plain and EXTENSIBLE headers)
into planar float32 [channels, samples]; encodes 32-bit float.  FLAC streams go through `flac.py` (written from the format
description, bit exact); MP3 is not part of this build and is rejected with Unimplemented.
"""
from __future__ import annotations

import struct
from typing import Optional, Tuple

import numpy as np
import torch

from ..core.matrix import OaMatrix
from ..core.types import OaStatus, OaStatusCode
from .fn_audio import OaAudio, OaLayoutForChannels


class OaAudioDecoder:
    @staticmethod
    def LoadMemory(data: bytes) -> Tuple[Optional[OaAudio], OaStatus]:
        if data[:4] == b"fLaC":
            from .flac import DecodeFlac
            try:
                pcm_i, rate, bits = DecodeFlac(data)
            except (ValueError, KeyError, IndexError, struct.error) as e:
                return None, OaStatus(OaStatusCode.DataLoss, f"corrupt FLAC stream: {e}")
            x = torch.from_numpy((pcm_i.astype(np.float64) / float(1 << (bits - 1))).astype(np.float32))
            return OaAudio(OaMatrix(x.contiguous()), int(rate), OaLayoutForChannels(x.shape[0])), OaStatus.Ok()
        if data[:3] == b"ID3" or (len(data) > 1 and data[0] == 0xFF and (data[1] & 0xE0) == 0xE0):
            return None, OaStatus(OaStatusCode.Unimplemented, "MP3 decoding is not part of this build")
        if len(data) < 12 or data[:4] != b"RIFF" or data[8:12] != b"WAVE":
            return None, OaStatus(OaStatusCode.InvalidArgument, "not a RIFF/WAVE stream")
        pos, fmt, pcm = 12, None, None
        while pos + 8 <= len(data):
            tag, size = data[pos:pos + 4], struct.unpack("<I", data[pos + 4:pos + 8])[0]
            body = data[pos + 8:pos + 8 + size]
            if tag == b"fmt ":
                fmt = body
            elif tag == b"data":
                pcm = body
            pos += 8 + size + (size & 1)
        if fmt is None or pcm is None or len(fmt) < 16:
            return None, OaStatus(OaStatusCode.DataLoss, "WAVE stream lacks a format or a data chunk")
        kind, channels, rate, _, _, bits = struct.unpack("<HHIIHH", fmt[:16])
        if kind == 0xFFFE and len(fmt) >= 26:
            kind = struct.unpack("<H", fmt[24:26])[0]
        if channels == 0 or rate == 0:
            return None, OaStatus(OaStatusCode.DataLoss, "WAVE format names no channels or no sample rate")
        frame = channels * bits // 8
        n = len(pcm) // frame if frame else 0
        raw = np.frombuffer(pcm[:n * frame], dtype=np.uint8)
        if kind == 1 and bits == 8:
            x = (raw.astype(np.float32) - 128.0) / 128.0
        elif kind == 1 and bits == 16:
            x = raw.view("<i2").astype(np.float32) / 32768.0
        elif kind == 1 and bits == 24:
            b = raw.reshape(-1, 3).astype(np.int32)
            v = b[:, 0] | (b[:, 1] << 8) | (b[:, 2] << 16)
            x = np.where(v & 0x800000, v - (1 << 24), v).astype(np.float32) / 8388608.0
        elif kind == 1 and bits == 32:
            x = (raw.view("<i4").astype(np.float64) / 2147483648.0).astype(np.float32)
        elif kind == 3 and bits == 32:
            x = raw.view("<f4").astype(np.float32)
        elif kind == 3 and bits == 64:
            x = raw.view("<f8").astype(np.float32)
        else:
            return None, OaStatus(OaStatusCode.Unimplemented, f"WAVE format tag {kind} with {bits} bits is not supported")
        planar = torch.from_numpy(np.ascontiguousarray(x.reshape(n, channels).T))
        return OaAudio(OaMatrix(planar), rate, OaLayoutForChannels(channels)), OaStatus.Ok()

    @staticmethod
    def LoadFile(path: str) -> Tuple[Optional[OaAudio], OaStatus]:
        try:
            with open(path, "rb") as f:
                return OaAudioDecoder.LoadMemory(f.read())
        except OSError as e:
            return None, OaStatus(OaStatusCode.NotFound, str(e))


class OaAudioEncoder:
    @staticmethod
    def EncodeWavF32(audio: OaAudio) -> Tuple[Optional[bytes], OaStatus]:
        if audio.IsEmpty() or not audio.Validate():
            return None, OaStatus(OaStatusCode.InvalidArgument, "audio must be a non-empty planar fp32 [channels, samples] clip")
        t = audio.AsMatrix().Tensor().detach().float().cpu()
        c, n = t.shape
        pcm = t.T.contiguous().numpy().astype("<f4").tobytes()
        fmt = struct.pack("<HHIIHH", 3, c, audio.SampleRate(), audio.SampleRate() * c * 4, c * 4, 32)
        fact = struct.pack("<I", n)
        body = b"WAVE" + b"fmt " + struct.pack("<I", len(fmt)) + fmt + b"fact" + struct.pack("<I", 4) + fact + b"data" + struct.pack("<I", len(pcm)) + pcm
        return b"RIFF" + struct.pack("<I", len(body)) + body, OaStatus.Ok()

    @staticmethod
    def SaveWavF32(audio: OaAudio, path: str) -> OaStatus:
        blob, st = OaAudioEncoder.EncodeWavF32(audio)
        if blob is None:
            return st
        try:
            with open(path, "wb") as f:
                f.write(blob)
        except OSError as e:
            return OaStatus(OaStatusCode.Unavailable, str(e))
        return OaStatus.Ok()
