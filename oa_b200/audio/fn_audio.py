"""OaFnAudio: waveform operations (return OaAudio) and feature / measurement operations (return OaMatrix).

Reference: Source/Public/Oa/Audio/Type.h (OaAudio: planar fp32 [Channels, Samples] + sample rate + layout; configs) and
Source/Private/Oa/Audio/FnAudio/{Signal/FnAudioSignal.cpp, Transform/FnAudioTransform.cpp} with the kernels under
Audio/Shader/Compute.  The STFT is GEMM-shaped here: windowed frames [C*F, fft] times a [2*bins, fft] cosine / -sine
basis (fp32 GEMM), then magnitudes; the mel filterbank and the MFCC DCT-II are GEMMs too.  Invalid inputs return None
(the reference returns an empty value and logs).
"""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass, field
from functools import lru_cache
from typing import Optional

import torch

from .. import _native as N
from ..core import fn_matrix as F
from ..core.matrix import OaMatrix
from ..ops import kernels as K


class OaChannelLayout(enum.IntEnum):
    Mono = 0
    Stereo = 1
    Surround5_1 = 2
    Surround7_1 = 3
    Unknown = 255


def OaChannelsForLayout(layout: OaChannelLayout) -> int:
    return {OaChannelLayout.Mono: 1, OaChannelLayout.Stereo: 2, OaChannelLayout.Surround5_1: 6, OaChannelLayout.Surround7_1: 8}.get(layout, 0)


def OaLayoutForChannels(channels: int) -> OaChannelLayout:
    return {1: OaChannelLayout.Mono, 2: OaChannelLayout.Stereo, 6: OaChannelLayout.Surround5_1, 8: OaChannelLayout.Surround7_1}.get(channels, OaChannelLayout.Unknown)


class OaAudio:
    """Planar float32 audio [Channels, Samples] with its sample rate and channel layout."""

    def __init__(self, data: Optional[OaMatrix] = None, sample_rate: int = 44100, layout: OaChannelLayout = OaChannelLayout.Mono):
        self.Data_, self.SampleRate_, self.Layout_ = data, int(sample_rate), layout

    def AsMatrix(self) -> Optional[OaMatrix]: return self.Data_
    def IsEmpty(self) -> bool: return self.Data_ is None or self.Data_.IsEmpty()
    def Channels(self) -> int: return 0 if self.IsEmpty() else int(self.Data_.Tensor().shape[0])
    def Samples(self) -> int: return 0 if self.IsEmpty() or self.Data_.Tensor().dim() < 2 else int(self.Data_.Tensor().shape[1])
    def SampleRate(self) -> int: return self.SampleRate_
    def Layout(self) -> OaChannelLayout: return self.Layout_
    def DurationSeconds(self) -> float: return self.Samples() / self.SampleRate_ if self.SampleRate_ > 0 else 0.0

    def Validate(self) -> bool:
        if self.IsEmpty():
            return True
        t = self.Data_.Tensor()
        if t.dim() != 2 or t.shape[0] <= 0 or t.shape[1] <= 0 or self.SampleRate_ == 0 or t.dtype != torch.float32:
            return False
        want = OaChannelsForLayout(self.Layout_)
        return want == 0 or t.shape[0] == want


@dataclass
class OaStftConfig:
    FftSize: int = 1024
    HopSize: int = 256
    WinSize: int = 0          # 0 = FftSize
    Window: int = 0           # 0 Hann, 1 Hamming, 2 Blackman, 3 rectangular
    Center: bool = True


@dataclass
class OaMelConfig:
    FftSize: int = 1024
    HopSize: int = 256
    NumMels: int = 80
    FMin: float = 0.0
    FMax: float = 0.0         # 0 = SampleRate / 2
    LogScale: bool = True
    Normalize: bool = False


@dataclass
class OaMfccConfig:
    NumCoeffs: int = 13
    Mel: OaMelConfig = field(default_factory=OaMelConfig)


@dataclass
class OaResampleConfig:
    OutRate: int = 16000
    FilterHalfWidth: int = 64


@dataclass
class OaNormalizeAudioConfig:
    Mode: int = 0             # 0 peak, 1 RMS
    TargetDb: float = -3.0


LN10_OVER_20_INV = 8.68588963806504


def _ok(a: OaAudio) -> bool:
    return a is not None and a.Validate() and not a.IsEmpty()


def _like(t: torch.Tensor, a: OaAudio) -> OaAudio:
    return OaAudio(OaMatrix(t), a.SampleRate(), a.Layout())


def _db(db: float) -> float:
    return 10.0 ** (db / 20.0)


def _t(a: OaAudio) -> torch.Tensor:
    return F._c(a.AsMatrix().Tensor())


# ---------------------------------------------------------------------------------------------------------- waveform
def Normalize(audio: OaAudio, target_db=-3.0, mode: int = 0) -> Optional[OaAudio]:
    if isinstance(target_db, OaNormalizeAudioConfig):
        target_db, mode = target_db.TargetDb, target_db.Mode
    if not _ok(audio) or not math.isfinite(target_db) or mode not in (0, 1):
        return None
    F._ctx_add("AudioNormalize")
    x = _t(audio)
    level = x.abs().max().item() if mode == 0 else math.sqrt((x * x).mean().item())
    return _like(x * (_db(target_db) / level) if level > 0.0 else x.clone(), audio)


def Gain(audio: OaAudio, gain_db: float) -> Optional[OaAudio]:
    if not _ok(audio) or not math.isfinite(gain_db) or not -300.0 <= gain_db <= 100.0:
        return None
    return _like(F.Scale(audio.AsMatrix(), _db(gain_db)).Tensor(), audio)


def Clip(audio: OaAudio, minimum: float = -1.0, maximum: float = 1.0) -> Optional[OaAudio]:
    if not _ok(audio) or not math.isfinite(minimum) or not math.isfinite(maximum) or minimum > maximum:
        return None
    return _like(F.ClampMax(F.ClampMin(audio.AsMatrix(), minimum), maximum).Tensor(), audio)


def PreEmphasis(audio: OaAudio, alpha: float = 0.97) -> Optional[OaAudio]:
    """y[n] = x[n] - alpha x[n-1] (y[0] = x[0])."""
    if not _ok(audio) or not math.isfinite(alpha):
        return None
    F._ctx_add("AudioPreEmphasis")
    x = _t(audio)
    y = x.clone()
    if x.shape[1] >= 2:
        y[:, 1:] -= alpha * x[:, :-1]
    return _like(y, audio)


def ToMono(audio: OaAudio) -> Optional[OaAudio]:
    if not _ok(audio):
        return None
    x = _t(audio)
    out = x.clone() if x.shape[0] == 1 else F.Mean(audio.AsMatrix(), 0).Tensor().reshape(1, -1)
    return OaAudio(OaMatrix(out), audio.SampleRate(), OaChannelLayout.Mono)


def Fade(audio: OaAudio, fade_in_samples: int, fade_out_samples: int) -> Optional[OaAudio]:
    """Linear ramps: sample s is scaled by s / fade_in at the head and (S - 1 - s) / fade_out at the tail."""
    if not _ok(audio) or fade_in_samples < 0 or fade_out_samples < 0:
        return None
    F._ctx_add("AudioFade")
    x = _t(audio)
    S = x.shape[1]
    fi, fo = min(int(fade_in_samples), S), min(int(fade_out_samples), S)
    if x.is_cuda:
        out = torch.empty_like(x)
        K._launch(N.require().oa_audio_fade(x.data_ptr(), out.data_ptr(), x.numel(), S, fi, fo, N.stream()), "oa_audio_fade")
        return _like(out, audio)
    s = torch.arange(S, dtype=torch.float32)
    env = torch.ones(S)
    if fi > 0:
        env = torch.where(s < fi, s / fi, env)
    if fo > 0:
        rev = S - 1 - s
        env = torch.where(rev < fo, torch.minimum(env, rev / fo), env)
    return _like(x * env, audio)


def Mix(a: OaAudio, b: OaAudio, gain_a: float = 1.0, gain_b: float = 1.0) -> Optional[OaAudio]:
    if not _ok(a) or not _ok(b) or a.SampleRate() != b.SampleRate() or a.Layout() != b.Layout() \
            or a.AsMatrix().Tensor().shape != b.AsMatrix().Tensor().shape or not math.isfinite(gain_a) or not math.isfinite(gain_b):
        return None
    F._ctx_add("AudioMix")
    x, y = _t(a), _t(b)
    if x.is_cuda:
        out = torch.empty_like(x)
        K._launch(N.require().oa_audio_mix(x.data_ptr(), y.data_ptr(), out.data_ptr(), x.numel(), float(gain_a), float(gain_b), N.stream()),
                  "oa_audio_mix")
        return _like(out, a)
    return _like(x * gain_a + y * gain_b, a)


def Resample(audio: OaAudio, out_rate=16000, filter_half_width: int = 64) -> Optional[OaAudio]:
    """Hann-windowed sinc interpolation at exact rational positions; the sinc is scaled to the output Nyquist when
    down-sampling.  Output length = floor(samples * out / in)."""
    if isinstance(out_rate, OaResampleConfig):
        out_rate, filter_half_width = out_rate.OutRate, out_rate.FilterHalfWidth
    if not _ok(audio) or out_rate <= 0 or not 1 <= filter_half_width <= 1024:
        return None
    x = _t(audio)
    in_rate = audio.SampleRate()
    if in_rate == out_rate:
        return _like(x.clone(), audio)
    g = math.gcd(in_rate, out_rate)
    in_r, out_r = in_rate // g, out_rate // g
    C, S = x.shape
    So = S * out_r // in_r
    if So == 0:
        return None
    F._ctx_add("AudioResample")
    if x.is_cuda:
        out = torch.empty(C, So, dtype=torch.float32, device=x.device)
        K._launch(N.require().oa_audio_resample(x.data_ptr(), out.data_ptr(), C, S, So, in_r, out_r, int(filter_half_width), N.stream()),
                  "oa_audio_resample")
        return OaAudio(OaMatrix(out), out_rate, audio.Layout())
    j = torch.arange(So, dtype=torch.int64)
    num = (j % out_r) * in_r
    n0 = (j // out_r) * in_r + num // out_r
    frac = (num % out_r).float() / out_r
    scale, hw = min(1.0, out_r / in_r), float(filter_half_width)
    taps = torch.arange(-filter_half_width, filter_half_width + 1)
    t = taps[None, :].float() - frac[:, None]
    inside = t.abs() <= hw
    st = scale * t
    sinc = torch.where(st.abs() < 1e-7, torch.ones_like(st), torch.sin(math.pi * st) / (math.pi * st))
    kern = torch.where(inside, scale * sinc * 0.5 * (1.0 + torch.cos(math.pi * t / hw)), torch.zeros_like(t))
    ksum = kern.sum(1)
    n = n0[:, None] + taps[None, :]
    valid = (n >= 0) & (n < S)
    vals = x[:, n.clamp(0, S - 1)] * (kern * valid)[None]
    out = torch.where(ksum > 1e-7, vals.sum(-1) / ksum, torch.zeros_like(ksum))
    return OaAudio(OaMatrix(out.contiguous()), out_rate, audio.Layout())


# ---------------------------------------------------------------------------------------------------- measurements
def AmplitudeToDb(audio: OaAudio, floor_db: float = -100.0) -> Optional[OaMatrix]:
    if not _ok(audio) or not math.isfinite(floor_db) or not -300.0 <= floor_db <= 0.0:
        return None
    return F.Scale(F.Log(F.ClampMin(F.Abs(audio.AsMatrix()), _db(floor_db))), LN10_OVER_20_INV)


def WaveformEnvelope(audio: OaAudio, bins: int = 2048) -> Optional[OaMatrix]:
    """[bins, 2] (min, max) over all channels; every sample belongs to exactly one bin."""
    if not _ok(audio) or not 1 <= bins <= 65536:
        return None
    F._ctx_add("AudioWaveformEnvelope")
    x = _t(audio)
    C, S = x.shape
    if x.is_cuda:
        out = torch.empty(bins, 2, dtype=torch.float32, device=x.device)
        K._launch(N.require().oa_audio_envelope(x.data_ptr(), out.data_ptr(), C, S, int(bins), N.stream()), "oa_audio_envelope")
        return OaMatrix(out)
    width, rem = S // bins, S % bins
    out = torch.zeros(bins, 2)
    for b in range(bins):
        begin = b * width + min(b, rem)
        end = begin + width + (1 if b < rem else 0)
        if begin < end:
            seg = x[:, begin:end]
            out[b, 0], out[b, 1] = seg.min(), seg.max()
    return OaMatrix(out)


# ------------------------------------------------------------------------------------------------------- transforms
def _pow2(n: int) -> bool:
    return n > 0 and n & (n - 1) == 0


def _window(win: int, fft: int, kind: int) -> torch.Tensor:
    k = torch.arange(fft, dtype=torch.float32)
    ph = 2.0 * math.pi * k / win
    w = {0: 0.5 * (1 - torch.cos(ph)), 1: 0.54 - 0.46 * torch.cos(ph), 2: 0.42 - 0.5 * torch.cos(ph) + 0.08 * torch.cos(2 * ph),
         3: torch.ones(fft)}[kind]
    return torch.where(k < win, w, torch.zeros(fft))


@lru_cache(maxsize=16)
def _dft_basis(fft: int) -> torch.Tensor:
    """[2*bins, fft]: rows 0..bins-1 = cos(2 pi b k / fft), rows bins.. = -sin(2 pi b k / fft) (float64 angles, fp32 out)."""
    bins = fft // 2 + 1
    ang = 2.0 * math.pi * (torch.arange(bins, dtype=torch.float64)[:, None] * torch.arange(fft, dtype=torch.float64)[None, :] % fft) / fft
    return torch.cat((torch.cos(ang), -torch.sin(ang)), 0).float().contiguous()


def _stft_frames(samples: int, fft: int, hop: int) -> int:
    return 1 if samples < fft else 1 + (samples - fft) // hop


def Stft(audio: OaAudio, cfg: Optional[OaStftConfig] = None) -> Optional[OaMatrix]:
    """Magnitude spectrogram [Channels, Frames, FftSize / 2 + 1]; Center pads FftSize / 2 zeros on both sides; a last
    frame that runs past the end reads zeros."""
    cfg = cfg or OaStftConfig()
    if not _ok(audio) or not _pow2(cfg.FftSize) or not 16 <= cfg.FftSize <= 1024 or cfg.HopSize <= 0:
        return None
    win = cfg.WinSize or cfg.FftSize
    if win > cfg.FftSize or not 0 <= cfg.Window <= 3:
        return None
    F._ctx_add("Stft")
    x = _t(audio)
    C, S = x.shape
    pad = cfg.FftSize // 2 if cfg.Center else 0
    frames = _stft_frames(S + 2 * pad, cfg.FftSize, cfg.HopSize)
    bins = cfg.FftSize // 2 + 1
    basis = _dft_basis(cfg.FftSize).to(x.device)
    if x.is_cuda:
        lib, st = N.require(), N.stream()
        fr = torch.empty(C * frames, cfg.FftSize, dtype=torch.float32, device=x.device)
        K._launch(lib.oa_audio_stft_frame(x.data_ptr(), fr.data_ptr(), C, S, frames, cfg.FftSize, cfg.HopSize, win, cfg.Window, pad, st),
                  "oa_audio_stft_frame")
        reim = K.gemm(fr, basis)
        spec = torch.empty(C * frames, bins, dtype=torch.float32, device=x.device)
        K._launch(lib.oa_audio_magnitude(reim.data_ptr(), spec.data_ptr(), C * frames, bins, st), "oa_audio_magnitude")
        return OaMatrix(spec.reshape(C, frames, bins))
    need = (frames - 1) * cfg.HopSize + cfg.FftSize
    xp = torch.nn.functional.pad(x, (pad, max(0, need - S - pad)))
    fr = xp.unfold(1, cfg.FftSize, cfg.HopSize)[:, :frames] * _window(win, cfg.FftSize, cfg.Window)
    reim = fr.reshape(C * frames, cfg.FftSize) @ basis.t()
    return OaMatrix(torch.sqrt(reim[:, :bins] ** 2 + reim[:, bins:] ** 2).reshape(C, frames, bins))


def _mel_filterbank(cfg: OaMelConfig, sample_rate: int) -> torch.Tensor:
    """HTK mel scale, triangular filters, [NumMels, bins] (fp32 arithmetic as in the reference's host builder)."""
    bins = cfg.FftSize // 2 + 1
    f_max = cfg.FMax if cfg.FMax > 0 else sample_rate * 0.5
    hz2mel = lambda f: 2595.0 * math.log10(1.0 + f / 700.0)
    mel2hz = lambda m: 700.0 * (10.0 ** (m / 2595.0) - 1.0)
    lo, hi = hz2mel(cfg.FMin), hz2mel(f_max)
    pts = torch.tensor([mel2hz(lo + i * (hi - lo) / (cfg.NumMels + 1)) for i in range(cfg.NumMels + 2)], dtype=torch.float32)
    hz = torch.arange(bins, dtype=torch.float32) * (sample_rate / cfg.FftSize)
    l, c, h = pts[:-2, None], pts[1:-1, None], pts[2:, None]
    up = torch.where((hz >= l) & (hz <= c) & (c > l), (hz - l) / (c - l).clamp(min=1e-30), torch.zeros(()))
    down = torch.where((hz > c) & (hz <= h) & (h > c), (h - hz) / (h - c).clamp(min=1e-30), torch.zeros(()))
    return (up + down).contiguous()


def _mel_ok(cfg: OaMelConfig, sample_rate: int) -> bool:
    nyq = sample_rate * 0.5
    f_max = cfg.FMax if cfg.FMax > 0 else nyq
    return (sample_rate > 0 and _pow2(cfg.FftSize) and 16 <= cfg.FftSize <= 1024 and cfg.HopSize > 0 and 0 < cfg.NumMels <= 4096
            and math.isfinite(cfg.FMin) and math.isfinite(f_max) and 0.0 <= cfg.FMin < f_max <= nyq)


def _mel_native(audio: OaAudio, cfg: OaMelConfig) -> Optional[torch.Tensor]:
    """[C, Frames, Mels]"""
    if not _ok(audio) or not _mel_ok(cfg, audio.SampleRate()):
        return None
    spec = Stft(audio, OaStftConfig(cfg.FftSize, cfg.HopSize, cfg.FftSize))
    if spec is None:
        return None
    F._ctx_add("MelFilterbank")
    s = spec.Tensor()
    C, Fr, bins = s.shape
    fb = _mel_filterbank(cfg, audio.SampleRate()).to(s.device)
    mel = K.gemm(s.reshape(C * Fr, bins), fb) if s.is_cuda else s.reshape(C * Fr, bins) @ fb.t()
    if cfg.LogScale:
        mel = torch.log(mel + 1e-9)
    return mel.reshape(C, Fr, cfg.NumMels)


def MelSpectrogram(audio: OaAudio, cfg: Optional[OaMelConfig] = None) -> Optional[OaMatrix]:
    """[Channels, NumMels, Frames] (log(mel + 1e-9) when LogScale; per-channel instance normalisation when Normalize)."""
    cfg = cfg or OaMelConfig()
    mel = _mel_native(audio, cfg)
    if mel is None:
        return None
    out = mel.transpose(1, 2).contiguous()
    if cfg.Normalize:
        flat = out.reshape(out.shape[0], -1)
        cen = flat - flat.mean(1, keepdim=True)
        out = (cen / torch.sqrt((cen * cen).mean(1, keepdim=True) + 1e-5)).reshape(out.shape)
    return OaMatrix(out)


def Mfcc(audio: OaAudio, cfg: Optional[OaMfccConfig] = None) -> Optional[OaMatrix]:
    """[Channels, NumCoeffs, Frames]: orthonormal DCT-II of the log-mel spectrogram."""
    cfg = cfg or OaMfccConfig()
    if cfg.NumCoeffs <= 0 or cfg.NumCoeffs > cfg.Mel.NumMels:
        return None
    mc = OaMelConfig(**{**cfg.Mel.__dict__, "LogScale": True})
    mel = _mel_native(audio, mc)
    if mel is None:
        return None
    F._ctx_add("Mfcc")
    C, Fr, Mn = mel.shape
    k, m = torch.arange(cfg.NumCoeffs, dtype=torch.float32)[:, None], torch.arange(Mn, dtype=torch.float32)[None, :]
    dct = torch.cos(math.pi / Mn * (m + 0.5) * k) * torch.where(k == 0, math.sqrt(1.0 / Mn), math.sqrt(2.0 / Mn))
    dct = dct.to(mel.device).contiguous()
    flat = mel.reshape(C * Fr, Mn).contiguous()
    coef = K.gemm(flat, dct) if mel.is_cuda else flat @ dct.t()
    return OaMatrix(coef.reshape(C, Fr, cfg.NumCoeffs).transpose(1, 2).contiguous())
