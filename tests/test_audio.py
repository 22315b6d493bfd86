"""OaFnAudio against torch.stft / closed forms on CPU; the CUDA kernels against the CPU path."""
import math

import pytest
import torch

from oa_b200.audio import fn_audio as A
from oa_b200.core.matrix import OaMatrix


def _audio(device="cpu", C=2, S=4000, rate=16000, seed=0):
    g = torch.Generator().manual_seed(seed)
    t = torch.arange(S) / rate
    x = torch.stack([0.5 * torch.sin(2 * math.pi * (440 + 220 * c) * t) + 0.05 * torch.randn(S, generator=g) for c in range(C)])
    return A.OaAudio(OaMatrix(x.float().to(device)), rate, A.OaLayoutForChannels(C))


def test_audio_value_and_signal_ops_cpu():
    a = _audio()
    assert a.Validate() and a.Channels() == 2 and a.Samples() == 4000 and abs(a.DurationSeconds() - 0.25) < 1e-9
    assert not A.OaAudio(OaMatrix(torch.zeros(3, 10)), 16000, A.OaChannelLayout.Stereo).Validate()
    x = a.AsMatrix().Tensor()
    n = A.Normalize(a, -6.0, 0).AsMatrix().Tensor()
    assert abs(n.abs().max().item() - 10 ** (-6 / 20)) < 1e-5
    r = A.Normalize(a, A.OaNormalizeAudioConfig(1, -20.0)).AsMatrix().Tensor()
    assert abs(math.sqrt((r * r).mean().item()) - 0.1) < 1e-5
    assert torch.allclose(A.Gain(a, 6.0).AsMatrix().Tensor(), x * 10 ** 0.3, atol=1e-6) and A.Gain(a, 500.0) is None
    assert A.Clip(a, -0.1, 0.1).AsMatrix().Tensor().abs().max() <= 0.1 + 1e-7 and A.Clip(a, 1.0, -1.0) is None
    p = A.PreEmphasis(a, 0.97).AsMatrix().Tensor()
    assert torch.allclose(p[:, 1:], x[:, 1:] - 0.97 * x[:, :-1], atol=1e-6) and torch.equal(p[:, 0], x[:, 0])
    m = A.ToMono(a)
    assert m.Layout() == A.OaChannelLayout.Mono and torch.allclose(m.AsMatrix().Tensor()[0], x.mean(0), atol=1e-6)
    f = A.Fade(a, 100, 200).AsMatrix().Tensor()
    assert f[0, 0] == 0 and torch.allclose(f[:, 50], x[:, 50] * 0.5) and f[0, -1] == 0 and torch.allclose(f[:, -101], x[:, -101] * 0.5)
    assert torch.equal(f[:, 1000], x[:, 1000])
    mix = A.Mix(a, a, 0.25, 0.5).AsMatrix().Tensor()
    assert torch.allclose(mix, 0.75 * x, atol=1e-6) and A.Mix(a, _audio(S=100)) is None
    db = A.AmplitudeToDb(a, -80.0).Tensor()
    assert torch.allclose(db, 20 * torch.log10(x.abs().clamp(min=1e-4)), atol=1e-4)
    env = A.WaveformEnvelope(a, 7).Tensor()
    assert env.shape == (7, 2) and abs(env[:, 0].min().item() - x.min().item()) < 1e-7 and abs(env[:, 1].max().item() - x.max().item()) < 1e-7
    assert torch.allclose(env[0], torch.stack((x[:, :572].min(), x[:, :572].max())))


def test_resample_preserves_tones_cpu():
    a = _audio(C=1, S=8000, rate=16000, seed=1)
    down = A.Resample(a, 8000, 32)
    assert down.SampleRate() == 8000 and down.Samples() == 4000
    t = torch.arange(4000) / 8000
    want = 0.5 * torch.sin(2 * math.pi * 440 * t)
    got = down.AsMatrix().Tensor()[0]
    assert (got - want)[100:-100].abs().mean() < 0.05             # the 440 Hz tone survives; the added noise is mostly removed
    up = A.Resample(a, A.OaResampleConfig(24000, 16))
    assert up.Samples() == 12000
    same = A.Resample(a, 16000)
    assert torch.equal(same.AsMatrix().Tensor(), a.AsMatrix().Tensor()) and A.Resample(a, 0) is None


def test_stft_mel_mfcc_match_torch_cpu():
    a = _audio(C=2, S=4000)
    x = a.AsMatrix().Tensor()
    for center, kind, win in ((True, 0, 0), (False, 1, 200)):
        cfg = A.OaStftConfig(256, 64, win, kind, center)
        got = A.Stft(a, cfg).Tensor()
        w = {0: torch.hann_window, 1: torch.hamming_window}[kind](win or 256, periodic=True)
        w = torch.nn.functional.pad(w, (0, 256 - (win or 256)))
        xin = torch.nn.functional.pad(x, (128, 128)) if center else x
        ref = torch.stft(xin, 256, 64, 256, window=w, center=False, return_complex=True).abs().transpose(1, 2)
        assert got.shape == ref.shape == (2, got.shape[1], 129), (got.shape, ref.shape)
        assert (got - ref).abs().max() < 2e-3
    peak = A.Stft(a, A.OaStftConfig(512, 128)).Tensor()[0].mean(0).argmax().item()
    assert abs(peak * 16000 / 512 - 440) < 32
    mel = A.MelSpectrogram(a, A.OaMelConfig(256, 64, 20)).Tensor()
    assert mel.shape[:2] == (2, 20) and torch.isfinite(mel).all()
    lin = A.MelSpectrogram(a, A.OaMelConfig(256, 64, 20, LogScale=False)).Tensor()
    assert torch.allclose(mel, torch.log(lin + 1e-9), atol=1e-5) and lin.min() >= 0
    nrm = A.MelSpectrogram(a, A.OaMelConfig(256, 64, 20, Normalize=True)).Tensor()
    assert abs(nrm[0].mean().item()) < 1e-4 and abs(nrm[0].std(unbiased=False).item() - 1) < 1e-2
    mf = A.Mfcc(a, A.OaMfccConfig(13, A.OaMelConfig(256, 64, 20))).Tensor()
    assert mf.shape == (2, 13, mel.shape[2])
    k, m = torch.arange(13.0)[:, None], torch.arange(20.0)[None, :]
    dct = torch.cos(math.pi / 20 * (m + 0.5) * k) * torch.where(k == 0, math.sqrt(1 / 20), math.sqrt(2 / 20))
    assert torch.allclose(mf, torch.einsum("km,cmf->ckf", dct, mel), atol=1e-4)
    assert A.Stft(a, A.OaStftConfig(300, 64)) is None and A.Mfcc(a, A.OaMfccConfig(40, A.OaMelConfig(256, 64, 20))) is None
    assert A.MelSpectrogram(a, A.OaMelConfig(256, 64, 20, FMax=9000.0)) is None


@pytest.mark.gpu
def test_audio_kernels_match_cpu_path():
    from oa_b200.ops import kernels as K
    ac, ag = _audio("cpu", 2, 20000), _audio("cuda", 2, 20000)
    eq = lambda f, tol=1e-5: (f(ac).AsMatrix().Tensor() - f(ag).AsMatrix().Tensor().cpu()).abs().max().item() < tol
    assert eq(lambda a: A.Fade(a, 1000, 3000)) and eq(lambda a: A.Mix(a, a, 0.3, 0.6)) and eq(lambda a: A.Resample(a, 11025, 32), 1e-4)
    assert eq(lambda a: A.Resample(a, 48000, 16), 1e-4)
    assert torch.equal(A.WaveformEnvelope(ac, 333).Tensor(), A.WaveformEnvelope(ag, 333).Tensor().cpu())
    for cfg in (A.OaStftConfig(1024, 256), A.OaStftConfig(64, 16, 48, 2, False)):
        c, g = A.Stft(ac, cfg).Tensor(), A.Stft(ag, cfg).Tensor().cpu()
        assert c.shape == g.shape and (c - g).abs().max() < 1e-3 * max(1.0, c.abs().max().item())
    mc, mg = A.Mfcc(ac).Tensor(), A.Mfcc(ag).Tensor().cpu()
    assert mc.shape == mg.shape and (mc - mg).abs().max() < 5e-3
    K.check_status()
