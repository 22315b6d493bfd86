"""KV-cache decoding against full-window recomputation (CPU), and the decode kernels against their PyTorch statement (GPU)."""
import math

import pytest
import torch

from oa_b200.core import fn_matrix as F
from oa_b200.core.matrix import OaMatrix
from oa_b200.ml import autograd as AG
from oa_b200.models import OaGptConfig, OaGptModel
from oa_b200.ops import kernels as K
from oa_b200.serve import OaGptDecoder


def _full_window_greedy(model, prompt, n):
    ids = prompt.clone()
    with AG.OaGradNo():
        for _ in range(n):
            logits = model.Forward(OaMatrix(ids.contiguous())).Tensor().reshape(ids.shape[0], ids.shape[1], -1)
            ids = torch.cat([ids, logits[:, -1].float().argmax(-1).to(torch.int32).reshape(-1, 1)], 1)
    return ids


@pytest.mark.parametrize("kind", ["rope_swiglu", "learned_gelu"])
def test_cached_generation_matches_full_window(kind):
    F.SetRngSeed(5)
    if kind == "rope_swiglu":
        cfg = OaGptConfig(64, 32, 2, 4, 64, 32, "rms", "swiglu", 10000.0, False, 1e-5, 0.3)
    else:
        cfg = OaGptConfig(64, 32, 2, 4, 64, 32, "layer", "gelu", 0.0, True, 1e-5, 0.3)
    model = OaGptModel(cfg)
    prompt = torch.randint(0, 64, (3, 9), dtype=torch.int32)
    dec = OaGptDecoder(model, batch=3, max_seq=32)
    got = dec.Generate(prompt, 10)
    want = _full_window_greedy(model, prompt, 10)
    assert torch.equal(got, want)
    assert dec.Cache.Length == 9 + 9


@pytest.mark.gpu
@pytest.mark.parametrize("hd", [64, 128])
def test_decode_kernels(hd):
    torch.manual_seed(0)
    B, H, S, L = 3, 4, 300, 261
    kc = torch.zeros(B, H, S, hd, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    qkv = torch.randn(B * L, 3 * H * hd, device="cuda").bfloat16()
    D = H * hd
    K.kv_append(qkv[:, D:2 * D], qkv[:, 2 * D:], kc, vc, B, L, 0)
    kr = qkv[:, D:2 * D].reshape(B, L, H, hd).permute(0, 2, 1, 3)
    assert torch.equal(kc[:, :, :L], kr)
    q = torch.randn(B, 3 * D, device="cuda").bfloat16()
    out = K.decode_attn(q[:, :D], kc, vc, L)
    ref = K.decode_attn(q[:, :D].cpu(), kc.cpu(), vc.cpu(), L)
    assert (out.float().cpu() - ref.float()).abs().max().item() < 2e-2


@pytest.mark.gpu
@pytest.mark.parametrize("hd", [64, 128])
def test_streamed_decode_attention_lengths_and_splits(hd, monkeypatch):
    """The streamed kernel against the fp32 reference for lengths around tile and split edges, with a device-resident
    position, more items than persistent CTAs, and against the one-CTA-per-head kernel it replaces."""
    torch.manual_seed(1)
    B, H, S = 5, 8, 1100
    kc = (torch.randn(B, H, S, hd, device="cuda") * 0.5).bfloat16()
    vc = torch.randn(B, H, S, hd, device="cuda").bfloat16()
    q = torch.randn(B, H * hd, device="cuda").bfloat16()
    kcc, vcc, qc = kc.cpu(), vc.cpu(), q.cpu()
    tile = 64 if hd == 128 else 128
    for L in (1, 7, tile - 1, tile, tile + 1, 3 * tile + 5, 517, 1024, 1100):
        out = K.decode_attn(q, kc, vc, L)
        ref = K.decode_attn(qc, kcc, vcc, L)
        assert (out.float().cpu() - ref.float()).abs().max().item() < 2e-2, L
    pos = torch.tensor([300], dtype=torch.int32, device="cuda")
    out = K.decode_attn(q, kc, vc, 217, pos_dev=pos)
    assert (out.float().cpu() - K.decode_attn(qc, kcc, vcc, 517).float()).abs().max().item() < 2e-2
    monkeypatch.setenv("OA_DECODE_ATTN", "v1")
    old = K.decode_attn(q, kc, vc, 517)
    monkeypatch.delenv("OA_DECODE_ATTN")
    assert (old.float() - K.decode_attn(q, kc, vc, 517).float()).abs().max().item() < 2e-2
    # 40 x 16 heads x 2 splits = 1280 items over 296 persistent CTAs: several items per CTA through one pipeline
    B2, H2, S2 = 40, 16, 600
    k2 = (torch.randn(B2, H2, S2, hd, device="cuda") * 0.5).bfloat16()
    v2 = torch.randn(B2, H2, S2, hd, device="cuda").bfloat16()
    q2 = torch.randn(B2, H2 * hd, device="cuda").bfloat16()
    out = K.decode_attn(q2, k2, v2, 555)
    ref = K.decode_attn(q2.cpu(), k2.cpu(), v2.cpu(), 555)
    assert (out.float().cpu() - ref.float()).abs().max().item() < 2e-2
    K.check_status()


@pytest.mark.gpu
def test_cached_generation_gpu_bf16():
    from oa_b200.runtime import engine as RT
    F.SetRngSeed(5)
    prev = F.GetWeightDtype()
    F.SetWeightDtype(torch.bfloat16)
    try:
        cfg = OaGptConfig(256, 128, 2, 2, 256, 64, "rms", "swiglu", 10000.0, False, 1e-5, 0.2)
        model = OaGptModel(cfg)
        prompt = torch.randint(0, 256, (2, 17), dtype=torch.int32, device="cuda")
        dec = OaGptDecoder(model, batch=2, max_seq=64)
        logits = dec.Prefill(prompt)
        with AG.OaGradNo():
            full = model.Forward(OaMatrix(prompt)).Tensor().reshape(2, 17, -1)[:, -1]
        assert (logits.float() - full.float()).abs().max().item() < 5e-2 * max(1.0, full.float().abs().max().item())
        nxt = logits.float().argmax(-1).to(torch.int32).reshape(-1, 1)
        step = dec.Step(nxt)
        with AG.OaGradNo():
            full2 = model.Forward(OaMatrix(torch.cat([prompt, nxt], 1))).Tensor().reshape(2, 18, -1)[:, -1]
        assert (step.float() - full2.float()).abs().max().item() < 5e-2 * max(1.0, full2.float().abs().max().item())
    finally:
        F.SetWeightDtype(prev)
    K.check_status()
