"""Animation language model on small configurations: shapes, a reference CLIP block in plain PyTorch, tokenizer
round trip and training signal, prior conditioning and generation, one-file save / load."""
import math

import pytest
import torch

from oa_b200.core import fn_matrix as F
from oa_b200.core.matrix import OaMatrix
from oa_b200.extensions.alm import (OaAlmAg, OaAlmFfnType, OaAlmPriorAg, OaAlmPriorConfig, OaAlmTokenizerAg, OaAlmTokenizerConfig,
                                    OaClipTextAg, OaClipTextConfig, OaClipTextWeightName, OaClipTokenizer)
from oa_b200.ml import autograd as AG
from oa_b200.ml.optim import OaAdamW


def _clip_cfg():
    return OaClipTextConfig(VocabSize=300, ContextLength=12, HiddenSize=32, IntermediateSize=64, NumHeads=4, NumLayers=2,
                            ProjectionDim=16, BosToken=298, EosToken=299, PadToken=299)


def _clip_reference(model: OaClipTextAg, ids: torch.Tensor) -> torch.Tensor:
    """The same network written with plain tensor operations in fp32."""
    c = model.Config()
    P = {n.Name: n.Param.Data.Tensor().float() for n in model.AllNamedParameterPtrs()}
    B, S = ids.shape
    x = P["token_embedding.weight"][ids.long()] + P["position_embedding.weight"][:S][None]
    mask = torch.full((S, S), float("-inf")).triu(1)
    hd = c.HiddenSize // c.NumHeads
    for i in range(c.NumLayers):
        p = lambda n: P[f"layers.{i}.{n}"]
        h = torch.nn.functional.layer_norm(x, (c.HiddenSize,), p("layer_norm1.weight"), p("layer_norm1.bias"), c.LayerNormEps)
        q, k, v = (h @ p(f"self_attn.{n}_proj.weight").T + p(f"self_attn.{n}_proj.bias") for n in "qkv")
        sp = lambda t: t.view(B, S, c.NumHeads, hd).transpose(1, 2)
        a = torch.softmax(sp(q) @ sp(k).transpose(-1, -2) / math.sqrt(hd) + mask, -1) @ sp(v)
        x = x + a.transpose(1, 2).reshape(B, S, c.HiddenSize) @ p("self_attn.out_proj.weight").T + p("self_attn.out_proj.bias")
        h = torch.nn.functional.layer_norm(x, (c.HiddenSize,), p("layer_norm2.weight"), p("layer_norm2.bias"), c.LayerNormEps)
        h = h @ p("fc1.weight").T + p("fc1.bias")
        x = x + (h * torch.sigmoid(c.QuickGeluAlpha * h)) @ p("fc2.weight").T + p("fc2.bias")
    x = torch.nn.functional.layer_norm(x, (c.HiddenSize,), P["final_layer_norm.weight"], P["final_layer_norm.bias"], c.LayerNormEps)
    eos = (ids == c.EosToken).int().argmax(1)
    return x[torch.arange(B), eos] @ P["text_projection.weight"].T


def test_clip_text_encoder_matches_plain_torch():
    torch.manual_seed(0)
    model = OaClipTextAg(_clip_cfg())
    tok = OaClipTokenizer(config=model.Config())
    ids = tok.EncodeBatch(["a person walks forward", "jump"])
    assert ids.Size(0) == 2 and ids.Size(1) == 12 and int(ids.Tensor()[1, 0]) == 298
    with AG.OaGradNo():
        out = model.Forward(ids).Tensor().float()
        same = model.ForwardTokens(ids, tok.EosRows(ids)).Tensor().float()
    ref = _clip_reference(model, ids.Tensor().cpu())
    assert out.shape == (2, 16) and torch.allclose(out, same) and torch.allclose(out.cpu(), ref, atol=2e-4, rtol=1e-3)
    model.Freeze()
    assert all(not p.Data.RequiresGrad() for p in model.AllParameterPtrs())
    assert not OaClipTextConfig(HiddenSize=30, NumHeads=4).Validate().IsOk()


def test_clip_tokenizer_merges_and_names():
    vocab = {"w": 0, "a": 1, "l": 2, "k</w>": 3, "wa": 4, "wal": 5, "walk</w>": 6, "s</w>": 7, "<|endoftext|>": 9}
    tok = OaClipTokenizer(vocab, [("w", "a"), ("wa", "l"), ("wal", "k</w>")], OaClipTextConfig(VocabSize=12, ContextLength=6, BosToken=10, EosToken=11, PadToken=11))
    assert tok.Encode("Walk  walks") == [10, 6, 5, 9, 7, 11] and tok.Encode("") == [10, 11, 11, 11, 11, 11]
    assert OaClipTextWeightName("text_model.encoder.layers.3.mlp.fc1.weight") == "layers.3.fc1.weight"
    assert OaClipTextWeightName("text_model.encoder.layers.0.self_attn.q_proj.bias") == "layers.0.self_attn.q_proj.bias"
    assert OaClipTextWeightName("text_model.embeddings.token_embedding.weight") == "token_embedding.weight"
    assert OaClipTextWeightName("vision_model.encoder.layers.0.mlp.fc1.weight") is None and OaClipTextWeightName("logit_scale") is None
    model = OaClipTextAg(_clip_cfg())
    names = {n.Name for n in model.AllNamedParameterPtrs()}
    assert {"layers.1.fc2.bias", "layers.0.self_attn.k_proj.weight", "final_layer_norm.bias", "text_projection.weight"} <= names


def _tok_cfg():
    return OaAlmTokenizerConfig(InputDim=11, Width=16, CodeDim=8, NumCodes=12, DownT=2, Depth=1, SeqLen=16)


def test_motion_tokenizer_shapes_and_training_signal():
    torch.manual_seed(1)
    tk = OaAlmTokenizerAg(_tok_cfg())
    assert tk.DownsampleFactor() == 4
    B, T = 3, 16
    x = OaMatrix(torch.randn(B * T, 11))
    with AG.OaGradNo():
        z = tk.Encode(x, B, T)
        assert z.Tensor().shape == (B * 4, 8) and torch.allclose(z.Tensor().float().pow(2).mean(1), torch.ones(B * 4), atol=1e-3)
        idx = tk.Tokenize(x, B, T)
        assert len(idx) == 1 and idx[0].Tensor().numel() == B * 4 and int(idx[0].Tensor().max()) < 12
        recon = tk.Detokenize(idx, B, 4)
        assert recon.Tensor().shape == (B * T, 11)
    with pytest.raises(ValueError):
        tk.Encode(OaMatrix(torch.randn(B * 6, 11)), B, 6)
    opt = OaAdamW(tk.AllParameterPtrs(), 3e-3)
    losses = []
    for _ in range(12):
        with AG.OaGradientTape() as tape:
            loss, res = tk.ReconstructionLoss(x, B, T)
        tape.Backward(loss)
        opt.Step(); opt.ZeroGrad()
        tk.EmaUpdate(res)
        losses.append(float(loss.Tensor()))
    assert all(math.isfinite(l) for l in losses) and min(losses[-3:]) < losses[0]


def test_prior_conditioning_generation_and_moe_layout():
    torch.manual_seed(2)
    cfg = OaAlmPriorConfig(DModel=32, NumHeads=2, NumLayers=2, DFfn=64, TextFeatureDim=16, SeqLen=8, MaxSeqLen=24)
    cfg.SyncVocab(12)
    assert (cfg.VocabSize, cfg.SomToken, cfg.EomToken, cfg.PadToken) == (15, 12, 13, 14)
    prior = OaAlmPriorAg(cfg)
    ids = F.FromInt32([12, 1, 2, 3, 12, 4, 5, 6], [2, 4])
    text = OaMatrix(torch.randn(2, 16))
    with AG.OaGradNo():
        plain, cond = prior.Forward(ids).Tensor(), prior.ForwardConditioned(ids, text).Tensor()
        cond2 = prior.ForwardConditioned(ids, OaMatrix(text.Tensor() * -1)).Tensor()
    assert plain.shape == (2, 4 * 15) and cond.shape == (2, 4 * 15) and not torch.allclose(cond, cond2)
    # causal: changing the last token leaves earlier positions untouched
    ids_b = F.FromInt32([12, 1, 2, 9, 12, 4, 5, 9], [2, 4])
    with AG.OaGradNo():
        other = prior.Forward(ids_b).Tensor()
    assert torch.allclose(plain.view(2, 4, 15)[:, :3], other.view(2, 4, 15)[:, :3], atol=1e-5)
    toks = prior.GenerateConditioned(text, temperature=0.0, max_len=10).Tensor()
    assert toks.shape[0] == 2 and 2 <= toks.shape[1] <= 11 and bool((toks[:, 0] == 12).all()) and int(toks.max()) <= 14
    again = prior.GenerateConditioned(text, temperature=0.0, max_len=10).Tensor()
    assert torch.equal(toks, again)
    sampled = prior.Generate(3, temperature=1.0, top_k=5, top_p=0.9, max_len=6, seed=3).Tensor()
    assert sampled.shape[0] == 3 and bool((sampled[:, 1:] != 12).all())
    with pytest.raises(ValueError):
        prior.ForwardConditioned(ids, OaMatrix(torch.randn(2, 7)))
    hybrid = OaAlmPriorConfig(DModel=32, NumHeads=2, NumLayers=4, DFfn=64, SeqLen=8, MaxSeqLen=16, FfnType=OaAlmFfnType.Hybrid, MoeEvery=2)
    assert [hybrid.UsesMoe(i) for i in range(4)] == [False, True, False, True]
    with pytest.raises(ValueError):
        OaAlmPriorAg(OaAlmPriorConfig(DModel=30, NumHeads=4))


def test_assembled_model_generates_and_round_trips(tmp_path):
    torch.manual_seed(3)
    tk = OaAlmTokenizerAg(_tok_cfg())
    pcfg = OaAlmPriorConfig(DModel=32, NumHeads=2, NumLayers=1, DFfn=64, TextFeatureDim=16, SeqLen=8, MaxSeqLen=24)
    pcfg.SyncVocab(12)
    model = OaAlmAg(tk, OaAlmPriorAg(pcfg), OaClipTextAg(_clip_cfg()))
    motions = model.Generate(["walk", "a person sits down"], temperature=0.0, max_len=6)
    assert len(motions) == 2
    for m in motions:
        assert m.IsEmpty() or (m.Tensor().shape[1] == 11 and m.Tensor().shape[0] % 4 == 0)
    path = tmp_path / "alm.oam"
    assert model.Save(str(path)).IsOk()
    back = OaAlmAg.LoadOam(str(path))
    assert back.Prior.GetConfig().TextFeatureDim == 16 and back.Tokenizer.Config().NumCodes == 12 and back.Text is not None
    a = {n.Name: n.Param.Data.Tensor() for n in model.AllNamedParameterPtrs()}
    b = {n.Name: n.Param.Data.Tensor() for n in back.AllNamedParameterPtrs()}
    assert a.keys() == b.keys() and all(torch.equal(a[k].cpu(), b[k].cpu()) for k in a)
    again = back.Generate(["walk", "a person sits down"], temperature=0.0, max_len=6)
    assert all(x.IsEmpty() == y.IsEmpty() and (x.IsEmpty() or torch.allclose(x.Tensor(), y.Tensor(), atol=1e-5)) for x, y in zip(motions, again))
    bad = OaAlmPriorConfig(DModel=32, NumHeads=2, NumLayers=1, DFfn=64, TextFeatureDim=16, SeqLen=8, MaxSeqLen=24)
    with pytest.raises(ValueError):
        OaAlmAg(tk, OaAlmPriorAg(bad))          # 512 codes against the tokenizer's 12
