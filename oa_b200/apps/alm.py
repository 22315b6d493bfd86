"""trainalm / genalm: train and run the animation language model from the command line.

    python -m oa_b200.apps.alm train --dataset /data/HumanML3D --out var/Alm.oam --tok-steps 5000 --lm-steps 5000
    python -m oa_b200.apps.alm gen --model var/Alm.oam --prompt "a person walks forward" --out walk.npy

`train` is the two-stage trainer of Apps/Ml/Gen3dAnim/trainalm.cpp: stage 1 fits the convolutional VQ tokenizer on
random windows of the clips (reconstruction + commitment loss, EMA codebook, live-code count and perplexity reported
per interval), stage 2 tokenizes every clip and fits the Transformer prior on [SOM] codes [EOM] sequences, conditioned
on the clip's caption when a text encoder is part of the bundle.  `gen` is Apps/Ml/Gen3dAnim/genalm.cpp: one bundle
in, one motion per prompt out (normalised features are mapped back with the dataset statistics when `--dataset` is
given).  Both own only policy (steps, sampling); the architecture travels inside the `.oam` bundle.
"""
from __future__ import annotations

import argparse
import math
import sys
from typing import List, Optional

import numpy as np
import torch

from ..core import fn_matrix as F
from ..core.matrix import OaMatrix
from ..data.datasets import OaDsHumanMl3d
from ..extensions.alm import (OaAlmAg, OaAlmPriorAg, OaAlmPriorConfig, OaAlmTokenizerAg, OaAlmTokenizerConfig, OaClipTextAg,
                              OaClipTextConfig)
from ..ml import autograd as AG
from ..ml import fn_loss as L
from ..ml.optim import OaAdamW


def _windows(ds: OaDsHumanMl3d, batch: int, seq: int, gen: torch.Generator) -> Optional[torch.Tensor]:
    """[batch * seq, features] random windows of normalised clips at least `seq` frames long."""
    eligible = [i for i in range(ds.NumClips()) if ds.ClipFrames(i) >= seq]
    if not eligible:
        return None
    rows = []
    for _ in range(batch):
        i = eligible[int(torch.randint(len(eligible), (1,), generator=gen))]
        clip = ds.GetItem(i).Tensor()
        s = int(torch.randint(clip.shape[0] - seq + 1, (1,), generator=gen))
        rows.append(clip[s:s + seq])
    return torch.cat(rows, 0)


def CodebookStats(indices: torch.Tensor, num_codes: int):
    """(live codes, perplexity) of a batch of code ids."""
    counts = torch.bincount(indices.reshape(-1).long().cpu(), minlength=num_codes).float()
    p = counts / counts.sum().clamp_min(1)
    nz = p[p > 0]
    return int((counts > 0).sum()), float(torch.exp(-(nz * nz.log()).sum()))


def TrainTokenizer(tok: OaAlmTokenizerAg, ds: OaDsHumanMl3d, steps: int, out=print, log_every: int = 50, seed: int = 0) -> List[float]:
    c = tok.Config()
    gen = torch.Generator().manual_seed(seed)
    opt = OaAdamW(tok.AllParameterPtrs(), c.LearningRate)
    device = tok.AllParameterPtrs()[0].Data.Tensor().device
    losses = []
    for step in range(steps):
        x = _windows(ds, c.BatchSize, c.SeqLen, gen)
        if x is None:
            raise ValueError(f"no clip has {c.SeqLen} frames")
        xm = OaMatrix(x.to(device))
        if step == 0:
            with AG.OaGradNo():
                tok.Seed(tok.Encode(xm, c.BatchSize, c.SeqLen))
        with AG.OaGradientTape() as tape:
            loss, res = tok.ReconstructionLoss(xm, c.BatchSize, c.SeqLen)
        tape.Backward(loss)
        opt.Step(); opt.ZeroGrad()
        tok.EmaUpdate(res)
        losses.append(float(loss.Tensor()))
        if (step + 1) % log_every == 0 or step + 1 == steps:
            live, ppl = CodebookStats(res.Idx[0].Tensor(), c.NumCodes)
            out(f"  tokenizer step {step + 1}/{steps}: loss {losses[-1]:.6f} | codebook {live}/{c.NumCodes} live | ppl {ppl:.1f} | "
                f"commit {float(res.CommitLoss.Tensor()):.6f}")
    return losses


def TokenizeClips(tok: OaAlmTokenizerAg, ds: OaDsHumanMl3d, prior_cfg: OaAlmPriorConfig) -> List[List[int]]:
    """[SOM] codes [EOM] per clip, cut to the prior's maximum length."""
    f, seqs = tok.DownsampleFactor(), []
    device = tok.AllParameterPtrs()[0].Data.Tensor().device
    budget = prior_cfg.MaxSeqLen - 3
    with AG.OaGradNo():
        for i in range(ds.NumClips()):
            frames = (ds.ClipFrames(i) // f) * f
            if frames == 0:
                seqs.append([])
                continue
            x = OaMatrix(ds.GetItem(i).Tensor()[:frames].contiguous().to(device))
            codes = tok.Tokenize(x, 1, frames)[0].Tensor().reshape(-1).cpu().tolist()[:budget]
            seqs.append([prior_cfg.SomToken] + [int(c) for c in codes] + [prior_cfg.EomToken])
    return seqs


def TrainPrior(model: OaAlmAg, ds: OaDsHumanMl3d, steps: int, out=print, log_every: int = 50, seed: int = 0) -> List[float]:
    prior, c = model.Prior, model.Prior.GetConfig()
    seqs = [(i, s) for i, s in enumerate(TokenizeClips(model.Tokenizer, ds, c)) if len(s) >= 3]
    if not seqs:
        raise ValueError("no clip is long enough to tokenize")
    device = prior.AllParameterPtrs()[0].Data.Tensor().device
    text_cache = {}
    if model.Text is not None and c.TextFeatureDim > 0:
        for i, _ in seqs:
            text_cache[i] = model.TextFeatures([ds.ClipText(i) or "motion"]).Tensor()
    gen = torch.Generator().manual_seed(seed)
    opt = OaAdamW(prior.AllParameterPtrs(), c.LearningRate)
    T = min(c.SeqLen, c.MaxSeqLen - 1)
    losses = []
    for step in range(steps):
        pick = [seqs[int(torch.randint(len(seqs), (1,), generator=gen))] for _ in range(c.BatchSize)]
        ids = torch.full((c.BatchSize, T + 1), c.PadToken, dtype=torch.int32)
        for r, (_, s) in enumerate(pick):
            s = s[:T + 1]
            ids[r, :len(s)] = torch.tensor(s, dtype=torch.int32)
        inp = F.FromInt32(ids[:, :-1].reshape(-1).tolist(), [c.BatchSize, T])
        tgt = ids[:, 1:].clone().long()
        tgt[tgt == c.PadToken] = -100
        with AG.OaGradientTape() as tape:
            if text_cache:
                text = OaMatrix(torch.cat([text_cache[i] for i, _ in pick], 0).to(device))
                logits = prior.ForwardConditioned(inp, text)
            else:
                logits = prior.Forward(inp)
            loss = L.CrossEntropy(logits.Reshape([c.BatchSize * T, c.VocabSize]), OaMatrix(tgt.reshape(-1).to(torch.int32).to(device)))
        tape.Backward(loss)
        opt.Step(); opt.ZeroGrad()
        losses.append(float(loss.Tensor()))
        if (step + 1) % log_every == 0 or step + 1 == steps:
            out(f"  prior step {step + 1}/{steps}: loss {losses[-1]:.4f} | ppl {math.exp(min(20.0, losses[-1])):.1f}")
    return losses


def BuildModel(ds: OaDsHumanMl3d, width: int, codes: int, d_model: int, layers: int, heads: int, with_text: bool,
               text_cfg: Optional[OaClipTextConfig] = None, seq_len: int = 64, batch: int = 32) -> OaAlmAg:
    tcfg = OaAlmTokenizerConfig(InputDim=ds.FeatDim(), Width=width, CodeDim=width, NumCodes=codes, SeqLen=seq_len, BatchSize=batch)
    text = OaClipTextAg(text_cfg or OaClipTextConfig.ViTL14()) if with_text else None
    pcfg = OaAlmPriorConfig(DModel=d_model, NumHeads=heads, NumLayers=layers, DFfn=4 * d_model, BatchSize=batch,
                            TextFeatureDim=text.Config().ProjectionDim if text is not None else 0)
    pcfg.SyncVocab(codes)
    pcfg.SeqLen = min(pcfg.SeqLen, pcfg.MaxSeqLen - 2)
    if text is not None:
        text.Freeze()
    return OaAlmAg(OaAlmTokenizerAg(tcfg), OaAlmPriorAg(pcfg), text)


def trainalm_main(a, out=print) -> int:
    ds = OaDsHumanMl3d(a.dataset, a.split, a.max_clips, a.feat_dim)
    if not ds.Ok():
        out(f"Error: no clips under {a.dataset} (split {a.split})")
        return 1
    out(f"  dataset: {ds.NumClips()} clips, {ds.TotalFrames()} frames, {ds.FeatDim()} features")
    model = BuildModel(ds, a.width, a.codes, a.d_model, a.layers, a.heads, a.text, seq_len=a.seq_len, batch=a.batch)
    try:
        TrainTokenizer(model.Tokenizer, ds, a.tok_steps, out, a.log_every, a.seed)
        TrainPrior(model, ds, a.lm_steps, out, a.log_every, a.seed)
    except ValueError as e:
        out(f"Error: {e}")
        return 1
    st = model.Save(a.out)
    if not st.IsOk():
        out(f"Error: {st.message}")
        return 1
    out(f"  saved {a.out} ({model.NumParameters():,} parameters)")
    return 0


def genalm_main(a, out=print) -> int:
    try:
        model = OaAlmAg.LoadOam(a.model)
    except ValueError as e:
        out(f"Error: {e}")
        return 1
    model.Eval()
    if model.Text is not None:
        motions = model.Generate([a.prompt], a.temperature, a.top_k, a.top_p, a.max_len, a.seed)
    else:
        toks = model.Prior.Generate(1, a.temperature, a.top_k, a.top_p, a.max_len, a.seed)
        motions = model.Prior.DecodeToMotion(toks, model.Tokenizer)
    m = motions[0]
    if m.IsEmpty():
        out("  the model ended the motion before producing a code")
        return 2
    feats = m.Tensor().float().cpu()
    if a.dataset:
        ds = OaDsHumanMl3d(a.dataset, a.split, 1, feats.shape[1])
        if ds.Ok():
            feats = ds.Denormalize(feats)
    np.save(a.out, feats.numpy())
    out(f"  wrote {a.out}: {feats.shape[0]} frames x {feats.shape[1]} features")
    return 0


def main(argv=None, out=print) -> int:
    ap = argparse.ArgumentParser(prog="alm", description="Train and run the animation language model")
    sub = ap.add_subparsers(dest="cmd", required=True)
    t = sub.add_parser("train")
    t.add_argument("--dataset", required=True); t.add_argument("--split", default="train"); t.add_argument("--out", required=True)
    t.add_argument("--max-clips", type=int, default=0); t.add_argument("--feat-dim", type=int, default=263)
    t.add_argument("--tok-steps", type=int, default=5000); t.add_argument("--lm-steps", type=int, default=5000)
    t.add_argument("--width", type=int, default=512); t.add_argument("--codes", type=int, default=512)
    t.add_argument("--d-model", type=int, default=384); t.add_argument("--layers", type=int, default=6); t.add_argument("--heads", type=int, default=6)
    t.add_argument("--seq-len", type=int, default=64); t.add_argument("--batch", type=int, default=32)
    t.add_argument("--text", action="store_true", help="bundle a CLIP ViT-L/14 text encoder and condition the prior on captions")
    t.add_argument("--log-every", type=int, default=50); t.add_argument("--seed", type=int, default=0)
    g = sub.add_parser("gen")
    g.add_argument("--model", required=True); g.add_argument("--prompt", default="a person walks forward"); g.add_argument("--out", default="motion.npy")
    g.add_argument("--dataset", default=""); g.add_argument("--split", default="train")
    g.add_argument("--temperature", type=float, default=1.0); g.add_argument("--top-k", type=int, default=0); g.add_argument("--top-p", type=float, default=0.9)
    g.add_argument("--max-len", type=int, default=64); g.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    return trainalm_main(a, out) if a.cmd == "train" else genalm_main(a, out)


if __name__ == "__main__":
    sys.exit(main())
