"""chatlm: talk to a language model stored in an `.oam` file.

    python -m oa_b200.apps.chatlm -m model.oam                       # interactive
    python -m oa_b200.apps.chatlm -m model.oam -p "Once upon a time" -t 0.5 -n 200

The architecture is read from the file (Apps/Ml/chatlm/main.cpp: `ResolveArchName`, single-prompt mode with `-p`,
temperature `-t`, generation statistics with `-v`).  Supported here: the GPT family of `oa_b200.models.gpt`
(`OaGpt`) and the small-suite models (`OaNlpSuiteModel`).  Text is handled as UTF-8 bytes; models with a larger
vocabulary see the byte values as token ids.  On a GPU with rotary positions the KV-cache decoder runs the
generation; otherwise the last context window is re-run per token.
"""
from __future__ import annotations

import argparse
import struct
import sys
import time
from typing import List, Optional, Tuple

import torch

from ..core import fn_matrix as F
from ..core.matrix import OaMatrix
from ..io.oam import OamModel
from ..ml import autograd as AG
from ..models.gpt import OaGptConfig, OaGptModel


def ResolveArchName(oam_arch: str) -> str:
    a = oam_arch.lower()
    if a in ("oagpt", "oagpt_v1", "gpt", "gpt2", "oagptmodel"):
        return "gpt"
    if a.startswith("oanlpsuite"):
        return "nlpsuite"
    if a.startswith("oallm") or a == "llm":
        return "llm"
    return a


def _gpt_config_from(oam: OamModel) -> OaGptConfig:
    cfg = oam.GetConfig()
    blob = cfg["ArchConfig"]
    if len(blob) < 32:
        raise ValueError("the file carries no GPT architecture record")
    vocab, d, layers, heads, dff, seq, rms, swiglu = struct.unpack("<8I", blob[:32])
    names = {w.Name for w in oam.Weights()}
    return OaGptConfig(vocab, d, layers, heads, dff, seq, "rms" if rms else "layer", "swiglu" if swiglu else "gelu",
                       RopeTheta=0.0 if "pos_embed.weight" in names else 10000.0, Bias="head.bias" in names)


def LoadModel(path: str):
    """(model, kind) from an `.oam` file; raises ValueError with the reason when it cannot be served."""
    oam, st = OamModel.Load(path)
    if oam is None:
        raise ValueError(st.message)
    kind = ResolveArchName(oam.GetConfig()["Architecture"])
    if kind == "gpt":
        model = OaGptModel(_gpt_config_from(oam))
    elif kind == "nlpsuite":
        from ..ml.nlp_suite import OaNlpSuiteModel
        model = OaNlpSuiteModel.FromOam(oam) if hasattr(OaNlpSuiteModel, "FromOam") else None
        if model is None:
            raise ValueError("small-suite checkpoints are restored through OaNlpSuiteModel(recipe).Load(path)")
    else:
        raise ValueError(f"architecture '{oam.GetConfig()['Architecture']}' is not served by chatlm")
    st = model.LoadFrom(oam)
    if not st.IsOk():
        raise ValueError(st.message)
    model.Eval()
    return model, kind


def _sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, gen: torch.Generator) -> int:
    logits = logits.float().cpu()
    if temperature <= 0:
        return int(logits.argmax())
    logits = logits / temperature
    if top_k > 0:
        kth = torch.topk(logits, min(top_k, logits.numel())).values[-1]
        logits = torch.where(logits < kth, torch.full_like(logits, float("-inf")), logits)
    probs = torch.softmax(logits, -1)
    if 0 < top_p < 1:
        sp, si = torch.sort(probs, descending=True)
        keep = torch.cumsum(sp, 0) - sp < top_p
        mask = torch.zeros_like(probs, dtype=torch.bool)
        mask[si[keep]] = True
        probs = torch.where(mask, probs, torch.zeros_like(probs))
        probs = probs / probs.sum()
    return int(torch.multinomial(probs, 1, generator=gen))


def GenerateTokens(model: OaGptModel, prompt: List[int], new_tokens: int, temperature: float = 0.8, top_k: int = 0,
                   top_p: float = 0.95, seed: int = 0, stop_token: Optional[int] = None, on_token=None) -> List[int]:
    """Prompt + generated ids.  `on_token(id)` is called as each id is produced (streaming)."""
    cfg = model.Cfg
    toks = list(prompt) or [0]
    gen = torch.Generator().manual_seed(seed)
    device = model.Embed.Weight.Tensor().device
    with AG.OaGradNo():
        decoder = None
        if device.type == "cuda" and cfg.RopeTheta > 0 and len(toks) + new_tokens <= cfg.SeqLen:
            from ..serve.decoder import OaGptDecoder
            decoder = OaGptDecoder(model, 1, len(toks) + new_tokens)
            logits = decoder.Prefill(torch.tensor([toks], dtype=torch.int32, device=device))[0]
        for _ in range(new_tokens):
            if decoder is None:
                window = toks[-cfg.SeqLen:]
                logits = model.Forward(F.FromInt32(window, [1, len(window)])).Tensor()[len(window) - 1]
            nxt = _sample(logits.reshape(-1)[:cfg.Vocab], temperature, top_k, top_p, gen)
            toks.append(nxt)
            if on_token is not None:
                on_token(nxt)
            if stop_token is not None and nxt == stop_token:
                break
            if decoder is not None:
                logits = decoder.Step(torch.tensor([nxt], dtype=torch.int32, device=device))[0]
    return toks


def GenerateText(model: OaGptModel, prompt: str, new_tokens: int, **kw) -> Tuple[str, float]:
    """(prompt + continuation decoded as UTF-8 with replacement, seconds spent generating)."""
    ids = [b % model.Cfg.Vocab for b in prompt.encode("utf-8")]
    t0 = time.perf_counter()
    out = GenerateTokens(model, ids, new_tokens, **kw)
    dt = time.perf_counter() - t0
    return bytes(t & 0xFF for t in out).decode("utf-8", errors="replace"), dt


def main(argv=None, out=print, read=input) -> int:
    ap = argparse.ArgumentParser(prog="chatlm", description="Chat with a model stored in an .oam file")
    ap.add_argument("-m", "--model", required=True)
    ap.add_argument("-p", "--prompt", default=None, help="answer one prompt and exit")
    ap.add_argument("-t", "--temperature", type=float, default=0.8)
    ap.add_argument("-n", "--tokens", type=int, default=128)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=0.95)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("-v", "--verbose", action="store_true")
    a = ap.parse_args(argv)
    try:
        model, kind = LoadModel(a.model)
    except ValueError as e:
        out(f"Error: {e}")
        return 1
    if kind != "gpt":
        out(f"Error: generation for '{kind}' models goes through their own tutorial entry points")
        return 1
    kw = dict(temperature=a.temperature, top_k=a.top_k, top_p=a.top_p, seed=a.seed)

    def answer(prompt: str) -> None:
        text, dt = GenerateText(model, prompt, a.tokens, **kw)
        out(text)
        if a.verbose:
            n = max(0, len(text.encode("utf-8", errors="replace")) - len(prompt.encode("utf-8")))
            out(f"  gen: {n} tok in {dt * 1e3:.2f} ms ({n / dt if dt > 1e-9 else 0:.0f} tok/s)")

    if a.prompt is not None:
        answer(a.prompt)
        return 0
    out(f"chatlm: {a.model} ({model.NumParameters():,} parameters); empty line or Ctrl-D to quit")
    while True:
        try:
            line = read("> ")
        except (EOFError, KeyboardInterrupt):
            break
        if not line.strip():
            break
        answer(line)
    return 0


if __name__ == "__main__":
    sys.exit(main())
