"""chatlm and the ALM trainer / generator on tiny models."""
import os

import numpy as np
import torch

from oa_b200.apps import alm as alm_app
from oa_b200.apps import chatlm
from oa_b200.models.gpt import OaGptConfig, OaGptModel


def test_chatlm_single_prompt_and_repl(tmp_path):
    torch.manual_seed(0)
    cfg = OaGptConfig(Vocab=256, DModel=32, NLayers=1, NHeads=2, DFf=64, SeqLen=16)
    model = OaGptModel(cfg)
    path = str(tmp_path / "tiny.oam")
    assert model.Save(path).IsOk()
    loaded, kind = chatlm.LoadModel(path)
    assert kind == "gpt" and loaded.Cfg.DModel == 32 and loaded.Cfg.RopeTheta == 0.0 and loaded.Cfg.Bias
    ids = chatlm.GenerateTokens(loaded, [104, 105], 20, temperature=0.0)
    assert len(ids) == 22 and ids[:2] == [104, 105] and ids == chatlm.GenerateTokens(loaded, [104, 105], 20, temperature=0.0)
    streamed = []
    sampled = chatlm.GenerateTokens(loaded, [1], 8, temperature=1.0, top_k=10, top_p=0.9, seed=5, on_token=streamed.append)
    assert sampled[1:] == streamed and sampled == chatlm.GenerateTokens(loaded, [1], 8, temperature=1.0, top_k=10, top_p=0.9, seed=5)
    lines = []
    assert chatlm.main(["-m", path, "-p", "to be", "-n", "12", "-t", "0", "-v"], out=lines.append) == 0
    assert lines[0].startswith("to be") and "tok/s" in lines[1]
    feed = iter(["hello", ""])
    lines.clear()
    assert chatlm.main(["-m", path, "-n", "4"], out=lines.append, read=lambda _: next(feed)) == 0 and lines[1].startswith("hello")
    assert chatlm.main(["-m", str(tmp_path / "nope.oam"), "-p", "x"], out=lines.append) == 1
    assert chatlm.ResolveArchName("oagpt_v1") == "gpt" and chatlm.ResolveArchName("oallm_v6") == "llm"


def _fake_humanml(root, clips=4, frames=40, feat=23):
    rng = np.random.default_rng(0)
    os.makedirs(root / "new_joint_vecs"); os.makedirs(root / "texts")
    np.save(root / "Mean.npy", np.zeros(feat, np.float32)); np.save(root / "Std.npy", np.ones(feat, np.float32))
    ids = [f"{i:06d}" for i in range(clips)]
    (root / "train.txt").write_text("\n".join(ids) + "\n")
    t = np.linspace(0, 6, frames)[:, None]
    for k, cid in enumerate(ids):
        np.save(root / "new_joint_vecs" / f"{cid}.npy", (np.sin(t * (k + 1) + np.arange(feat)[None]) + 0.05 * rng.standard_normal((frames, feat))).astype(np.float32))
        (root / "texts" / f"{cid}.txt").write_text(f"motion number {k}#x#0.0#0.0\n")


def test_trainalm_then_genalm(tmp_path):
    torch.manual_seed(0)
    _fake_humanml(tmp_path)
    out_path, lines = str(tmp_path / "alm.oam"), []
    rc = alm_app.main(["train", "--dataset", str(tmp_path), "--out", out_path, "--feat-dim", "23", "--tok-steps", "6", "--lm-steps", "6",
                       "--width", "16", "--codes", "8", "--d-model", "32", "--layers", "1", "--heads", "2", "--seq-len", "16", "--batch", "4",
                       "--log-every", "3"], out=lines.append)
    assert rc == 0 and os.path.exists(out_path), lines
    assert any("codebook" in l and "ppl" in l for l in lines) and any(l.strip().startswith("prior step 6/6") for l in lines)
    npy = str(tmp_path / "gen.npy")
    rc = alm_app.main(["gen", "--model", out_path, "--out", npy, "--max-len", "5", "--temperature", "0", "--dataset", str(tmp_path)], out=lines.append)
    assert rc in (0, 2)
    if rc == 0:
        m = np.load(npy)
        assert m.shape[1] == 23 and m.shape[0] % 4 == 0 and np.isfinite(m).all()
    assert alm_app.main(["train", "--dataset", str(tmp_path / "void"), "--out", out_path], out=lines.append) == 1
    live, ppl = alm_app.CodebookStats(torch.tensor([0, 0, 1, 1]), 8)
    assert live == 2 and abs(ppl - 2.0) < 1e-5
