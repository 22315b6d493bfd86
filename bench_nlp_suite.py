"""The OaNlpSuite benchmark of the reference (Docs/Benchmarks/OaNlpSuite.md): 5 architectures x 3 tokenizers, batch 64,
context 16, width 32, 300 AdamW steps on the 576-byte corpus, on one GPU.

    python bench_nlp_suite.py [--steps 300] [--eager] [--out results.json]

Per recipe it reports wall ms / step, device ms / step (CUDA events around the step), tokens / s (batch x context / wall
time, the reference's figure), the final cross-entropy and next-token accuracy on the last batch, and the ratio to the
reference's published wall-time number (measured by its authors on their hardware; it does not build on this machine).
Steps run as a captured CUDA graph from step 2 on (`OaItTrainingConfig.Program`), `--eager` disables that.
"""
from __future__ import annotations

import argparse
import json
import sys
import time

import torch

# published by the reference (wall ms / step, token/s): Docs/Benchmarks/OaNlpSuite.md:106-140
PUBLISHED = {
    ("rnn", "byte"): (5.00, 204.69e3), ("rnn", "bpe"): (5.39, 189.99e3), ("rnn", "char"): (4.75, 215.66e3),
    ("gru", "byte"): (11.17, 92.82e3), ("gru", "bpe"): (10.85, 94.55e3), ("gru", "char"): (10.92, 93.97e3),
    ("transformer", "byte"): (7.99, 128.94e3), ("transformer", "bpe"): (7.93, 129.50e3), ("transformer", "char"): (6.89, 148.63e3),
    ("moe", "byte"): (8.62, 118.80e3), ("moe", "bpe"): (8.84, 115.78e3), ("moe", "char"): (8.36, 122.77e3),
    ("mamba3", "byte"): (33.34, 30.72e3), ("mamba3", "bpe"): (33.39, 30.67e3), ("mamba3", "char"): (32.45, 31.55e3),
}


def run_recipe(arch, tok, steps: int, eager: bool) -> dict:
    from oa_b200.core import fn_matrix as F
    from oa_b200.ml import fn_loss as L
    from oa_b200.ml import nlp_suite as NS
    from oa_b200.ml.autograd import OaGradientTape
    from oa_b200.ml.optim import OaAdamW
    from oa_b200.ml.training import OaItTraining, OaItTrainingConfig

    F.SetRngSeed(NS.OaNlpSuiteRngSeed)
    recipe = NS.OaNlpSuiteRecipe(arch, tok)
    model = NS.OaNlpSuiteModel(recipe)
    sampler = NS.OaNlpSuiteSampler(recipe, NS.OaNlpSuiteBatchSize)
    opt = OaAdamW(model.AllParameterPtrs(), recipe.LearningRate())
    B, S = NS.OaNlpSuiteBatchSize, recipe.ContextLength()
    batches = []
    for _ in range(steps):
        x, y = sampler.Next()
        pin = (lambda t: t.pin_memory()) if torch.cuda.is_available() else (lambda t: t)
        batches.append((pin(x.Tensor().cpu()), pin(y.Tensor().cpu())))
    dev = F._dev()
    ids = F.FromTensor(torch.empty((B, S), dtype=torch.int32, device=dev))
    tgt = F.FromTensor(torch.empty((B * S,), dtype=torch.int32, device=dev))
    training = OaItTraining(opt, OaItTrainingConfig(TotalSteps=steps, BatchSize=B, SequenceLength=S, TimerName=recipe.TimerName(),
                                                    Program=not eager))
    state = {"i": 0, "logits": None}

    def prepare():
        x, y = batches[state["i"]]
        state["i"] += 1
        ids.Tensor().copy_(x, non_blocking=True)
        tgt.Tensor().copy_(y.reshape(-1), non_blocking=True)

    def record():
        opt.ZeroGrad()
        with OaGradientTape() as tape:
            logits = model.Forward(ids)
            state["logits"] = logits
            loss = L.CrossEntropy(logits, tgt)
            tape.Backward(loss)
        return loss

    sync = torch.cuda.synchronize if torch.cuda.is_available() else (lambda: None)
    sync()
    walls = []
    while not training.IsDone():
        t0 = time.perf_counter()
        training.Step(prepare, record)
        walls.append((time.perf_counter() - t0) * 1e3)
    training.Finish()
    sync()
    with torch.no_grad():
        from oa_b200.ml.autograd import OaGradNo
        with OaGradNo():
            logits = model.Forward(ids).Tensor().float().reshape(B * S, -1)
    acc = (logits.argmax(1) == tgt.Tensor().long()).float().mean().item()
    steady = sorted(walls[5:])
    wall = sum(steady) / len(steady)
    gpu = training.GpuTimingStats()
    key = (recipe.ArchitectureId(), recipe.TokenizerId())
    pub_ms, pub_tps = PUBLISHED[key]
    return {"architecture": recipe.ArchitectureName(), "tokenizer": recipe.TokenizerName(), "params": sum(p.Data.NumElements() for p in model.AllParameterPtrs()),
            "steps": steps, "wall_ms_per_step": wall, "wall_p50_ms": steady[len(steady) // 2], "gpu_ms_per_step": gpu.MeanMs,
            "tokens_per_s": B * S / (wall / 1e3), "final_ce": training.LastLoss(), "final_accuracy": acc,
            "published_wall_ms": pub_ms, "published_tokens_per_s": pub_tps, "speedup_vs_published": pub_ms / wall,
            "executor": "eager" if eager else "cuda graph replay"}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--eager", action="store_true")
    ap.add_argument("--only", default="")
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    from oa_b200.core.types import OaPrecision
    from oa_b200.ml import nlp_suite as NS
    from oa_b200.ops import kernels as K
    from oa_b200.runtime.engine import OaEngineConfig, OaInitComputeEngine
    assert OaInitComputeEngine(OaEngineConfig(Precision=OaPrecision.FP32, DeviceIndex=0))      # the reference trains this suite in FP32
    results = []
    for arch in NS.OaNlpArchitecture:
        for tok in NS.OaNlpTokenizerKind:
            if args.only and args.only not in (NS.OaNlpSuiteRecipe(arch, tok).ArchitectureId(),):
                continue
            r = run_recipe(arch, tok, args.steps, args.eager)
            results.append(r)
            print(json.dumps(r), flush=True)
    K.check_status()
    if args.out:
        with open(args.out, "w") as f:
            json.dump(results, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
