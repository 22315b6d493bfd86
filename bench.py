#!/usr/bin/env python
"""Flagship benchmark: training throughput (tokens/s) of the dense GPT-style Transformer LM, data parallel.

Config: vocab 32000, d_model 1024, 24 layers, 16 heads (head_dim 64), FFN 4096 GELU,
RMSNorm, RoPE, seq 2048, micro-batch 8 per GPU, bf16 compute with fp32 master weights and AdamW, token ids
uniform over the vocabulary from a seed, weights N(0, 0.02).  Weak scaling: per-GPU work is fixed.

  python bench.py --gpus N --steps K --warmup W            (N>1: launched by torchrun, one rank per GPU)
  python bench.py --impl reference ...                      (the reference arm: the unmodified reference through its own public API; it is a
                                                            Vulkan-only library and does not install on an image without a Vulkan SDK, in which
                                                            case this prints one line saying why it is unavailable and exits 0)

Prints ONE JSON line on rank 0.  `value` is timed on the device with CUDA events around exactly K steps
(barrier + synchronize on both sides, max over ranks); `e2e` is the same metric through the public
OaItTraining API including the per-step pinned-host -> device input copy and the loss readback.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)


def reference_arm(args) -> int:
    # The reference is a Vulkan-only C++ library; its wheel cannot be built offline on this image
    # (CMake: "Neither VulkanHeaders (vcpkg) nor Vulkan SDK found", and it requires Clang), and no
    # Vulkan loader / ICD / software renderer exists on the GPU box.
    ref = os.path.join(REPO, "baseline", "_ref", "oa")
    if not os.path.isdir(ref):
        print(json.dumps({"impl": "reference",
                          "unavailable": "reference (Vulkan-only) does not build offline: no Vulkan headers/SDK or loader on this image; unavailable on this box"}))
        return 0
    print(json.dumps({"impl": "reference", "unavailable": "reference installed but no Vulkan ICD on this box"}))
    return 0


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for ln in self.proc.stdout:
            self.lines.append(ln.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx = float(f[2])
            except ValueError:
                continue
            for nm, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="oa_b200")
    ap.add_argument("--model", default="gpt350m", choices=["gpt350m", "tiny", "mamba3", "mamba3-tiny", "moe", "char"])
    ap.add_argument("--micro-batch", type=int, default=0, help="sequences per GPU; 0 = the configuration's own (8 GPT, 4 Mamba-3 / MoE, 16 char LM)")
    ap.add_argument("--seq", type=int, default=0)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--dp-mode", default="fused", choices=["fused", "nccl"])
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            print(f"bench.py: --gpus {args.gpus} needs torchrun with {args.gpus} ranks", file=sys.stderr)
            return 2
    args.warmup = max(args.warmup, 3)
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    import oa_b200 as oa
    from oa_b200 import _native
    from oa_b200.core import fn_matrix as F
    from oa_b200.core.types import OaPrecision
    from oa_b200.ml.autograd import OaGradientTape
    from oa_b200.ml.optim import OaAdamW
    from oa_b200.ml.training import OaItTraining, OaItTrainingConfig
    from oa_b200.models import OaGptConfig, OaGptModel
    from oa_b200.runtime.engine import OaContextGetDefault, OaEngineConfig, OaInitComputeEngine

    if args.micro_batch <= 0:
        args.micro_batch = {"mamba3": 4, "moe": 4, "char": 16}.get(args.model, 8)
    cfg_e = OaEngineConfig(Precision=OaPrecision.FP32 if args.model == "char" else OaPrecision.BF16, DeviceIndex=local_rank)
    assert OaInitComputeEngine(cfg_e)
    from oa_b200.models import OaMamba3Config, OaMamba3LmModel
    names = {"gpt350m": "dense GPT 24x1024, 16 heads, FFN 4096 GELU, RMSNorm, RoPE, vocab 32000", "tiny": "tiny",
             "mamba3": "Mamba-3 32x1536, state 128, expand 2, head dim 64, chunk 256, vocab 32000", "mamba3-tiny": "mamba3-tiny",
             "char": "char-level Transformer LM, FP32: vocab 256, d 128, 4 layers, 4 heads, FFN 512 GELU, pre-LayerNorm, learned positions",
             "moe": "sparse MoE 16x2048, 64 experts top-2, SwiGLU 1408, 1 shared expert, vocab 32000 (single-GPU experts)"}
    if args.model in ("mamba3", "mamba3-tiny"):
        mcfg = OaMamba3Config.Mamba3_32x1536() if args.model == "mamba3" else OaMamba3Config(1024, 256, 2, 32, 2, 16, 256, 64)
    elif args.model == "moe":
        mcfg = OaGptConfig.Moe16x2048()
    elif args.model == "char":
        mcfg = OaGptConfig.CharLm()
    else:
        mcfg = OaGptConfig.Gpt350M() if args.model == "gpt350m" else OaGptConfig(1024, 256, 2, 4, 1024, 256, "rms", "gelu", 10000.0, False, 1e-5, 0.02)
    if args.seq:
        mcfg.SeqLen = args.seq
    B, S = args.micro_batch, mcfg.SeqLen
    F.SetRngSeed(20260714)                      # same weights on every rank
    model = OaMamba3LmModel(mcfg) if args.model.startswith("mamba3") else OaGptModel(mcfg)
    params = model.AllParameterPtrs()
    opt = OaAdamW(params, 3e-4, weight_decay=0.1)
    dp = None
    if world > 1:
        from oa_b200.parallel.dp import OaDataParallel
        dp = OaDataParallel(model, opt, mode=args.dp_mode)
    dev = torch.device("cuda", local_rank)
    gen = torch.Generator().manual_seed(1234 + rank)
    n_host = 8
    host_tokens = [torch.randint(0, mcfg.Vocab, (B, S + 1), generator=gen, dtype=torch.int32).pin_memory() for _ in range(n_host)]
    ids = F.FromTensor(torch.empty((B, S), dtype=torch.int32, device=dev))
    tgt = F.FromTensor(torch.empty((B, S), dtype=torch.int32, device=dev))
    h2d_bytes = 2 * B * S * 4
    step_counter = {"i": 0}

    def prepare():
        t = host_tokens[step_counter["i"] % n_host]
        step_counter["i"] += 1
        ids.Tensor().copy_(t[:, :S], non_blocking=True)
        tgt.Tensor().copy_(t[:, 1:], non_blocking=True)

    def record():
        opt.ZeroGrad()
        with OaGradientTape() as tape:
            loss = model.Loss(ids, tgt)
            tape.Backward(loss)
        return loss

    tcfg = OaItTrainingConfig(TotalSteps=10 ** 9, BatchSize=B * world, SequenceLength=S, Program=not args.no_graph)
    training = OaItTraining(opt, tcfg)
    ctx = OaContextGetDefault()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- warm-up through the public API (step 1 eager, step 2 captures the program)
    launches_before_capture = None
    for w in range(args.warmup):
        training.IsDone()
        n0 = _native.launches()
        training.Step(prepare, record)
        if w == 1 or args.no_graph:
            launches_before_capture = _native.launches() - n0
    launches_per_step = launches_before_capture or 0
    loss_warm = training.LastLoss()

    # ---- device-timed region: exactly K steps, inputs resident, no host sync inside
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    prog = training.Program()
    for _ in range(args.steps):
        if prog is not None and prog.IsCaptured():
            prog.Replay()
            opt.NotifyProgramReplay()
        else:
            record()
            opt.Step()
    e1.record()
    barrier()
    dev_ms = e0.elapsed_time(e1)
    clocks = sampler.stop()

    # ---- end-to-end region: public API, H2D of the inputs and D2H of the loss every step
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        training.IsDone()
        training.Step(prepare, record)
    f1.record()
    barrier()
    e2e_ms = max(f0.elapsed_time(f1), (time.perf_counter() - t0) * 1e3)
    final_loss = training.LastLoss()
    st = ctx.Sync()

    if world > 1:
        t = torch.tensor([dev_ms, e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms, e2e_ms = float(t[0]), float(t[1])
    tokens = B * S * world * args.steps
    value = tokens / (dev_ms / 1e3)
    e2e_value = tokens / (e2e_ms / 1e3)
    flops_per_token = model.FlopsPerToken()
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(REPO, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak_tf = peaks.get("bf16_tflops_sustained", 1400.0)
    out = {
        "metric": "train tokens/s (device-timed, max over ranks)", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp32" if args.model == "char" else "bf16", "data": "synthetic (uniform token ids, random-init N(0,0.02) weights)",
        "config": {"model": names[args.model],
                   "global_batch": B * world, "seq_len": S, "parallelism": f"dp{world}", "optimizer": "AdamW fp32 master",
                   "l2": "inputs larger than L2 (activations and weights >> 126 MB per step)",
                   "executor": "cuda graph replay" if (prog is not None and prog.IsCaptured()) else "eager stream",
                   "dp": (args.dp_mode if world > 1 else "none")},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": 4,
                "ms_per_step": e2e_ms / args.steps},
        "gpu_launches": launches_per_step * args.steps,
        "launches_per_step": launches_per_step,
        "model_tflops_per_gpu": value / world * flops_per_token / 1e12,
        "frac_of_measured_bf16_sustained": (value / world * flops_per_token / 1e12) / peak_tf,
        "loss_after_warmup": loss_warm, "final_loss": final_loss, "status": "ok" if st else repr(st),
    }
    if rank == 0:
        print(json.dumps(out))
    if dp is not None:
        dp.Close()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
