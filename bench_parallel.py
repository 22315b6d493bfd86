"""Expert-parallel and tensor-parallel training benchmarks (the MoE and 7B-class configurations), one node.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 bench_parallel.py --mode ep
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 bench_parallel.py --mode tp

--mode ep: sparse MoE Transformer 16 x 2048, 64 experts top-2 (SwiGLU 1408) + 1 shared expert, seq 2048, micro-batch 4 per
GPU; routed experts sharded over the ranks (all-to-all dispatch / combine through peer memory), every other parameter
data-parallel with the fused reduce-scatter + AdamW + all-gather step.
--mode tp: 7B-class Transformer (32 x 4096, 32 heads, SwiGLU 11008), seq 4096, micro-batch 1 with gradient accumulation
to 32 sequences per optimizer step; column / row parallel projections through the fused all-gather -> GEMM and
GEMM -> reduce-scatter kernels, sequence-sharded norms, vocabulary-parallel cross-entropy.
Timing: W untimed steps, then K steps between CUDA events with a barrier + synchronize on both sides, max over ranks;
rank 0 prints one JSON line.  Synthetic uniform token ids, random-init N(0, 0.02) weights, bf16 with fp32 master AdamW.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", choices=["ep", "tp", "tp-decode"], required=True)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--accum", type=int, default=32)
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (0 = the configuration's own)")
    args = ap.parse_args()
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from oa_b200 import _native
    from oa_b200.core import fn_matrix as F
    from oa_b200.core.types import OaPrecision
    from oa_b200.ml.autograd import OaGradientTape
    from oa_b200.ml.optim import OaAdamW
    from oa_b200.models import OaGptConfig, OaGptModel
    from oa_b200.ops import kernels as K
    from oa_b200.parallel.mesh import OaDeviceMesh
    from oa_b200.runtime.engine import OaEngineConfig, OaInitComputeEngine
    assert OaInitComputeEngine(OaEngineConfig(Precision=OaPrecision.BF16, DeviceIndex=local))
    dev = torch.device("cuda", local)
    mesh = OaDeviceMesh()
    F.SetRngSeed(20260714)
    gen = torch.Generator().manual_seed(99 if args.mode == "tp" else 1234 + rank)   # TP ranks see the same batch

    if args.mode == "tp-decode":
        # batch-32 greedy decoding of 256 tokens after a 2048-token prompt, weights / KV cache / heads sharded over the ranks
        from oa_b200.parallel.tp_model import OaTpGptModel
        from oa_b200.serve.tp_decoder import OaTpGptDecoder
        cfg = OaGptConfig.Llama7B()
        if args.layers:
            cfg.NLayers = args.layers
        Bd, prompt_len, new = 32, 2048, 256
        model = OaTpGptModel(cfg, mesh, 1)
        dec = OaTpGptDecoder(model, Bd, prompt_len + new)
        prompt = torch.randint(0, cfg.Vocab, (Bd, prompt_len), generator=gen, dtype=torch.int32).to(dev)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        dec.Generate(prompt[:, :256], 8)                       # warm-up
        dist.barrier()
        torch.cuda.synchronize()
        ev[0].record()
        logits = dec.Prefill(prompt)
        ev[1].record()
        for _ in range(new):
            logits = dec.Step(logits.float().argmax(-1).to(torch.int32))
        ev[2].record()
        torch.cuda.synchronize()
        t = torch.tensor([ev[0].elapsed_time(ev[1]), ev[1].elapsed_time(ev[2])], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        K.check_status()
        if rank == 0:
            print(json.dumps({"metric": "greedy decode tokens/s (device-timed, max over ranks)", "value": Bd * new / (float(t[1]) / 1e3),
                              "unit": "tokens/s", "n_gpus": world, "ms_per_token": float(t[1]) / new, "prefill_ms": float(t[0]),
                              "prefill_tokens_per_s": Bd * prompt_len / (float(t[0]) / 1e3), "dtype": "bf16",
                              "config": {"model": "7B-class Transformer 32x4096", "layers": cfg.NLayers, "batch": Bd, "prompt": prompt_len,
                                         "new_tokens": new, "parallelism": f"tp{world}, one-shot all-reduce over peer memory"},
                              "kv_cache_gib_per_gpu": round(dec.Cache.Bytes() / 2 ** 30, 2)}), flush=True)
        mesh.Close()
        dist.destroy_process_group()
        return 0
    if args.mode == "ep":
        from oa_b200.parallel.dp import OaDataParallel
        from oa_b200.parallel.ep import OaExpertParallel
        cfg = OaGptConfig.Moe16x2048()
        if args.layers:
            cfg.NLayers = args.layers
        B, S, micro_steps = 4, cfg.SeqLen, 1
        model = OaGptModel(cfg)
        ep = OaExpertParallel(model, mesh, tokens_per_rank=B * S, capacity_factor=2.0)
        expert_params = ep.ExpertParameters()
        expert_ids = {id(p) for p in expert_params}
        dense_params = [p for p in model.AllParameterPtrs() if id(p) not in expert_ids]
        opt_dense, opt_exp = OaAdamW(dense_params, 3e-4, weight_decay=0.1), OaAdamW(expert_params, 3e-4, weight_decay=0.1)
        OaDataParallel(model, opt_dense, mode="fused", mesh=mesh)
        opt_exp.SetGradScale(1.0 / world)
        opts = [opt_dense, opt_exp]
        loss_fn, after_backward = model.Loss, (lambda: None)
        name, par = "sparse MoE 16x2048, 64 experts top-2, SwiGLU 1408, 1 shared expert, vocab 32000", f"ep{world} (experts) x dp{world} (rest)"
        tokens_per_step = B * S * world
    else:
        from oa_b200.parallel.tp_model import OaTpGptModel
        cfg = OaGptConfig.Llama7B()
        if args.layers:
            cfg.NLayers = args.layers
        B, S, micro_steps = 1, cfg.SeqLen, args.accum
        model = OaTpGptModel(cfg, mesh, B)
        opt = OaAdamW(model.AllParameterPtrs(), 3e-4, weight_decay=0.1)
        opt.SetGradScale(1.0 / micro_steps)
        opts = [opt]
        loss_fn, after_backward = model.Loss, model.SyncReplicatedGrads
        name, par = "7B-class Transformer 32x4096, 32 heads, SwiGLU 11008, RMSNorm, RoPE, vocab 32000", f"tp{world} + sequence parallel"
        tokens_per_step = B * S * micro_steps
    n_host = 4
    host = [torch.randint(0, cfg.Vocab, (B, S + 1), generator=gen, dtype=torch.int32).pin_memory() for _ in range(n_host)]
    ids = F.FromTensor(torch.empty((B, S), dtype=torch.int32, device=dev))
    tgt = F.FromTensor(torch.empty((B, S), dtype=torch.int32, device=dev))
    counter = {"i": 0}

    def step():
        for o in opts:
            o.ZeroGrad()
        loss = None
        for _ in range(micro_steps):
            t = host[counter["i"] % n_host]
            counter["i"] += 1
            ids.Tensor().copy_(t[:, :S], non_blocking=True)
            tgt.Tensor().copy_(t[:, 1:], non_blocking=True)
            with OaGradientTape() as tape:
                loss = loss_fn(ids, tgt)
                tape.Backward(loss)
        after_backward()
        for o in opts:
            o.Step()
        return loss

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    n0 = _native.launches()
    for _ in range(max(3, args.warmup)):
        loss = step()
    launches = (_native.launches() - n0) // max(3, args.warmup)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        loss = step()
    e1.record()
    barrier()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    K.check_status()
    final = loss.Item()
    mem = torch.cuda.max_memory_allocated() / 2 ** 30
    if rank == 0:
        per_step = float(ms[0]) / args.steps
        print(json.dumps({"metric": "train tokens/s (device-timed, max over ranks)", "value": tokens_per_step / (per_step / 1e3), "unit": "tokens/s",
                          "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": per_step, "higher_is_better": True,
                          "dtype": "bf16", "data": "synthetic (uniform token ids, random-init N(0,0.02) weights)",
                          "config": {"model": name, "layers": cfg.NLayers, "tokens_per_step": tokens_per_step, "seq_len": S,
                                     "micro_batch": B, "micro_steps": micro_steps, "parallelism": par, "executor": "eager stream"},
                          "gpu_launches_per_step": launches, "final_loss": final, "peak_memory_gib": round(mem, 1)}), flush=True)
    mesh.Close()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
