"""Run under torchrun on >= 2 GPUs: the fused all-gather->GEMM and GEMM->reduce-scatter kernels against NCCL + a plain
matmul, then a tensor-parallel Transformer (loss, shard gradients) against the same model on one device.
Prints 'TP_CHECK_OK' on success."""
import os
import sys

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
    from oa_b200.models import OaGptConfig, OaGptModel
    from oa_b200.ops import kernels as K
    from oa_b200.parallel import tp as TP
    from oa_b200.parallel.mesh import OaDeviceMesh
    from oa_b200.parallel.tp_model import OaTpGptModel
    from oa_b200.runtime.engine import OaEngineConfig, OaInitComputeEngine
    assert OaInitComputeEngine(OaEngineConfig(Precision=OaPrecision.BF16, DeviceIndex=local))
    mesh = OaDeviceMesh()
    dev = torch.device("cuda", local)

    def close(a, b, tol, what):
        err = (a.float() - b.float()).abs().max().item()
        scale = b.float().abs().max().item() + 1e-9
        assert err <= tol * scale, f"rank {rank} {what}: err {err} scale {scale}"

    # ---- 1. the two fused kernels, three calls each (the epoch of a call site advances on the device)
    M, Kd, Nn = 256 * world, 320, 448
    arena = TP.OaTpArena(mesh, 64 << 20)
    ag, rs = TP.OaTpAgSite(arena, M, Kd), TP.OaTpRsSite(arena, M, Nn)
    rs_mn = TP.OaTpRsSite(arena, M, Kd)
    for it in range(3):
        g = torch.Generator(device="cpu").manual_seed(10 * it + rank)
        xs = torch.randn(M // world, Kd, generator=g).to(dev).bfloat16()
        w = (torch.randn(Nn, Kd, generator=torch.Generator().manual_seed(99 + it)) * 0.1).to(dev).bfloat16()
        y = TP.ag_gemm(ag, xs, w)
        parts = [torch.empty_like(xs) for _ in range(world)]
        dist.all_gather(parts, xs)
        xf = torch.cat(parts, 0)
        close(y, xf.float() @ w.float().t(), 2e-2, f"all-gather->GEMM call {it}")
        close(ag.gathered(), xf, 0.0, "gathered copy")
        a = torch.randn(M, Kd, generator=g).to(dev).bfloat16()
        res = torch.randn(M // world, Nn, generator=g).to(dev).bfloat16()
        out = TP.gemm_rs(rs, a, w, residual=res)
        full = (a.float() @ w.float().t())
        dist.all_reduce(full)
        want = full[rank * (M // world):(rank + 1) * (M // world)] + res.float()
        close(out, want, 2e-2, f"GEMM->reduce-scatter call {it}")
        # MN-major weight operand (the backward form): [M, Nn] @ W[Nn, Kd]
        gy = torch.randn(M, Nn, generator=g).to(dev).bfloat16()
        dx = TP.gemm_rs(rs_mn, gy, w, b_mn=True)
        fullx = gy.float() @ w.float()
        dist.all_reduce(fullx)
        close(dx, fullx[rank * (M // world):(rank + 1) * (M // world)], 2e-2, f"GEMM(MN)->reduce-scatter call {it}")
    torch.cuda.synchronize()
    K.check_status()

    # ---- 2. tensor-parallel model against the single-device model
    cfg = OaGptConfig(512, 256, 2, 4, 512, 128, "rms", "swiglu", 10000.0, False, 1e-5, 0.05)
    B = 2 * world
    F.SetRngSeed(7)
    full_model = OaGptModel(cfg)
    tp_model = OaTpGptModel(cfg, mesh, B, full=full_model)
    gen = torch.Generator().manual_seed(5)
    tok = torch.randint(0, cfg.Vocab, (B, cfg.SeqLen + 1), generator=gen, dtype=torch.int32).to(dev)
    ids, tg = F.FromTensor(tok[:, :-1].contiguous()), F.FromTensor(tok[:, 1:].contiguous())
    with OaGradientTape() as tape:
        lf = full_model.Loss(ids, tg)
        tape.Backward(lf)
    for step in range(2):                       # twice: buffers and epochs are reused
        for p in tp_model.AllParameterPtrs():
            p.Data.ZeroGrad()
        with OaGradientTape() as tape:
            lt = tp_model.Loss(ids, tg)
            tape.Backward(lt)
        tp_model.SyncReplicatedGrads()
        torch.cuda.synchronize()
        K.check_status()
        assert abs(lt.Item() - lf.Item()) < 2e-2 * max(1.0, abs(lf.Item())), (lt.Item(), lf.Item())
        W, r = world, rank
        D, Fd, V = cfg.DModel, cfg.DFf, cfg.Vocab
        Dl, Fl, Vl = D // W, Fd // W, V // W
        fb, tb = full_model.Blocks[0], tp_model.Blocks[0]
        gq = fb.Attention.QProj.Weight.Data.GradTensor()[r * Dl:(r + 1) * Dl]
        close(tb.Qkv.Data.GradTensor()[:Dl], gq, 6e-2, "q_proj grad")
        close(tb.Out.Data.GradTensor(), fb.Attention.OutProj.Weight.Data.GradTensor()[:, r * Dl:(r + 1) * Dl], 6e-2, "out_proj grad")
        close(tb.Up.Data.GradTensor()[:Fl], fb.Ffn.Gate.Weight.Data.GradTensor()[r * Fl:(r + 1) * Fl], 6e-2, "gate grad")
        close(tb.Down.Data.GradTensor(), fb.Ffn.Down.Weight.Data.GradTensor()[:, r * Fl:(r + 1) * Fl], 6e-2, "down grad")
        close(tp_model.Head.Data.GradTensor(), full_model.Head.Weight.Data.GradTensor()[r * Vl:(r + 1) * Vl], 6e-2, "head grad")
        close(tp_model.Embed.Data.GradTensor(), full_model.Embed.Weight.Data.GradTensor(), 6e-2, "embedding grad")
        close(tb.LnAttn.Weight.Data.GradTensor(), fb.LnAttn.Weight.Data.GradTensor(), 6e-2, "norm grad")
    dist.barrier()
    if rank == 0:
        print("TP_CHECK_OK")
    mesh.Close()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
