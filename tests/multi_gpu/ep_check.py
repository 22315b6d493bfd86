"""Run under torchrun on >= 2 GPUs: expert-parallel MoE layer (peer-memory dispatch / combine) against the same layer
computed without expert parallelism on every rank's own tokens: once with the learned-at-random router, once with a
router that sends (nearly) every token to expert 0 (eight times the mean load with 16 experts and top-2), which must pass without
a dropped route and with the row buffers grown past their first size.  Prints 'EP_CHECK_OK' on success."""
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
    from oa_b200.ml.nn.moe import OaMoE
    from oa_b200.ops import kernels as K
    from oa_b200.parallel.ep import OaExpertParallel
    from oa_b200.parallel.mesh import OaDeviceMesh
    from oa_b200.runtime.engine import OaEngineConfig, OaInitComputeEngine
    assert OaInitComputeEngine(OaEngineConfig(Precision=OaPrecision.BF16, DeviceIndex=local))
    def case(T, D, Fh, E, k, skew):
        def make():
            F.SetRngSeed(11)
            m = OaMoE(D, Fh, E, k, num_shared_experts=0, expert_bias=False)
            if skew:
                # feature 0 is a constant of every token (set below) and expert 0 reads it with a large weight, so expert 0 is
                # in every token's top-k: it receives T rows from every rank, 8x the mean of T * k / E
                rw = m.Router.Weight.Data.Tensor()
                rw[0, 0] = 1.5                   # +6 on expert 0's logit; the other logits are about N(0, 1)
            return m

        ref, ep = make(), make()
        plan = OaExpertParallel(ep, mesh, tokens_per_rank=T, capacity_factor=1.0 if skew else 1.25)
        torch.manual_seed(100 + rank)
        xt = torch.randn(T, D, device="cuda")
        if skew:
            xt[:, 0] = 4.0
        xt = xt.bfloat16()
        gt = torch.randn(T, D, device="cuda").bfloat16()

        def run(layer):
            x = F.FromTensor(xt.clone()).SetRequiresGrad(True)
            with OaGradientTape() as tape:
                y = layer.Forward(x)
                tape.Backward(y, grad=gt.clone())
            return y.Tensor().float(), x.GradTensor().float()

        yr, dxr = run(ref)
        for rep in range(2):                     # the second pass reuses every buffer (and the grown ones)
            for p in ep.AllParameterPtrs():
                if p.Data.GradTensor() is not None:
                    p.Data.GradTensor().zero_()
            ye, dxe = run(ep)
        torch.cuda.synchronize()
        K.check_status()

        def close(a, b, tol, what):
            err = (a - b).abs().max().item()
            scale = b.abs().max().item() + 1e-9
            assert err <= tol * scale, f"rank {rank} skew={skew} {what}: err {err} scale {scale}"

        close(ye, yr, 3e-2, "forward")
        close(dxe, dxr, 5e-2, "dx")
        El = E // world
        for name in ("GateUpW", "DownW"):
            gref = getattr(ref, name).Data.GradTensor().float().clone()
            dist.all_reduce(gref)
            gep = getattr(ep, name).Data.GradTensor().float()
            close(gep, gref[rank * El:(rank + 1) * El], 5e-2, name + " grad")
        gr_ref = ref.Router.Weight.Data.GradTensor().float()
        close(ep.Router.Weight.Data.GradTensor().float(), gr_ref, 8e-2, "router grad")
        d = ep.Dispatcher
        counts = d.counts_global.cpu()
        assert int(counts.sum()) == world * T * k, "every route of every rank is accounted for"
        if skew:
            assert int(counts[0]) >= int(0.99 * world * T), f"expert 0 holds {int(counts[0])} rows, expected about {world * T}"
            grown = torch.tensor([d.Grown], device="cuda")
            dist.all_reduce(grown, op=dist.ReduceOp.MIN)
            assert int(grown) >= 1, "the first buffer size cannot hold the skewed load: it must have grown (on every rank)"
        return d.Grown

    mesh = OaDeviceMesh()
    case(1024, 256, 384, 8, 2, skew=False)
    case(1024, 256, 384, 16, 2, skew=True)
    dist.barrier()
    if rank == 0:
        print("EP_CHECK_OK")
    mesh.Close()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
