"""Run under torchrun on >= 2 GPUs: expert-parallel MoE layer (peer-memory dispatch / combine) against the same layer
computed without expert parallelism on every rank's own tokens.  Prints 'EP_CHECK_OK' on success."""
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
    T, D, Fh, E, k = 1024, 256, 384, 8, 2

    def make():
        F.SetRngSeed(11)
        m = OaMoE(D, Fh, E, k, num_shared_experts=0, expert_bias=False)
        return m

    ref, ep = make(), make()
    mesh = OaDeviceMesh()
    plan = OaExpertParallel(ep, mesh, tokens_per_rank=T, capacity_factor=3.0)
    torch.manual_seed(100 + rank)
    xt = torch.randn(T, D, device="cuda").bfloat16()
    gt = torch.randn(T, D, device="cuda").bfloat16()

    def run(layer):
        x = F.FromTensor(xt.clone()).SetRequiresGrad(True)
        with OaGradientTape() as tape:
            y = layer.Forward(x)
            tape.Backward(y, grad=gt.clone())
        return y.Tensor().float(), x.GradTensor().float()

    yr, dxr = run(ref)
    ye, dxe = run(ep)
    torch.cuda.synchronize()
    K.check_status()

    def close(a, b, tol, what):
        err = (a - b).abs().max().item()
        scale = b.abs().max().item() + 1e-9
        assert err <= tol * scale, f"rank {rank} {what}: err {err} scale {scale}"

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
    dist.barrier()
    if rank == 0:
        print("EP_CHECK_OK")
    mesh.Close()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
