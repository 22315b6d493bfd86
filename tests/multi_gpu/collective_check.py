"""Run under torchrun on >= 2 GPUs: every OaCollective verb over peer memory against torch.distributed (NCCL), for a small
message (one pass) and a large one (reduce-scatter + all-gather form of AllReduce).  Prints 'COLLECTIVE_CHECK_OK'."""
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
    from oa_b200.ops import kernels as K
    from oa_b200.parallel.collective import OaCollective
    from oa_b200.parallel.mesh import OaDeviceMesh, OaReduceOp
    mesh = OaDeviceMesh()
    col = OaCollective(mesh, staging_bytes=32 << 20)
    assert col.Peer
    dev = torch.device("cuda", local)
    torch.manual_seed(7 + rank)
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
        for n in (1024 * world, 512 * 1024 * world):
            t = torch.randn(n, 4, device=dev).to(dtype)
            for op, top in ((OaReduceOp.Sum, dist.ReduceOp.SUM), (OaReduceOp.Max, dist.ReduceOp.MAX)):
                ref = t.clone()
                dist.all_reduce(ref, op=top)
                got = col.AllReduce(t, op)
                assert (got.float() - ref.float()).abs().max().item() <= tol * (ref.float().abs().max().item() + 1), ("allreduce", dtype, n, op)
            ref = torch.empty(n // world, 4, device=dev, dtype=dtype)
            dist.reduce_scatter_tensor(ref, t.clone())
            got = col.ReduceScatter(t)
            assert (got.float() - ref.float()).abs().max().item() <= tol * (ref.float().abs().max().item() + 1), ("reduce_scatter", dtype, n)
            ref = torch.empty(n * world, 4, device=dev, dtype=dtype)
            dist.all_gather_into_tensor(ref, t)
            assert torch.equal(col.AllGather(t), ref), ("all_gather", dtype, n)
            ref = t.clone()
            dist.broadcast(ref, src=world - 1)
            assert torch.equal(col.Broadcast(t, root=world - 1), ref), ("broadcast", dtype, n)
            ref = torch.empty_like(t)
            dist.all_to_all_single(ref, t)
            assert torch.equal(col.AllToAll(t), ref), ("all_to_all", dtype, n)
            got = col.Scatter(t if rank == 0 else None, root=0, shape=t.shape, dtype=dtype)
            src = t.clone()
            dist.broadcast(src, src=0)
            blk = n // world
            assert torch.equal(got, src[rank * blk:(rank + 1) * blk]), ("scatter", dtype, n)
    col.Barrier()
    torch.cuda.synchronize()
    K.check_status()
    mesh.Close()
    dist.destroy_process_group()
    if rank == 0:
        print("COLLECTIVE_CHECK_OK")
    return 0


if __name__ == "__main__":
    sys.exit(main())
