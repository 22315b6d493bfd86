"""Tensor-parallel decoding on 2 GPUs: the one-shot all-reduce kernel against NCCL, and greedy generation of the sharded
model against the single-device decoder on the unsharded model."""
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
    from oa_b200.models import OaGptConfig, OaGptModel
    from oa_b200.ops import kernels as K
    from oa_b200.parallel.mesh import OaDeviceMesh
    from oa_b200.parallel.tp_model import OaTpGptModel
    from oa_b200.runtime.engine import OaEngineConfig, OaInitComputeEngine
    from oa_b200.serve import OaGptDecoder
    from oa_b200.serve.tp_decoder import OaOneShotAllReduce, OaTpGptDecoder
    assert OaInitComputeEngine(OaEngineConfig(Precision=OaPrecision.BF16, DeviceIndex=local))
    mesh = OaDeviceMesh()

    # ---- the all-reduce kernel: 9 calls (both staging halves, several sizes), with and without a residual
    ar = OaOneShotAllReduce(mesh, 32 * 1024)
    g = torch.Generator(device="cuda").manual_seed(10 + rank)
    for call, n in enumerate((8, 4096, 32 * 1024, 2048, 24, 32 * 1024, 8192, 16, 1024)):
        src = torch.randn(n, device="cuda", generator=g).bfloat16()
        res = torch.randn(n, device="cuda", generator=torch.Generator(device="cuda").manual_seed(call)).bfloat16() if call % 2 else None
        got = ar(src, res).float()
        want = src.float().clone()
        dist.all_reduce(want)
        if res is not None:
            want = want + res.float()
        err = (got - want).abs().max().item()
        assert err <= 2e-2 * max(1.0, want.abs().max().item()), (call, n, err)
    torch.cuda.synchronize()
    K.check_status()

    # ---- generation
    cfg = OaGptConfig(512, 256, 2, 4, 512, 64, "rms", "swiglu", 10000.0, False, 1e-5, 0.05)
    F.SetRngSeed(3)
    full = OaGptModel(cfg)
    B, S, new = 8, 24, 12
    tp = OaTpGptModel(cfg, mesh, B, full=full)
    prompt = torch.randint(0, cfg.Vocab, (B, S), generator=torch.Generator().manual_seed(5), dtype=torch.int32).cuda()
    ref_dec, tp_dec = OaGptDecoder(full, B, S + new), OaTpGptDecoder(tp, B, S + new)
    l_ref, l_tp = ref_dec.Prefill(prompt).float(), tp_dec.Prefill(prompt).float()
    assert l_tp.shape == l_ref.shape
    err = (l_tp - l_ref).abs().max().item()
    assert err <= 5e-2 * max(1.0, l_ref.abs().max().item()), ("prefill logits", err)
    nxt = l_ref.argmax(-1).to(torch.int32)
    s_ref, s_tp = ref_dec.Step(nxt).float(), tp_dec.Step(nxt).float()
    err = (s_tp - s_ref).abs().max().item()
    assert err <= 5e-2 * max(1.0, s_ref.abs().max().item()), ("step logits", err)
    out_ref, out_tp = ref_dec.Generate(prompt, new), tp_dec.Generate(prompt, new)
    assert out_tp.shape == (B, S + new) and torch.equal(out_tp[:, :S], prompt)
    agree = (out_ref[:, S:] == out_tp[:, S:]).float().mean().item()
    assert agree >= 0.8, agree          # bf16 partial sums are added in a different order; near-ties may flip
    gathered = [torch.empty_like(out_tp) for _ in range(world)]
    dist.all_gather(gathered, out_tp)
    assert all(torch.equal(gathered[0], t) for t in gathered)          # every rank generated the same tokens
    torch.cuda.synchronize()
    K.check_status()
    dist.barrier()
    if rank == 0:
        print("TP_DECODE_CHECK_OK")
    mesh.Close()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
