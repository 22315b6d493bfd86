"""VQ and quantisation kernels against their CPU (PyTorch) statements."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_vq_kernels_match_cpu_path():
    from oa_b200.core.matrix import OaMatrix as M
    from oa_b200.ml.nn import vq as VQ
    from oa_b200.ops import kernels as K
    g = torch.Generator().manual_seed(0)
    n, d, k = 3000, 64, 512
    z, e = torch.randn(n, d, generator=g), torch.randn(k, d, generator=g)
    rc, rg = VQ.VqAssign(M(z), M(e)), VQ.VqAssign(M(z.cuda()), M(e.cuda()))
    dist = ((z[:, None, :] - e[None]) ** 2).sum(-1)
    got = rg.Idx.Tensor().cpu().long()
    # a different index is acceptable only where the two codes are equally near within rounding
    picked, best = dist.gather(1, got[:, None])[:, 0], dist.min(1).values
    assert (picked - best).max() < 1e-3 and (got != rc.Idx.Tensor().long()).float().mean() < 0.01
    assert torch.equal(rg.Zq.Tensor().cpu(), e[got])
    idx = rc.Idx.Tensor()
    idx[idx >= 500] = 0                                   # leave some codes without rows
    state = lambda dev: [t.clone().to(dev) for t in (torch.randn(k, d, generator=torch.Generator().manual_seed(1)),
                                                     torch.rand(k, generator=torch.Generator().manual_seed(2)) * 3, torch.zeros(k, d))]
    for normalize in (False, True):
        sc, sg = state("cpu"), state("cuda")
        VQ.VqEmaUpdate(M(z), M(idx), M(sc[0]), M(sc[1]), M(sc[2]), 0.9, 1e-5, 0.6, 5, normalize)
        VQ.VqEmaUpdate(M(z.cuda()), M(idx.cuda()), M(sg[0]), M(sg[1]), M(sg[2]), 0.9, 1e-5, 0.6, 5, normalize)
        for a, b in zip(sc, sg):
            assert (a - b.cpu()).abs().max() < 1e-4
    K.check_status()


def test_quant_kernels_match_cpu_path():
    from oa_b200.ops import kernels as K
    from oa_b200.ops import quant as Q
    g = torch.Generator().manual_seed(3)
    x = torch.randn(100_003, generator=g) * 2
    xg = x.cuda()
    sc, sg = Q.q4_0_scale(x), Q.q4_0_scale(xg)
    assert torch.equal(sc, sg.cpu())
    qc, qg = Q.q4_0_quantize(x, sc), Q.q4_0_quantize(xg, sg)
    assert (qc != qg.cpu()).float().mean() < 1e-4          # division rounding may differ on exact .5 ties only
    assert torch.equal(Q.q4_0_dequantize(qc, sc, x.numel()), Q.q4_0_dequantize(qc.cuda(), sg, x.numel()).cpu())
    x8 = x[:100_000 // 32 * 32]
    bc, bg = Q.q8_0_quantize(x8), Q.q8_0_quantize(x8.cuda())
    assert (bc != bg.cpu()).float().mean() < 1e-4
    assert torch.equal(Q.q8_0_dequantize(bc), Q.q8_0_dequantize(bc.cuda()).cpu())
    s = torch.tensor([x.abs().max().item() / 127])
    ic, ig = Q.int8_quantize(x, s), Q.int8_quantize(xg, s.cuda())
    assert (ic != ig.cpu()).float().mean() < 1e-4
    assert torch.equal(Q.int8_dequantize(ic, s), Q.int8_dequantize(ic.cuda(), s.cuda()).cpu())
    K.check_status()
