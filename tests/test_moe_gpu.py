"""MoE kernels on the GPU against the CPU statement of the same math (router, plan, gather/combine, grouped GEMMs),
including an empty expert, duplicate routes of one token, and the sparse layer against its dense oracle."""
import pytest
import torch

from oa_b200.ops import kernels as K
from oa_b200.ops import moe as M

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(got, ref, rtol, what=""):
    got, ref = got.float().cpu(), ref.float().cpu()
    scale = ref.abs().max().item() + 1e-12
    err = (got - ref).abs().max().item()
    assert err <= rtol * scale, f"{what}: max err {err:.4g} > {rtol * scale:.4g}"


@pytest.fixture(autouse=True)
def _status():
    yield
    torch.cuda.synchronize()
    K.check_status()


@pytest.mark.parametrize("T,E,k", [(300, 8, 2), (4096, 64, 2), (1000, 5, 1)])
def test_router_and_plan(T, E, k):
    torch.manual_seed(0)
    logits = torch.randn(T, E, device=DEV)
    if E >= 8:
        logits[:, 3] = -50.0            # expert 3 never selected: empty segment
    bias = torch.randn(E, device=DEV) * 0.1
    bias[3 % E] = 0.0
    probs, idx, w = M.router(logits, k, bias)
    pr, ir, wr = M.router(logits.cpu(), k, bias.cpu())
    _close(probs, pr, 1e-5, "probs")
    assert torch.equal(idx.cpu(), ir), "top-k indices (ties to the lower index)"
    _close(w, wr, 1e-5, "route weights")
    P = M.plan(idx, E)
    Pr = M.plan(ir, E)
    assert torch.equal(P.counts.cpu(), Pr.counts) and torch.equal(P.offsets.cpu(), Pr.offsets)
    assert torch.equal(P.inverse.cpu(), Pr.inverse), "stable expert-major order"
    assert torch.equal(P.packed_token.cpu(), Pr.packed_token)
    dw = torch.randn(T, k, device=DEV)
    col = torch.rand(E, device=DEV)
    _close(M.router_bwd(probs, idx, w, dw, col, 0.3, torch.float32), M.router_bwd(pr, ir, wr, dw.cpu(), col.cpu(), 0.3, torch.float32), 1e-4, "router bwd")


def test_gather_grouped_combine():
    torch.manual_seed(1)
    T, E, k, D, Fh = 700, 8, 2, 256, 384
    logits = torch.randn(T, E, device=DEV)
    logits[:, 5] = -50.0
    probs, idx, w = M.router(logits, k)
    P = M.plan(idx, E)
    Pc = M.plan(idx.cpu(), E)
    x = (torch.randn(T, D, device=DEV)).bfloat16()
    W1 = (torch.randn(E, Fh, D, device=DEV) * 0.05).bfloat16()
    b1 = torch.randn(E, Fh, device=DEV).bfloat16()
    c = lambda t: t.cpu().float()
    px = M.gather(x, P)
    pxr = M.gather(c(x), Pc)
    _close(px, pxr, 0.0 + 1e-6, "gather")
    y = M.grouped_linear(px, W1, b1, P)
    yr = M.grouped_linear(pxr, c(W1), c(b1), Pc)
    live = Pc.packed_token >= 0
    _close(y.cpu()[live], yr[live], 1e-2, "grouped linear")
    base = torch.randn(T, Fh, device=DEV).bfloat16()
    out = M.combine(y, w, P, base=base)
    outr = M.combine(yr, w.cpu(), Pc, base=c(base))
    _close(out, outr, 1e-2, "combine")
    dout = torch.randn(T, Fh, device=DEV).bfloat16()
    dy, dg = M.combine_bwd(y, w, P, dout)
    dyr, dgr = M.combine_bwd(yr, w.cpu(), Pc, c(dout))
    _close(dy, dyr, 1e-2, "combine bwd dpacked")
    _close(dg, dgr, 2e-2, "combine bwd dgate")
    dpx = M.grouped_linear(dy, W1, None, P, b_mn=True)
    dpxr = M.grouped_linear(dyr, c(W1), None, Pc, b_mn=True)
    used = int(Pc.offsets[-1])          # rows past the last segment are never written nor read
    _close(dpx[:used], dpxr[:used], 1e-2, "grouped data grad")
    dW = M.grouped_weight_grad(dy, px, P, out=torch.zeros(E, Fh, D, device=DEV))
    dWr = M.grouped_weight_grad(dyr, pxr, Pc, out=torch.zeros(E, Fh, D))
    _close(dW, dWr, 1e-2, "grouped weight grad")
    assert dW[5].abs().max().item() == 0.0, "empty expert must get a zero gradient"
    _close(M.grouped_bias_grad(dy, P), M.grouped_bias_grad(dyr, Pc), 2e-2, "grouped bias grad")
    _close(M.gather_bwd(dpx, P), M.gather_bwd(dpxr, Pc), 1e-2, "gather bwd")


def test_moe_layer_sparse_vs_dense_oracle():
    from oa_b200.core import fn_matrix as F
    from oa_b200.core.types import OaPrecision
    from oa_b200.ml.autograd import OaGradientTape
    from oa_b200.ml.nn.moe import OaMoE
    from oa_b200.runtime.engine import OaEngineConfig, OaInitComputeEngine, OaShutdownComputeEngine
    OaShutdownComputeEngine()
    assert OaInitComputeEngine(OaEngineConfig(Precision=OaPrecision.BF16, DeviceIndex=0))
    try:
        F.SetRngSeed(5)
        m = OaMoE(128, 192, 8, 2, num_shared_experts=1)
        m.SetAuxLossAlpha(0.01)
        x = F.RandN([512, 128], std=1.0).SetRequiresGrad(True)

        def run(sparse):
            m.SetSparseExecution(sparse)
            for p in m.AllParameterPtrs():
                p.Data._meta.grad, p.Data._meta.grad_fresh = None, True
            x._meta.grad = None
            with OaGradientTape() as tape:
                y = m.Forward(x)
                loss = F.Add(F.Cast(F.Mean(F.Mul(y, y)), 0), m.AuxLoss())
                tape.Backward(loss)
            return y.Tensor().float().clone(), x.GradTensor().float().clone(), {n.Name: n.Param.Data.GradTensor().float().clone() for n in m.AllNamedParameterPtrs()}

        ys, gxs, gs = run(True)
        yd, gxd, gd = run(False)
        _close(ys, yd, 3e-2, "moe forward")
        _close(gxs, gxd, 6e-2, "moe dx")
        for name in gs:
            _close(gs[name], gd[name], 8e-2, "moe grad " + name)
    finally:
        OaShutdownComputeEngine()
