"""Mamba-3 SISO: the PyTorch statement against a naive scalar recurrence, decode step against the full forward,
module gradients against torch.autograd (CPU), and the CUDA kernels against the PyTorch statement (GPU)."""
import math

import pytest
import torch

from oa_b200.ops import mamba3 as M3


def _dims(H=2, P=4, N=8, A=2, has_z=True, chunk=16):
    return M3.Mamba3Dims(d_inner=H * P, heads=H, headdim=P, d_state=N, angles=A, has_z=has_z, chunk=chunk)


def _inputs(d, B, L, device="cpu", dtype=torch.float32, seed=0):
    g = torch.Generator().manual_seed(seed)
    proj = torch.randn(B * L, d.d_in_proj, generator=g)
    o = d.offsets()
    proj[:, o[4]:o[4] + d.heads] -= 3.0                 # dt around softplus(-3 + bias): inside the clamp for most entries
    proj[:, o[7]:] *= 3.0                               # visible rotation
    dt_bias = torch.rand(1, d.heads, generator=g)
    Bb = 1.0 + 0.1 * torch.randn(d.heads, d.d_state, generator=g)
    Cb = 1.0 + 0.1 * torch.randn(d.heads, d.d_state, generator=g)
    D = 0.5 * torch.randn(d.heads, generator=g)
    mv = lambda t, dt_=torch.float32: t.to(device=device, dtype=dt_)
    return mv(proj, dtype), mv(dt_bias), mv(Bb), mv(Cb), mv(D)


def _naive(proj, dt_bias, Bb, Cb, D, d, B, L):
    """Scalar loops, look-ahead form: scale_t = gamma_t + dt_{t+1} (1 - sigmoid(trap_{t+1}))."""
    z, x, Bn, Cn, dt, adt, trap, angle = [t.double() for t in M3.reference_preprocess(proj, dt_bias, d, B, L)]
    H, P, N, A = d.heads, d.headdim, d.d_state, d.angles
    y = torch.zeros(B, L, H, P, dtype=torch.float64)
    for b in range(B):
        for h in range(H):
            Hs = torch.zeros(P, N, dtype=torch.float64)
            th = torch.zeros(A, dtype=torch.float64)
            for t in range(L):
                th = th + angle[b, t] * dt[b, t, h]
                C = Cn[b, t] + Cb[h].double()
                Bv = Bn[b, t] + Bb[h].double()
                Cr, Br = C.clone(), Bv.clone()
                for k in range(A):
                    c, s = math.cos(th[k]), math.sin(th[k])
                    Cr[2 * k], Cr[2 * k + 1] = C[2 * k] * c - C[2 * k + 1] * s, C[2 * k] * s + C[2 * k + 1] * c
                    Br[2 * k], Br[2 * k + 1] = Bv[2 * k] * c - Bv[2 * k + 1] * s, Bv[2 * k] * s + Bv[2 * k + 1] * c
                a = math.exp(adt[b, t, h])
                gamma = dt[b, t, h] * torch.sigmoid(trap[b, t, h])
                sg = dt[b, t + 1, h] * (1 - torch.sigmoid(trap[b, t + 1, h])) if t + 1 < L else 0.0
                qk = (Cr * Br).sum()
                xt = x[b, t, h * P:(h + 1) * P]
                yt = (a * Hs) @ Cr + (D[h].double() + gamma * qk) * xt
                if d.has_z:
                    zt = z[b, t, h * P:(h + 1) * P]
                    yt = yt * zt * torch.sigmoid(zt)
                y[b, t, h] = yt
                Hs = a * Hs + (gamma + sg) * xt[:, None] * Br[None, :]
    return y.reshape(B * L, H * P)


@pytest.mark.parametrize("has_z", [True, False])
def test_reference_matches_naive_recurrence(has_z):
    d = _dims(has_z=has_z)
    B, L = 2, 9
    args = _inputs(d, B, L)
    got = M3.reference_core(*args, d, B, L)
    want = _naive(*args, d, B, L)
    assert (got.double() - want).abs().max().item() < 1e-5


def test_step_matches_forward_cpu():
    d = _dims()
    B, L = 2, 7
    proj, dtb, Bb, Cb, D = _inputs(d, B, L)
    full = M3.reference_core(proj, dtb, Bb, Cb, D, d, B, L).reshape(B, L, -1)
    state = {}
    p3 = proj.reshape(B, L, -1)
    for t in range(L):
        y = M3.step(p3[:, t].contiguous(), dtb, Bb, Cb, D, d, state)
        assert (y - full[:, t]).abs().max().item() < 1e-5
    # prefill 4 tokens, then step the rest
    st = {}
    M3.core_fwd(p3[:, :4].reshape(B * 4, -1).contiguous(), dtb, Bb, Cb, D, d, B, 4, save=False, final=st)
    for t in range(4, L):
        y = M3.step(p3[:, t].contiguous(), dtb, Bb, Cb, D, d, st)
        assert (y - full[:, t]).abs().max().item() < 1e-5


@pytest.mark.parametrize("norm", [False, True])
def test_module_gradients_cpu(norm):
    from oa_b200.core.matrix import OaMatrix
    from oa_b200.ml import autograd as AG
    from oa_b200.core import fn_matrix as F
    from oa_b200.ml.nn.mamba3 import OaMamba3Module

    torch.manual_seed(0)
    m = OaMamba3Module(16, d_state=16, expand=2, headdim=8, is_outproj_norm=norm, chunk=8)
    B, L = 2, 6
    x = torch.randn(B, L, 16)
    for p in m.Parameters():
        p.Data.Tensor().copy_(p.Data.Tensor() + 0.05 * torch.randn_like(p.Data.Tensor()))
    tape = AG.OaGradientTape()
    xm = OaMatrix(x.clone())
    xm.SetRequiresGrad(True)
    out = m.Forward(xm)
    w = torch.randn(B, L, 16)
    loss = F.Sum(F.Mul(out, OaMatrix(w)))
    tape.Backward(loss)
    tape.Close()
    # the same composite in plain torch
    leaves = {p.Name: p.Data.Tensor().detach().clone().requires_grad_(True) for p in m.Parameters()}
    xt = x.clone().requires_grad_(True)
    proj = xt.reshape(B * L, 16) @ leaves["in_proj"].t()
    y = M3.reference_core(proj, leaves["dt_bias"], leaves["B_bias"], leaves["C_bias"], leaves["D"], m.Dims, B, L)
    if norm:
        H, P = m.NHeads, m.HeadDim
        yf = y.reshape(B * L, H, P)
        zf = proj[:, :m.DInner].reshape(B * L, H, P)
        y = (yf * torch.rsqrt((yf * yf).mean(-1, keepdim=True) + 1e-5) * leaves["norm_weight"].reshape(1, H, P)
             * torch.nn.functional.silu(zf)).reshape(B * L, H * P)
    ref_out = (y @ leaves["out_proj"].t()).reshape(B, L, 16)
    assert (out.Tensor() - ref_out).abs().max().item() < 1e-4
    (ref_out * w).sum().backward()
    assert (xm.GradTensor() - xt.grad).abs().max().item() < 1e-4
    for p in m.Parameters():
        g, r = p.Grad().Tensor().float(), leaves[p.Name].grad
        assert (g.reshape(r.shape) - r).abs().max().item() <= 1e-4 * max(1.0, r.abs().max().item()), p.Name


# --------------------------------------------------------------------------------------------------------------- GPU
CASES = [
    dict(H=4, P=16, N=32, A=8, B=2, L=41, chunk=16),       # several chunks, ragged last chunk and sub-chunk
    dict(H=2, P=64, N=128, A=32, B=2, L=70, chunk=32),     # the large-model head shape
    dict(H=3, P=8, N=16, A=0, B=1, L=9, chunk=8),          # no rotary angles, small head
]


@pytest.mark.gpu
@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("has_z", [True, False])
def test_scan_kernels_match_reference(case, has_z):
    from oa_b200.ops import kernels as K
    c = dict(case)
    B, L = c.pop("B"), c.pop("L")
    d = _dims(has_z=has_z, **c)
    cpu = _inputs(d, B, L)
    gpu = tuple(t.cuda() for t in cpu)
    y, saved = M3.core_fwd(gpu[0], *gpu[1:], d, B, L, save=True)
    want = M3.reference_core(*cpu, d, B, L)
    assert (y.cpu() - want).abs().max().item() <= 2e-4 * max(1.0, want.abs().max().item())
    dy = torch.randn(B * L, d.d_inner, generator=torch.Generator().manual_seed(1))
    got = M3.core_bwd(saved, dy.cuda())
    _, scpu = M3.core_fwd(cpu[0], *cpu[1:], d, B, L)
    ref = M3.core_bwd(scpu, dy)
    for g, r, nm in zip(got, ref, ("dproj", "ddt_bias", "dB_bias", "dC_bias", "dD")):
        scale = max(1.0, r.abs().max().item())
        err = (g.cpu().float().reshape(r.shape) - r.float()).abs().max().item()
        assert err <= 5e-4 * scale, (nm, err, scale)
    torch.cuda.synchronize()
    K.check_status()


@pytest.mark.gpu
def test_step_kernel_matches_forward():
    d = _dims(H=4, P=16, N=32, A=8, chunk=16)
    B, L = 3, 12
    cpu = _inputs(d, B, L)
    gpu = tuple(t.cuda() for t in cpu)
    full = M3.reference_core(*cpu, d, B, L).reshape(B, L, -1)
    p3 = gpu[0].reshape(B, L, -1)
    st = {}
    for t in range(L):
        y = M3.step(p3[:, t].contiguous(), *gpu[1:], d, st)
        assert (y.cpu() - full[:, t]).abs().max().item() < 2e-4, t
    st = {}
    M3.core_fwd(p3[:, :5].reshape(B * 5, -1).contiguous(), *gpu[1:], d, B, 5, save=False, final=st)
    for t in range(5, L):
        y = M3.step(p3[:, t].contiguous(), *gpu[1:], d, st)
        assert (y.cpu() - full[:, t]).abs().max().item() < 2e-4, t


@pytest.mark.gpu
@pytest.mark.parametrize("P", [16, 64])
def test_gated_norm_kernels(P):
    H, rows = 4, 37
    d = M3.Mamba3Dims(d_inner=H * P, heads=H, headdim=P, d_state=16, angles=2, has_z=False)
    g = torch.Generator().manual_seed(0)
    y = torch.randn(rows, H * P, generator=g)
    proj = torch.randn(rows, d.d_in_proj, generator=g)
    w = 1 + 0.1 * torch.randn(H, P, generator=g)
    do = torch.randn(rows, H * P, generator=g)
    out_r, rstd_r = M3.gated_norm_fwd(y, proj, w, d)
    dproj_r = torch.zeros_like(proj)
    dy_r, dw_r = M3.gated_norm_bwd(y, proj, w, rstd_r, do, d, dproj_r)
    out, rstd = M3.gated_norm_fwd(y.cuda(), proj.cuda(), w.cuda(), d)
    dproj = torch.zeros_like(proj).cuda()
    dy, dw = M3.gated_norm_bwd(y.cuda(), proj.cuda(), w.cuda(), rstd, do.cuda(), d, dproj)
    for a, b in ((out, out_r), (dy, dy_r), (dw, dw_r), (dproj, dproj_r)):
        assert (a.cpu() - b).abs().max().item() <= 1e-4 * max(1.0, b.abs().max().item())


@pytest.mark.gpu
def test_module_bf16_runs_and_tracks_fp32():
    from oa_b200.core.matrix import OaMatrix
    from oa_b200.ml.nn.mamba3 import OaMamba3Module
    from oa_b200.ops import kernels as K

    d = _dims(H=4, P=16, N=32, A=8, chunk=16)
    B, L = 2, 33
    cpu = _inputs(d, B, L)
    y, saved = M3.core_fwd(cpu[0].cuda().bfloat16(), *[t.cuda() for t in cpu[1:]], d, B, L)
    want = M3.reference_core(cpu[0].bfloat16().float(), *cpu[1:], d, B, L)
    assert (y.float().cpu() - want).abs().max().item() <= 3e-2 * max(1.0, want.abs().max().item())
    dy = torch.randn(B * L, d.d_inner).bfloat16()
    got = M3.core_bwd(saved, dy.cuda())
    _, scpu = M3.core_fwd(cpu[0].bfloat16().float(), *cpu[1:], d, B, L)
    ref = M3.core_bwd(scpu, dy.float())
    for g, r in zip(got, ref):
        assert (g.cpu().float().reshape(r.shape) - r).abs().max().item() <= 4e-2 * max(1.0, r.abs().max().item())
    K.check_status()


# ------------------------------------------------------------------------------------------ chunked (tensor-core) scan
def _ssd_vs_reference(d, B, L, Q, device, gemm_dtype, tol):
    from oa_b200.ops import mamba3_ssd as SSD
    H, P = d.heads, d.headdim
    cpu = _inputs(d, B, L)
    leaves = [t.clone().requires_grad_(True) for t in cpu]
    want = M3.reference_core(*leaves, d, B, L)
    dy = torch.randn(B * L, d.d_inner, generator=torch.Generator().manual_seed(1))
    ref = torch.autograd.grad(want, leaves, dy)
    lv = [t.clone().requires_grad_(True) for t in cpu[:2]]
    z, x, Bn, Cn, dt, adt, trap, angle = M3.reference_preprocess(lv[0], lv[1], d, B, L)
    ins = [x.reshape(B, L, H, P), z.reshape(B, L, H, P) if d.has_z else None, Bn, Cn, dt, adt, trap, angle]
    dev = [t.detach().to(device) if t is not None else None for t in ins]
    y, saved = SSD.ssd_fwd(*dev, *[t.to(device) for t in cpu[2:]], d, B, L, Q, gemm_dtype=gemm_dtype)
    assert (y.cpu().reshape(B * L, -1) - want).abs().max().item() <= tol * max(1.0, want.abs().max().item())
    gs = SSD.ssd_bwd(saved, dy.reshape(B, L, H, P).to(device))
    gs = {k: (v.cpu() if v is not None else None) for k, v in gs.items()}
    outs = [ins[0], ins[2], ins[3], ins[4], ins[5], ins[6], ins[7]] + ([ins[1]] if d.has_z else [])
    gl = [gs["x"], gs["Bn"], gs["Cn"], gs["dt"], gs["adt"], gs["trap"], gs["angle"]] + ([gs["z"]] if d.has_z else [])
    chain = torch.autograd.grad(outs, lv, gl)
    for got, r, nm in zip((chain[0], chain[1], gs["Bb"], gs["Cb"], gs["D"]), ref, ("dproj", "ddt_bias", "dB_bias", "dC_bias", "dD")):
        err = (got.reshape(r.shape) - r).abs().max().item()
        assert err <= tol * max(1.0, r.abs().max().item()), (nm, err)


@pytest.mark.parametrize("has_z", [True, False])
@pytest.mark.parametrize("A", [4, 0])
def test_ssd_math_matches_recurrence_cpu(has_z, A):
    """The chunked form (masked score GEMMs + chunk-state recurrence) and its hand-written backward equal the
    token-by-token recurrence and torch.autograd through it."""
    d = _dims(H=2, P=8, N=16, A=A, has_z=has_z)
    _ssd_vs_reference(d, 2, 32, 8, "cpu", torch.float32, 2e-5)


@pytest.mark.gpu
def test_ssd_bf16_gemms_track_fp32_reference():
    from oa_b200.ops import kernels as K
    d = _dims(H=4, P=64, N=128, A=32)
    _ssd_vs_reference(d, 2, 256, 128, "cuda", torch.bfloat16, 3e-2)
    K.check_status()


@pytest.mark.gpu
def test_core_uses_chunked_scan_for_bf16_training():
    """core_fwd / core_bwd on bf16 CUDA input with a whole number of chunks take the tensor-core path and agree with
    the sequential kernels on the same input."""
    import os
    from oa_b200.ops import kernels as K
    d = _dims(H=4, P=64, N=128, A=32, chunk=64)
    B, L = 2, 256
    cpu = _inputs(d, B, L)
    args = [cpu[0].cuda().bfloat16()] + [t.cuda() for t in cpu[1:]]
    y, sv = M3.core_fwd(*args, d, B, L)
    assert sv.ssd is not None
    dy = torch.randn(B * L, d.d_inner).bfloat16().cuda()
    got = M3.core_bwd(sv, dy)
    os.environ["OA_MAMBA3_SSD"] = "0"
    try:
        y0, sv0 = M3.core_fwd(*args, d, B, L)
        assert sv0.ssd is None
        ref = M3.core_bwd(sv0, dy)
    finally:
        os.environ.pop("OA_MAMBA3_SSD")
    assert (y.float() - y0.float()).abs().max().item() <= 3e-2 * max(1.0, y0.float().abs().max().item())
    for g, r, nm in zip(got, ref, ("dproj", "ddt_bias", "dB_bias", "dC_bias", "dD")):
        err = (g.float() - r.float().reshape(g.shape)).abs().max().item()
        assert err <= 4e-2 * max(1.0, r.float().abs().max().item()), (nm, err)
    # the fused glue kernels and the tensor-expression glue are the same algorithm: tight agreement
    os.environ["OA_MAMBA3_SSD_FUSED"] = "0"
    try:
        y1, sv1 = M3.core_fwd(*args, d, B, L)
        ref1 = M3.core_bwd(sv1, dy)
    finally:
        os.environ.pop("OA_MAMBA3_SSD_FUSED")
    assert (y.float() - y1.float()).abs().max().item() <= 1e-2 * max(1.0, y1.float().abs().max().item())
    for g, r, nm in zip(got, ref1, ("dproj", "ddt_bias", "dB_bias", "dC_bias", "dD")):
        err = (g.float() - r.float().reshape(g.shape)).abs().max().item()
        assert err <= 1.5e-2 * max(1.0, r.float().abs().max().item()), (nm, err)
    K.check_status()


def test_empyrealm_core_modes_cpu():
    """Byte mode, custom-projection mode and embedded-only mode share the mixer + residual path."""
    from oa_b200.core import fn_matrix as F
    from oa_b200.core.matrix import OaMatrix
    from oa_b200.ml import autograd as AG
    from oa_b200.ml.nn.empyrealm import OaEmpyrealmCore
    from oa_b200.ml.nn.layers import OaLinear
    F.SetRngSeed(11)
    core = OaEmpyrealmCore(50, 16, d_state=8, headdim=8)
    ids = OaMatrix(torch.randint(0, 50, (2, 6), dtype=torch.int32))
    tape = AG.OaGradientTape()
    out = core.Forward(ids)
    tape.Backward(F.Sum(F.Mul(out, out)))
    tape.Close()
    assert tuple(out.Tensor().shape) == (12, 16)
    names = [n.Name for n in core.AllNamedParameterPtrs()]
    assert any(n.startswith("embed.") for n in names) and any(n.startswith("mixer.") for n in names)
    assert all(n.Param.Data.GradTensor() is not None for n in core.AllNamedParameterPtrs())
    emb = core.Embed.Forward(ids).Tensor().reshape(2, 6, 16)
    mixed = core.Mixer().Forward(OaMatrix(emb)).Tensor().reshape(12, 16)
    assert torch.allclose(out.Tensor(), mixed + emb.reshape(12, 16), atol=1e-6)            # residual around the mixer
    # sequences of a batch do not leak into each other
    ids2 = ids.Tensor().clone()
    ids2[1] = (ids2[1] + 7) % 50
    out2 = core.Forward(OaMatrix(ids2)).Tensor()
    assert torch.equal(out2[:6], out.Tensor()[:6]) and not torch.equal(out2[6:], out.Tensor()[6:])
    only = OaEmpyrealmCore.EmbeddedOnly(16, d_state=8, headdim=8)
    assert not any(n.Name.startswith("embed.") for n in only.AllNamedParameterPtrs())
    with pytest.raises(RuntimeError):
        only.Forward(ids)
    assert tuple(only.ForwardEmbedded(OaMatrix(torch.randn(2, 6, 16))).Tensor().shape) == (12, 16)
    assert tuple(only.ForwardEmbedded(OaMatrix(torch.randn(9, 16))).Tensor().shape) == (9, 16)

    class Pose(OaLinear):
        def Forward(self, x):
            return super().Forward(x.Reshape([x.Size(0) * x.Size(1), x.Size(2)])).Reshape([x.Size(0), x.Size(1), 16])

    custom = OaEmpyrealmCore(Pose(5, 16), 16, d_state=8, headdim=8)
    assert tuple(custom.Forward(OaMatrix(torch.randn(3, 4, 5))).Tensor().shape) == (12, 16)
    custom.ResetState(3)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_benchmark_variant_kernels_match_the_composed_ops(dtype):
    """Causal depthwise convolution + SiLU and the learned-decay fill (mamba3_conv.cu) against the same options composed from
    differentiable tensor ops on the CPU: forward values and every gradient."""
    from oa_b200.core import fn_matrix as F
    from oa_b200.core.matrix import OaMatrix
    from oa_b200.core.types import OaPrecision
    from oa_b200.ml.autograd import OaGradientTape
    from oa_b200.ml.nn.mamba3 import OaMamba3Module
    from oa_b200.runtime import engine as RT
    B, L = 2, 150

    def run(device):
        cfg = RT.OaEngineConfig(Precision=OaPrecision.FP32 if dtype == torch.float32 else OaPrecision.BF16)
        if device == "cpu":
            cfg.DevicePreference = RT.OaDevicePreference.Cpu
            cfg.Precision = OaPrecision.FP32
        eng = RT.OaEngine.Create(cfg)
        eng.SetAsGlobal()
        F.SetRngSeed(4)
        m = OaMamba3Module(32, d_state=16, expand=2, headdim=16, conv_width=4, a_log=True)
        g = torch.Generator().manual_seed(9)
        wref = {n.Name: torch.randn(n.Param.Tensor().shape, generator=g) * 0.3 for n in m.AllNamedParameterPtrs()}
        for n in m.AllNamedParameterPtrs():
            n.Param.Tensor().copy_(wref[n.Name].to(n.Param.Tensor().dtype))
        x = torch.randn(B * L, m.DInProj, generator=g)
        up = torch.randn(B * L, m.DInProj, generator=g)
        dev = eng.Device()
        proj = OaMatrix(x.to(device=dev, dtype=dtype if device != "cpu" else torch.float32)).SetRequiresGrad(True)
        with OaGradientTape() as tape:
            out = m._prepare(proj, B, L)
            tape.Backward(out, grad=up.to(device=dev, dtype=out.Tensor().dtype))
        return (out.Tensor().float().cpu(), proj.GradTensor().float().cpu(), m.ConvWeight.Data.GradTensor().float().cpu(),
                m.ALog.Data.GradTensor().float().cpu())

    got, ref = run("cuda"), run("cpu")
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    for a, b, what in zip(got, ref, ("forward", "dproj", "dconv_weight", "dA_log")):
        scale = b.abs().max().item() + 1e-9
        assert (a - b).abs().max().item() <= tol * scale, (what, (a - b).abs().max().item(), scale)
