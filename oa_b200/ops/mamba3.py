"""Mamba-3 SISO core on raw tensors: preprocess + selective scan (+ gated output norm), forward, backward and decode step.

The math is the reference recurrence (Test/Ml/Nn/TestMamba3.cpp:107-142; preprocess in
Shader/Compute/Nn/Ssm/Mamba3/Mamba3Preprocess.slang:1-14).  `reference_core` states it in plain fp32 PyTorch and is
differentiable by torch.autograd: it is the CPU path (forward and backward) and the oracle of the GPU tests.  CUDA
tensors run the kernels of csrc/kernels/mamba3.cu.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch

from .. import _native as N
from . import kernels as K


@dataclass
class Mamba3Dims:
    d_inner: int
    heads: int
    headdim: int
    d_state: int
    angles: int
    has_z: bool = True            # silu(z) gate inside the scan (off when the gated output norm does it)
    eps: float = 1e-5
    dt_min: float = 1e-3
    dt_max: float = 0.1
    afloor: float = 1e-4
    chunk: int = 256

    @property
    def d_in_proj(self) -> int:
        return 2 * self.d_inner + 2 * self.d_state + 3 * self.heads + self.angles

    def offsets(self):
        z, x = 0, self.d_inner
        b = 2 * self.d_inner
        c = b + self.d_state
        dd_dt = c + self.d_state
        dd_a = dd_dt + self.heads
        trap = dd_a + self.heads
        angle = trap + self.heads
        return z, x, b, c, dd_dt, dd_a, trap, angle


def _rot(v: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, A: int) -> torch.Tensor:
    """Rotates pairs (2k, 2k+1), k < A, of the last dimension."""
    if A == 0:
        return v
    head = v[..., :2 * A].reshape(*v.shape[:-1], A, 2)
    v0, v1 = head[..., 0], head[..., 1]
    r = torch.stack((v0 * cos - v1 * sin, v0 * sin + v1 * cos), -1).reshape(*v.shape[:-1], 2 * A)
    return torch.cat((r, v[..., 2 * A:]), -1)


def reference_preprocess(proj: torch.Tensor, dt_bias: torch.Tensor, d: Mamba3Dims, B: int, L: int):
    pf = proj.float().reshape(B, L, -1)
    o = d.offsets()
    H, Nn, A = d.heads, d.d_state, d.angles
    z, x = pf[..., o[0]:o[0] + d.d_inner], pf[..., o[1]:o[1] + d.d_inner]
    Bm, Cm = pf[..., o[2]:o[2] + Nn], pf[..., o[3]:o[3] + Nn]
    dd_dt, dd_a = pf[..., o[4]:o[4] + H], pf[..., o[5]:o[5] + H]
    trap, angle = pf[..., o[6]:o[6] + H], pf[..., o[7]:o[7] + A]
    Bn = Bm * torch.rsqrt((Bm * Bm).mean(-1, keepdim=True) + d.eps)
    Cn = Cm * torch.rsqrt((Cm * Cm).mean(-1, keepdim=True) + d.eps)
    dt = torch.clamp(torch.nn.functional.softplus(dd_dt + dt_bias.float().reshape(1, 1, H)), d.dt_min, d.dt_max)
    ht = torch.where(dd_a >= 0, 1.0 + dd_a, 1.0 / (1.0 - torch.clamp(dd_a, max=0.0)))
    adt = torch.minimum(-ht, torch.full_like(ht, -d.afloor)) * dt
    return z, x, Bn, Cn, dt, adt, trap, angle


def reference_core(proj: torch.Tensor, dt_bias, Bb, Cb, D, d: Mamba3Dims, B: int, L: int, state: Optional[dict] = None):
    """y [B*L, d_inner] fp32 of the whole core; `state` (decode) carries H, theta, K, V between calls and is updated."""
    H, P, Nn, A = d.heads, d.headdim, d.d_state, d.angles
    z, x, Bn, Cn, dt, adt, trap, angle = reference_preprocess(proj, dt_bias, d, B, L)
    tr = torch.sigmoid(trap)
    gamma = dt * tr
    late = dt * (1.0 - tr)                                    # coefficient of the previous token's x (x) B~ term
    x4, z4 = x.reshape(B, L, H, P), z.reshape(B, L, H, P)
    Cb_, Bb_ = Cb.float().reshape(1, H, Nn), Bb.float().reshape(1, H, Nn)
    Dv = D.float().reshape(1, H) if D is not None else torch.zeros(1, H, device=proj.device)
    if state is not None and state.get("H") is not None:
        Hs, theta, Kp, Vp = state["H"], state["theta"], state["K"], state["V"]
        first = False
    else:
        Hs = torch.zeros(B, H, P, Nn, device=proj.device)
        theta = torch.zeros(B, H, A, device=proj.device)
        Kp = torch.zeros(B, H, Nn, device=proj.device)
        Vp = torch.zeros(B, H, P, device=proj.device)
        first = True
    ys = []
    for t in range(L):
        theta = theta + angle[:, t].reshape(B, 1, A) * dt[:, t].reshape(B, H, 1)
        cos, sin = torch.cos(theta), torch.sin(theta)
        Ct = _rot(Cn[:, t].reshape(B, 1, Nn) + Cb_, cos, sin, A)
        Bt = _rot(Bn[:, t].reshape(B, 1, Nn) + Bb_, cos, sin, A)
        if not (first and t == 0):
            Hs = Hs + late[:, t].reshape(B, H, 1, 1) * Vp.unsqueeze(-1) * Kp.unsqueeze(-2)
        a = torch.exp(adt[:, t]).reshape(B, H, 1, 1)
        Hd = a * Hs
        qk = (Ct * Bt).sum(-1)
        xt = x4[:, t]
        y = torch.einsum("bhn,bhpn->bhp", Ct, Hd) + (Dv + gamma[:, t] * qk).unsqueeze(-1) * xt
        if d.has_z:
            y = y * torch.nn.functional.silu(z4[:, t])
        ys.append(y)
        Hs = Hd + gamma[:, t].reshape(B, H, 1, 1) * xt.unsqueeze(-1) * Bt.unsqueeze(-2)
        Kp, Vp = Bt, xt
    if state is not None:
        state.update(H=Hs.detach(), theta=theta.detach(), K=Kp.detach(), V=Vp.detach())
    return torch.stack(ys, 1).reshape(B * L, H * P)


def _f32(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    if t is None:
        return None
    return t.contiguous() if t.dtype == torch.float32 else K.cast(t.contiguous(), torch.float32)


def _use_ssd(proj: torch.Tensor, d: "Mamba3Dims", L: int) -> bool:
    """The chunked tensor-core scan serves bf16 training on CUDA when the sequence is a whole number of chunks; fp32
    inputs, ragged lengths and decode prefill (which needs the recurrent state) use the sequential kernels.
    OA_MAMBA3_SSD=0 forces the sequential kernels."""
    if os.environ.get("OA_MAMBA3_SSD", "1") == "0" or not proj.is_cuda or proj.dtype != torch.bfloat16:
        return False
    from . import mamba3_ssd as SSD
    return SSD.supported(d, L, SSD.CHUNK)


class Saved:
    __slots__ = ("proj", "params", "pre", "Hck", "Tck", "dims", "B", "L", "ssd")


def core_fwd(proj: torch.Tensor, dt_bias, Bb, Cb, D, d: Mamba3Dims, B: int, L: int, save: bool = True, final: Optional[dict] = None):
    """proj [B*L, d_in_proj] -> (y [B*L, d_inner] in proj's dtype, saved).  `final`, when given, receives the decode state."""
    rows = B * L
    assert proj.shape == (rows, d.d_in_proj) and proj.is_contiguous()
    if not proj.is_cuda:
        st = {} if final is not None else None
        y = reference_core(proj, dt_bias, Bb, Cb, D, d, B, L, st)
        if final is not None:
            final.update(st)
        s = Saved()
        s.proj, s.params, s.dims, s.B, s.L = proj, (dt_bias, Bb, Cb, D), d, B, L
        return y.to(proj.dtype), s
    lib, dev, st_ = N.require(), proj.device, N.stream()
    H, P, Nn, A = d.heads, d.headdim, d.d_state, d.angles
    f = lambda *shape: torch.empty(shape, dtype=torch.float32, device=dev)
    Bn, Cn, rstd = f(rows, Nn), f(rows, Nn), f(rows, 2)
    dt, adt, trap, angle = f(rows, H), f(rows, H), f(rows, H), f(rows, max(A, 1))
    dtb, Bb32, Cb32, D32 = _f32(dt_bias), _f32(Bb), _f32(Cb), _f32(D)
    K._launch(lib.oa_mamba3_pre_fwd(K.dt(proj), proj.data_ptr(), d.d_in_proj, dtb.data_ptr(), rows, H, Nn, A, d.d_inner, d.eps, d.dt_min,
                                    d.dt_max, d.afloor, Bn.data_ptr(), Cn.data_ptr(), rstd.data_ptr(), dt.data_ptr(), adt.data_ptr(),
                                    trap.data_ptr(), angle.data_ptr(), st_), "oa_mamba3_pre_fwd")
    if final is None and _use_ssd(proj, d, L):
        # chunked tensor-core path: the same preprocessed inputs, GEMM-shaped scan
        from . import mamba3_ssd as SSD
        s = Saved()
        s.proj, s.params, s.dims, s.B, s.L = proj, (dtb, Bb32, Cb32, D32), d, B, L
        s.pre, s.Hck, s.Tck = (Bn, Cn, rstd, dt, adt, trap, angle), None, None
        if os.environ.get("OA_MAMBA3_SSD_FUSED", "1") != "0":
            y, sv = SSD.ssd_fwd_cuda(proj, Bn, Cn, dt, adt, trap, angle, Bb32, Cb32, D32, d, B, L, save)
            s.ssd = sv
            return y, s
        o = d.offsets()
        v4 = lambda c0: proj[:, c0:c0 + d.d_inner].reshape(B, L, H, P)
        r3 = lambda t, w: t.reshape(B, L, w)
        y4, sv = SSD.ssd_fwd(v4(o[1]), v4(o[0]) if d.has_z else None, r3(Bn, Nn), r3(Cn, Nn), r3(dt, H), r3(adt, H), r3(trap, H),
                             r3(angle, max(A, 1))[..., :A], Bb32, Cb32, D32, d, B, L, SSD.CHUNK)
        s.ssd = sv if save else None
        return y4.reshape(rows, d.d_inner).to(proj.dtype), s
    nC = (L + d.chunk - 1) // d.chunk
    Hck = f(B, H, nC, P, Nn) if save else None
    Tck = f(B, H, nC, max(A, 1)) if save else None
    y = torch.empty((rows, d.d_inner), dtype=proj.dtype, device=dev)
    es = proj.element_size()
    o = d.offsets()
    if final is not None:
        final.update(H=f(B, H, P, Nn), theta=torch.zeros(B, H, max(A, 1), dtype=torch.float32, device=dev), K=f(B, H, Nn), V=f(B, H, P))
    K._launch(lib.oa_mamba3_scan_fwd(K.dt(proj), proj.data_ptr() + o[1] * es, proj.data_ptr() + o[0] * es if d.has_z else None,
                                     d.d_in_proj, Cn.data_ptr(), Bn.data_ptr(), dt.data_ptr(), adt.data_ptr(), trap.data_ptr(),
                                     angle.data_ptr(), Cb32.data_ptr(), Bb32.data_ptr(), N.ptr(D32), y.data_ptr(), d.d_inner,
                                     N.ptr(Hck), N.ptr(Tck), N.ptr(final["H"]) if final is not None else None,
                                     N.ptr(final["theta"]) if final is not None else None,
                                     N.ptr(final["K"]) if final is not None else None, N.ptr(final["V"]) if final is not None else None,
                                     B, L, H, P, Nn, A, d.chunk, st_), "oa_mamba3_scan_fwd")
    s = Saved()
    s.proj, s.params, s.dims, s.B, s.L = proj, (dtb, Bb32, Cb32, D32), d, B, L
    s.pre, s.Hck, s.Tck, s.ssd = (Bn, Cn, rstd, dt, adt, trap, angle), Hck, Tck, None
    return y, s


def core_bwd(s: Saved, dy: torch.Tensor, dproj: Optional[torch.Tensor] = None):
    """Returns (dproj [B*L, d_in_proj], ddt_bias [H], dBb [H,N], dCb [H,N], dD [H]) - parameter gradients in fp32.
    With `dproj` given, only the columns this op owns are written (the z columns stay untouched when has_z is off)."""
    d, B, L, proj = s.dims, s.B, s.L, s.proj
    rows = B * L
    H, P, Nn, A = d.heads, d.headdim, d.d_state, d.angles
    if not proj.is_cuda:
        dt_bias, Bb, Cb, D = s.params
        leaves = [proj.detach().float().requires_grad_(True)] + [t.detach().float().requires_grad_(True) for t in (dt_bias, Bb, Cb)]
        Dl = D.detach().float().requires_grad_(True) if D is not None else None
        with torch.enable_grad():
            y = reference_core(leaves[0], leaves[1], leaves[2], leaves[3], Dl, d, B, L)
            gs = torch.autograd.grad(y, leaves + ([Dl] if Dl is not None else []), dy.float(), allow_unused=True)
        gp = gs[0].to(proj.dtype)
        if dproj is not None:
            if d.has_z:
                dproj.copy_(gp)
            else:
                dproj[:, d.d_inner:] = gp[:, d.d_inner:]
            gp = dproj
        z0 = lambda g, like: g if g is not None else torch.zeros_like(like)
        return gp, z0(gs[1], leaves[1]), z0(gs[2], leaves[2]), z0(gs[3], leaves[3]), (z0(gs[4], Dl) if Dl is not None else None)
    lib, dev, st_ = N.require(), proj.device, N.stream()
    Bn, Cn, rstd, dt, adt, trap, angle = s.pre
    dtb, Bb32, Cb32, D32 = s.params
    Am = max(A, 1)
    sizes = [rows * Nn, rows * Nn, rows * H, rows * H, rows * H, rows * Am, H * Nn, H * Nn, H, H]
    flat = torch.zeros(sum(sizes), dtype=torch.float32, device=dev)
    parts, off = [], 0
    for n in sizes:
        parts.append(flat[off:off + n])
        off += n
    dCn, dBn, ddt, dadt, dtrap, dangle, dCb, dBb, dD, ddtb = parts
    if dproj is None:
        dproj = torch.empty_like(proj)
        if not d.has_z:
            dproj[:, :d.d_inner].zero_()
    es = proj.element_size()
    o = d.offsets()
    if s.ssd is not None:
        from . import mamba3_ssd as SSD
        if isinstance(s.ssd, SSD.SsdSavedCuda):
            g = SSD.ssd_bwd_cuda(s.ssd, proj, dy, dproj)
        else:
            g = SSD.ssd_bwd(s.ssd, dy.reshape(B, L, H, P))
            dproj[:, o[1]:o[1] + d.d_inner] = g["x"].reshape(rows, d.d_inner)
            if d.has_z:
                dproj[:, o[0]:o[0] + d.d_inner] = g["z"].reshape(rows, d.d_inner)
        c32 = lambda t: t.reshape(rows, -1).float().contiguous()
        dBn, dCn, ddt, dadt, dtrap = c32(g["Bn"]), c32(g["Cn"]), c32(g["dt"]), c32(g["adt"]), c32(g["trap"])
        if A:
            dangle = c32(g["angle"])
        dBb, dCb = g["Bb"].contiguous(), g["Cb"].contiguous()
        if D32 is not None:
            dD = g["D"]
        K._launch(lib.oa_mamba3_pre_bwd(K.dt(proj), proj.data_ptr(), dproj.data_ptr(), d.d_in_proj, dtb.data_ptr(), rows, H, Nn, A, d.d_inner,
                                        d.eps, d.dt_min, d.dt_max, d.afloor, Bn.data_ptr(), Cn.data_ptr(), rstd.data_ptr(), dBn.data_ptr(),
                                        dCn.data_ptr(), ddt.data_ptr(), dadt.data_ptr(), dtrap.data_ptr(), dangle.data_ptr(),
                                        ddtb.data_ptr(), st_), "oa_mamba3_pre_bwd")
        return dproj, ddtb, dBb.view(H, Nn), dCb.view(H, Nn), (dD if D32 is not None else None)
    scratch = K.scratch(dev, 4 * int(lib.oa_mamba3_scratch_floats(B, H, P, Nn, d.chunk)), "mamba3_bwd")
    dy = dy.contiguous()
    K._launch(lib.oa_mamba3_scan_bwd(K.dt(proj), proj.data_ptr() + o[1] * es, proj.data_ptr() + o[0] * es if d.has_z else None,
                                     d.d_in_proj, Cn.data_ptr(), Bn.data_ptr(), dt.data_ptr(), adt.data_ptr(), trap.data_ptr(),
                                     angle.data_ptr(), Cb32.data_ptr(), Bb32.data_ptr(), N.ptr(D32), dy.data_ptr(), d.d_inner,
                                     dproj.data_ptr() + o[1] * es, dproj.data_ptr() + o[0] * es if d.has_z else None, d.d_in_proj,
                                     dCn.data_ptr(), dBn.data_ptr(), ddt.data_ptr(), dadt.data_ptr(), dtrap.data_ptr(),
                                     dangle.data_ptr(), dCb.data_ptr(), dBb.data_ptr(), dD.data_ptr(), s.Hck.data_ptr(),
                                     s.Tck.data_ptr(), scratch.data_ptr(), B, L, H, P, Nn, A, d.chunk, st_), "oa_mamba3_scan_bwd")
    K._launch(lib.oa_mamba3_pre_bwd(K.dt(proj), proj.data_ptr(), dproj.data_ptr(), d.d_in_proj, dtb.data_ptr(), rows, H, Nn, A, d.d_inner,
                                    d.eps, d.dt_min, d.dt_max, d.afloor, Bn.data_ptr(), Cn.data_ptr(), rstd.data_ptr(), dBn.data_ptr(),
                                    dCn.data_ptr(), ddt.data_ptr(), dadt.data_ptr(), dtrap.data_ptr(), dangle.data_ptr(),
                                    ddtb.data_ptr(), st_), "oa_mamba3_pre_bwd")
    return dproj, ddtb, dBb.view(H, Nn), dCb.view(H, Nn), (dD if D32 is not None else None)


def step(proj: torch.Tensor, dt_bias, Bb, Cb, D, d: Mamba3Dims, state: dict) -> torch.Tensor:
    """One decode token per sequence: proj [B, d_in_proj] -> y [B, d_inner]; `state` is created on first use."""
    Bsz = proj.shape[0]
    if not proj.is_cuda:
        return reference_core(proj, dt_bias, Bb, Cb, D, d, Bsz, 1, state).to(proj.dtype)
    lib, dev, st_ = N.require(), proj.device, N.stream()
    H, P, Nn, A = d.heads, d.headdim, d.d_state, d.angles
    Am = max(A, 1)
    f = lambda *shape: torch.zeros(shape, dtype=torch.float32, device=dev)
    first = state.get("H") is None
    if first:
        state.update(H=f(Bsz, H, P, Nn), theta=f(Bsz, H, Am), K=f(Bsz, H, Nn), V=f(Bsz, H, P))
    if "theta2" not in state:
        state.update(theta2=f(Bsz, H, Am), K2=f(Bsz, H, Nn))
    Bn, Cn = (torch.empty((Bsz, Nn), dtype=torch.float32, device=dev) for _ in range(2))
    rstd = torch.empty((Bsz, 2), dtype=torch.float32, device=dev)
    dt, adt, trap = (torch.empty((Bsz, H), dtype=torch.float32, device=dev) for _ in range(3))
    angle = torch.empty((Bsz, Am), dtype=torch.float32, device=dev)
    dtb, Bb32, Cb32, D32 = _f32(dt_bias), _f32(Bb), _f32(Cb), _f32(D)
    proj = proj.contiguous()
    K._launch(lib.oa_mamba3_pre_fwd(K.dt(proj), proj.data_ptr(), d.d_in_proj, dtb.data_ptr(), Bsz, H, Nn, A, d.d_inner, d.eps, d.dt_min,
                                    d.dt_max, d.afloor, Bn.data_ptr(), Cn.data_ptr(), rstd.data_ptr(), dt.data_ptr(), adt.data_ptr(),
                                    trap.data_ptr(), angle.data_ptr(), st_), "oa_mamba3_pre_fwd")
    y = torch.empty((Bsz, d.d_inner), dtype=proj.dtype, device=dev)
    es = proj.element_size()
    o = d.offsets()
    K._launch(lib.oa_mamba3_step(K.dt(proj), proj.data_ptr() + o[1] * es, proj.data_ptr() + o[0] * es if d.has_z else None, d.d_in_proj,
                                 Cn.data_ptr(), Bn.data_ptr(), dt.data_ptr(), adt.data_ptr(), trap.data_ptr(), angle.data_ptr(),
                                 Cb32.data_ptr(), Bb32.data_ptr(), N.ptr(D32), y.data_ptr(), d.d_inner, state["H"].data_ptr(),
                                 state["V"].data_ptr(), state["theta"].data_ptr(), state["K"].data_ptr(), state["theta2"].data_ptr(),
                                 state["K2"].data_ptr(), Bsz, H, P, Nn, A, 1 if first else 0, st_), "oa_mamba3_step")
    state["theta"], state["theta2"] = state["theta2"], state["theta"]
    state["K"], state["K2"] = state["K2"], state["K"]
    return y


def gated_norm_fwd(y: torch.Tensor, proj: torch.Tensor, w: torch.Tensor, d: Mamba3Dims, eps: float = 1e-5):
    """out = rmsnorm_per_head(y) * w * silu(z), z = proj[:, :d_inner].  Returns (out, rstd)."""
    rows = y.shape[0]
    H, P = d.heads, d.headdim
    if not y.is_cuda:
        yf = y.float().reshape(rows, H, P)
        rstd = torch.rsqrt((yf * yf).mean(-1) + eps)
        zf = proj[:, :d.d_inner].float().reshape(rows, H, P)
        out = yf * rstd.unsqueeze(-1) * w.float().reshape(1, H, P) * torch.nn.functional.silu(zf)
        return out.reshape(rows, H * P).to(y.dtype), rstd.reshape(-1)
    out = torch.empty_like(y)
    rstd = torch.empty(rows * H, dtype=torch.float32, device=y.device)
    K._launch(N.require().oa_gated_norm_fwd(K.dt(y), y.data_ptr(), proj.data_ptr(), proj.shape[1], _f32(w).data_ptr(), out.data_ptr(),
                                            rstd.data_ptr(), rows, H, P, eps, N.stream()), "oa_gated_norm_fwd")
    return out, rstd


def gated_norm_bwd(y, proj, w, rstd, dout, d: Mamba3Dims, dproj: torch.Tensor):
    """Returns (dy, dw fp32 [H*P]); dz is written into dproj[:, :d_inner]."""
    rows = y.shape[0]
    H, P = d.heads, d.headdim
    if not y.is_cuda:
        n = y.float().reshape(rows, H, P) * rstd.reshape(rows, H, 1)
        zf = proj[:, :d.d_inner].float().reshape(rows, H, P)
        sg = torch.sigmoid(zf)
        g = dout.float().reshape(rows, H, P)
        wf = w.float().reshape(1, H, P)
        dn = g * wf * zf * sg
        dy = rstd.reshape(rows, H, 1) * (dn - n * (dn * n).mean(-1, keepdim=True))
        dproj[:, :d.d_inner] = (g * n * wf * sg * (1 + zf * (1 - sg))).reshape(rows, H * P).to(dproj.dtype)
        dw = (g * n * zf * sg).sum(0).reshape(-1)
        return dy.reshape(rows, H * P).to(y.dtype), dw
    dy = torch.empty_like(y)
    dw = torch.zeros(H * P, dtype=torch.float32, device=y.device)
    K._launch(N.require().oa_gated_norm_bwd(K.dt(y), y.data_ptr(), proj.data_ptr(), proj.shape[1], _f32(w).data_ptr(), rstd.data_ptr(),
                                            dout.contiguous().data_ptr(), dy.data_ptr(), dproj.data_ptr(), dproj.shape[1], dw.data_ptr(),
                                            rows, H, P, N.stream()), "oa_gated_norm_bwd")
    return dy, dw
