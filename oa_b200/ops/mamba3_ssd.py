"""Chunked (state-space-duality) form of the Mamba-3 SISO core: the training path on tensor cores.

With a per-head scalar decay the recurrence of ops/mamba3.py unrolls, inside a chunk of Q tokens that starts from state
H_in, to
    y_t = sum_{s<t} exp(cum_t - cum_s) scale_s (C~_t.B~_s) x_s + (D + gamma_t C~_t.B~_t) x_t + exp(cum_t) C~_t H_in^T
    H_out = exp(cum_Q) H_in + sum_s exp(cum_Q - cum_s) scale_s x_s (x) B~_s
(cum = inclusive prefix sum of a*dt inside the chunk), i.e. per (batch, head, chunk):
    G = C~ B~^T                      [Q, Q]    batched GEMM
    M = mask(G, cum, scale, gamma, D)          one elementwise pass (strict lower triangle decayed, exact diagonal)
    Y = M X + (C~ exp(cum)) H_in^T   [Q, P]    two batched GEMMs
    S = (w . X)^T B~                 [P, N]    batched GEMM, w_s = exp(cum_Q - cum_s) scale_s
and a short recurrence over the chunk states.  The backward pass is the same GEMM shapes transposed plus the
row / column reductions of dM.  Every GEMM runs through ops.kernels.bgemm (tcgen05 on CUDA, fp32 torch on CPU); the
sequential kernels of csrc/kernels/mamba3.cu remain the exact fp32 path, the decode path and the oracle.
The elementwise glue between the GEMMs is written with tensor expressions here and is the next thing to fuse into kernels.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from . import kernels as K
from . import mamba3 as M3

TWO_PI = 2.0 * math.pi
CHUNK = 128


class SsdSaved:
    pass


def _rot(v, cos, sin, A):
    if A == 0:
        return v
    head = v[..., :2 * A].reshape(*v.shape[:-1], A, 2)
    v0, v1 = head[..., 0], head[..., 1]
    r = torch.stack((v0 * cos - v1 * sin, v0 * sin + v1 * cos), -1).reshape(*v.shape[:-1], 2 * A)
    return torch.cat((r, v[..., 2 * A:]), -1)


def _rot_bwd(g, vr, cos, sin, A):
    """Given dL/d(rotated) `g` and the rotated values `vr`: returns (dL/d(unrotated), dL/dtheta [..., A])."""
    if A == 0:
        return g, None
    gh = g[..., :2 * A].reshape(*g.shape[:-1], A, 2)
    vh = vr[..., :2 * A].reshape(*vr.shape[:-1], A, 2)
    g0, g1 = gh[..., 0], gh[..., 1]
    dth = -g0 * vh[..., 1] + g1 * vh[..., 0]
    u = torch.stack((g0 * cos + g1 * sin, -g0 * sin + g1 * cos), -1).reshape(*g.shape[:-1], 2 * A)
    return torch.cat((u, g[..., 2 * A:]), -1), dth


def _chunks(t, B, L, H, Q):
    """[B, L, H, ...] -> [B*H*nC, Q, ...]"""
    nC = L // Q
    rest = t.shape[3:]
    return t.reshape(B, nC, Q, H, *rest).permute(0, 3, 1, 2, *range(4, 4 + len(rest))).reshape(B * H * nC, Q, *rest)


def _unchunks(t, B, L, H, Q):
    """[B*H*nC, Q, ...] -> [B, L, H, ...]"""
    nC = L // Q
    rest = t.shape[2:]
    return t.reshape(B, H, nC, Q, *rest).permute(0, 2, 3, 1, *range(4, 4 + len(rest))).reshape(B, L, H, *rest)


def supported(d: M3.Mamba3Dims, L: int, Q: int = 128) -> bool:
    return L % Q == 0 and d.headdim % 8 == 0 and d.d_state % 8 == 0 and d.d_state <= 128 and d.angles <= 128


def ssd_fwd(x, z, Bn, Cn, dt, adt, trap, angle, Bb, Cb, D, d: M3.Mamba3Dims, B: int, L: int, Q: int = 128, gemm_dtype=None):
    """x, z [B, L, H, P] (z None without the in-scan gate); Bn, Cn [B, L, N]; dt, adt, trap [B, L, H]; angle [B, L, A]
    (fp32).  Returns (y [B, L, H, P] fp32, saved)."""
    H, P, Nn, A = d.heads, d.headdim, d.d_state, d.angles
    dev = x.device
    gd = gemm_dtype or (torch.bfloat16 if x.is_cuda else torch.float32)
    nC = L // Q
    G = B * H * nC
    tr = torch.sigmoid(trap)
    gamma = dt * tr
    late = dt * (1.0 - tr)
    sg = torch.cat((late[:, 1:], torch.zeros_like(late[:, :1])), 1)
    scale = gamma + sg
    theta = torch.cumsum(angle[:, :, None, :] * dt[:, :, :, None], 1) if A else None      # [B, L, H, A]
    if A:
        theta = theta - TWO_PI * torch.round(theta / TWO_PI)
        cos, sin = torch.cos(theta), torch.sin(theta)
    else:
        cos = sin = None
    Ct = _rot(Cn[:, :, None, :] + Cb.float()[None, None], cos, sin, A)                 # [B, L, H, N]
    Bt = _rot(Bn[:, :, None, :] + Bb.float()[None, None], cos, sin, A)
    qk = (Ct * Bt).sum(-1)                                                                # [B, L, H]
    c = lambda t: _chunks(t, B, L, H, Q)
    adt_c = c(adt.unsqueeze(-1)).squeeze(-1)                                              # [G, Q]
    cum = torch.cumsum(adt_c, 1)
    cumQ = cum[:, -1:]
    gamma_c, scale_c, qk_c = c(gamma.unsqueeze(-1)).squeeze(-1), c(scale.unsqueeze(-1)).squeeze(-1), c(qk.unsqueeze(-1)).squeeze(-1)
    Ct_c, Bt_c = c(Ct), c(Bt)                                                             # [G, Q, N] fp32
    X4 = c(x.float())                                                                     # [G, Q, P]
    w = torch.exp(cumQ - cum) * scale_c                                                   # [G, Q]
    ecum = torch.exp(cum)
    Ct_g, Bt_g = Ct_c.to(gd).contiguous(), Bt_c.to(gd).contiguous()
    Ce_g = (Ct_c * ecum[..., None]).to(gd).contiguous()
    X_g = X4.to(gd).contiguous()
    Xw_g = (X4 * w[..., None]).to(gd).contiguous()
    Dh = (D.float() if D is not None else torch.zeros(H, device=dev)).reshape(1, H, 1).expand(B, H, nC).reshape(G, 1)
    Gm = K.bgemm(Ct_g, Bt_g, out_dtype=torch.float32)                                     # [G, Q, Q]
    tri = torch.tril(torch.ones(Q, Q, device=dev, dtype=torch.bool), -1)
    E = torch.exp((cum[:, :, None] - cum[:, None, :]).masked_fill(~tri, float("-inf")))  # strict lower triangle, 0 elsewhere
    Mm = Gm * E * scale_c[:, None, :]
    Mm = Mm + torch.diag_embed(Dh + gamma_c * qk_c)
    Mm_g = Mm.to(gd).contiguous()
    Y = K.bgemm(Mm_g, X_g, b_mn=True, out_dtype=torch.float32)                            # [G, Q, P]
    S = K.bgemm(Xw_g, Bt_g, a_mn=True, b_mn=True, out_dtype=torch.float32)                # [G, P, N]
    S5 = S.reshape(B * H, nC, P, Nn)
    dec = torch.exp(cumQ).reshape(B * H, nC, 1, 1)
    Hin = torch.empty_like(S5)
    h = torch.zeros(B * H, P, Nn, device=dev)
    for ci in range(nC):
        Hin[:, ci] = h
        h = dec[:, ci] * h + S5[:, ci]
    Hin_g = Hin.reshape(G, P, Nn).to(gd).contiguous()
    Y = K.bgemm(Ce_g, Hin_g, out=Y, accumulate=True)
    y = _unchunks(Y, B, L, H, Q)                                                          # [B, L, H, P]
    s = SsdSaved()
    s.y_raw = y if z is not None else None
    if z is not None:
        y = y * torch.nn.functional.silu(z.float())
    # kept for the backward pass: the GEMM operands and the per-token scalars; G, E and M are recomputed there
    s.__dict__.update(dims=d, B=B, L=L, Q=Q, gd=gd, z=z, dt=dt, tr=tr, angle=angle, gamma_c=gamma_c, scale_c=scale_c, qk_c=qk_c, cum=cum,
                      cumQ=cumQ, w=w, Ct_g=Ct_g, Bt_g=Bt_g, Ce_g=Ce_g, X_g=X_g, Xw_g=Xw_g, Hin_g=Hin_g, dec=dec, theta=theta, Dh=Dh,
                      has_d=D is not None, final_state=h)
    return y, s


def ssd_bwd(s: SsdSaved, dy: torch.Tensor):
    """dy [B, L, H, P] -> dict of fp32 gradients: x, z, Bn, Cn [B, L, N], dt, adt, trap [B, L, H], angle [B, L, A], Bb, Cb [H, N], D [H]."""
    d, B, L, Q, gd = s.dims, s.B, s.L, s.Q, s.gd
    H, P, Nn, A = d.heads, d.headdim, d.d_state, d.angles
    nC = L // Q
    G = B * H * nC
    dev = dy.device
    dy = dy.float()
    out = {}
    if s.z is not None:
        zf = s.z.float()
        sgz = torch.sigmoid(zf)
        out["z"] = dy * s.y_raw * sgz * (1 + zf * (1 - sgz))
        dy = dy * zf * sgz
    else:
        out["z"] = None
    c = lambda t: _chunks(t, B, L, H, Q)
    dY = c(dy)                                                                             # [G, Q, P]
    dY_g = dY.to(gd).contiguous()
    # recompute the masked score matrix of the forward pass
    s.Ct_c, s.Bt_c, s.X4 = s.Ct_g.float(), s.Bt_g.float(), s.X_g.float()
    s.ecum = torch.exp(s.cum)
    s.Gm = K.bgemm(s.Ct_g, s.Bt_g, out_dtype=torch.float32)
    tri0 = torch.tril(torch.ones(Q, Q, device=dev, dtype=torch.bool), -1)
    s.E = torch.exp((s.cum[:, :, None] - s.cum[:, None, :]).masked_fill(~tri0, float("-inf")))
    s.Mm_g = (s.Gm * s.E * s.scale_c[:, None, :] + torch.diag_embed(s.Dh + s.gamma_c * s.qk_c)).to(gd).contiguous()
    if A:
        s.cos, s.sin = torch.cos(s.theta), torch.sin(s.theta)
    else:
        s.cos = s.sin = None
    # ---- through Y = M X + Ce Hin^T
    dM = K.bgemm(dY_g, s.X_g, out_dtype=torch.float32)                                     # [G, Q(t), Q(s)]
    dX = K.bgemm(s.Mm_g, dY_g, a_mn=True, b_mn=True, out_dtype=torch.float32)              # [G, Q(s), P]
    dCe = K.bgemm(dY_g, s.Hin_g, b_mn=True, out_dtype=torch.float32)                       # [G, Q, N]
    T = K.bgemm(dY_g, s.Ce_g, a_mn=True, b_mn=True, out_dtype=torch.float32)               # [G, P, N]
    # ---- reverse recurrence over the chunk states
    T5 = T.reshape(B * H, nC, P, Nn)
    Hin5 = s.Hin_g.float().reshape(B * H, nC, P, Nn)
    dHout = torch.empty_like(T5)
    dcumQ = torch.zeros(B * H, nC, device=dev)
    g = torch.zeros(B * H, P, Nn, device=dev)
    for ci in range(nC - 1, -1, -1):
        dHout[:, ci] = g
        dcumQ[:, ci] = (g * Hin5[:, ci]).sum((1, 2)) * s.dec[:, ci, 0, 0]
        g = s.dec[:, ci] * g + T5[:, ci]
    dcumQ = dcumQ.reshape(G, 1)
    dHout_g = dHout.reshape(G, P, Nn).to(gd).contiguous()
    # ---- through S = Xw^T B~
    dXw = K.bgemm(s.Bt_g, dHout_g, out_dtype=torch.float32)                                # [G, Q, P]
    dBt = K.bgemm(s.Xw_g, dHout_g, b_mn=True, out_dtype=torch.float32)                     # [G, Q, N]
    dw = (dXw * s.X4).sum(-1)                                                              # [G, Q]
    dX = dX + dXw * s.w[..., None]
    # ---- through M
    tri = s.E > 0
    dMl = torch.where(tri, dM, torch.zeros_like(dM))
    GE = s.Gm * s.E
    dG = dMl * s.E * s.scale_c[:, None, :]
    dMM = dMl * GE * s.scale_c[:, None, :]                                                 # dM * M on the strict lower triangle
    dcum = dMM.sum(2) - dMM.sum(1)                                                         # rows: +, columns: -
    dscale = (dMl * GE).sum(1)
    diag = torch.diagonal(dM, dim1=1, dim2=2)
    dgamma = diag * s.qk_c
    dqk = diag * s.gamma_c
    out["D"] = diag.reshape(B, H, nC * Q).sum((0, 2)) if s.has_d else None
    dG_g = dG.to(gd).contiguous()
    dCt = K.bgemm(dG_g, s.Bt_g, b_mn=True, out_dtype=torch.float32)                        # [G, Q, N]
    dBt = K.bgemm(dG_g, s.Ct_g, a_mn=True, b_mn=True, out=dBt, accumulate=True)
    # ---- Ce = C~ exp(cum), w = exp(cumQ - cum) scale, qk = C~.B~
    dCt = dCt + dCe * s.ecum[..., None] + dqk[..., None] * s.Bt_c
    dBt = dBt + dqk[..., None] * s.Ct_c
    dcum = dcum + (dCe * s.Ct_c).sum(-1) * s.ecum - dw * s.w
    dcumQ = dcumQ + (dw * s.w).sum(1, keepdim=True)
    dscale = dscale + dw * torch.exp(s.cumQ - s.cum)
    dcum[:, -1:] += dcumQ
    dadt_c = torch.flip(torch.cumsum(torch.flip(dcum, [1]), 1), [1])                       # cum is an inclusive prefix sum
    u = lambda t: _unchunks(t.unsqueeze(-1), B, L, H, Q).squeeze(-1)
    out["adt"] = u(dadt_c)
    dgamma_l, dscale_l = u(dgamma), u(dscale)
    out["x"] = _unchunks(dX, B, L, H, Q)
    # ---- rotation, biases, angles
    dCt_l, dBt_l = _unchunks(dCt, B, L, H, Q), _unchunks(dBt, B, L, H, Q)                  # [B, L, H, N]
    Ct_l, Bt_l = _unchunks(s.Ct_c, B, L, H, Q), _unchunks(s.Bt_c, B, L, H, Q)
    gC, thC = _rot_bwd(dCt_l, Ct_l, s.cos, s.sin, A)
    gB, thB = _rot_bwd(dBt_l, Bt_l, s.cos, s.sin, A)
    out["Cn"], out["Bn"] = gC.sum(2), gB.sum(2)
    out["Cb"], out["Bb"] = gC.sum((0, 1)), gB.sum((0, 1))
    ddt = torch.zeros_like(s.dt)
    if A:
        dth = thC + thB                                                                    # [B, L, H, A]
        gth = torch.flip(torch.cumsum(torch.flip(dth, [1]), 1), [1])                       # theta is a prefix sum over the sequence
        out["angle"] = (gth * s.dt[..., None]).sum(2)
        ddt = ddt + (gth * s.angle[:, :, None, :]).sum(-1)
    else:
        out["angle"] = torch.zeros_like(s.angle)
    # ---- gamma = dt tr; scale_l = gamma_l + dt_{l+1} (1 - tr_{l+1})
    dgam = dgamma_l + dscale_l
    ddt = ddt + dgam * s.tr
    dtr = dgam * s.dt
    ddt[:, 1:] += dscale_l[:, :-1] * (1 - s.tr[:, 1:])
    dtr[:, 1:] -= dscale_l[:, :-1] * s.dt[:, 1:]
    out["dt"] = ddt
    out["trap"] = dtr * s.tr * (1 - s.tr)
    return out


# ====================================================================================== fused CUDA path (bf16 projection)
def _unchunk_small(t: torch.Tensor, B: int, L: int, H: int) -> torch.Tensor:
    """[G, Q] -> [B, L, H]"""
    return t.reshape(B, H, L // CHUNK, CHUNK).permute(0, 2, 3, 1).reshape(B, L, H)


class SsdSavedCuda:
    __slots__ = ("Ct", "Bt", "Ce", "X", "Xw", "M", "Hin", "cum", "gamma", "scale", "w", "qk", "theta", "yraw", "dims", "B", "L", "dt",
                 "trap", "angle", "Dh")


def ssd_fwd_cuda(proj: torch.Tensor, Bn, Cn, dt, adt, trap, angle, Bb, Cb, D, d: M3.Mamba3Dims, B: int, L: int, save: bool = True):
    """The chunked scan with the glue in csrc/kernels/mamba3_ssd.cu.  proj bf16 [B*L, d_in_proj]; Bn, Cn [B*L, N];
    dt, adt, trap [B*L, H]; angle [B*L, max(A, 1)] (fp32).  Returns (y bf16 [B*L, d_inner], saved)."""
    from .. import _native as N
    lib, st, dev = N.require(), N.stream(), proj.device
    H, P, Nn, A = d.heads, d.headdim, d.d_state, d.angles
    Q, nC, rows = CHUNK, L // CHUNK, B * L
    G = B * H * nC
    o = d.offsets()
    es = proj.element_size()
    bf = lambda *s: torch.empty(s, dtype=torch.bfloat16, device=dev)
    f32 = lambda *s: torch.empty(s, dtype=torch.float32, device=dev)
    theta = None
    if A:
        theta, tot = f32(B, L, H, A), f32(B, nC, H, A)
        K._launch(lib.oa_ssd_theta_fwd(angle.data_ptr(), angle.shape[-1], dt.data_ptr(), tot.data_ptr(), theta.data_ptr(), B, L, H, A, st),
                  "oa_ssd_theta_fwd", 2)
    Ct, Bt, Ce, X, Xw = bf(G, Q, Nn), bf(G, Q, Nn), bf(G, Q, Nn), bf(G, Q, P), bf(G, Q, P)
    cum, gamma, scale, w, qk = f32(G, Q), f32(G, Q), f32(G, Q), f32(G, Q), f32(G, Q)
    K._launch(lib.oa_ssd_prep_fwd(proj.data_ptr() + o[1] * es, d.d_in_proj, Bn.data_ptr(), Cn.data_ptr(), Bb.data_ptr(), Cb.data_ptr(),
                                  dt.data_ptr(), adt.data_ptr(), trap.data_ptr(), N.ptr(theta), Ct.data_ptr(), Bt.data_ptr(), Ce.data_ptr(),
                                  X.data_ptr(), Xw.data_ptr(), cum.data_ptr(), gamma.data_ptr(), scale.data_ptr(), w.data_ptr(),
                                  qk.data_ptr(), B, L, H, P, Nn, A, st), "oa_ssd_prep_fwd")
    Gm = K.bgemm(Ct, Bt, out_dtype=torch.float32)
    M = bf(G, Q, Q)
    K._launch(lib.oa_ssd_mask_fwd(Gm.data_ptr(), cum.data_ptr(), scale.data_ptr(), gamma.data_ptr(), qk.data_ptr(), N.ptr(D), M.data_ptr(),
                                  G, H, nC, st), "oa_ssd_mask_fwd")
    del Gm
    Y = K.bgemm(M, X, b_mn=True, out_dtype=torch.float32)
    S = K.bgemm(Xw, Bt, a_mn=True, b_mn=True, out_dtype=torch.float32)
    Hin = bf(G, P, Nn)
    K._launch(lib.oa_ssd_state_fwd(S.data_ptr(), cum.data_ptr(), Hin.data_ptr(), B * H, nC, P * Nn, st), "oa_ssd_state_fwd")
    del S
    K.bgemm(Ce, Hin, out=Y, accumulate=True)
    y = bf(rows, d.d_inner)
    yraw = bf(rows, d.d_inner) if d.has_z else None
    K._launch(lib.oa_ssd_out_fwd(Y.data_ptr(), proj.data_ptr() + o[0] * es if d.has_z else None, d.d_in_proj, y.data_ptr(), N.ptr(yraw),
                                 d.d_inner, B, L, H, P, st), "oa_ssd_out_fwd")
    if not save:
        return y, None
    s = SsdSavedCuda()
    s.Ct, s.Bt, s.Ce, s.X, s.Xw, s.M, s.Hin = Ct, Bt, Ce, X, Xw, M, Hin
    s.cum, s.gamma, s.scale, s.w, s.qk, s.theta, s.yraw = cum, gamma, scale, w, qk, theta, yraw
    s.dims, s.B, s.L, s.dt, s.trap, s.angle, s.Dh = d, B, L, dt, trap, angle, D
    return y, s


def ssd_bwd_cuda(s: SsdSavedCuda, proj: torch.Tensor, dy: torch.Tensor, dproj: torch.Tensor) -> dict:
    """Writes dx (and dz) into their columns of dproj and returns the fp32 gradients the preprocess backward needs:
    Bn, Cn [B*L, N], dt, adt, trap [B*L, H], angle [B*L, max(A, 1)], Bb, Cb [H, N], D [H]."""
    from .. import _native as N
    lib, st, dev = N.require(), N.stream(), dy.device
    d, B, L = s.dims, s.B, s.L
    H, P, Nn, A = d.heads, d.headdim, d.d_state, d.angles
    Q, nC, rows = CHUNK, L // CHUNK, B * L
    G = B * H * nC
    o = d.offsets()
    es = proj.element_size()
    bf = lambda *sh: torch.empty(sh, dtype=torch.bfloat16, device=dev)
    f32 = lambda *sh: torch.empty(sh, dtype=torch.float32, device=dev)
    z32 = lambda *sh: torch.zeros(sh, dtype=torch.float32, device=dev)
    dy = dy.contiguous()
    dY = bf(G, Q, P)
    K._launch(lib.oa_ssd_dy_prep(dy.data_ptr(), N.ptr(s.yraw), d.d_inner, proj.data_ptr() + o[0] * es if d.has_z else None, d.d_in_proj,
                                 dproj.data_ptr() + o[0] * es if d.has_z else None, d.d_in_proj, dY.data_ptr(), B, L, H, P, st),
              "oa_ssd_dy_prep")
    dM = K.bgemm(dY, s.X, out_dtype=torch.float32)
    dX = K.bgemm(s.M, dY, a_mn=True, b_mn=True, out_dtype=torch.float32)
    dCe = K.bgemm(dY, s.Hin, b_mn=True, out_dtype=torch.float32)
    T = K.bgemm(dY, s.Ce, a_mn=True, b_mn=True, out_dtype=torch.float32)
    dHout, dcumQ = bf(G, P, Nn), z32(G)
    K._launch(lib.oa_ssd_state_bwd(T.data_ptr(), s.cum.data_ptr(), s.Hin.data_ptr(), dHout.data_ptr(), dcumQ.data_ptr(), B * H, nC, P * Nn, st),
              "oa_ssd_state_bwd")
    del T
    dXw = K.bgemm(s.Bt, dHout, out_dtype=torch.float32)
    dBt = K.bgemm(s.Xw, dHout, b_mn=True, out_dtype=torch.float32)
    Gm = K.bgemm(s.Ct, s.Bt, out_dtype=torch.float32)
    dG, row_mm, col_mm, col_ge, diag = bf(G, Q, Q), f32(G, Q), f32(G, Q), f32(G, Q), f32(G, Q)
    K._launch(lib.oa_ssd_mask_bwd(dM.data_ptr(), Gm.data_ptr(), s.cum.data_ptr(), s.scale.data_ptr(), dG.data_ptr(), row_mm.data_ptr(),
                                  col_mm.data_ptr(), col_ge.data_ptr(), diag.data_ptr(), G, st), "oa_ssd_mask_bwd")
    del dM, Gm
    dCt = K.bgemm(dG, s.Bt, b_mn=True, out_dtype=torch.float32)
    K.bgemm(dG, s.Ct, a_mn=True, b_mn=True, out=dBt, accumulate=True)
    dqk = K.binary("mul", diag, s.gamma)
    dCn, dBn, dCb, dBb = f32(rows, Nn), f32(rows, Nn), z32(H, Nn), z32(H, Nn)
    dtheta = f32(B, L, H, A) if A else None
    dcum_ce = f32(G, Q)
    K._launch(lib.oa_ssd_prep_bwd(dCt.data_ptr(), dBt.data_ptr(), dCe.data_ptr(), s.Ct.data_ptr(), s.Bt.data_ptr(), s.cum.data_ptr(),
                                  dqk.data_ptr(), N.ptr(s.theta), dCn.data_ptr(), dBn.data_ptr(), dCb.data_ptr(), dBb.data_ptr(),
                                  N.ptr(dtheta), dcum_ce.data_ptr(), B, L, H, Nn, A, st), "oa_ssd_prep_bwd")
    del dCt, dBt, dCe
    dw = f32(G, Q)
    K._launch(lib.oa_ssd_dx_out(dX.data_ptr(), dXw.data_ptr(), s.X.data_ptr(), s.w.data_ptr(), dproj.data_ptr() + o[1] * es, d.d_in_proj,
                                dw.data_ptr(), B, L, H, P, st), "oa_ssd_dx_out")
    # ---- per-token scalar tail ([G, Q] / [B, L, H] sized tensors): three small kernels
    out = {"Bn": dBn, "Cn": dCn, "Bb": dBb, "Cb": dCb}
    ddt_theta = None
    if A:
        lda = s.angle.shape[-1]
        dangle, ddt_theta, tot = z32(rows, lda), f32(B, L, H), f32(B, nC, H, A)
        K._launch(lib.oa_ssd_theta_bwd(dtheta.data_ptr(), s.angle.data_ptr(), lda, s.dt.data_ptr(), tot.data_ptr(), dangle.data_ptr(),
                                       ddt_theta.data_ptr(), B, L, H, A, st), "oa_ssd_theta_bwd", 2)
        out["angle"] = dangle
    else:
        out["angle"] = z32(rows, 1)
    dadt, ddt, dtrap = f32(rows, H), f32(rows, H), f32(rows, H)
    dD = f32(H) if s.Dh is not None else None
    scratch = K.scratch(dev, (2 * rows * H + G) * 4, "ssd_tail")
    K._launch(lib.oa_ssd_tail(dw.data_ptr(), s.w.data_ptr(), col_ge.data_ptr(), row_mm.data_ptr(), col_mm.data_ptr(), dcum_ce.data_ptr(),
                              diag.data_ptr(), s.qk.data_ptr(), s.cum.data_ptr(), dcumQ.data_ptr(), s.dt.data_ptr(), s.trap.data_ptr(),
                              N.ptr(ddt_theta), dadt.data_ptr(), ddt.data_ptr(), dtrap.data_ptr(), N.ptr(dD), scratch.data_ptr(), B, L, H, st),
              "oa_ssd_tail", 3 if dD is not None else 2)
    out["adt"], out["dt"], out["trap"], out["D"] = dadt, ddt, dtrap, dD
    return out
