"""OaMamba3Module: the Mamba-3 SISO mixer (Source/Private/Oa/Ml/Nn/Mamba3/Mamba3.cpp:28-135 constructor, :160-250 Forward,
Step / ResetState below it).

Parameters, in registration order: in_proj [d_in_proj, d_model] (row blocks z | x | B | C | dd_dt | dd_A | trap | angle),
dt_bias [1, H], B_bias [H, N] (ones), C_bias [H, N] (ones), D [H] (zeros), out_proj [d_model, d_inner] and, with the
gated output norm, norm_weight [H, P].  Forward is in_proj GEMM -> one fused core op (preprocess + selective scan [+
gated per-head RMSNorm], csrc/kernels/mamba3.cu) -> out_proj GEMM; the core writes every gradient of the projected row
into one [B*S, d_in_proj] buffer, so the in_proj backward is two GEMMs on it.  Step keeps the recurrent state
(StepSsm / StepAngle / StepK / StepV in the reference) for token-by-token decoding.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ...core import fn_matrix as F
from ...core.matrix import OaMatrix
from ...ops import kernels as K
from ...ops import mamba3 as M3
from .. import autograd as AG
from ..module import OaModule


def _param_grad(p: OaMatrix, g32: Optional[torch.Tensor]):
    """Hands an fp32 parameter gradient to the tape in the parameter's shape and dtype."""
    if g32 is None or p is None or not p.RequiresGrad():
        return None
    t = p.Tensor()
    g = g32.reshape(t.shape)
    return g if g.dtype == t.dtype else K.cast(g.contiguous(), t.dtype)


def Mamba3Core(proj: OaMatrix, dt_bias: OaMatrix, b_bias: OaMatrix, c_bias: OaMatrix, d_skip: Optional[OaMatrix],
               norm_weight: Optional[OaMatrix], dims: M3.Mamba3Dims, batch: int, seq: int) -> OaMatrix:
    """proj [B*S, d_in_proj] -> mixed [B*S, d_inner]: preprocess, scan and (with norm_weight) the gated output norm."""
    F._ctx_add("Mamba3Siso")
    tp = F._c(proj.Tensor())
    params = [dt_bias, b_bias, c_bias, d_skip]
    pt = [m.Tensor() if m is not None else None for m in params]
    need = AG.IsEnabled() and (proj.RequiresGrad() or any(m is not None and m.RequiresGrad() for m in params + [norm_weight]))
    y, saved = M3.core_fwd(tp, pt[0], pt[1], pt[2], pt[3], dims, batch, seq, save=need)
    rstd = None
    out_t = y
    if norm_weight is not None:
        F._ctx_add("Mamba3GatedNorm")
        out_t, rstd = M3.gated_norm_fwd(y, tp, norm_weight.Tensor(), dims)
    out = OaMatrix(out_t)

    def back(g):
        F._ctx_add("Mamba3SisoBwd")
        g = F._c(g)
        dproj = torch.empty_like(tp)
        if norm_weight is None and not dims.has_z:
            dproj[:, :dims.d_inner].zero_()        # nobody reads z in this configuration: its gradient columns are zero
        dnw = None
        if norm_weight is not None:
            g, dnw = M3.gated_norm_bwd(y, tp, norm_weight.Tensor(), rstd, g, dims, dproj)
        dproj, ddtb, dBb, dCb, dD = M3.core_bwd(saved, g, dproj)
        return (dproj, _param_grad(dt_bias, ddtb), _param_grad(b_bias, dBb), _param_grad(c_bias, dCb), _param_grad(d_skip, dD),
                _param_grad(norm_weight, dnw))

    return AG.attach("Mamba3Siso", out, [proj, dt_bias, b_bias, c_bias, d_skip, norm_weight], back)


def Mamba3Prepare(proj: OaMatrix, conv_weight: Optional[OaMatrix], a_log: Optional[OaMatrix], conv_cols, alog_cols,
                  batch: int, seq: int) -> OaMatrix:
    """CUDA path of the benchmark-variant options (csrc/kernels/mamba3_conv.cu), IN PLACE on the projected rows: causal
    depthwise convolution + SiLU over columns `conv_cols`, dd_A columns `alog_cols` := exp(A_log) - 1.  The projection's own
    backward does not need its output, so overwriting it is safe; the convolution keeps a copy of its inputs."""
    from ... import _native as N
    lib = N.require()
    F._ctx_add("Mamba3Prepare")
    tp = F._c(proj.Tensor())
    rows, ld = tp.shape
    dt_code = K.dt(tp)
    saved = None
    if conv_weight is not None:
        lo, hi = conv_cols
        wt = conv_weight.Tensor()
        saved = torch.empty((rows, hi - lo), dtype=tp.dtype, device=tp.device)
        K._launch(lib.oa_mamba3_conv_fwd(dt_code, tp.data_ptr(), ld, lo, saved.data_ptr(), wt.data_ptr(), batch, seq, hi - lo, wt.shape[0],
                                         N.stream()), "oa_mamba3_conv_fwd", 2)
    if a_log is not None:
        lo, hi = alog_cols
        K._launch(lib.oa_mamba3_alog_fill(dt_code, tp.data_ptr(), ld, lo, a_log.Tensor().data_ptr(), rows, hi - lo, N.stream()),
                  "oa_mamba3_alog_fill")
    out = OaMatrix(tp)

    def back(g):
        F._ctx_add("Mamba3PrepareBwd")
        g = F._c(g)
        dw = da = None
        if a_log is not None:
            lo, hi = alog_cols
            col = K.contiguous(g[:, lo:hi])
            da = K.binary("mul", K.col_sum(col, out=torch.empty(hi - lo, dtype=torch.float32, device=g.device)),
                          K.unary("exp", a_log.Tensor().reshape(-1))).reshape(a_log.Tensor().shape)
            g[:, lo:hi].zero_()                     # the projection's dd_A outputs are not used by this variant
        if conv_weight is not None:
            lo, hi = conv_cols
            wt = conv_weight.Tensor()
            kw, C = wt.shape
            nblk = batch * ((seq + 63) // 64)
            parts = torch.empty((nblk, kw * C), dtype=torch.float32, device=g.device)
            gbuf = torch.empty((rows, C), dtype=g.dtype, device=g.device)
            K._launch(lib.oa_mamba3_conv_bwd(dt_code, g.data_ptr(), ld, lo, saved.data_ptr(), wt.data_ptr(), parts.data_ptr(), gbuf.data_ptr(),
                                             batch, seq, C, kw, N.stream()), "oa_mamba3_conv_bwd", 2)
            dw = K.col_sum(parts, out=torch.empty(kw * C, dtype=torch.float32, device=g.device)).reshape(kw, C)
        return (g, dw, da)

    return AG.attach("Mamba3Prepare", out, [proj, conv_weight, a_log], back)


class OaMamba3Module(OaModule):
    """Variants beyond the plain SISO mixer are composed from the fused SISO core:
      * `is_mimo`: R independent SISO states (Mamba3.cpp:193-219): rank r scans x * mimo_x[r] (gate z * mimo_z[r]) with its
        own B, C slice and bias, the outputs are recombined as sum_r y_r * mimo_o[r]; parameters mimo_x / mimo_z / mimo_o
        [H, R, P], B_bias / C_bias [H, R, N];
      * `ngroups == n_heads`: every head has its own B, C projection (Mamba3.cpp:314-317); the core then runs once per head
        on that head's columns (`ngroups` values other than 1 and n_heads do not broadcast in the reference either);
      * `conv_width > 0` and `a_log=True` are the options of the benchmark's Mamba-3 configuration, not of the reference:
        a depthwise causal convolution + SiLU over the x | B | C columns before the scan, and a learned per-head decay
        A = -exp(A_log) (A_log ~ log U(1, 16)) in place of the data-dependent one.  The defaults keep reference parity."""

    def __init__(self, d_model: int, d_state: int = 128, expand: int = 2, headdim: int = 64, ngroups: int = 1,
                 rope_fraction: float = 0.5, is_mimo: bool = False, mimo_rank: int = 4, dt_min: float = 1e-3, dt_max: float = 0.1,
                 dt_init_floor: float = 1e-4, a_floor: float = 1e-4, is_outproj_norm: bool = False, chunk: int = 256,
                 conv_width: int = 0, a_log: bool = False):
        super().__init__()
        self.DModel, self.DState, self.Expand, self.HeadDim = d_model, d_state, expand, headdim
        self.DInner = expand * d_model
        if self.DInner % headdim:
            raise ValueError("expand * d_model must be a multiple of headdim")
        self.NHeads = self.DInner // headdim
        if ngroups not in (1, self.NHeads):
            raise ValueError(f"ngroups must be 1 or n_heads ({self.NHeads}), got {ngroups}")
        if is_mimo and ngroups != 1:
            raise ValueError("the MIMO variant needs ngroups == 1")
        if is_mimo and mimo_rank < 1:
            raise ValueError("mimo_rank must be >= 1")
        self.NGroups, self.IsMimo, self.MimoRank = ngroups, bool(is_mimo), (int(mimo_rank) if is_mimo else 1)
        self.ConvWidth, self.HasALog = int(conv_width), bool(a_log)
        self.RopeDim = int(d_state * rope_fraction) & ~1
        self.NumRopeAngles = self.RopeDim // 2
        self.IsOutprojNorm = is_outproj_norm
        self.Dims = M3.Mamba3Dims(self.DInner, self.NHeads, headdim, d_state, self.NumRopeAngles, has_z=not is_outproj_norm,
                                  dt_min=dt_min, dt_max=dt_max, afloor=a_floor, chunk=chunk)
        H, GR = self.NHeads, self.NGroups * self.MimoRank
        self.BCWidth = d_state * GR
        self.DInProj = 2 * self.DInner + 2 * self.BCWidth + 3 * H + self.NumRopeAngles
        self.InProj = self.RegisterParameter("in_proj", F.RandGlorotUniform([self.DInProj, d_model]))
        # dt_bias = inverse softplus of dt drawn log-uniformly from [dt_min, dt_max] and floored
        r = F.Rand([H], torch.float32).Tensor().float().cpu()
        dtv = torch.exp(r * (math.log(dt_max) - math.log(dt_min)) + math.log(dt_min)).clamp_min(dt_init_floor)
        dt_bias = dtv + torch.log(-torch.expm1(-dtv))
        wdev = self.InProj.Data.Tensor().device
        self.DtBias = self.RegisterParameter("dt_bias", OaMatrix(dt_bias.reshape(1, H).to(wdev)))
        bias_shape = [H, self.MimoRank, d_state] if self.IsMimo else [H, d_state]
        self.BBias = self.RegisterParameter("B_bias", F.Ones(bias_shape, torch.float32))
        self.CBias = self.RegisterParameter("C_bias", F.Ones(bias_shape, torch.float32))
        self.MimoX = self.MimoZ = self.MimoO = None
        if self.IsMimo:
            R = self.MimoRank
            self.MimoX = self.RegisterParameter("mimo_x", F.Full([H, R, headdim], 1.0 / R, torch.float32))
            self.MimoZ = self.RegisterParameter("mimo_z", F.Ones([H, R, headdim], torch.float32))
            self.MimoO = self.RegisterParameter("mimo_o", F.Full([H, R, headdim], 1.0 / R, torch.float32))
        self.D = self.RegisterParameter("D", F.Zeros([H], torch.float32))
        self.OutProj = self.RegisterParameter("out_proj", F.RandGlorotUniform([d_model, self.DInner]))
        self.NormWeight = self.RegisterParameter("norm_weight", F.Ones([H, headdim], torch.float32)) if is_outproj_norm else None
        self.ConvWeight = self.ALog = None
        if self.ConvWidth > 0:
            cw = self.DInner + 2 * self.BCWidth
            w0 = torch.zeros(self.ConvWidth, cw)
            w0[0] = 1.0                                            # starts as the identity (tap 0 = the current token)
            self.ConvWeight = self.RegisterParameter("conv_weight", OaMatrix((w0 + 0.02 * torch.randn(self.ConvWidth, cw)).to(wdev)))
        if self.HasALog:
            u = F.Rand([H], torch.float32).Tensor().float().cpu()
            self.ALog = self.RegisterParameter("A_log", OaMatrix(torch.log(1.0 + 15.0 * u).reshape(1, H).to(wdev)))
        self._state: Optional[dict] = None
        self._plain = not self.IsMimo and self.NGroups == 1 and self.ConvWidth == 0 and not self.HasALog

    # ---- column layout of the projected row: z | x | B | C | dd_dt | dd_A | trap | angle
    def _columns(self):
        DI, W, H, A = self.DInner, self.BCWidth, self.NHeads, self.NumRopeAngles
        names, widths, off, out = ("z", "x", "B", "C", "dd_dt", "dd_A", "trap", "angle"), (DI, DI, W, W, H, H, H, A), 0, {}
        for n, w in zip(names, widths):
            out[n] = (off, off + w)
            off += w
        return out

    def _prepare(self, proj: OaMatrix, batch: int, seq: int) -> OaMatrix:
        """The benchmark-variant options, applied to the projected rows: causal depthwise convolution + SiLU over x | B | C,
        learned decay written into the dd_A columns (dd_A = exp(A_log) - 1 >= 0 makes the decay exactly -exp(A_log))."""
        c = self._columns()
        if proj.Tensor().is_cuda and self.ConvWidth <= 8:
            return Mamba3Prepare(proj, self.ConvWeight.Data if self.ConvWidth > 0 else None, self.ALog.Data if self.HasALog else None,
                                 (c["x"][0], c["C"][1]), c["dd_A"], batch, seq)
        if self.ConvWidth > 0:
            lo, hi = c["x"][0], c["C"][1]
            xbc = F.Slice(proj, 1, lo, hi).Reshape([batch, seq, hi - lo])
            acc = None
            for k in range(self.ConvWidth):                        # y[t] = sum_k w[k] * x[t - k], zero before the sequence start
                if k >= seq:
                    break
                sh = xbc if k == 0 else F.Concat([F.Zeros([batch, k, hi - lo], xbc.Tensor().dtype), F.Slice(xbc, 1, 0, seq - k)], 1)
                wk = F.Slice(self.ConvWeight.Data, 0, k, k + 1).Reshape([hi - lo])
                wk = wk if wk.Tensor().dtype == sh.Tensor().dtype else F.Cast(wk, sh.Tensor().dtype)
                term = F.Mul(sh.Reshape([batch * seq, hi - lo]), wk)
                acc = term if acc is None else F.Add(acc, term)
            proj = F.Concat([F.Slice(proj, 1, 0, lo), F.Silu(acc), F.Slice(proj, 1, hi, self.DInProj)], 1)
        if self.HasALog:
            lo, hi = c["dd_A"]
            a = F.AddScalar(F.Exp(self.ALog.Data), -1.0)           # [1, H]
            a = a if a.Tensor().dtype == proj.Tensor().dtype else F.Cast(a, proj.Tensor().dtype)
            rows = F.Add(F.Zeros([batch * seq, self.NHeads], proj.Tensor().dtype), a.Reshape([self.NHeads]))
            proj = F.Concat([F.Slice(proj, 1, 0, lo), rows, F.Slice(proj, 1, hi, self.DInProj)], 1)
        return proj

    def _mix(self, proj: OaMatrix, batch: int, seq: int) -> OaMatrix:
        """proj [B*S, DInProj] -> mixed [B*S, d_inner] for every variant."""
        nw = self.NormWeight.Data if self.NormWeight is not None else None
        if self._plain:
            return Mamba3Core(proj, self.DtBias.Data, self.BBias.Data, self.CBias.Data, self.D.Data, nw, self.Dims, batch, seq)
        proj = self._prepare(proj, batch, seq)
        c = self._columns()
        H, P, Nn, DI = self.NHeads, self.HeadDim, self.DState, self.DInner
        col = lambda name: F.Slice(proj, 1, *c[name])
        if self.IsMimo:
            z, x, tail = col("z"), col("x"), F.Slice(proj, 1, c["dd_dt"][0], self.DInProj)
            dims = M3.Mamba3Dims(DI, H, P, Nn, self.NumRopeAngles, has_z=self.Dims.has_z, dt_min=self.Dims.dt_min, dt_max=self.Dims.dt_max,
                                 afloor=self.Dims.afloor, chunk=self.Dims.chunk)
            total = None
            for r in range(self.MimoRank):
                flat = lambda m: F.Slice(m.Data, 1, r, r + 1).Reshape([DI])
                cast = lambda m: m if m.Tensor().dtype == proj.Tensor().dtype else F.Cast(m, proj.Tensor().dtype)
                pr = F.Concat([F.Mul(z, cast(flat(self.MimoZ))), F.Mul(x, cast(flat(self.MimoX))),
                               F.Slice(proj, 1, c["B"][0] + r * Nn, c["B"][0] + (r + 1) * Nn),
                               F.Slice(proj, 1, c["C"][0] + r * Nn, c["C"][0] + (r + 1) * Nn), tail], 1)
                bb = F.Slice(self.BBias.Data, 1, r, r + 1).Reshape([H, Nn])
                cb = F.Slice(self.CBias.Data, 1, r, r + 1).Reshape([H, Nn])
                yr = Mamba3Core(pr, self.DtBias.Data, bb, cb, self.D.Data, None, dims, batch, seq)
                contrib = F.Mul(yr, cast(flat(self.MimoO)))
                total = contrib if total is None else F.Add(total, contrib)
            y = total
            if nw is not None:                                      # gated per-head RMSNorm with the UNSCALED z
                rows = batch * seq * H
                ones = F.Ones([P], y.Tensor().dtype)
                n = F.RmsNormGated(y.Reshape([rows, P]), ones, None, z.Reshape([rows, P]), 1e-5, True).Reshape([batch * seq, DI])
                w = nw.Reshape([DI])
                y = F.Mul(n, w if w.Tensor().dtype == n.Tensor().dtype else F.Cast(w, n.Tensor().dtype))
            return y
        if self.NGroups == H:
            dims = M3.Mamba3Dims(P, 1, P, Nn, self.NumRopeAngles, has_z=self.Dims.has_z, dt_min=self.Dims.dt_min, dt_max=self.Dims.dt_max,
                                 afloor=self.Dims.afloor, chunk=self.Dims.chunk)
            outs = []
            for h in range(H):
                one = lambda name: F.Slice(proj, 1, c[name][0] + h, c[name][0] + h + 1)
                ph = F.Concat([F.Slice(proj, 1, c["z"][0] + h * P, c["z"][0] + (h + 1) * P),
                               F.Slice(proj, 1, c["x"][0] + h * P, c["x"][0] + (h + 1) * P),
                               F.Slice(proj, 1, c["B"][0] + h * Nn, c["B"][0] + (h + 1) * Nn),
                               F.Slice(proj, 1, c["C"][0] + h * Nn, c["C"][0] + (h + 1) * Nn),
                               one("dd_dt"), one("dd_A"), one("trap"), col("angle")], 1)
                sl = lambda m, d=0: F.Slice(m, d, h, h + 1)
                outs.append(Mamba3Core(ph, sl(self.DtBias.Data, 1), sl(self.BBias.Data), sl(self.CBias.Data), sl(self.D.Data),
                                       sl(nw) if nw is not None else None, dims, batch, seq))
            return F.Concat(outs, 1)
        # ngroups == 1 with the benchmark-variant options only
        return Mamba3Core(proj, self.DtBias.Data, self.BBias.Data, self.CBias.Data, self.D.Data, nw, self.Dims, batch, seq)

    # ---- training / prefill
    def Forward(self, x: OaMatrix) -> OaMatrix:
        if x.Rank() != 3:
            raise ValueError(f"OaMamba3Module.Forward expects rank-3 [batch, seq, d_model], got rank {x.Rank()}")
        batch, seq = x.Size(0), x.Size(1)
        flat = x.Reshape([batch * seq, self.DModel])
        proj = F.Linear(flat, self.InProj.Data, None, name="Mamba3InProj")
        mixed = self._mix(proj, batch, seq)
        out = F.Linear(mixed, self.OutProj.Data, None, name="Mamba3OutProj")
        return out.Reshape([batch, seq, self.DModel])

    # ---- decoding
    def ResetState(self, batch: int = 0) -> None:
        """Drops the recurrent decode state; the next Step allocates it for whatever batch it receives."""
        self._state = None
        self._window = None

    def Step(self, x: OaMatrix) -> OaMatrix:
        """x [batch, d_model] -> [batch, d_model]; the recurrent state lives in the module until ResetState()."""
        if not self._plain:
            return self._step_by_window(x)
        if self._state is None:
            self._state = {}
        with AG.OaGradNo():
            proj = F.Linear(x, self.InProj.Data, None, name="Mamba3InProj")
            tp = F._c(proj.Tensor())
            y = M3.step(tp, self.DtBias.Data.Tensor(), self.BBias.Data.Tensor(), self.CBias.Data.Tensor(), self.D.Data.Tensor(),
                        self.Dims, self._state)
            if self.NormWeight is not None:
                y, _ = M3.gated_norm_fwd(y, tp, self.NormWeight.Data.Tensor(), self.Dims)
            return F.Linear(OaMatrix(y), self.OutProj.Data, None, name="Mamba3OutProj")

    def _step_by_window(self, x: OaMatrix) -> OaMatrix:
        """Decode step of the composed variants (MIMO, per-head groups, convolution, learned decay): the tokens seen so far
        are kept and the mixer is re-run over them, so a step costs O(length).  The plain SISO mixer has the constant-cost
        recurrent step; these variants are training-side options."""
        with AG.OaGradNo():
            t = x.Tensor().unsqueeze(1)
            self._window = t if getattr(self, "_window", None) is None else torch.cat((self._window, t), 1)
            full = self.Forward(OaMatrix(self._window.contiguous()))
            return OaMatrix(full.Tensor()[:, -1].contiguous())

    def Prefill(self, x: OaMatrix) -> OaMatrix:
        """Forward over a prompt [batch, seq, d_model] that also leaves the decode state behind (no autograd)."""
        batch, seq = x.Size(0), x.Size(1)
        if not self._plain:
            with AG.OaGradNo():
                self._window = x.Tensor().clone()
                return self.Forward(x)
        self._state = {}
        with AG.OaGradNo():
            proj = F.Linear(x.Reshape([batch * seq, self.DModel]), self.InProj.Data, None, name="Mamba3InProj")
            tp = F._c(proj.Tensor())
            y, _ = M3.core_fwd(tp, self.DtBias.Data.Tensor(), self.BBias.Data.Tensor(), self.CBias.Data.Tensor(), self.D.Data.Tensor(),
                               self.Dims, batch, seq, save=False, final=self._state)
            if self.NormWeight is not None:
                y, _ = M3.gated_norm_fwd(y, tp, self.NormWeight.Data.Tensor(), self.Dims)
            out = F.Linear(OaMatrix(y), self.OutProj.Data, None, name="Mamba3OutProj")
        return out.Reshape([batch, seq, self.DModel])
