"""OaGruCell / OaGru / OaRnnCell / OaRnn (Source/Private/Oa/Ml/Nn/Gru/Gru.cpp:32-201, Nn/Rnn/Rnn.cpp).

Parameters per cell: weight_ih [G*H, I], weight_hh [G*H, H], bias_ih [G*H], bias_hh [G*H] (G = 3 for the GRU with gate
order reset | update | candidate, G = 1 for the tanh RNN); stacked layers are children `layer0`, `layer1`, ...
Forward takes [batch, seq, input]: the input projection of all time steps is one GEMM, the recurrence is one scan
kernel per layer (OA_DISABLE_GRU_SCAN / OA_DISABLE_RNN_SCAN fall back to per-step cells, the differential-test path).
"""
from __future__ import annotations

from typing import Optional

import torch

from ...core import fn_matrix as F
from ...core.matrix import OaMatrix
from ...ops import kernels as K
from ...utils import envflag
from .. import autograd as AG
from ..module import OaModule


def RecurrentScan(gates_i: OaMatrix, w_hh: OaMatrix, b_hh: Optional[OaMatrix], gates: int, name: str) -> OaMatrix:
    """Scan over time of a GRU (gates=3) or RNN (gates=1); gates_i [B, S, G*H] -> [B, S, H]."""
    F._ctx_add(name)
    tg, tw = F._c(gates_i.Tensor()), F._c(w_hh.Tensor())
    tb = b_hh.Tensor() if b_hh is not None else None
    need = AG.IsEnabled() and (gates_i.RequiresGrad() or w_hh.RequiresGrad())
    out_t, hprev = K.rnn_scan_fwd(tg, tw, tb, gates, save=need)
    out = OaMatrix(out_t)

    def back(g):
        F._ctx_add(name + "Bwd")
        dgi, dgh, _ = K.rnn_scan_bwd(tg, tw, tb, hprev, F._c(g), gates)
        B, S, GH = dgh.shape
        H = GH // gates
        dgh2, hp2 = dgh.reshape(B * S, GH), hprev.reshape(B * S, H)
        dw = None
        if w_hh.RequiresGrad():
            buf, acc, direct = F._grad_out(w_hh, tw.shape, tw.dtype, tw.device)
            if (B * S) % 8 == 0 or not dgh2.is_cuda or dgh2.dtype == torch.float32:
                K.gemm(dgh2, hp2, a_mn=True, b_mn=True, out=buf, accumulate=acc)
            else:                                       # odd row counts: exact fp32 product
                v = K.gemm(K.cast(dgh2, torch.float32), K.cast(hp2, torch.float32), a_mn=True, b_mn=True)
                buf.copy_(v + buf.float() if acc else v)
            dw = None if direct else buf
        db = F._bias_grad(b_hh, dgh2)
        return (dgi, dw, db)

    return AG.attach(name, out, [gates_i, w_hh, b_hh], back)


class _Cell(OaModule):
    Gates = 1
    Kernel = "RnnScan"

    def __init__(self, input_size: int, hidden_size: int, bias: bool = True):
        super().__init__()
        G = self.Gates
        self.InputSize, self.HiddenSize, self.HasBias = input_size, hidden_size, bias
        self.WeightIh = self.RegisterParameter("weight_ih", F.RandXavier([G * hidden_size, input_size]))
        self.WeightHh = self.RegisterParameter("weight_hh", F.RandXavier([G * hidden_size, hidden_size]))
        self.BiasIh = self.RegisterParameter("bias_ih", F.Zeros([G * hidden_size])) if bias else None
        self.BiasHh = self.RegisterParameter("bias_hh", F.Zeros([G * hidden_size])) if bias else None

    def ZeroState(self, batch: int) -> OaMatrix:
        return F.Zeros([batch, self.HiddenSize])

    def InputProjection(self, x2d: OaMatrix) -> OaMatrix:
        return F.Linear(x2d, self.WeightIh.Data, self.BiasIh.Data if self.BiasIh else None, name=self.Kernel.replace("Scan", "CellLinear"))

    def Step(self, x: OaMatrix, hidden: OaMatrix) -> OaMatrix:
        """One time step: x [B, I], hidden [B, H] -> new hidden (generic differentiable ops)."""
        gi = self.InputProjection(x)
        gh = F.Linear(hidden, self.WeightHh.Data, self.BiasHh.Data if self.BiasHh else None)
        return self._pointwise(gi, gh, hidden)

    def _pointwise(self, gi, gh, hidden):
        return F.Tanh(F.Add(gi, gh))

    def Forward(self, x):
        raise RuntimeError("cells are stepped: use Step(x, hidden)")


class OaRnnCell(_Cell):
    Gates, Kernel = 1, "RnnScan"


class OaGruCell(_Cell):
    Gates, Kernel = 3, "GruScan"

    def _pointwise(self, gi, gh, hidden):
        H = self.HiddenSize
        ir, iz, inn = F.Split(gi, [H, H, H], -1)
        hr, hz, hn = F.Split(gh, [H, H, H], -1)
        r = F.Sigmoid(F.Add(ir, hr))
        z = F.Sigmoid(F.Add(iz, hz))
        n = F.Tanh(F.Add(inn, F.Mul(r, hn)))
        one_minus_z = F.AddScalar(F.Neg(z), 1.0)
        return F.Add(F.Mul(one_minus_z, n), F.Mul(z, hidden))


class _Stack(OaModule):
    CellType = OaRnnCell
    DisableFlag = "OA_DISABLE_RNN_SCAN"

    def __init__(self, input_size: int, hidden_size: int, num_layers: int = 1, bias: bool = True):
        super().__init__()
        self.InputSize, self.HiddenSize, self.NumLayers, self.HasBias = input_size, hidden_size, num_layers, bias
        self.Layers = []
        for i in range(num_layers):
            cell = self.CellType(input_size if i == 0 else hidden_size, hidden_size, bias)
            self.Layers.append(self.RegisterModule(f"layer{i}", cell))

    def ZeroState(self, batch: int, layer: int = 0) -> OaMatrix:
        return self.Layers[layer].ZeroState(batch)

    def Step(self, x: OaMatrix, hidden: OaMatrix, layer: int = 0) -> OaMatrix:
        return self.Layers[layer].Step(x, hidden)

    def Forward(self, x: OaMatrix) -> OaMatrix:
        if x.Rank() != 3:
            raise ValueError(f"{type(self).__name__}.Forward expects rank-3 [batch, seq, input], got rank {x.Rank()}")
        batch, seq = x.Size(0), x.Size(1)
        use_scan = not envflag.IsSet(self.DisableFlag)
        cur = x
        for cell in self.Layers:
            flat = cur.Reshape([batch * seq, cell.InputSize])
            gates_i = cell.InputProjection(flat)
            if use_scan:
                g3 = gates_i.Reshape([batch, seq, cell.Gates * cell.HiddenSize])
                cur = RecurrentScan(g3, cell.WeightHh.Data, cell.BiasHh.Data if cell.BiasHh else None, cell.Gates, cell.Kernel)
            else:
                g3 = gates_i.Reshape([batch, seq, cell.Gates * cell.HiddenSize])
                h = cell.ZeroState(batch)
                outs = []
                for t in range(seq):
                    gi = F.Reshape(F.Slice(g3, 1, t, t + 1), [batch, cell.Gates * cell.HiddenSize])
                    gh = F.Linear(h, cell.WeightHh.Data, cell.BiasHh.Data if cell.BiasHh else None)
                    h = cell._pointwise(gi, gh, h)
                    outs.append(F.Reshape(h, [batch, 1, cell.HiddenSize]))
                cur = F.Concat(outs, 1)
        return cur


class OaRnn(_Stack):
    CellType, DisableFlag = OaRnnCell, "OA_DISABLE_RNN_SCAN"


class OaGru(_Stack):
    CellType, DisableFlag = OaGruCell, "OA_DISABLE_GRU_SCAN"
