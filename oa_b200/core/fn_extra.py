"""Row compaction / scatter with a device-resident count, accuracy counters, stochastic rounding, the int8 matrix product,
and the composite functions that complete the matrix-function namespace.

Contracts: Source/Public/Oa/Core/FnMatrix.h:170-176 (accuracy counters), :239-266 (ScatterAddRows, CompactRows and its
result record, CompactRowsBwd, ScatterRows, ScatterRowsBwdSource), Source/Public/Oa/Ml/FnMatrix.h (LinearDataReluBwd,
LinearReluBwdData), the loss kernels MaskedMse / SmoothL1Mean / VelSmoothL1 of Ml/Shader/Compute/Loss, the Sr and
Quantize kernels.  CUDA tensors run `csrc/kernels/rows.cu`; CPU tensors run the same definitions in PyTorch.

Compaction keeps a FIXED capacity (the input's row count): Values is [T, D] with the first Count rows valid and the
rest zero, RowMap [T] and Count [1] stay on the device, so nothing here reads a mask on the host and every consumer
sizes its work by the device-side count.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from .. import _native as N
from ..ml import autograd as AG
from ..ops import kernels as K
from .matrix import OaMatrix


def _c(t: torch.Tensor) -> torch.Tensor:
    return t if t.is_contiguous() else t.contiguous()


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return N.CONST["OA_F32"]
    if t.dtype == torch.bfloat16:
        return N.CONST["OA_BF16"]
    raise TypeError(f"unsupported dtype {t.dtype}")


def _mask_u8(mask: OaMatrix, rows: int) -> torch.Tensor:
    m = mask.Tensor().reshape(-1)
    if m.numel() != rows:
        raise ValueError(f"mask has {m.numel()} entries for {rows} rows")
    return _c((m != 0).to(torch.uint8))


@dataclass
class OaCompactRowsResult:
    Values: OaMatrix         # [T, D]: first Count rows valid, remaining rows zero
    RowMap: OaMatrix         # int32 [T]: packed row -> source row for the first Count entries
    Count: OaMatrix          # int32 [1]
    DispatchArgs: OaMatrix   # int32 [3]: ceil(Count * D / 256), 1, 1 (kept for consumers that size a launch by it)


def _compact(x: torch.Tensor, mask: torch.Tensor):
    T, D = x.shape
    if x.is_cuda:
        lib = N.require()
        pos = torch.empty(T, dtype=torch.int32, device=x.device)
        count = torch.empty(1, dtype=torch.int32, device=x.device)
        values = torch.zeros_like(x)
        rowmap = torch.zeros(T, dtype=torch.int32, device=x.device)
        scratch = torch.empty(int(lib.oa_rows_scan_scratch_ints(T)), dtype=torch.int32, device=x.device)
        K._launch(lib.oa_rows_scan(mask.data_ptr(), pos.data_ptr(), count.data_ptr(), scratch.data_ptr(), T, N.stream()), "oa_rows_scan")
        K._launch(lib.oa_rows_compact(x.data_ptr(), mask.data_ptr(), pos.data_ptr(), values.data_ptr(), rowmap.data_ptr(), T, D,
                                      x.element_size(), N.stream()), "oa_rows_compact")
    else:
        idx = torch.nonzero(mask, as_tuple=False).reshape(-1)
        count = torch.tensor([idx.numel()], dtype=torch.int32)
        values = torch.zeros_like(x)
        values[:idx.numel()] = x[idx]
        rowmap = torch.zeros(T, dtype=torch.int32)
        rowmap[:idx.numel()] = idx.to(torch.int32)
    args = torch.stack(((count[0].to(torch.int64) * D + 255) // 256, torch.ones((), dtype=torch.int64, device=x.device),
                        torch.ones((), dtype=torch.int64, device=x.device))).to(torch.int32)
    return values, rowmap, count, args


def _scatter(packed: torch.Tensor, rowmap: torch.Tensor, count: torch.Tensor, out: torch.Tensor, add: bool) -> torch.Tensor:
    """out[rowmap[i]] (=|+=) packed[i] for i < count, in place on `out`."""
    cap, D = packed.shape
    if out.is_cuda:
        K._launch(N.require().oa_rows_scatter(packed.data_ptr(), rowmap.data_ptr(), count.data_ptr(), out.data_ptr(), cap, out.shape[0], D,
                                              _dt(out), int(add), N.stream()), "oa_rows_scatter")
        return out
    n = min(int(count[0]), cap)
    idx = rowmap[:n].long()
    if add:
        out.index_add_(0, idx, packed[:n])
    else:
        out[idx] = packed[:n]
    return out


def _gather(src: torch.Tensor, rowmap: torch.Tensor, count: torch.Tensor, capacity: int) -> torch.Tensor:
    D = src.shape[1]
    if src.is_cuda:
        out = torch.empty(capacity, D, dtype=src.dtype, device=src.device)
        K._launch(N.require().oa_rows_gather(src.data_ptr(), rowmap.data_ptr(), count.data_ptr(), out.data_ptr(), capacity, src.shape[0], D,
                                             src.element_size(), N.stream()), "oa_rows_gather")
        return out
    out = torch.zeros(capacity, D, dtype=src.dtype)
    n = min(int(count[0]), capacity)
    out[:n] = src[rowmap[:n].long()]
    return out


def _rows2d(m: OaMatrix) -> torch.Tensor:
    t = _c(m.Tensor())
    if t.dim() != 2:
        raise ValueError("expected a [rows, width] matrix")
    return t


def CompactRows(x: OaMatrix, mask: OaMatrix) -> OaCompactRowsResult:
    """Selected rows (mask != 0) moved to the front in order; records on the gradient tape."""
    tx = _rows2d(x)
    values, rowmap, count, args = _compact(tx, _mask_u8(mask, tx.shape[0]))
    out = AG.attach("CompactRows", OaMatrix(values), [x], lambda g: (_scatter(_c(g), rowmap, count, torch.zeros_like(tx), False),))
    return OaCompactRowsResult(out, OaMatrix(rowmap), OaMatrix(count), OaMatrix(args))


def CompactRowsBwd(grad_out: OaMatrix, row_map: OaMatrix, count: OaMatrix, input_shape: Sequence[int]) -> OaMatrix:
    g = _rows2d(grad_out)
    return OaMatrix(_scatter(g, row_map.Tensor(), count.Tensor(), torch.zeros(*input_shape, dtype=g.dtype, device=g.device), False))


def ScatterRows(self_: OaMatrix, source: OaMatrix, row_map, count: Optional[OaMatrix] = None) -> OaMatrix:
    """Copy of `self_` with source[i] written to row row_map[i] for i < count.  `row_map` may be a CompactRows result."""
    if isinstance(row_map, OaCompactRowsResult):
        row_map, count = row_map.RowMap, row_map.Count
    base, src = _rows2d(self_), _rows2d(source)
    rm, cn = row_map.Tensor(), count.Tensor()
    out = _scatter(src, rm, cn, base.clone(), False)

    def back(g):
        g = _c(g)
        g_self = _scatter(torch.zeros_like(src), rm, cn, g.clone(), False)          # overwritten rows pass nothing to self
        return g_self, _gather(g, rm, cn, src.shape[0])

    return AG.attach("ScatterRows", OaMatrix(out), [self_, source], back)


def ScatterRowsBwdSource(grad_out: OaMatrix, row_map: OaMatrix, count: OaMatrix) -> OaMatrix:
    g = _rows2d(grad_out)
    return OaMatrix(_gather(g, row_map.Tensor(), count.Tensor(), row_map.Tensor().numel()))


def ScatterAddRows(source: OaMatrix, indices: OaMatrix, out_rows: int) -> OaMatrix:
    """out[indices[i]] += source[i] over all rows of `source` ([out_rows, D] result).  Rows named more than once add up; on
    the GPU their order of addition is not fixed."""
    src = _rows2d(source)
    idx = _c(indices.Tensor().reshape(-1).to(torch.int32))
    if idx.numel() != src.shape[0]:
        raise ValueError("one index per source row is required")
    count = torch.tensor([src.shape[0]], dtype=torch.int32, device=src.device)
    out = _scatter(src, idx, count, torch.zeros(out_rows, src.shape[1], dtype=src.dtype, device=src.device), True)
    return AG.attach("ScatterAddRows", OaMatrix(out), [source], lambda g: (_gather(_c(g), idx, count, src.shape[0]),))


def _accuracy(logits: OaMatrix, labels: OaMatrix, mask: Optional[OaMatrix]) -> torch.Tensor:
    t = _c(logits.Tensor())
    t = t.reshape(-1, t.shape[-1])
    y = _c(labels.Tensor().reshape(-1).to(torch.int32))
    if y.numel() != t.shape[0]:
        raise ValueError("one label per row is required")
    m = _mask_u8(mask, t.shape[0]) if mask is not None else None
    if t.is_cuda:
        out = torch.zeros(2, dtype=torch.int32, device=t.device)
        K._launch(N.require().oa_accuracy_count(t.data_ptr(), y.data_ptr(), m.data_ptr() if m is not None else None, out.data_ptr(), t.shape[0],
                                                t.shape[1], _dt(t), N.stream()), "oa_accuracy_count")
        return out
    hit = t.float().argmax(-1).to(torch.int32) == y          # argmax returns the lowest index among equal maxima
    keep = m.bool() if m is not None else torch.ones_like(hit)
    return torch.stack(((hit & keep).sum(), keep.sum())).to(torch.int32)


def CategoricalAccuracyCount(logits: OaMatrix, labels: OaMatrix) -> OaMatrix:
    """Device int32 scalar: rows whose last-axis arg-max equals the label."""
    return OaMatrix(_accuracy(logits, labels, None)[:1])


def MaskedCategoricalAccuracyCount(logits: OaMatrix, labels: OaMatrix, mask: OaMatrix) -> OaMatrix:
    """Device int32 scalar: correct rows among those whose mask is non-zero (divide by the number of such rows)."""
    return OaMatrix(_accuracy(logits, labels, mask)[:1])


def SrRoundBf16(x: OaMatrix, seed: int = 0) -> OaMatrix:
    """fp32 -> bf16 with stochastic rounding (unbiased: the mean of many roundings converges to the input)."""
    t = _c(x.Tensor().float())
    seed = int(seed) & 0xFFFFFFFFFFFFFFFF
    if t.is_cuda:
        out = torch.empty_like(t, dtype=torch.bfloat16)
        K._launch(N.require().oa_sr_round_bf16(t.data_ptr(), out.data_ptr(), t.numel(), seed & 0xFFFFFFFF, seed >> 32, N.stream()), "oa_sr_round_bf16")
        return OaMatrix(out)
    from ..ops.lunar import _mix32
    i = torch.arange(t.numel(), dtype=torch.int64)
    r = _mix32(torch.tensor(seed & 0xFFFFFFFF) ^ _mix32(((seed >> 32) + i * 0x9E3779B9 + (i >> 32)) & 0xFFFFFFFF)) & 0xFFFF
    bits = t.reshape(-1).view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    finite = (bits & 0x7F800000) != 0x7F800000
    bits = torch.where(finite, (bits + r) & 0xFFFFFFFF, bits)
    hi = (bits >> 16).to(torch.int32).to(torch.int16)        # wraps to the signed pattern of the same 16 bits
    return OaMatrix(hi.view(torch.bfloat16).reshape(t.shape))


def GemmInt8(a: OaMatrix, b: OaMatrix, row_scale: Optional[OaMatrix] = None, col_scale: Optional[OaMatrix] = None) -> OaMatrix:
    """A [M, K] int8 times B [N, K] int8 transposed: int32 [M, N], or fp32 scaled by row_scale[m] * col_scale[n] when scales
    are given (the dequantised product of two per-row quantised operands)."""
    ta, tb = _c(a.Tensor()), _c(b.Tensor())
    if ta.dtype != torch.int8 or tb.dtype != torch.int8 or ta.dim() != 2 or tb.dim() != 2 or ta.shape[1] != tb.shape[1]:
        raise ValueError("GemmInt8 takes int8 [M, K] and [N, K]")
    M, Kd = ta.shape
    Nn = tb.shape[0]
    scaled = row_scale is not None or col_scale is not None
    rs = _c(row_scale.Tensor().float().reshape(-1)) if row_scale is not None else None
    cs = _c(col_scale.Tensor().float().reshape(-1)) if col_scale is not None else None
    if ta.is_cuda:
        out = torch.empty(M, Nn, dtype=torch.float32 if scaled else torch.int32, device=ta.device)
        K._launch(N.require().oa_gemm_int8(ta.data_ptr(), tb.data_ptr(), None if scaled else out.data_ptr(), out.data_ptr() if scaled else None,
                                           rs.data_ptr() if rs is not None else None, cs.data_ptr() if cs is not None else None, M, Nn, Kd,
                                           N.stream()), "oa_gemm_int8")
        return OaMatrix(out)
    acc = ta.to(torch.int32) @ tb.to(torch.int32).T
    if not scaled:
        return OaMatrix(acc)
    out = acc.float()
    if rs is not None:
        out = out * rs[:, None]
    if cs is not None:
        out = out * cs[None, :]
    return OaMatrix(out)


# ------------------------------------------------------------------------------------------ composites
def _F():
    from . import fn_matrix as F
    return F


def LinearDataReluBwd(dy: OaMatrix, w: OaMatrix, pre_activation: OaMatrix) -> OaMatrix:
    """Data gradient through a Linear whose INPUT came out of a ReLU: (dy W) gated by pre_activation > 0."""
    F = _F()
    return F.ReluBwd(pre_activation, F.LinearDataBwd(dy, w))


def LinearReluBwdData(dy: OaMatrix, y: OaMatrix, w: OaMatrix) -> OaMatrix:
    """Data gradient of y = relu(x W^T + b): (dy gated by y > 0) W."""
    F = _F()
    return F.LinearDataBwd(F.ReluBwd(y, dy), w)


def SumDim(m: OaMatrix, dim: int) -> OaMatrix:
    return _F().Sum(m, dim)


def ReduceCols(m: OaMatrix) -> OaMatrix:
    """Column sums of a [rows, cols] matrix ([cols] result), e.g. a bias gradient."""
    return _F().Sum(m, 0)


def MeanBwd(grad_out: OaMatrix, input_shape: Sequence[int]) -> OaMatrix:
    """Gradient of the mean over all elements: the upstream scalar spread evenly."""
    n = 1
    for s in input_shape:
        n *= int(s)
    F = _F()
    return F.Scale(F.Add(F.Zeros(list(input_shape), grad_out.Tensor().dtype), grad_out), 1.0 / n)


def MaxBwd(x: OaMatrix, y: OaMatrix, grad_out: OaMatrix) -> OaMatrix:
    """Gradient of a last-axis max: the upstream value goes to the first position that attains the maximum."""
    tx = x.Tensor()
    idx = (tx == y.Tensor().unsqueeze(-1)).to(torch.int32).argmax(-1, keepdim=True)
    out = torch.zeros_like(tx)
    out.scatter_(-1, idx, grad_out.Tensor().unsqueeze(-1).to(tx.dtype))
    return OaMatrix(out)


def LogSoftmaxBwd(y: OaMatrix, grad_out: OaMatrix) -> OaMatrix:
    """dx = g - exp(y) * sum(g) along the last axis, from the saved log-probabilities y."""
    F = _F()
    s = F.Sum(grad_out, -1)
    return F.Sub(grad_out, F.Mul(F.Exp(y), F.Reshape(s, list(s.Tensor().shape) + [1])))


def CopyAtOffset(dst: OaMatrix, src: OaMatrix, element_offset: int) -> None:
    """dst.flat[offset : offset + src.numel] = src.flat, in place."""
    d, s = dst.Tensor(), src.Tensor()
    if not d.is_contiguous() or element_offset < 0 or element_offset + s.numel() > d.numel():
        raise ValueError("CopyAtOffset needs a contiguous destination that holds the source at that offset")
    d.view(-1)[element_offset:element_offset + s.numel()].copy_(s.reshape(-1))


def MatrixCopyRegion(dst: OaMatrix, src: OaMatrix, dst_row: int, dst_col: int, src_row: int = 0, src_col: int = 0,
                     rows: Optional[int] = None, cols: Optional[int] = None) -> None:
    """Rectangle copy between two 2-D matrices, in place on `dst`."""
    d, s = dst.Tensor(), src.Tensor()
    rows = s.shape[0] - src_row if rows is None else rows
    cols = s.shape[1] - src_col if cols is None else cols
    if min(dst_row, dst_col, src_row, src_col, rows, cols) < 0 or dst_row + rows > d.shape[0] or dst_col + cols > d.shape[1] \
            or src_row + rows > s.shape[0] or src_col + cols > s.shape[1]:
        raise ValueError("region outside a matrix")
    d[dst_row:dst_row + rows, dst_col:dst_col + cols].copy_(s[src_row:src_row + rows, src_col:src_col + cols])


def TransposeBatched(m: OaMatrix) -> OaMatrix:
    """[B, R, C] -> [B, C, R], materialised."""
    return _F().Transpose(m, 1, 2)


def GemmStrided(a: OaMatrix, b: OaMatrix) -> OaMatrix:
    """Batched product of arbitrarily strided operands: [B, M, K] x [B, K, N] (views are made contiguous first, then
    the batched tensor-core product runs)."""
    F = _F()
    return F.Bmm(OaMatrix(_c(a.Tensor())), OaMatrix(_c(b.Tensor())))


# ------------------------------------------------------------------------------------------ losses
def MaskedMse(pred: OaMatrix, target: OaMatrix, mask: OaMatrix) -> OaMatrix:
    """Mean of (pred - target)^2 over the elements whose mask is non-zero (mask broadcast over the last axis when it has
    one entry per row)."""
    F = _F()
    tp = pred.Tensor()
    m = mask.Tensor().to(tp.dtype)
    if m.numel() != tp.numel():
        m = m.reshape(-1, 1).expand(-1, tp.numel() // m.numel())
    m = OaMatrix(_c(m.reshape(tp.shape)))
    d = F.Mul(F.Sub(pred, target), m)
    denom = float(m.Tensor().sum().clamp_min(1.0))
    return F.Scale(F.Sum(F.Mul(d, d)), 1.0 / denom)


def SmoothL1Mean(pred: OaMatrix, target: OaMatrix, beta: float = 1.0) -> OaMatrix:
    """Huber loss averaged over all elements."""
    from ..ml import fn_loss as L
    loss = L.SmoothL1(pred, target, beta)
    return loss if loss.NumElements() == 1 else _F().Mean(loss)


def VelSmoothL1(pred: OaMatrix, target: OaMatrix, batch: int, frames: int, beta: float = 1.0) -> OaMatrix:
    """Huber loss on frame-to-frame differences of [batch * frames, D] sequences (penalises velocity error, not pose)."""
    F = _F()
    D = pred.Tensor().shape[-1]
    if frames < 2:
        raise ValueError("velocity needs at least two frames")

    def vel(m: OaMatrix) -> OaMatrix:
        x = F.Reshape(m, [batch, frames, D])
        return F.Reshape(F.Sub(F.Slice(x, 1, 1, frames), F.Slice(x, 1, 0, frames - 1)), [batch * (frames - 1), D])

    return SmoothL1Mean(vel(pred), vel(target), beta)
