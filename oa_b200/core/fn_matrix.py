"""OaFnMatrix: the operation library on OaMatrix, core and ML ops, each with its autograd node.

Reference: Source/Public/Oa/Core/FnMatrix.h:21-537 (factories, elementwise, reductions, indexing),
Source/Public/Oa/Ml/FnMatrix.h:15-813 (Linear family, activations, norms, attention, Swiglu), the
generated backward catalogue Source/Private/Oa/Ml/Autograd/Matrix/AutogradMatrix.h, and the Python
manifest Source/Python/oa/_surface.py:172-263 (the names exported as `oa.OaFnMatrix`).

Every function launches this package's kernels through `oa_b200.ops.kernels`; on a CPU engine the same
functions run the fp32 statement of the math.  Conventions kept from the reference: weights are
`[out, in]` and `MatMulNt(A[M,K], B[N,K]) = A @ B^T`; GELU is the tanh approximation; CrossEntropy
and friends live in `OaFnLoss`.
"""
from __future__ import annotations

import math
import struct
from typing import Optional, Sequence

import torch

from .. import _native as N
from ..ml import autograd as AG
from ..ops import kernels as K
from ..runtime import engine as RT
from .matrix import OaMatrix
from .types import OaScalarType, to_torch_dtype

_rng = {"seed": 0x1234ABCD, "offset": 0}


def _dev() -> torch.device:
    return RT.get_engine().Device()


def _ctx_add(name: str) -> None:
    RT.OaContext.GetDefault().Add(name)


def _w(t: torch.Tensor) -> OaMatrix:
    return OaMatrix(t)


def _dtype(d) -> torch.dtype:
    if d is None:
        return RT.get_engine().WeightDtype()
    return to_torch_dtype(d)


# ======================================================================= factories
def Empty(shape, dtype=None) -> OaMatrix:
    return _w(torch.empty(tuple(shape), dtype=_dtype(dtype), device=_dev()))


def EmptyOn(shape, device_index: int, dtype=None) -> OaMatrix:
    return _w(torch.empty(tuple(shape), dtype=_dtype(dtype), device=torch.device("cuda", device_index)))


def Full(shape, value: float, dtype=None) -> OaMatrix:
    t = torch.empty(tuple(shape), dtype=_dtype(dtype), device=_dev())
    K.fill_(t, float(value))
    return _w(t)


def Zeros(shape, dtype=None) -> OaMatrix:
    return Full(shape, 0.0, dtype)


def Ones(shape, dtype=None) -> OaMatrix:
    return Full(shape, 1.0, dtype)


def SetRngSeed(seed: int) -> None:
    _rng["seed"] = int(seed) & 0xFFFFFFFFFFFFFFFF
    _rng["offset"] = 0


def _next_offset(n: int) -> int:
    off = _rng["offset"]
    _rng["offset"] = off + (n + 3) // 4
    return off


# ---- random numbers inside a captured training program.  A launch argument is frozen in a CUDA graph, so a captured
# Dropout with host-side (seed, offset) would repeat the same mask on every replay.  While a program is being captured the
# random ops read (seed, base offset) from a device word pair instead and pass only the offset RELATIVE to the start of
# the step; the program closes the step with a one-thread kernel that adds the counters the step consumed to the base
# (the reference rewrites Philox nodes the same way: Source/Private/Oa/Ml/TrainingProgram.cpp:245-324).  Eager step k and
# replayed step k therefore draw the same counters.
_rng_capture = {"state": None, "base": 0}


def BeginProgramRng():
    """Called by OaTrainingProgram right before capture: device state := host (seed, offset)."""
    dev = _dev()
    if dev.type != "cuda":
        return None
    st = _rng_capture["state"]
    if st is None or st.device != dev:
        st = torch.zeros(2, dtype=torch.int64, device=dev)
    seed, off = _rng["seed"], _rng["offset"]
    st.copy_(torch.tensor([seed - (1 << 64) if seed >= (1 << 63) else seed, off], dtype=torch.int64))
    _rng_capture["state"], _rng_capture["base"] = st, off
    _rng_capture["active"] = True
    return st


def EndProgramRng() -> int:
    """Called at the end of the captured body: appends the advance launch; returns the counters one step consumes.  The
    host offset goes back to its value before the capture (the capture pass itself executed nothing)."""
    st = _rng_capture["state"]
    used = _rng["offset"] - _rng_capture["base"]
    if st is not None and used > 0:
        K.philox_state_advance(st, used)
    _rng["offset"] = _rng_capture["base"]
    _rng_capture["active"] = False
    return used


def AdvanceHostRng(counters: int) -> None:
    """A replayed step consumed `counters` Philox counters on the device: keep the host offset in step."""
    _rng["offset"] += int(counters)


def _rng_args(n: int):
    """(seed, offset, state) for one random launch of n values."""
    off = _next_offset(n)
    if _rng_capture.get("active"):
        return 0, off - _rng_capture["base"], _rng_capture["state"]
    return _rng["seed"], off, None


def _philox(shape, dtype, normal: bool, a: float, b: float) -> OaMatrix:
    dt = _dtype(dtype)
    t = torch.empty(tuple(shape), dtype=torch.float32 if dt not in (torch.float32, torch.bfloat16) else dt, device=_dev())
    seed, off, state = _rng_args(t.numel())
    K.philox_(t, seed, off, normal=normal, a=a, b=b, state=state)
    return _w(t if t.dtype == dt else t.to(dt))


def Rand(shape, dtype=None) -> OaMatrix:
    """U[0,1)."""
    return _philox(shape, dtype, False, 0.0, 1.0)


def PhiloxUniform(shape, lo: float = 0.0, hi: float = 1.0, dtype=None) -> OaMatrix:
    return _philox(shape, dtype, False, lo, hi)


def PhiloxNormal(shape, mean: float = 0.0, std: float = 1.0, dtype=None) -> OaMatrix:
    return _philox(shape, dtype, True, mean, std)


def RandN(shape, dtype=None, std: Optional[float] = None) -> OaMatrix:
    """N(0, sqrt(2/fan_in)) for rank 2 (fan_in = dim 1), N(0, 0.02) otherwise
    (Source/Private/Oa/Core/FnMatrix/Alloc/FnMatrixAlloc.cpp:105-167)."""
    shape = tuple(shape)
    if std is None:
        std = math.sqrt(2.0 / shape[1]) if len(shape) == 2 else 0.02
    return _philox(shape, dtype, True, 0.0, std)


def RandXavier(shape, dtype=None) -> OaMatrix:
    shape = tuple(shape)
    bound = math.sqrt(1.0 / shape[-1])
    return _philox(shape, dtype, False, -bound, bound)


def RandGlorotUniform(shape, dtype=None) -> OaMatrix:
    shape = tuple(shape)
    fo, fi = (shape[0], shape[1]) if len(shape) >= 2 else (shape[0], shape[0])
    bound = math.sqrt(6.0 / (fi + fo))
    return _philox(shape, dtype, False, -bound, bound)


def RandKaimingUniform(shape, dtype=None) -> OaMatrix:
    shape = tuple(shape)
    fi = shape[1] if len(shape) >= 2 else shape[0]
    bound = math.sqrt(6.0 / fi)
    return _philox(shape, dtype, False, -bound, bound)


def FromFloats(values, shape=None, dtype=None) -> OaMatrix:
    t = torch.tensor(list(values), dtype=torch.float32)
    if shape is not None:
        t = t.reshape(tuple(shape))
    return _w(t.to(device=_dev(), dtype=_dtype(dtype) if dtype is not None else torch.float32))


def FromInt32(values, shape=None) -> OaMatrix:
    t = torch.tensor(list(values), dtype=torch.int32)
    if shape is not None:
        t = t.reshape(tuple(shape))
    return _w(t.to(_dev()))


def FromBytes(data: bytes, shape, dtype) -> OaMatrix:
    dt = to_torch_dtype(dtype)
    t = torch.frombuffer(bytearray(data), dtype=dt).reshape(tuple(shape))
    return _w(t.to(_dev()))


def FromTensor(t: torch.Tensor) -> OaMatrix:
    return _w(t)


def CausalMask(seq: int, dtype=None) -> OaMatrix:
    """Additive [seq, seq] mask: 0 on and below the diagonal, a large negative value above."""
    m = torch.full((seq, seq), -1e9, dtype=torch.float32).triu(1)
    return _w(m.to(device=_dev(), dtype=_dtype(dtype)))


def GetWeightDtype() -> OaScalarType:
    from .types import from_torch_dtype
    return from_torch_dtype(RT.get_engine().WeightDtype())


def SetWeightDtype(dtype) -> None:
    RT.get_engine().SetWeightDtype(to_torch_dtype(dtype))


def CopyToHost(m: OaMatrix):
    RT.OaContext.GetDefault().Sync()
    return m.Tensor().detach().float().cpu().reshape(-1).tolist()


def CopyToHost2D(m: OaMatrix):
    RT.OaContext.GetDefault().Sync()
    return m.Tensor().detach().float().cpu().reshape(m.Size(0), -1).tolist()


def Scalar(m: OaMatrix) -> float:
    RT.OaContext.GetDefault().Sync()
    return m.Item()


def Detach(m: OaMatrix) -> OaMatrix:
    return m.Detach()


def Cast(m: OaMatrix, dtype) -> OaMatrix:
    dt = to_torch_dtype(dtype)
    x = m.Tensor()
    if x.dtype == dt:
        return m
    _ctx_add("Cast")
    out = _w(K.cast(x, dt))
    src_dt = x.dtype
    return AG.attach("Cast", out, [m], lambda g: (K.cast(g, src_dt),))


# ======================================================================= elementwise
def _c(t: torch.Tensor) -> torch.Tensor:
    return t if t.is_contiguous() else K.contiguous(t)


def _unary(name: str, op: str, m: OaMatrix, s0: float, bwd) -> OaMatrix:
    _ctx_add(name)
    x = _c(m.Tensor())
    y = K.unary(op, x, s0)
    out = _w(y)
    if bwd is None:
        return out
    return AG.attach(name, out, [m], lambda g: (bwd(x, y, _c(g)),))


def Neg(m): return _unary("Neg", "neg", m, 0.0, lambda x, y, g: K.unary("neg", g))
def Abs(m): return _unary("Abs", "abs", m, 0.0, lambda x, y, g: K.binary("abs_bwd", x, g))
def Log(m): return _unary("Log", "log", m, 0.0, lambda x, y, g: K.binary("log_bwd", x, g))
def Exp(m): return _unary("Exp", "exp", m, 0.0, lambda x, y, g: K.binary("mul", y, g))
def Sqrt(m): return _unary("Sqrt", "sqrt", m, 0.0, lambda x, y, g: K.binary("sqrt_bwd", y, g))
def Sin(m): return _unary("Sin", "sin", m, 0.0, lambda x, y, g: K.binary("mul", K.unary("cos", x), g))
def Cos(m): return _unary("Cos", "cos", m, 0.0, lambda x, y, g: K.unary("neg", K.binary("mul", K.unary("sin", x), g)))
def Reciprocal(m): return _unary("Reciprocal", "recip", m, 0.0, lambda x, y, g: K.binary("recip_bwd", y, g))
def Scale(m, s: float): return _unary("Scale", "scale", m, float(s), lambda x, y, g: K.unary("scale", g, float(s)))
def AddScalar(m, s: float): return _unary("AddScalar", "add_scalar", m, float(s), lambda x, y, g: g)
def SubScalar(m, s: float): return _unary("SubScalar", "add_scalar", m, -float(s), lambda x, y, g: g)
def DivScalar(m, s: float): return _unary("DivScalar", "scale", m, 1.0 / float(s), lambda x, y, g: K.unary("scale", g, 1.0 / float(s)))
def Square(m): return _unary("Square", "square", m, 0.0, lambda x, y, g: K.unary("scale", K.binary("mul", x, g), 2.0))


def Pow(m, e: float):
    e = float(e)
    return _unary("Pow", "pow", m, e, lambda x, y, g: K.unary("scale", K.binary("mul", K.unary("pow", x, e - 1.0), g), e))


def ClampMax(m, v: float):
    v = float(v)
    return _unary("ClampMax", "clamp_max", m, v,
                  lambda x, y, g: K.binary("mul", g, K.binary("ge", K.unary("rsub_scalar", x, v), torch.zeros(1, dtype=x.dtype, device=x.device))))


def ClampMin(m, v: float):
    v = float(v)
    return _unary("ClampMin", "clamp_min", m, v,
                  lambda x, y, g: K.binary("mul", g, K.binary("ge", K.unary("add_scalar", x, -v), torch.zeros(1, dtype=x.dtype, device=x.device))))


def Relu(m): return _unary("Relu", "relu", m, 0.0, lambda x, y, g: K.binary("relu_bwd", x, g))
def Gelu(m): return _unary("Gelu", "gelu", m, 0.0, lambda x, y, g: K.binary("gelu_bwd", x, g))
def Silu(m): return _unary("Silu", "silu", m, 0.0, lambda x, y, g: K.binary("silu_bwd", x, g))
def Tanh(m): return _unary("Tanh", "tanh", m, 0.0, lambda x, y, g: K.binary("tanh_bwd", y, g))
def Sigmoid(m): return _unary("Sigmoid", "sigmoid", m, 0.0, lambda x, y, g: K.binary("sigmoid_bwd", y, g))
def Softplus(m): return _unary("Softplus", "softplus", m, 0.0, lambda x, y, g: K.binary("softplus_bwd", x, g))
def LeakyRelu(m, slope: float = 0.01):
    # d/dx = slope + (1 - slope) * [x > 0]
    return _unary("LeakyRelu", "leaky_relu", m, slope,
                  lambda x, y, g: K.binary("add", K.unary("scale", K.binary("relu_bwd", x, g), 1.0 - slope), K.unary("scale", g, slope)))
def Elu(m, alpha: float = 1.0):
    def bwd(x, y, g):           # d/dx = 1 for x > 0, y + alpha otherwise
        r = K.binary("relu_bwd", x, g)
        return K.binary("add", r, K.binary("mul", K.binary("sub", g, r), K.unary("add_scalar", y, alpha)))
    return _unary("Elu", "elu", m, alpha, bwd)
def Mish(m): return _unary("Mish", "mish", m, 0.0, lambda x, y, g: K.binary("mish_bwd", x, g))


def ReluBwd(x: OaMatrix, dy: OaMatrix) -> OaMatrix: return _w(K.binary("relu_bwd", _c(x.Tensor()), _c(dy.Tensor())))
def GeluBwd(x: OaMatrix, dy: OaMatrix) -> OaMatrix: return _w(K.binary("gelu_bwd", _c(x.Tensor()), _c(dy.Tensor())))
def SiluBwd(x: OaMatrix, dy: OaMatrix) -> OaMatrix: return _w(K.binary("silu_bwd", _c(x.Tensor()), _c(dy.Tensor())))
def TanhBwd(y: OaMatrix, dy: OaMatrix) -> OaMatrix: return _w(K.binary("tanh_bwd", _c(y.Tensor()), _c(dy.Tensor())))


def _reduce_to(g: torch.Tensor, shape) -> torch.Tensor:
    """Sums a gradient over the dimensions along which `shape` was broadcast."""
    shape = tuple(shape)
    if tuple(g.shape) == shape:
        return g
    n = 1
    for d in shape:
        n *= d
    if n == 1:
        return K.row_reduce("sum", g.reshape(1, -1)).reshape(shape)
    if n == g.shape[-1] and shape[-1] == g.shape[-1]:
        return K.col_sum(g.reshape(-1, g.shape[-1])).reshape(shape)
    if g.dim() >= 1 and n == g.numel() // g.shape[-1] and shape[-1] == 1 and len(shape) == g.dim():
        return K.row_reduce("sum", g.reshape(-1, g.shape[-1])).reshape(shape)
    # general case: one dimension at a time, [outer, d, inner] -> [outer, inner]
    padded = (1,) * (g.dim() - len(shape)) + shape
    cur = g
    for i in range(g.dim()):
        if padded[i] == cur.shape[i]:
            continue
        if padded[i] != 1:
            raise ValueError(f"cannot reduce gradient {tuple(g.shape)} to {shape}")
        outer = 1
        for d in cur.shape[:i]:
            outer *= d
        dsz = cur.shape[i]
        inner = cur.numel() // (outer * dsz)
        v = _c(cur).reshape(outer, dsz, inner)
        if inner == 1:
            r = K.row_reduce("sum", v.reshape(outer, dsz))
        elif outer == 1:
            r = K.col_sum(v.reshape(dsz, inner))
        else:
            r = K.row_reduce("sum", K.contiguous(v.permute(0, 2, 1)).reshape(outer * inner, dsz))
        cur = r.reshape(*cur.shape[:i], 1, *cur.shape[i + 1:])
    return cur.reshape(shape)


def _fast_broadcast(big: torch.Tensor, small: torch.Tensor) -> bool:
    """True when ops.kernels.binary handles (big, small) without materialising the broadcast."""
    if big.shape == small.shape or small.numel() == 1:
        return True
    if small.numel() == big.shape[-1] and (small.dim() == 1 or all(d == 1 for d in small.shape[:-1])):
        return True
    return small.dim() == big.dim() and small.shape[-1] == 1 and small.numel() == big.numel() // big.shape[-1]


def _binary(name: str, op: str, a: OaMatrix, b: OaMatrix, bwd) -> OaMatrix:
    _ctx_add(name)
    ta, tb = _c(a.Tensor()), _c(b.Tensor())
    if ta.shape != tb.shape:
        full = torch.broadcast_shapes(ta.shape, tb.shape)
        big, small = (ta, tb) if ta.numel() >= tb.numel() else (tb, ta)
        if tuple(big.shape) != tuple(full) or not _fast_broadcast(big, small):
            xa, xb = K.contiguous(ta.expand(full)), K.contiguous(tb.expand(full))
            y = K.binary(op, xa, xb)
            out = _w(y)
            if bwd is None:
                return out

            def back_full(g):
                ga, gb = bwd(xa, xb, y, _c(g))
                return (_reduce_to(ga, ta.shape) if ga is not None else None, _reduce_to(gb, tb.shape) if gb is not None else None)

            return AG.attach(name, out, [a, b], back_full)
    swap = ta.numel() < tb.numel()
    if swap and op in ("add", "mul"):
        y = K.binary(op, tb, ta)
    elif swap:
        # broadcast on the left operand: expand explicitly (rare path)
        y = K.binary(op, _c(ta.expand_as(tb)), tb)
    else:
        y = K.binary(op, ta, tb)
    out = _w(y)
    if bwd is None:
        return out

    def back(g):
        g = _c(g)
        ga, gb = bwd(ta, tb, y, g)
        return (_reduce_to(ga, ta.shape) if ga is not None else None, _reduce_to(gb, tb.shape) if gb is not None else None)

    return AG.attach(name, out, [a, b], back)


def Add(a, b): return _binary("Add", "add", a, b, lambda ta, tb, y, g: (g, g))
def Sub(a, b): return _binary("Sub", "sub", a, b, lambda ta, tb, y, g: (g, K.unary("neg", g)))


def Mul(a, b):
    def bwd(ta, tb, y, g):
        big_a = ta.numel() >= tb.numel()
        ga = K.binary("mul", g, tb) if big_a else K.binary("mul", g, _c(tb))
        gb = K.binary("mul", g, ta) if not big_a or ta.shape == tb.shape else K.binary("mul", g, ta)
        return ga, gb
    return _binary("Mul", "mul", a, b, bwd)


def Div(a, b):
    def bwd(ta, tb, y, g):
        ga = K.binary("div", g, tb)
        gb = K.unary("neg", K.binary("div", K.binary("mul", g, y), tb))
        return ga, gb
    return _binary("Div", "div", a, b, bwd)


def Equal(a, b): return _binary("Equal", "eq", a, b, None)
def GreaterEqual(a, b): return _binary("GreaterEqual", "ge", a, b, None)
def Maximum(a, b): return _binary("Maximum", "max", a, b, None)


def AddInPlace(dst: OaMatrix, src: OaMatrix) -> None:
    _ctx_add("AddInPlace")
    K.binary("add", dst.Tensor(), _c(src.Tensor()), out=dst.Tensor())


def ScaleInPlace(dst: OaMatrix, s: float) -> None:
    _ctx_add("ScaleInPlace")
    K.unary("scale", dst.Tensor(), float(s), out=dst.Tensor())


def Fill(dst: OaMatrix, v: float) -> None:
    _ctx_add("Fill")
    K.fill_(dst.Tensor(), float(v))


def MultiFill(mats, v: float) -> None:
    for m in mats:
        Fill(m, v)


def MultiAdd(dsts, srcs) -> None:
    for d, s in zip(dsts, srcs):
        AddInPlace(d, s)


def FlushDeferredAccum() -> None:
    """Gradient accumulation is never deferred here (kernels run in stream order); kept for API parity."""


def Dropout(m: OaMatrix, p: float, training: bool = True) -> OaMatrix:
    if not training or p <= 0.0:
        return m
    _ctx_add("Dropout")
    x = _c(m.Tensor())
    seed, off, state = _rng_args(x.numel())
    out = _w(K.dropout(x, p, seed, off, state))
    return AG.attach("Dropout", out, [m], lambda g: (K.dropout(_c(g), p, seed, off, state),))


# ======================================================================= shape ops
def Reshape(m: OaMatrix, shape) -> OaMatrix:
    shape = tuple(int(s) for s in shape)
    t = m.Tensor()
    out = _w(t.reshape(shape) if t.is_contiguous() else K.contiguous(t).reshape(shape))
    src = tuple(t.shape)
    return AG.attach("Reshape", out, [m], lambda g: (g.reshape(src),))


def Transpose(m: OaMatrix, d0: int = 0, d1: int = 1) -> OaMatrix:
    _ctx_add("Transpose")
    out = _w(K.contiguous(m.Tensor().transpose(d0, d1)))
    return AG.attach("Transpose", out, [m], lambda g: (K.contiguous(g.transpose(d0, d1)),))


def Permute(m: OaMatrix, dims) -> OaMatrix:
    dims = tuple(dims)
    inv = [0] * len(dims)
    for i, d in enumerate(dims):
        inv[d] = i
    _ctx_add("Permute")
    out = _w(K.contiguous(m.Tensor().permute(dims)))
    return AG.attach("Permute", out, [m], lambda g: (K.contiguous(g.permute(inv)),))


def Slice(m: OaMatrix, dim: int, start: int, end: int) -> OaMatrix:
    _ctx_add("Slice")
    t = m.Tensor()
    out = _w(K.contiguous(t.narrow(dim, start, end - start)))

    def back(g):
        full = torch.empty_like(t)
        K.fill_(full, 0.0)
        full.narrow(dim, start, end - start).copy_(g)
        return (full,)

    return AG.attach("Slice", out, [m], back)


def Concat(mats: Sequence[OaMatrix], dim: int = 0) -> OaMatrix:
    _ctx_add("Concat")
    ts = [x.Tensor() for x in mats]
    shape = list(ts[0].shape)
    shape[dim] = sum(t.shape[dim] for t in ts)
    out_t = torch.empty(shape, dtype=ts[0].dtype, device=ts[0].device)
    sizes, off = [], 0
    for t in ts:
        out_t.narrow(dim, off, t.shape[dim]).copy_(t)
        sizes.append((off, t.shape[dim]))
        off += t.shape[dim]
    out = _w(out_t)
    return AG.attach("Concat", out, list(mats), lambda g: tuple(K.contiguous(g.narrow(dim, o, n)) for o, n in sizes))


def Split(m: OaMatrix, sizes: Sequence[int], dim: int = -1):
    outs, off = [], 0
    if dim < 0:
        dim += m.Rank()
    for n in sizes:
        outs.append(Slice(m, dim, off, off + n))
        off += n
    return outs


def RepeatInterleave(m: OaMatrix, repeats: int, dim: int = 0) -> OaMatrix:
    _ctx_add("RepeatInterleave")
    t = m.Tensor()
    out = _w(K.contiguous(t.unsqueeze(dim + 1).expand(*t.shape[: dim + 1], repeats, *t.shape[dim + 1:])).reshape(
        *t.shape[:dim], t.shape[dim] * repeats, *t.shape[dim + 1:]))

    def back(g):
        return (_repeat_bwd(_c(g), t.shape, dim, repeats),)

    return AG.attach("RepeatInterleave", out, [m], back)


def _repeat_bwd(g, shape, dim, repeats):
    gg = g.reshape(*shape[: dim + 1], repeats, *shape[dim + 1:])
    gg = K.contiguous(gg.movedim(dim + 1, -1))
    return K.row_reduce("sum", gg.reshape(-1, repeats)).reshape(shape)


# ======================================================================= reductions
def _rows(t: torch.Tensor):
    return _c(t).reshape(-1, t.shape[-1])


def Sum(m: OaMatrix, dim: Optional[int] = None) -> OaMatrix:
    _ctx_add("Sum")
    t = m.Tensor()
    if dim is None:
        out = _w(K.row_reduce("sum", _c(t).reshape(1, -1)).reshape(1))
        return AG.attach("Sum", out, [m], lambda g: (K.binary("mul", torch.ones_like(t), g.reshape(1)),))
    if dim < 0:
        dim += t.dim()
    if dim == t.dim() - 1:
        out = _w(K.row_reduce("sum", _rows(t)).reshape(t.shape[:-1]))
        return AG.attach("Sum", out, [m], lambda g: (K.binary("mul", torch.ones_like(t), _c(g).reshape(*t.shape[:-1], 1)),))
    if dim == 0 and t.dim() == 2:
        out = _w(K.col_sum(_c(t)))
        return AG.attach("Sum", out, [m], lambda g: (K.binary("add", torch.zeros_like(t), _c(g)),))
    moved = K.contiguous(t.movedim(dim, -1))
    out = _w(K.row_reduce("sum", moved.reshape(-1, moved.shape[-1])).reshape(moved.shape[:-1]))

    def back(g):
        full = K.binary("mul", torch.ones_like(moved), _c(g).reshape(*moved.shape[:-1], 1))
        return (K.contiguous(full.movedim(-1, dim)),)

    return AG.attach("Sum", out, [m], back)


def Mean(m: OaMatrix, dim: Optional[int] = None) -> OaMatrix:
    n = m.NumElements() if dim is None else m.Size(dim)
    return Scale(Sum(m, dim), 1.0 / n)


def Max(m: OaMatrix, dim: int = -1) -> OaMatrix:
    _ctx_add("Max")
    t = m.Tensor()
    rows = _rows(t)
    y = K.row_reduce("max", rows)
    out = _w(y.reshape(t.shape[:-1]))

    def back(g):
        mask = K.binary("eq", rows, y.reshape(-1, 1))
        return (K.binary("mul", mask, _c(g).reshape(-1, 1)).reshape(t.shape),)

    return AG.attach("Max", out, [m], back)


def Argmax(m: OaMatrix, dim: int = -1) -> OaMatrix:
    _ctx_add("Argmax")
    t = m.Tensor()
    if t.dim() == 1:
        return _w(K.row_reduce("argmax", _c(t).reshape(1, -1)).reshape(()))
    return _w(K.row_reduce("argmax", _rows(t)).reshape(t.shape[:-1]))


def Softmax(m: OaMatrix, dim: int = -1) -> OaMatrix:
    _ctx_add("Softmax")
    t = m.Tensor()
    y = K.softmax(_rows(t))
    out = _w(y.reshape(t.shape))
    return AG.attach("Softmax", out, [m], lambda g: (K.softmax_bwd(y, _rows(g)).reshape(t.shape),))


def LogSoftmax(m: OaMatrix, dim: int = -1) -> OaMatrix:
    _ctx_add("LogSoftmax")
    t = m.Tensor()
    y = K.softmax(_rows(t), log=True)
    out = _w(y.reshape(t.shape))
    return AG.attach("LogSoftmax", out, [m], lambda g: (K.softmax_bwd(y, _rows(g), log=True).reshape(t.shape),))


def SoftmaxBwd(y: OaMatrix, dy: OaMatrix) -> OaMatrix:
    return _w(K.softmax_bwd(_rows(y.Tensor()), _rows(dy.Tensor())).reshape(y.Tensor().shape))


def SoftmaxScaledMasked(scores: OaMatrix, scale: float, mask: Optional[OaMatrix] = None) -> OaMatrix:
    """softmax(scores * scale + mask) over the last dimension; the additive mask has the scores' shape or is one
    [rows, cols] block that repeats over the leading dimensions (a [S, S] causal mask for [B*H, S, S] scores)."""
    _ctx_add("SoftmaxScaledMasked")
    t = scores.Tensor()
    mk = _rows(mask.Tensor()) if mask is not None else None
    y = K.softmax(_rows(t), scale=scale, mask=mk)
    out = _w(y.reshape(t.shape))
    return AG.attach("SoftmaxScaledMasked", out, [scores], lambda g: (K.softmax_bwd(y, _rows(g), scale=scale).reshape(t.shape),))


def TopK(m: OaMatrix, k: int):
    """Descending top-k over the last dimension, ties to the lower index (Flat/TopK.slang:39-77).
    Returns (values [rows,k], indices int32 [rows,k])."""
    from ..ops import moe as MOE
    _ctx_add("TopK")
    vals, idx = MOE.topk(_rows(m.Tensor()), k)
    return _w(vals), _w(idx)


def TopKMask(m: OaMatrix, k: int) -> OaMatrix:
    from ..ops import moe as MOE
    _ctx_add("TopKMask")
    rows = _rows(m.Tensor())
    _, idx = MOE.topk(rows, k)
    mask = torch.zeros_like(rows)
    mask.scatter_(1, idx.long(), 1.0)
    return _w(mask.reshape(m.Tensor().shape))


# ======================================================================= indexing
def Gather(table: OaMatrix, ids: OaMatrix) -> OaMatrix:
    """out[i,:] = table[ids[i],:] (Embedding lookup); ids any shape, output [ids.numel, dim]."""
    _ctx_add("Gather")
    tt, ti = table.Tensor(), ids.Tensor()
    out = _w(K.embedding_fwd(tt, ti))
    vocab = tt.shape[0]

    def back(g):
        gt = K.embedding_bwd(_c(g), ti, vocab)
        return (gt if tt.dtype == torch.float32 else K.cast(gt, tt.dtype), None)

    return AG.attach("Gather", out, [table, ids], back)


def GatherBwd(dout: OaMatrix, ids: OaMatrix, vocab: int) -> OaMatrix:
    return _w(K.embedding_bwd(_c(dout.Tensor()), ids.Tensor(), vocab))


def GatherLastDim(m: OaMatrix, idx: OaMatrix) -> OaMatrix:
    """out[r, j] = m[r, idx[r, j]]."""
    _ctx_add("GatherLastDim")
    rows = _rows(m.Tensor())
    ii = idx.Tensor().reshape(rows.shape[0], -1).long()
    out = _w(torch.gather(rows, 1, ii))

    def back(g):
        full = torch.zeros_like(rows)
        full.scatter_add_(1, ii, g.reshape(ii.shape).to(rows.dtype))
        return (full.reshape(m.Tensor().shape), None)

    return AG.attach("GatherLastDim", out, [m, idx], back)


# ======================================================================= linear algebra
def _grad_out(leaf: Optional[OaMatrix], shape, dtype, device):
    """Destination of a parameter gradient: the leaf's persistent buffer when it has one."""
    sink = leaf.GradSink() if (leaf is not None and leaf.IsLeaf() and leaf.RequiresGrad()) else None
    if sink is not None:
        return sink[0], sink[1], True
    return torch.empty(shape, dtype=dtype, device=device), False, False


def MatMulNt(a: OaMatrix, b: OaMatrix) -> OaMatrix:
    """C = A @ B^T with A [..., K] and B [N, K]; fp32 accumulation."""
    _ctx_add("MatMulNt")
    ta, tb = a.Tensor(), b.Tensor()
    a2 = _rows(ta)
    tb = _c(tb)
    y = K.gemm(a2, tb)
    out = _w(y.reshape(*ta.shape[:-1], tb.shape[0]))

    def back(g):
        g2 = _rows(g)
        da = K.gemm(g2, tb, b_mn=True).reshape(ta.shape) if a.RequiresGrad() else None
        db = None
        if b.RequiresGrad():
            buf, acc, direct = _grad_out(b, tb.shape, tb.dtype, tb.device)
            K.gemm(g2, a2, a_mn=True, b_mn=True, out=buf, accumulate=acc)
            db = None if direct else buf
        return (da, db)

    return AG.attach("MatMulNt", out, [a, b], back)


def _bias_grad(bias: Optional[OaMatrix], g2: torch.Tensor):
    if bias is None or not bias.RequiresGrad():
        return None
    sink = bias.GradSink() if bias.IsLeaf() else None
    if sink is not None:
        K.col_sum(g2, out=sink[0], accumulate=sink[1])
        return None
    return K.col_sum(g2)


def Linear(x: OaMatrix, w: OaMatrix, b: Optional[OaMatrix] = None, act: int = K.ACT_NONE, name: str = "Linear",
           residual: Optional[OaMatrix] = None) -> OaMatrix:
    """y = act(x @ W^T + b) (+ residual); W is [out, in].  act in {none, gelu, relu} is fused in the GEMM epilogue,
    the pre-activation is kept for the backward pass."""
    _ctx_add(name)
    tx, tw = x.Tensor(), _c(w.Tensor())
    x2 = _rows(tx)
    tb = b.Tensor() if b is not None else None
    z = torch.empty((x2.shape[0], tw.shape[0]), dtype=tx.dtype, device=tx.device) if act != K.ACT_NONE else None
    res2 = _rows(residual.Tensor()) if residual is not None else None
    y = K.gemm(x2, tw, bias=tb, act=act, aux_out=z, residual=res2)
    out = _w(y.reshape(*tx.shape[:-1], tw.shape[0]))

    def back(g):
        g2 = _rows(g)
        if act == K.ACT_GELU:
            gz = K.binary("gelu_bwd", z, g2)
        elif act == K.ACT_RELU:
            gz = K.binary("relu_bwd", z, g2)
        else:
            gz = g2
        dx = K.gemm(gz, tw, b_mn=True).reshape(tx.shape) if x.RequiresGrad() else None
        dw = None
        if w.RequiresGrad():
            buf, acc, direct = _grad_out(w, tw.shape, tw.dtype, tw.device)
            K.gemm(gz, x2, a_mn=True, b_mn=True, out=buf, accumulate=acc)
            dw = None if direct else buf
        db = _bias_grad(b, gz)
        if residual is not None:
            return (dx, dw, db, g)
        return (dx, dw, db)

    ins = [x, w, b] + ([residual] if residual is not None else [])
    return AG.attach(name, out, ins, back)


def LinearGelu(x, w, b=None): return Linear(x, w, b, K.ACT_GELU, "LinearGelu")
def LinearRelu(x, w, b=None): return Linear(x, w, b, K.ACT_RELU, "LinearRelu")


def LinearDataBwd(dy: OaMatrix, w: OaMatrix) -> OaMatrix:
    """dX = dY @ W."""
    return _w(K.gemm(_rows(dy.Tensor()), _c(w.Tensor()), b_mn=True))


class OaLinearWeightBiasBwdResult:
    def __init__(self, dw: OaMatrix, db: OaMatrix):
        self.WeightGrad = dw
        self.BiasGrad = db


def LinearWeightBwd(dy: OaMatrix, x: OaMatrix) -> OaMatrix:
    return _w(K.gemm(_rows(dy.Tensor()), _rows(x.Tensor()), a_mn=True, b_mn=True))


def LinearWeightBiasBwd(dy: OaMatrix, x: OaMatrix) -> OaLinearWeightBiasBwdResult:
    g2 = _rows(dy.Tensor())
    return OaLinearWeightBiasBwdResult(_w(K.gemm(g2, _rows(x.Tensor()), a_mn=True, b_mn=True)), _w(K.col_sum(g2)))


def PackedLinear(x: OaMatrix, weights: Sequence[OaMatrix], biases: Sequence[Optional[OaMatrix]]):
    """Several projections of one activation as ONE GEMM over the row-concatenated weights; returns the packed
    output [M, sum(N_i)] (reference: PackedLinear2/3, Source/Private/Oa/Ml/FnMatrix/Modules/FnMatrixPackedLinear.cpp:33-70).
    The checkpoint keeps the separate weights; callers that own a pre-packed weight should call Linear directly."""
    wcat = Concat(list(weights), 0)
    bcat = Concat([b for b in biases], 0) if all(b is not None for b in biases) and len(biases) else None
    return Linear(x, wcat, bcat, name=f"PackedLinear{len(weights)}")


def PackedLinear2(x, w0, w1, b0=None, b1=None): return PackedLinear(x, [w0, w1], [b0, b1])
def PackedLinear3(x, w0, w1, w2, b0=None, b1=None, b2=None): return PackedLinear(x, [w0, w1, w2], [b0, b1, b2])


def Bmm(a: OaMatrix, b: OaMatrix) -> OaMatrix:
    """out[n] = a[n] @ b[n], a [B,M,K], b [B,K,N] (exact fp32 products; bf16 inputs are widened)."""
    _ctx_add("Bmm")
    ta, tb = a.Tensor(), b.Tensor()
    fa, fb = (ta if ta.dtype == torch.float32 else K.cast(ta, torch.float32)), (tb if tb.dtype == torch.float32 else K.cast(tb, torch.float32))
    y = K.bmm_f32(fa, fb, b_mn=True)
    out = _w(y if ta.dtype == torch.float32 else K.cast(y, ta.dtype))

    def back(g):
        gf = _c(g if g.dtype == torch.float32 else K.cast(g, torch.float32))
        da = K.bmm_f32(gf, _c(fb), b_mn=False)                       # g @ b^T
        db = K.bmm_f32(K.contiguous(fa.transpose(1, 2)), gf, b_mn=True)  # a^T @ g
        if ta.dtype != torch.float32:
            da, db = K.cast(da, ta.dtype), K.cast(db, tb.dtype)
        return (da, db)

    return AG.attach("Bmm", out, [a, b], back)


# ======================================================================= norms
def RmsNorm(x: OaMatrix, w: OaMatrix, eps: float = 1e-6) -> OaMatrix:
    _ctx_add("RmsNorm")
    tx, tw = x.Tensor(), w.Tensor()
    x2 = _rows(tx)
    y, rstd, _ = K.rmsnorm_fwd(x2, tw, eps)
    out = _w(y.reshape(tx.shape))

    def back(g, pending=None):
        # `pending`: what x has already collected through the residual stream; the kernel adds it while it writes dx
        sink = w.GradSink() if (w.IsLeaf() and w.RequiresGrad()) else None
        dres = _rows(pending) if (pending is not None and pending.is_contiguous()) else None
        dx, dw = K.rmsnorm_bwd(x2, tw, _rows(g), rstd, dres=dres, dw_out=sink[0] if sink else None, accumulate_dw=bool(sink and sink[1]))
        dx = dx.reshape(tx.shape)
        if pending is not None and dres is None:
            dx = K.binary("add", pending, dx)
        return (dx, None if sink else dw)

    return AG.attach("RmsNorm", out, [x, w], back, fold=0)


def ResidualRmsNorm(x: OaMatrix, residual: OaMatrix, w: OaMatrix, eps: float = 1e-6):
    """(y, s) with s = x + residual and y = RmsNorm(s) in one pass."""
    _ctx_add("ResidualRmsNorm")
    s = Add(x, residual)
    return RmsNorm(s, w, eps), s


def RmsNormGated(x: OaMatrix, w: OaMatrix, bias: Optional[OaMatrix], z: OaMatrix, eps: float = 1e-5,
                 norm_before_gate: bool = True) -> OaMatrix:
    """norm_before_gate: (RmsNorm(x) * w + bias) * silu(z); otherwise RmsNorm(x * silu(z)) * w + bias
    (Source/Public/Oa/Ml/FnMatrix.h:503-506)."""
    if norm_before_gate:
        n = RmsNorm(x, w, eps)
        if bias is not None:
            n = Add(n, bias)
        return SiluMul(z, n)
    n = RmsNorm(SiluMul(z, x), w, eps)
    return Add(n, bias) if bias is not None else n


def LayerNorm(x: OaMatrix, w: OaMatrix, b: Optional[OaMatrix], eps: float = 1e-5) -> OaMatrix:
    _ctx_add("LayerNorm")
    tx = x.Tensor()
    x2 = _rows(tx)
    tw = w.Tensor()
    y, mean, rstd = K.layernorm_fwd(x2, tw, b.Tensor() if b is not None else None, eps)
    out = _w(y.reshape(tx.shape))

    def back(g):
        ws = w.GradSink() if (w.IsLeaf() and w.RequiresGrad()) else None
        bs = b.GradSink() if (b is not None and b.IsLeaf() and b.RequiresGrad()) else None
        if (ws is None) != (bs is None) or (ws and bs and ws[1] != bs[1]):
            ws = bs = None  # mixed states: fall back to returned gradients
        dx, dw, db = K.layernorm_bwd(x2, tw, _rows(g), mean, rstd, dw_out=ws[0] if ws else None,
                                     db_out=bs[0] if bs else None, accumulate=bool(ws and ws[1]), want_bias=b is not None)
        return (dx.reshape(tx.shape), None if ws else dw, None if bs else db)

    return AG.attach("LayerNorm", out, [x, w, b], back)


# ======================================================================= gated activations
def Swiglu(gate_up: OaMatrix) -> OaMatrix:
    """silu(A[:, :F]) * A[:, F:] on a packed [M, 2F] tensor."""
    _ctx_add("Swiglu")
    t = gate_up.Tensor()
    a2 = _rows(t)
    y = K.swiglu_fwd(a2)
    out = _w(y.reshape(*t.shape[:-1], t.shape[-1] // 2))
    return AG.attach("Swiglu", out, [gate_up], lambda g: (K.swiglu_bwd(a2, _rows(g)).reshape(t.shape),))


def SiluMul(gate: OaMatrix, up: OaMatrix) -> OaMatrix:
    return _binary("SiluMul", "silu_mul", gate, up, lambda tg, tu, y, g: (
        K.binary("mul", K.binary("silu_bwd", tg, g), tu), K.binary("silu_mul", tg, g)))


def Geglu(packed: OaMatrix) -> OaMatrix:
    """A[:, :F] * gelu(A[:, F:])."""
    F = packed.Size(-1) // 2
    a, b = Split(packed, [F, F], -1)
    return Mul(a, Gelu(b))


# ======================================================================= attention
def SplitHeads(x: OaMatrix, batch: int, seq: int, heads: int) -> OaMatrix:
    """[B*S, D] -> [B*H, S, D/H]."""
    d = x.Size(-1)
    return Reshape(Permute(Reshape(x, [batch, seq, heads, d // heads]), [0, 2, 1, 3]), [batch * heads, seq, d // heads])


def MergeHeads(x: OaMatrix, batch: int, seq: int, heads: int) -> OaMatrix:
    hd = x.Size(-1)
    return Reshape(Permute(Reshape(x, [batch, heads, seq, hd]), [0, 2, 1, 3]), [batch * seq, heads * hd])


def RoPE(x: OaMatrix, heads: int, head_dim: int, seq: int, pos_offset: int = 0, theta: float = 10000.0) -> OaMatrix:
    """Rotate-half RoPE on [B*S, heads*head_dim] rows (Nn/Rope/RopeApply.slang:39-56)."""
    _ctx_add("RopeApply")
    t = K.unary("copy", _rows(x.Tensor()))
    K.rope_(t, heads, head_dim, seq, pos_offset=pos_offset, theta=theta)
    out = _w(t.reshape(x.Tensor().shape))

    def back(g):
        gg = K.unary("copy", _rows(g))
        K.rope_(gg, heads, head_dim, seq, pos_offset=pos_offset, theta=theta, backward=True)
        return (gg.reshape(x.Tensor().shape),)

    return AG.attach("RopeApply", out, [x], back)


def FlashAttentionPacked(qkv: OaMatrix, batch: int, seq: int, heads: int, head_dim: int, *, causal: bool = True,
                         rope_theta: float = 0.0, pos_offset: int = 0, consume_input: bool = False) -> OaMatrix:
    """Attention over a packed projection output [B*S, 3*H*hd] (q | k | v side by side); returns [B*S, H*hd].
    With rope_theta > 0 rotate-half RoPE is applied to q and k in place first (on a copy while autograd records, unless
    the caller owns the projection output and passes consume_input: nothing else reads it)."""
    _ctx_add("FlashAttentionCausal" if causal else "FlashAttention")
    t = qkv.Tensor()
    D = heads * head_dim
    if rope_theta > 0:
        if AG.IsEnabled() and qkv.RequiresGrad() and not consume_input:
            t = K.unary("copy", _c(t))
        K.rope_(t[:, : 2 * D], 2 * heads, head_dim, seq, pos_offset=pos_offset, theta=rope_theta)
    q, k, v = t[:, :D], t[:, D:2 * D], t[:, 2 * D:]
    o, lse = K.flash_fwd(q, k, v, batch, seq, heads, head_dim, causal=causal)
    out = _w(o)

    def back(g):
        dqkv = torch.empty_like(t)
        K.flash_bwd(q, k, v, o, _c(g), lse, batch, seq, heads, head_dim, causal=causal, dqkv=dqkv)
        if rope_theta > 0:
            K.rope_(dqkv[:, : 2 * D], 2 * heads, head_dim, seq, pos_offset=pos_offset, theta=rope_theta, backward=True)
        return (dqkv,)

    return AG.attach("FlashAttentionCausal", out, [qkv], back)


def FlashAttentionCausal(q: OaMatrix, k: OaMatrix, v: OaMatrix, batch: int, seq: int, heads: int) -> OaMatrix:
    """q, k, v: [B*S, D] each -> [B*S, D]."""
    D = q.Size(-1)
    return FlashAttentionPacked(Concat([q, k, v], 1), batch, seq, heads, D // heads, causal=True)


# ======================================================================= embedding
def Embedding(table: OaMatrix, ids: OaMatrix, pos_table: Optional[OaMatrix] = None, seq_len: int = 0) -> OaMatrix:
    """table[ids] (+ pos_table[i % seq_len]) in one kernel; output [ids.numel, dim]."""
    _ctx_add("Embedding")
    tt, ti = table.Tensor(), ids.Tensor()
    tp = pos_table.Tensor() if pos_table is not None else None
    out = _w(K.embedding_fwd(tt, ti, tp, seq_len))
    vocab, dim = tt.shape

    def back(g):
        g = _c(g)
        gt = K.embedding_bwd(g, ti, vocab)
        gp = None
        if pos_table is not None and pos_table.RequiresGrad():
            n = g.shape[0]
            gp = K.col_sum(K.contiguous(g.reshape(n // seq_len, seq_len * dim))).reshape(seq_len, dim)
            if tp.shape[0] != seq_len:           # rows of the position table beyond the sequence get a zero gradient
                full = torch.empty_like(tp, dtype=gp.dtype)
                K.fill_(full, 0.0)
                K.unary("copy", gp, out=full[:seq_len])
                gp = full
        return (gt if tt.dtype == torch.float32 else K.cast(gt, tt.dtype), None, gp)

    return AG.attach("Embedding", out, [table, ids, pos_table], back)


# ======================================================================= quantisation, VQ, sampling (thin entry points)
def ComputeScaleQ4_0(m: OaMatrix) -> OaMatrix:
    """Per-32-element-block scale max|x| / 7 (1 for an all-zero block)  (Source/Public/Oa/Ml/FnMatrix.h:786-789)."""
    from ..ops import quant as Q
    _ctx_add("ComputeScaleQ4_0")
    return _w(Q.q4_0_scale(m.Tensor()))


def QuantizeQ4_0(m: OaMatrix, scale: OaMatrix) -> OaMatrix:
    """Packed Q4_0 bytes [blocks * 16]: two 4-bit codes per byte, code = clamp(round(x / scale), -7, 7) + 7."""
    from ..ops import quant as Q
    _ctx_add("QuantizeQ4_0")
    return _w(Q.q4_0_quantize(m.Tensor(), scale.Tensor()))


def DequantizeQ4_0(packed: OaMatrix, scale: OaMatrix, count: int) -> OaMatrix:
    from ..ops import quant as Q
    _ctx_add("DequantizeQ4_0")
    return _w(Q.q4_0_dequantize(packed.Tensor(), scale.Tensor(), int(count)))


def QuantizeQ8_0(m: OaMatrix) -> OaMatrix:
    """Q8_0 blocks of 34 bytes (fp16 scale + 32 int8)."""
    from ..ops import quant as Q
    _ctx_add("QuantizeQ8_0")
    return _w(Q.q8_0_quantize(m.Tensor()))


def DequantizeQ8_0(blocks: OaMatrix) -> OaMatrix:
    from ..ops import quant as Q
    _ctx_add("DequantizeQ8_0")
    return _w(Q.q8_0_dequantize(blocks.Tensor()))


def QuantizeInt8(m: OaMatrix, scale: OaMatrix) -> OaMatrix:
    from ..ops import quant as Q
    _ctx_add("QuantizeInt8")
    return _w(Q.int8_quantize(m.Tensor(), scale.Tensor()))


def DequantizeInt8(q: OaMatrix, scale: OaMatrix) -> OaMatrix:
    from ..ops import quant as Q
    _ctx_add("DequantizeInt8")
    return _w(Q.int8_dequantize(q.Tensor(), scale.Tensor()))


def VqAssign(ze: OaMatrix, codebook: OaMatrix):
    from ..ml.nn import vq as VQ
    return VQ.VqAssign(ze, codebook)


def VqEmaUpdate(ze, idx, embed_sum, cluster_size, codebook, decay: float, eps: float, dead_threshold: float, seed: int, normalize: bool) -> None:
    from ..ml.nn import vq as VQ
    VQ.VqEmaUpdate(ze, idx, embed_sum, cluster_size, codebook, decay, eps, dead_threshold, seed, normalize)


def SampleLogits(logits: OaMatrix, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0, seed: int = 0) -> OaMatrix:
    from ..ml.rl import fn_rl as FR
    return FR.SampleLogits(logits, temperature, top_k, top_p, seed)


# ======================================================================= channel-axis LayerNorm of [B, C, T] tensors
def _channel_norm_fwd(tx: torch.Tensor, tw: torch.Tensor, tb: Optional[torch.Tensor], B: int, C: int, L: int, eps: float, relu: bool):
    x3 = _c(tx).reshape(B, C, L)
    if not x3.is_cuda:
        xf = x3.float()
        mean = xf.mean(1)
        rstd = torch.rsqrt(xf.var(1, unbiased=False) + eps)
        y = (xf - mean[:, None]) * rstd[:, None] * tw.float().reshape(1, C, 1) + (tb.float().reshape(1, C, 1) if tb is not None else 0.0)
        if relu:
            y = torch.relu(y)
        return y.to(tx.dtype), mean.contiguous(), rstd.contiguous()
    y = torch.empty_like(x3)
    mean = torch.empty((B, L), dtype=torch.float32, device=x3.device)
    rstd = torch.empty((B, L), dtype=torch.float32, device=x3.device)
    K._launch(N.require().oa_channel_norm_fwd(K.dt(x3), x3.data_ptr(), _c(tw).data_ptr(), N.ptr(_c(tb) if tb is not None else None), y.data_ptr(),
                                              mean.data_ptr(), rstd.data_ptr(), B, C, L, float(eps), int(relu), N.stream()), "oa_channel_norm_fwd")
    return y, mean, rstd


def _channel_norm_bwd(tx, tw, tg, ty_relu, mean, rstd, B: int, C: int, L: int):
    x3, g3 = _c(tx).reshape(B, C, L), _c(tg).reshape(B, C, L)
    if not x3.is_cuda:
        gf = g3.float()
        if ty_relu is not None:
            gf = gf * (ty_relu.reshape(B, C, L).float() > 0)
        xhat = (x3.float() - mean[:, None]) * rstd[:, None]
        gw = gf * tw.float().reshape(1, C, 1)
        dx = rstd[:, None] * (gw - gw.mean(1, keepdim=True) - xhat * (gw * xhat).mean(1, keepdim=True))
        return dx.to(tx.dtype), (gf * xhat).sum((0, 2)), gf.sum((0, 2))
    dx = torch.empty_like(x3)
    dw = torch.empty(C, dtype=torch.float32, device=x3.device)
    db = torch.empty(C, dtype=torch.float32, device=x3.device)
    yr = _c(ty_relu).reshape(B, C, L) if ty_relu is not None else None
    K._launch(N.require().oa_channel_norm_bwd(K.dt(x3), x3.data_ptr(), _c(tw).data_ptr(), g3.data_ptr(), N.ptr(yr), mean.data_ptr(), rstd.data_ptr(),
                                              dx.data_ptr(), dw.data_ptr(), db.data_ptr(), B, C, L, N.stream()), "oa_channel_norm_bwd", 2)
    return dx, dw, db


def _channel_norm(name: str, x: OaMatrix, w: OaMatrix, b: Optional[OaMatrix], B: int, C: int, L: int, eps: float, relu: bool) -> OaMatrix:
    _ctx_add(name)
    tx, tw = x.Tensor(), w.Tensor()
    if tx.numel() != B * C * L or tw.numel() != C:
        raise ValueError(f"{name}: x has {tx.numel()} elements, expected {B}x{C}x{L}; weight has {tw.numel()}, expected {C}")
    y, mean, rstd = _channel_norm_fwd(tx, tw, b.Tensor() if b is not None else None, B, C, L, eps, relu)
    out = _w(y.reshape(tx.shape))

    def back(g):
        dx, dw, db = _channel_norm_bwd(tx, tw, g, y if relu else None, mean, rstd, B, C, L)
        return (dx.reshape(tx.shape), dw.to(tw.dtype).reshape(tw.shape), db.to(tw.dtype).reshape(b.Tensor().shape) if b is not None else None)

    return AG.attach(name, out, [x, w, b], back)


def ChannelNorm(x: OaMatrix, w: OaMatrix, b: Optional[OaMatrix], batch: int, channels: int, seq_len: int, eps: float = 1e-5) -> OaMatrix:
    """LayerNorm over the channel axis of [B, C, T] in one kernel, no transposes (Source/Public/Oa/Ml/FnMatrix.h:544-550)."""
    return _channel_norm("ChannelNorm", x, w, b, batch, channels, seq_len, eps, False)


def ChannelNormRelu(x: OaMatrix, w: OaMatrix, b: Optional[OaMatrix], batch: int, channels: int, seq_len: int, eps: float = 1e-5) -> OaMatrix:
    """ChannelNorm with the ReLU applied in the same kernel (Source/Public/Oa/Ml/FnMatrix.h:556-561)."""
    return _channel_norm("ChannelNormRelu", x, w, b, batch, channels, seq_len, eps, True)


def ChannelNormBwd(x: OaMatrix, w: OaMatrix, grad_out: OaMatrix, batch: int, channels: int, seq_len: int, eps: float = 1e-5):
    """Explicit backward: returns (DX, DWeight, DBias) (Source/Public/Oa/Ml/FnMatrix.h:552-555)."""
    tx, tw = x.Tensor(), w.Tensor()
    _, mean, rstd = _channel_norm_fwd(tx, tw, None, batch, channels, seq_len, eps, False)
    dx, dw, db = _channel_norm_bwd(tx, tw, grad_out.Tensor(), None, mean, rstd, batch, channels, seq_len)
    return _w(dx.reshape(tx.shape)), _w(dw.to(tw.dtype)), _w(db.to(tw.dtype))


def ChannelNormReluBwd(x: OaMatrix, w: OaMatrix, fwd_out: OaMatrix, grad_out: OaMatrix, batch: int, channels: int, seq_len: int, eps: float = 1e-5):
    tx, tw = x.Tensor(), w.Tensor()
    _, mean, rstd = _channel_norm_fwd(tx, tw, None, batch, channels, seq_len, eps, False)
    dx, dw, db = _channel_norm_bwd(tx, tw, grad_out.Tensor(), fwd_out.Tensor(), mean, rstd, batch, channels, seq_len)
    return _w(dx.reshape(tx.shape)), _w(dw.to(tw.dtype)), _w(db.to(tw.dtype))


# ======================================================================= 1-D convolution as im2col + one GEMM
def Im2Col1d(x: OaMatrix, k: int, stride: int, padding: int, dilation: int = 1) -> OaMatrix:
    """[N, InC, L] -> [N*OutL, InC*K] (row = n*OutL + ol, column = ic*K + k); differentiable, backward = Col2Im1d
    (Source/Public/Oa/Ml/FnMatrix.h:588-593)."""
    from ..ml.nn import conv as CV
    n, c, l = x.Tensor().shape
    return CV.Im2Col(x.Reshape([n, c, 1, l]), (1, k), (1, stride), (0, padding), (1, dilation))


def Col2Im1d(dcols: OaMatrix, n: int, c: int, l: int, k: int, stride: int, padding: int, dilation: int, out_l: int) -> OaMatrix:
    """Adjoint of Im2Col1d: [N*OutL, InC*K] -> [N, InC, L], overlapping windows accumulate (Source/Public/Oa/Ml/FnMatrix.h:595-600)."""
    from ..ml.nn import conv as CV
    from ..ops import conv as CO
    if CO.out_size(l, k, stride, padding, dilation) != out_l:
        raise ValueError("Col2Im1d: OutL does not match the convolution geometry")
    return CV.Col2Im(dcols, (n, c, 1, l), (1, k), (1, stride), (0, padding), (1, dilation)).Reshape([n, c, l])


def _conv1d_gemm(x: OaMatrix, w: OaMatrix, b: Optional[OaMatrix], stride: int, padding: int, dilation: int, relu: bool) -> OaMatrix:
    n, c, l = x.Tensor().shape
    o, _, k = w.Tensor().shape
    cols = Im2Col1d(x, k, stride, padding, dilation)
    y = Linear(cols, w.Reshape([o, c * k]), b, K.ACT_RELU if relu else K.ACT_NONE, "Conv1dReluGemm" if relu else "Conv1dGemm")
    return Permute(y.Reshape([n, cols.Size(0) // n, o]), [0, 2, 1])


def Conv1dGemm(x: OaMatrix, w: OaMatrix, b: Optional[OaMatrix], stride: int = 1, padding: int = 0, dilation: int = 1) -> OaMatrix:
    """x [N, InC, L], w [OutC, InC, K] -> [N, OutC, OutL]: im2col and one GEMM on the tensor cores (Source/Public/Oa/Ml/FnMatrix.h:571-580)."""
    return _conv1d_gemm(x, w, b, stride, padding, dilation, False)


def Conv1dReluGemm(x: OaMatrix, w: OaMatrix, b: Optional[OaMatrix], stride: int = 1, padding: int = 0, dilation: int = 1) -> OaMatrix:
    """Conv1dGemm with the ReLU in the GEMM epilogue (Source/Public/Oa/Ml/FnMatrix.h:582-586)."""
    return _conv1d_gemm(x, w, b, stride, padding, dilation, True)


# row compaction / scatter, accuracy counters, stochastic rounding, int8 product and the composite functions
from .fn_extra import (CategoricalAccuracyCount, CompactRows, CompactRowsBwd, CopyAtOffset, GemmInt8, GemmStrided, LinearDataReluBwd,  # noqa: E402,F401
                       LinearReluBwdData, LogSoftmaxBwd, MaskedCategoricalAccuracyCount, MaskedMse, MatrixCopyRegion, MaxBwd, MeanBwd,
                       OaCompactRowsResult, ReduceCols, ScatterAddRows, ScatterRows, ScatterRowsBwdSource, SmoothL1Mean, SrRoundBf16, SumDim,
                       TransposeBatched, VelSmoothL1)
