"""Raw-tensor entry points of the hot operations (no autograd here).

Each function takes `torch.Tensor`s.  CUDA tensors go to the hand-written sm_100a kernels through
`oa_b200._native`; CPU tensors run the plain fp32 PyTorch statement of the same math, which is both
the CPU execution path and the oracle the GPU tests compare against.  A CUDA tensor never falls back
to PyTorch math: a missing library or an unsupported shape raises.
"""
from __future__ import annotations

import math
import os
from typing import Optional

import torch

from .. import _native as N
from ..core import validation as V

C = N.CONST
ACT_NONE, ACT_GELU, ACT_RELU, ACT_SILU = C["OA_ACT_NONE"], C["OA_ACT_GELU"], C["OA_ACT_RELU"], C["OA_ACT_SILU"]
ACT_GELU_BWD, ACT_RELU_BWD = C["OA_ACT_GELU_BWD"], C["OA_ACT_RELU_BWD"]

_DT = {torch.float32: 0, torch.bfloat16: 1}


def dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise N.OaKernelError(f"unsupported dtype {t.dtype}") from None


# ---------------------------------------------------------------- per-device scratch and status
_status: dict[int, torch.Tensor] = {}
_workspace: dict[int, torch.Tensor] = {}
_scratch: dict[tuple, torch.Tensor] = {}
WORKSPACE_BYTES = 96 << 20


def status_word(device: torch.device) -> torch.Tensor:
    i = device.index if device.index is not None else torch.cuda.current_device()
    if i not in _status:
        _status[i] = torch.zeros(4, dtype=torch.int32, device=device)
    return _status[i]


def check_status(device: Optional[torch.device] = None) -> None:
    """Reads the kernels' error word (synchronises). Raises if a bounded wait ran out."""
    for i, t in list(_status.items()):
        if device is not None and device.index is not None and device.index != i:
            continue
        v = int(t[0].item())
        if v != 0:
            t.zero_()
            raise N.OaKernelError(f"a device-side wait ran out on cuda:{i} (kernel status {v})")


_STATUS_NAMES = {0: "none", 1: "wait for a TMA stage ran out", 2: "wait for a free stage ran out", 3: "wait for the accumulator ran out",
                 4: "wait for a free accumulator ran out", 5: "wait for a peer's flag ran out", 6: "wait for the softmax warps ran out",
                 7: "bad argument or index"}


def status_name(code: int) -> str:
    return _STATUS_NAMES.get(int(code), "unknown")


def peek_status(device: Optional[torch.device] = None) -> int:
    """The kernels' error word of the device (synchronises; does not clear it)."""
    for i, t in list(_status.items()):
        if device is not None and device.index is not None and device.index != i:
            continue
        v = int(t[0].item())
        if v != 0:
            return v
    return 0


def workspace(device: torch.device) -> torch.Tensor:
    i = device.index if device.index is not None else torch.cuda.current_device()
    if i not in _workspace:
        _workspace[i] = torch.empty(WORKSPACE_BYTES, dtype=torch.uint8, device=device)
    return _workspace[i]


def scratch(device: torch.device, nbytes: int, tag: str = "") -> torch.Tensor:
    """A persistent fp32 scratch buffer (grown on demand, keyed by tag) - stable across graph replays."""
    i = device.index if device.index is not None else torch.cuda.current_device()
    key = (i, tag)
    n = max(1, (nbytes + 3) // 4)
    cur = _scratch.get(key)
    if cur is None or cur.numel() < n:
        if torch.cuda.is_current_stream_capturing() and cur is not None:
            raise N.OaKernelError("scratch buffer would have to grow during graph capture")
        cur = torch.empty(n, dtype=torch.float32, device=device)
        _scratch[key] = cur
    return cur


def _launch(rc: int, what: str, n: int = 1, outputs=()) -> None:
    N.check(rc, what)
    N.count_launch(n)
    if V.OaValidation._enabled:
        V.AfterLaunch(what, outputs)


def _gelu_ref(x: torch.Tensor) -> torch.Tensor:
    return 0.5 * x * (1.0 + torch.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))


def _gelu_grad_ref(x: torch.Tensor) -> torch.Tensor:
    u = 0.7978845608028654 * (x + 0.044715 * x ** 3)
    t = torch.tanh(u)
    du = 0.7978845608028654 * (1.0 + 3 * 0.044715 * x * x)
    return 0.5 * (1 + t) + 0.5 * x * (1 - t * t) * du


# ---------------------------------------------------------------- GEMM
_gemm_planner = None      # (M, N, K, layout, epilogue, run(bn)) -> N tile; installed by runtime/gemm_tuner.py
# fp32 GEMMs on the tensor cores: 0 = off (exact fp32 FMA kernel), 2 = two bf16 parts per operand (3 products, ~2^-16 relative),
# 3 = three parts (6 products, fp32-grade).  OA_GEMM_F32_TENSOR sets the default; problems below _F32_TENSOR_MIN_FLOPS stay on
# the FMA kernel, where the launch latency of several tensor-core GEMMs would dominate.
_f32_tensor_terms = int(os.environ.get("OA_GEMM_F32_TENSOR", "0") or 0)
_F32_TENSOR_MIN_FLOPS = 1 << 28


def set_f32_tensor_terms(terms: int) -> None:
    global _f32_tensor_terms
    if terms not in (0, 2, 3):
        raise ValueError("fp32 tensor-core GEMM: 0 (off), 2 or 3 bf16 parts per operand")
    _f32_tensor_terms = int(terms)


def split_bf16(x: torch.Tensor, terms: int) -> torch.Tensor:
    """[terms, *x.shape] bf16 with x ~ sum of the parts (successive roundings of the remainder)."""
    x = x.contiguous()
    if not x.is_cuda:
        parts, r = [], x.float().clone()
        for _ in range(terms):
            h = r.bfloat16()
            parts.append(h)
            r = r - h.float()
        return torch.stack(parts)
    out = torch.empty((terms, *x.shape), dtype=torch.bfloat16, device=x.device)
    _launch(N.require().oa_split_bf16(x.data_ptr(), out.data_ptr(), x.numel(), terms, N.stream()), "oa_split_bf16")
    return out


def _gemm_f32_tensor(a, b, a_mn, b_mn, out, accumulate, alpha, terms) -> torch.Tensor:
    """out = alpha * A B^T in fp32 from bf16 products on the tensor cores: every pair of parts whose combined order is below
    `terms`, smallest contributions first, accumulated in the fp32 output."""
    pa, pb = split_bf16(a, terms), split_bf16(b, terms)
    pairs = sorted(((i, j) for i in range(terms) for j in range(terms) if i + j < terms), key=lambda p: -(p[0] + p[1]))
    for n, (i, j) in enumerate(pairs):
        gemm(pa[i], pb[j], a_mn=a_mn, b_mn=b_mn, out=out, accumulate=accumulate or n > 0, alpha=alpha)
    return out


def set_gemm_planner(fn) -> None:
    global _gemm_planner
    _gemm_planner = fn


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         bias: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None, act: int = ACT_NONE,
         aux_out: Optional[torch.Tensor] = None, aux_in: Optional[torch.Tensor] = None,
         out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None, accumulate: bool = False,
         alpha: float = 1.0, force_bn: int = 0) -> torch.Tensor:
    """out[M,N] = epilogue(alpha * A @ B^T) with A = a ([M,K]) or a^T (a is [K,M] when a_mn), B likewise.

    Epilogue order: + bias[N]; aux_out := value (pre-activation copy); act; * act'(aux_in) for the
    *_BWD modes; + residual[M,N]; + out when `accumulate`.
    """
    assert a.dim() == 2 and b.dim() == 2
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    Nn, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    if K != Kb:
        raise ValueError(f"gemm: reduction extents differ ({K} vs {Kb})")
    odt = out_dtype or (out.dtype if out is not None else a.dtype)
    if out is None:
        out = torch.empty((M, Nn), dtype=odt, device=a.device)
    if not a.is_cuda:
        A = (a.t() if a_mn else a).float()
        B = (b.t() if b_mn else b).float()
        v = alpha * (A @ B.t())
        if bias is not None:
            v = v + bias.float()
        if aux_out is not None:
            aux_out.copy_(v)
        if act == ACT_GELU:
            v = _gelu_ref(v)
        elif act == ACT_RELU:
            v = torch.relu(v)
        elif act == ACT_SILU:
            v = v * torch.sigmoid(v)
        elif act == ACT_GELU_BWD:
            v = v * _gelu_grad_ref(aux_in.float())
        elif act == ACT_RELU_BWD:
            v = v * (aux_in.float() > 0)
        if residual is not None:
            v = v + residual.float()
        if accumulate:
            v = v + out.float()
        out.copy_(v)
        return out
    lib = N.require()
    st = N.stream()
    if a.dtype == torch.bfloat16:
        assert b.dtype == torch.bfloat16
        assert a.stride(1) == 1 and b.stride(1) == 1 and out.stride(1) == 1
        ws = workspace(a.device)
        status = status_word(a.device)
        plain = bias is None and residual is None and aux_out is None and aux_in is None and act == ACT_NONE
        if V.OaValidation._enabled:
            for nm, t in (("gemm.a", a), ("gemm.b", b), ("gemm.out", out), ("gemm.residual", residual), ("gemm.aux_out", aux_out),
                          ("gemm.aux_in", aux_in)):
                V.ValidateTensor(nm, t, cuda=True, contiguous=False, align=16)
                if t is not None:      # TMA wants rows that start on 16-byte boundaries
                    V.OA_VALIDATE(t.stride(0) * t.element_size() % 16 == 0, V.OaValidationSeverity.Error, "Kernel",
                                  "%s: row pitch %d bytes is not a multiple of 16", nm, t.stride(0) * t.element_size())
            V.ValidateTensor("gemm.bias", bias, dtype=torch.bfloat16, cuda=True)
            V.OA_VALIDATE(Nn % 8 == 0 and K % 8 == 0, V.OaValidationSeverity.Error, "Kernel", "gemm: N=%d and K=%d must be multiples of 8", Nn, K)
            if force_bn == 0 and (M < 128 or Nn < 128):
                V.OaValidation.Report(V.OaValidationSeverity.Info, "Kernel", "gemm M=%d N=%d K=%d: tile larger than the problem", M, Nn, K)
        def launch(bn: int) -> int:
            return lib.oa_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, Nn, K, a.stride(0), b.stride(0),
                                    out.stride(0), int(a_mn), int(b_mn), N.ptr(bias), N.ptr(residual),
                                    residual.stride(0) if residual is not None else 0, N.ptr(aux_out), N.ptr(aux_in),
                                    (aux_out.stride(0) if aux_out is not None else (aux_in.stride(0) if aux_in is not None else 0)),
                                    act, int(out.dtype == torch.float32), int(accumulate), float(alpha),
                                    ws.data_ptr() if plain else None, ws.numel() if plain else 0, bn,
                                    status.data_ptr(), st)

        if _gemm_planner is not None and force_bn == 0 and not accumulate:
            # timing runs repeat the launch on the caller's operands, which is only harmless when the GEMM does not read `out`
            layout = int(a_mn) | (int(b_mn) << 1)
            epi = (act & 7) | (8 if bias is not None else 0) | (16 if residual is not None else 0) | (32 if aux_out is not None else 0) | \
                (64 if aux_in is not None else 0) | (128 if out.dtype == torch.float32 else 0)
            force_bn = _gemm_planner(M, Nn, K, layout, epi, lambda bn: N.check(launch(bn), "oa_gemm_bf16(tuning)"))
        rc = launch(force_bn)
        _launch(rc, f"oa_gemm_bf16 M={M} N={Nn} K={K}", outputs=(out,))
        return out
    if a.dtype == torch.float32:
        assert b.dtype == torch.float32 and out.dtype == torch.float32
        if (_f32_tensor_terms and 2.0 * M * Nn * K >= _F32_TENSOR_MIN_FLOPS and a.is_contiguous() and b.is_contiguous() and out.is_contiguous()
                and M % 8 == 0 and Nn % 8 == 0 and K % 8 == 0 and act == ACT_NONE and bias is None and residual is None and aux_out is None
                and aux_in is None):
            return _gemm_f32_tensor(a, b, a_mn, b_mn, out, accumulate, alpha, _f32_tensor_terms)
        if act in (ACT_GELU_BWD, ACT_RELU_BWD) or residual is not None or aux_out is not None:
            # composed from the plain product for the exact-fp32 path
            v = gemm(a, b, a_mn=a_mn, b_mn=b_mn, bias=bias, alpha=alpha)
            if aux_out is not None:
                aux_out.copy_(v)
            if act in (ACT_GELU, ACT_RELU, ACT_SILU):
                v = unary({ACT_GELU: "gelu", ACT_RELU: "relu", ACT_SILU: "silu"}[act], v)
            if act == ACT_GELU_BWD:
                v = binary("gelu_bwd", aux_in, v)
            elif act == ACT_RELU_BWD:
                v = binary("relu_bwd", aux_in, v)
            if residual is not None:
                v = binary("add", v, residual)
            if accumulate:
                v = binary("add", v, out)
            out.copy_(v)
            return out
        sam, sak = (a.stride(1), a.stride(0)) if a_mn else (a.stride(0), a.stride(1))
        sbn, sbk = (b.stride(1), b.stride(0)) if b_mn else (b.stride(0), b.stride(1))
        rc = lib.oa_gemm_f32(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, Nn, K, sam, sak, sbn, sbk, out.stride(0),
                             1, 0, 0, 0, N.ptr(bias), act, int(accumulate), float(alpha), st)
        _launch(rc, "oa_gemm_f32")
        return out
    raise N.OaKernelError(f"gemm: unsupported dtype {a.dtype}")


def bgemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False, out: Optional[torch.Tensor] = None,
          out_dtype: Optional[torch.dtype] = None, accumulate: bool = False, alpha: float = 1.0,
          residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Batched bf16 GEMM on the tensor cores: out[n] = alpha * A[n] @ B[n]^T (+ residual[n]) (+ out[n]).
    a is [n, M, K] (or [n, K, M] when a_mn), b is [n, N, K] (or [n, K, N] when b_mn); the last dimension of every
    operand must be contiguous, the batch and row strides are free."""
    nb = a.shape[0]
    M, Kd = (a.shape[2], a.shape[1]) if a_mn else (a.shape[1], a.shape[2])
    Nn, Kb = (b.shape[2], b.shape[1]) if b_mn else (b.shape[1], b.shape[2])
    assert Kd == Kb and b.shape[0] == nb
    odt = out_dtype or (out.dtype if out is not None else a.dtype)
    if out is None:
        out = torch.empty((nb, M, Nn), dtype=odt, device=a.device)
    if not a.is_cuda:
        A = (a.transpose(1, 2) if a_mn else a).float()
        B = (b.transpose(1, 2) if b_mn else b).float()
        v = alpha * torch.bmm(A, B.transpose(1, 2))
        if residual is not None:
            v = v + residual.float()
        if accumulate:
            v = v + out.float()
        out.copy_(v)
        return out
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a.stride(2) == 1 and b.stride(2) == 1 and out.stride(2) == 1
    lib = N.require()
    ws = workspace(a.device)
    plain = residual is None
    rc = lib.oa_gemm_bf16_batched(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, Nn, Kd, a.stride(1), b.stride(1), out.stride(1),
                                  int(a_mn), int(b_mn), None, N.ptr(residual), residual.stride(1) if residual is not None else 0,
                                  None, None, 0, ACT_NONE, int(out.dtype == torch.float32), int(accumulate), float(alpha),
                                  ws.data_ptr() if plain else None, ws.numel() if plain else 0, 0, nb, a.stride(0), b.stride(0),
                                  out.stride(0), residual.stride(0) if residual is not None else 0, 0, 0,
                                  status_word(a.device).data_ptr(), N.stream())
    _launch(rc, f"oa_gemm_bf16_batched n={nb} M={M} N={Nn} K={Kd}")
    return out


def bmm_f32(a: torch.Tensor, b: torch.Tensor, *, b_mn: bool = False, alpha: float = 1.0) -> torch.Tensor:
    """Batched fp32 product out[n] = a[n] @ (b[n] if b_mn else b[n]^T); a [B,M,K], b [B,N,K] or [B,K,N]."""
    Bn, M, K = a.shape
    Nn = b.shape[2] if b_mn else b.shape[1]
    if not a.is_cuda:
        bb = b if b_mn else b.transpose(1, 2)
        return (alpha * torch.bmm(a.float(), bb.float())).to(a.dtype)
    a = a.contiguous()
    b = b.contiguous()
    out = torch.empty((Bn, M, Nn), dtype=torch.float32, device=a.device)
    sbn, sbk = (1, b.stride(1)) if b_mn else (b.stride(1), 1)
    rc = N.require().oa_gemm_f32(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, Nn, K, a.stride(1), 1, sbn, sbk, Nn, Bn,
                                 a.stride(0), b.stride(0), out.stride(0), None, ACT_NONE, 0, float(alpha), N.stream())
    _launch(rc, "oa_gemm_f32(batched)")
    return out


# ---------------------------------------------------------------- elementwise
_U = {k[5:].lower(): v for k, v in C.items() if k.startswith("OA_U_") and k != "OA_U_COUNT"}
_B = {k[5:].lower(): v for k, v in C.items() if k.startswith("OA_B_") and k != "OA_B_COUNT"}
BC_NONE, BC_ROW, BC_COL, BC_SCALAR = C["OA_BC_NONE"], C["OA_BC_ROW"], C["OA_BC_COL"], C["OA_BC_SCALAR"]


def _softplus(x):
    return torch.nn.functional.softplus(x)


_U_REF = {
    "copy": lambda x, s0: x.clone(), "neg": lambda x, s0: -x, "abs": lambda x, s0: x.abs(), "log": lambda x, s0: x.log(),
    "exp": lambda x, s0: x.exp(), "sqrt": lambda x, s0: x.sqrt(), "sin": lambda x, s0: x.sin(), "cos": lambda x, s0: x.cos(),
    "recip": lambda x, s0: 1.0 / x, "scale": lambda x, s0: x * s0, "add_scalar": lambda x, s0: x + s0,
    "pow": lambda x, s0: x.pow(s0), "clamp_max": lambda x, s0: x.clamp(max=s0), "clamp_min": lambda x, s0: x.clamp(min=s0),
    "relu": lambda x, s0: x.relu(), "gelu": lambda x, s0: _gelu_ref(x), "silu": lambda x, s0: x * torch.sigmoid(x),
    "tanh": lambda x, s0: x.tanh(), "sigmoid": lambda x, s0: x.sigmoid(), "softplus": lambda x, s0: _softplus(x),
    "leaky_relu": lambda x, s0: torch.where(x > 0, x, s0 * x), "elu": lambda x, s0: torch.where(x > 0, x, s0 * (x.exp() - 1)),
    "mish": lambda x, s0: x * torch.tanh(_softplus(x)), "square": lambda x, s0: x * x, "rsub_scalar": lambda x, s0: s0 - x,
    "sign": lambda x, s0: torch.sign(x),
}


def _mish_bwd(a, b):
    sp = _softplus(a)
    t = torch.tanh(sp)
    return b * (t + a * (1 - t * t) * torch.sigmoid(a))


_B_REF = {
    "add": lambda a, b: a + b, "sub": lambda a, b: a - b, "mul": lambda a, b: a * b, "div": lambda a, b: a / b,
    "max": torch.maximum, "min": torch.minimum, "eq": lambda a, b: (a == b).float(), "ge": lambda a, b: (a >= b).float(),
    "relu_bwd": lambda a, b: b * (a > 0), "gelu_bwd": lambda a, b: b * _gelu_grad_ref(a),
    "silu_bwd": lambda a, b: b * torch.sigmoid(a) * (1 + a * (1 - torch.sigmoid(a))),
    "tanh_bwd": lambda a, b: b * (1 - a * a), "sigmoid_bwd": lambda a, b: b * a * (1 - a),
    "softplus_bwd": lambda a, b: b * torch.sigmoid(a), "leaky_relu_bwd": lambda a, b: torch.where(a > 0, b, 0.01 * b),
    "elu_bwd": lambda a, b: torch.where(a > 0, b, b * a.exp()), "mish_bwd": _mish_bwd,
    "abs_bwd": lambda a, b: b * torch.sign(a), "log_bwd": lambda a, b: b / a, "sqrt_bwd": lambda a, b: b * 0.5 / a,
    "recip_bwd": lambda a, b: -b * a * a, "silu_mul": lambda a, b: a * torch.sigmoid(a) * b,
}


def unary(op: str, x: torch.Tensor, s0: float = 0.0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    x = x.contiguous()
    if out is None:
        out = torch.empty_like(x)
    if not x.is_cuda:
        out.copy_(_U_REF[op](x.float(), s0))
        return out
    _launch(N.require().oa_unary(_U[op], dt(x), x.data_ptr(), out.data_ptr(), x.numel(), float(s0), 0.0, N.stream()),
            f"oa_unary({op})")
    return out


def binary(op: str, a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = op(a, b); b may be the same shape, a trailing-dimension vector, a per-row column or a scalar tensor."""
    a = a.contiguous()
    b = b.contiguous()
    mode, inner = BC_NONE, 1
    if b.shape != a.shape:
        if b.numel() == 1:
            mode = BC_SCALAR
        elif b.numel() == a.shape[-1] and (b.dim() == 1 or all(d == 1 for d in b.shape[:-1])):
            mode, inner = BC_ROW, a.shape[-1]
        elif a.dim() >= 1 and b.numel() == a.numel() // a.shape[-1] and (b.dim() == a.dim() and b.shape[-1] == 1):
            mode, inner = BC_COL, a.shape[-1]
        else:
            raise ValueError(f"binary({op}): cannot broadcast {tuple(b.shape)} to {tuple(a.shape)}")
    if out is None:
        out = torch.empty_like(a)
    if not a.is_cuda:
        out.copy_(_B_REF[op](a.float(), b.float() if mode != BC_ROW else b.float().reshape(-1)))
        return out
    assert a.dtype == b.dtype
    _launch(N.require().oa_binary(_B[op], dt(a), a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), inner, mode,
                                  N.stream()), f"oa_binary({op})")
    return out


def cast(x: torch.Tensor, dtype: torch.dtype, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    x = x.contiguous()
    if out is None:
        out = torch.empty(x.shape, dtype=dtype, device=x.device)
    if not x.is_cuda or x.dtype not in _DT or dtype not in _DT:
        out.copy_(x)
        return out
    _launch(N.require().oa_cast(dt(x), _DT[dtype], x.data_ptr(), out.data_ptr(), x.numel(), N.stream()), "oa_cast")
    return out


def fill_(x: torch.Tensor, value: float) -> torch.Tensor:
    if not x.is_cuda or x.dtype not in _DT or not x.is_contiguous():
        x.fill_(value)
        return x
    _launch(N.require().oa_fill(dt(x), x.data_ptr(), x.numel(), float(value), N.stream()), "oa_fill")
    return x


def contiguous(x: torch.Tensor) -> torch.Tensor:
    """Materialises a strided view (permute / slice / transpose) into a new contiguous tensor."""
    if x.is_contiguous():
        return x
    if not x.is_cuda or (x.dtype not in _DT and x.dtype != torch.int32) or x.dim() > 8:
        return x.contiguous()
    out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    import ctypes
    shape = (ctypes.c_longlong * x.dim())(*x.shape)
    strides = (ctypes.c_longlong * x.dim())(*x.stride())
    code = 4 if x.dtype == torch.int32 else dt(x)
    _launch(N.require().oa_copy_strided(code, x.data_ptr(), out.data_ptr(), x.dim(), ctypes.addressof(shape),
                                        ctypes.addressof(strides), N.stream()), "oa_copy_strided")
    return out


def swiglu_fwd(gate_up: torch.Tensor) -> torch.Tensor:
    rows, F2 = gate_up.shape
    F = F2 // 2
    out = torch.empty((rows, F), dtype=gate_up.dtype, device=gate_up.device)
    if not gate_up.is_cuda:
        g, u = gate_up.float()[:, :F], gate_up.float()[:, F:]
        out.copy_(g * torch.sigmoid(g) * u)
        return out
    _launch(N.require().oa_swiglu_fwd(dt(gate_up), gate_up.data_ptr(), out.data_ptr(), rows, F, N.stream()), "oa_swiglu_fwd")
    return out


def swiglu_bwd(gate_up: torch.Tensor, dout: torch.Tensor) -> torch.Tensor:
    rows, F2 = gate_up.shape
    F = F2 // 2
    dgu = torch.empty_like(gate_up)
    if not gate_up.is_cuda:
        g, u, d = gate_up.float()[:, :F], gate_up.float()[:, F:], dout.float()
        s = torch.sigmoid(g)
        dgu[:, :F] = d * u * s * (1 + g * (1 - s))
        dgu[:, F:] = d * g * s
        return dgu
    _launch(N.require().oa_swiglu_bwd(dt(gate_up), gate_up.data_ptr(), dout.contiguous().data_ptr(), dgu.data_ptr(), rows, F,
                                      N.stream()), "oa_swiglu_bwd")
    return dgu


def rope_(x: torch.Tensor, n_heads: int, head_dim: int, seq_len: int, *, pos_offset: int = 0, theta: float = 10000.0,
          backward: bool = False, pos_dev: Optional[torch.Tensor] = None) -> torch.Tensor:
    """In-place rotate-half RoPE on a [rows, >= n_heads*head_dim] view (row stride may exceed the width).  `pos_dev`
    (int32 [1] on the device) is added to pos_offset inside the kernel: decode steps replayed from a CUDA graph."""
    rows = x.shape[0]
    if not x.is_cuda:
        if pos_dev is not None:
            pos_offset += int(pos_dev.item())
        half = head_dim // 2
        pos = (torch.arange(rows) % seq_len + pos_offset).float()
        freq = theta ** (-2.0 * torch.arange(half).float() / head_dim)
        ang = pos[:, None] * freq[None, :]
        c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
        if backward:
            s = -s
        v = x[:, : n_heads * head_dim].float().reshape(rows, n_heads, head_dim)
        a, b = v[..., :half].clone(), v[..., half:].clone()
        v[..., :half] = a * c - b * s
        v[..., half:] = b * c + a * s
        x[:, : n_heads * head_dim] = v.reshape(rows, n_heads * head_dim).to(x.dtype)
        return x
    assert x.stride(1) == 1
    _launch(N.require().oa_rope(dt(x), x.data_ptr(), rows, x.stride(0), n_heads, head_dim, seq_len, pos_offset, float(theta),
                                int(backward), N.ptr(pos_dev), N.stream()), "oa_rope")
    return x


def embedding_fwd(table: torch.Tensor, ids: torch.Tensor, pos_table: Optional[torch.Tensor] = None, seq_len: int = 0):
    n = ids.numel()
    dim = table.shape[1]
    out = torch.empty((n, dim), dtype=table.dtype, device=table.device)
    if not table.is_cuda:
        idx = ids.reshape(-1).long()
        bad = (idx < 0) | (idx >= table.shape[0])
        v = table.float()[idx.clamp(0, table.shape[0] - 1)]
        v[bad] = float("nan")
        if pos_table is not None:
            v = v + pos_table.float()[torch.arange(n) % seq_len]
        out.copy_(v)
        return out
    ids = ids.reshape(-1).to(torch.int32).contiguous()
    _launch(N.require().oa_embedding_fwd(dt(table), table.data_ptr(), ids.data_ptr(), out.data_ptr(), n, dim, table.shape[0],
                                         N.ptr(pos_table), seq_len, N.stream()), "oa_embedding_fwd")
    return out


def embedding_bwd(dout: torch.Tensor, ids: torch.Tensor, vocab: int, dtable_f32: Optional[torch.Tensor] = None):
    """Scatter-adds dout rows into a fp32 table gradient (created zeroed when not given)."""
    n, dim = dout.shape
    if dtable_f32 is None:
        dtable_f32 = torch.zeros((vocab, dim), dtype=torch.float32, device=dout.device)
    if not dout.is_cuda:
        idx = ids.reshape(-1).long()
        ok = (idx >= 0) & (idx < vocab)
        dtable_f32.index_add_(0, idx[ok], dout.float()[ok])
        return dtable_f32
    ids = ids.reshape(-1).to(torch.int32).contiguous()
    _launch(N.require().oa_embedding_bwd(dt(dout), dout.contiguous().data_ptr(), ids.data_ptr(), dtable_f32.data_ptr(), n, dim,
                                         vocab, N.stream()), "oa_embedding_bwd")
    return dtable_f32


def col_sum(x: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
    rows, cols = x.shape
    if out is None:
        out = torch.empty(cols, dtype=x.dtype, device=x.device)
    if not x.is_cuda:
        s = x.float().sum(0)
        out.copy_(s + out.float() if accumulate else s)
        return out
    sc = scratch(x.device, ((rows + 255) // 256) * cols * 4, "colsum")
    _launch(N.require().oa_col_sum(dt(x), x.contiguous().data_ptr(), out.data_ptr(), dt(out), rows, cols, sc.data_ptr(),
                                   int(accumulate), N.stream()), "oa_col_sum", 2)
    return out


_R = {"sum": C["OA_R_SUM"], "mean": C["OA_R_MEAN"], "max": C["OA_R_MAX"], "argmax": C["OA_R_ARGMAX"]}


def row_reduce(op: str, x: torch.Tensor) -> torch.Tensor:
    """Reduces the last dimension of a 2-D tensor (sum / mean / max / argmax with ties to the lower index)."""
    rows, cols = x.shape
    odt = torch.int32 if op == "argmax" else x.dtype
    out = torch.empty(rows, dtype=odt, device=x.device)
    if not x.is_cuda:
        xf = x.float()
        out.copy_({"sum": lambda: xf.sum(1), "mean": lambda: xf.mean(1), "max": lambda: xf.max(1).values,
                   "argmax": lambda: xf.argmax(1)}[op]())
        return out
    _launch(N.require().oa_row_reduce(_R[op], dt(x), x.contiguous().data_ptr(), out.data_ptr(), rows, cols, N.stream()),
            f"oa_row_reduce({op})")
    return out


def softmax(x: torch.Tensor, *, log: bool = False, scale: float = 1.0, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Row softmax of x * scale + mask; the [mask_rows, cols] mask repeats every mask_rows rows of x."""
    rows, cols = x.shape
    out = torch.empty_like(x)
    mrows = mask.shape[0] if mask is not None else 0
    if mask is not None and (mask.shape[1] != cols or rows % mrows != 0):
        raise ValueError(f"softmax: mask {tuple(mask.shape)} does not tile scores {tuple(x.shape)}")
    if not x.is_cuda:
        v = x.float() * scale
        if mask is not None:
            v = (v.reshape(rows // mrows, mrows, cols) + mask.float()).reshape(rows, cols)
        out.copy_(torch.log_softmax(v, -1) if log else torch.softmax(v, -1))
        return out
    if mask is not None:
        mask = mask.contiguous() if mask.dtype == x.dtype else cast(mask.contiguous(), x.dtype)
    _launch(N.require().oa_softmax(dt(x), x.contiguous().data_ptr(), out.data_ptr(), rows, cols, int(log), float(scale),
                                   N.ptr(mask), mrows, N.stream()), "oa_softmax")
    return out


def softmax_bwd(y: torch.Tensor, dy: torch.Tensor, *, log: bool = False, scale: float = 1.0) -> torch.Tensor:
    rows, cols = y.shape
    dx = torch.empty_like(y)
    if not y.is_cuda:
        yf, df = y.float(), dy.float()
        if log:
            dx.copy_(scale * (df - yf.exp() * df.sum(-1, keepdim=True)))
        else:
            dx.copy_(scale * yf * (df - (df * yf).sum(-1, keepdim=True)))
        return dx
    _launch(N.require().oa_softmax_bwd(dt(y), y.contiguous().data_ptr(), dy.contiguous().data_ptr(), dx.data_ptr(), rows, cols,
                                       int(log), float(scale), N.stream()), "oa_softmax_bwd")
    return dx


def philox_(x: torch.Tensor, seed: int, offset: int, *, normal: bool, a: float, b: float,
            state: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Fills x with U[a,b) or N(a, b^2) from Philox4x32-10 (4 values per counter).  `state`: device int64[2] {seed, base
    offset}; when given the seed is read from it and `offset` counts from its base (replay-safe inside a captured step)."""
    if not x.is_cuda:
        g = torch.Generator().manual_seed((seed * 1000003 + offset) & 0x7FFFFFFFFFFFFFFF)
        if normal:
            x.copy_(torch.randn(x.shape, generator=g) * b + a)
        else:
            x.copy_(torch.rand(x.shape, generator=g) * (b - a) + a)
        return x
    _launch(N.require().oa_philox(dt(x), x.data_ptr(), x.numel(), seed, offset, int(normal), float(a), float(b), N.ptr(state),
                                  N.stream()), "oa_philox")
    return x


def philox_state_advance(state: torch.Tensor, delta: int) -> None:
    """state[1] += delta on the device (one thread): the last launch of a captured step that drew random numbers."""
    _launch(N.require().oa_philox_state_advance(state.data_ptr(), int(delta), N.stream()), "oa_philox_state_advance")


def dropout(x: torch.Tensor, p: float, seed: int, offset: int, state: Optional[torch.Tensor] = None) -> torch.Tensor:
    out = torch.empty_like(x)
    if not x.is_cuda:
        g = torch.Generator().manual_seed((seed * 1000003 + offset) & 0x7FFFFFFFFFFFFFFF)
        keep = (torch.rand(x.shape, generator=g) >= p).float() / (1 - p)
        out.copy_(x.float() * keep)
        return out
    _launch(N.require().oa_dropout(dt(x), x.contiguous().data_ptr(), out.data_ptr(), x.numel(), float(p), seed, offset,
                                   N.ptr(state), N.stream()), "oa_dropout")
    return out


# ---------------------------------------------------------------- norms
def rmsnorm_fwd(x, w, eps, residual=None):
    """Returns (y, rstd, residual_out).  With `residual`, normalises x + residual and also returns that sum."""
    rows, cols = x.shape
    y = torch.empty_like(x)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    res_out = torch.empty_like(x) if residual is not None else None
    if not x.is_cuda:
        xf = x.float() + (residual.float() if residual is not None else 0)
        if res_out is not None:
            res_out.copy_(xf)
            xf = res_out.float()
        r = torch.rsqrt(xf.pow(2).mean(-1) + eps)
        rstd.copy_(r)
        y.copy_(xf * r[:, None] * w.float())
        return y, rstd, res_out
    _launch(N.require().oa_rmsnorm_fwd(dt(x), x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(), rows, cols, float(eps),
                                       N.ptr(residual), N.ptr(res_out), N.stream()), "oa_rmsnorm_fwd")
    return y, rstd, res_out


def rmsnorm_bwd(x, w, dy, rstd, *, dres=None, dw_out=None, accumulate_dw=False):
    """Returns (dx, dw). dx includes `dres` (gradient arriving through a residual branch) when given."""
    rows, cols = x.shape
    dx = torch.empty_like(x)
    dw = dw_out if dw_out is not None else torch.empty(cols, dtype=w.dtype, device=x.device)
    if not x.is_cuda:
        xf, df, wf = x.float(), dy.float(), w.float()
        xh = xf * rstd[:, None]
        g = df * wf
        d = rstd[:, None] * (g - xh * (g * xh).mean(-1, keepdim=True))
        if dres is not None:
            d = d + dres.float()
        dx.copy_(d)
        s = (df * xh).sum(0)
        dw.copy_(s + dw.float() if accumulate_dw else s)
        return dx, dw
    sc = scratch(x.device, N.require().oa_norm_bwd_scratch_bytes(rows, cols), "norm")
    _launch(N.require().oa_rmsnorm_bwd(dt(x), x.data_ptr(), w.data_ptr(), dy.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                       dw.data_ptr(), dt(dw), rows, cols, N.ptr(dres), sc.data_ptr(), int(accumulate_dw),
                                       N.stream()), "oa_rmsnorm_bwd", 2)
    return dx, dw


def layernorm_fwd(x, w, b, eps):
    rows, cols = x.shape
    y = torch.empty_like(x)
    mean = torch.empty(rows, dtype=torch.float32, device=x.device)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    if not x.is_cuda:
        xf = x.float()
        m = xf.mean(-1)
        r = torch.rsqrt(xf.var(-1, unbiased=False) + eps)
        mean.copy_(m)
        rstd.copy_(r)
        v = (xf - m[:, None]) * r[:, None] * w.float()
        if b is not None:
            v = v + b.float()
        y.copy_(v)
        return y, mean, rstd
    _launch(N.require().oa_layernorm_fwd(dt(x), x.data_ptr(), w.data_ptr(), N.ptr(b), y.data_ptr(), mean.data_ptr(),
                                         rstd.data_ptr(), rows, cols, float(eps), N.stream()), "oa_layernorm_fwd")
    return y, mean, rstd


def layernorm_bwd(x, w, dy, mean, rstd, *, dw_out=None, db_out=None, accumulate=False, want_bias=True):
    rows, cols = x.shape
    dx = torch.empty_like(x)
    dw = dw_out if dw_out is not None else torch.empty(cols, dtype=w.dtype, device=x.device)
    db = db_out if db_out is not None else (torch.empty(cols, dtype=w.dtype, device=x.device) if want_bias else None)
    if not x.is_cuda:
        xf, df, wf = x.float(), dy.float(), w.float()
        xh = (xf - mean[:, None]) * rstd[:, None]
        g = df * wf
        dx.copy_(rstd[:, None] * (g - g.mean(-1, keepdim=True) - xh * (g * xh).mean(-1, keepdim=True)))
        s = (df * xh).sum(0)
        dw.copy_(s + dw.float() if accumulate else s)
        if db is not None:
            sb = df.sum(0)
            db.copy_(sb + db.float() if accumulate else sb)
        return dx, dw, db
    sc = scratch(x.device, N.require().oa_norm_bwd_scratch_bytes(rows, cols), "norm")
    _launch(N.require().oa_layernorm_bwd(dt(x), x.data_ptr(), w.data_ptr(), dy.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                         dx.data_ptr(), dw.data_ptr(), N.ptr(db), dt(dw), rows, cols, sc.data_ptr(),
                                         int(accumulate), N.stream()), "oa_layernorm_bwd", 3)
    return dx, dw, db


# ---------------------------------------------------------------- loss
def xent_fwd_bwd(logits: torch.Tensor, targets: torch.Tensor, *, grad_scale: Optional[float] = None,
                 dlogits: Optional[torch.Tensor] = None, ignore_index: int = -100):
    """Per-row loss (fp32) and, when grad_scale is given, dlogits = (softmax - onehot) * grad_scale.

    `dlogits` may be the logits tensor itself (in-place gradient).
    """
    rows, vocab = logits.shape
    row_loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
    want = grad_scale is not None
    if want and dlogits is None:
        dlogits = torch.empty_like(logits)
    if not logits.is_cuda:
        lf = logits.float()
        t = targets.reshape(-1).long()
        ign = t == ignore_index
        oor = (~ign) & ((t < 0) | (t >= vocab))
        tc = t.clamp(0, vocab - 1)
        lse = torch.logsumexp(lf, -1)
        loss = lse - lf.gather(1, tc[:, None])[:, 0]
        loss = torch.where(ign, torch.zeros_like(loss), loss)
        loss = torch.where(oor, torch.full_like(loss, float("nan")), loss)
        row_loss.copy_(loss)
        if want:
            g = torch.softmax(lf, -1)
            onehot = torch.zeros_like(g)
            valid = ~(ign | oor)
            onehot[valid, tc[valid]] = 1.0
            g = (g - onehot) * grad_scale
            g[ign] = 0
            dlogits.copy_(g)
        return row_loss, dlogits
    assert logits.stride(1) == 1
    tg = targets.reshape(-1).to(torch.int32).contiguous()
    _launch(N.require().oa_xent_fwd_bwd(dt(logits), logits.data_ptr(), tg.data_ptr(), row_loss.data_ptr(),
                                        dlogits.data_ptr() if want else None, rows, vocab, logits.stride(0),
                                        float(grad_scale or 0.0), ignore_index, N.stream()), "oa_xent_fwd_bwd")
    return row_loss, dlogits


def mean_f32(x: torch.Tensor, scale: Optional[float] = None) -> torch.Tensor:
    n = x.numel()
    s = (1.0 / n) if scale is None else scale
    out = torch.empty(1, dtype=torch.float32, device=x.device)
    if not x.is_cuda:
        out[0] = x.float().sum() * s
        return out
    _launch(N.require().oa_mean_f32(x.data_ptr(), out.data_ptr(), n, float(s), N.stream()), "oa_mean_f32")
    return out


# ---------------------------------------------------------------- optimizers
def optim_advance(state: torch.Tensor) -> None:
    if not state.is_cuda:
        state[0] += 1
        return
    _launch(N.require().oa_optim_advance(state.data_ptr(), N.stream()), "oa_optim_advance")


def adam_step(param, grad, master, m, v, state, *, decoupled: bool, inv_clip: Optional[torch.Tensor] = None) -> None:
    """One Adam/AdamW step over flat tensors. `state` = float[8] {step, lr, b1, b2, eps, wd, grad_scale, _}."""
    n = param.numel()
    if not param.is_cuda:
        step, lr, b1, b2, eps, wd, gs = [float(state[i]) for i in range(7)]
        g = grad.float().reshape(-1) * gs * (float(inv_clip[0]) if inv_clip is not None else 1.0)
        w = (master if master is not None else param).float().reshape(-1).clone()
        if decoupled:
            w = w - lr * wd * w
        else:
            g = g + wd * w
        m.mul_(b1).add_(g, alpha=1 - b1)
        v.mul_(b2).addcmul_(g, g, value=1 - b2)
        mh = m / (1 - b1 ** step)
        vh = v / (1 - b2 ** step)
        w = w - lr * mh / (vh.sqrt() + eps)
        if master is not None:
            master.copy_(w.reshape(master.shape))
        param.copy_(w.reshape(param.shape))
        return
    _launch(N.require().oa_adamw(dt(param), dt(grad), param.data_ptr(), grad.data_ptr(), N.ptr(master), m.data_ptr(),
                                 v.data_ptr(), n, state.data_ptr(), int(decoupled), N.ptr(inv_clip), N.stream()), "oa_adamw")


def sgd_step(param, grad, master, mom, *, lr: float, momentum: float, weight_decay: float) -> None:
    n = param.numel()
    if not param.is_cuda:
        g = grad.float().reshape(-1)
        w = (master if master is not None else param).float().reshape(-1).clone()
        upd = g
        if mom is not None:
            mom.mul_(momentum).add_(g)
            upd = mom
        w = w - (lr * upd + weight_decay * w)
        if master is not None:
            master.copy_(w.reshape(master.shape))
        param.copy_(w.reshape(param.shape))
        return
    _launch(N.require().oa_sgd(dt(param), dt(grad), param.data_ptr(), grad.data_ptr(), N.ptr(master), N.ptr(mom), n, float(lr),
                               float(momentum), float(weight_decay), N.stream()), "oa_sgd")


def sumsq(x: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> torch.Tensor:
    if not x.is_cuda:
        s = x.float().pow(2).sum()
        out[0] = s + out[0] if accumulate else s
        return out
    part = scratch(x.device, 1184 * 4 * 2, "sumsq")
    _launch(N.require().oa_sumsq(dt(x), x.data_ptr(), x.numel(), part.data_ptr(), out.data_ptr(), int(accumulate), N.stream()),
            "oa_sumsq", 2)
    return out


def clip_coef(sumsq_t: torch.Tensor, max_norm: float, coef: torch.Tensor) -> torch.Tensor:
    if not sumsq_t.is_cuda:
        nrm = float(sumsq_t[0]) ** 0.5
        coef[0] = max_norm / (nrm + 1e-6) if nrm > max_norm else 1.0
        return coef
    _launch(N.require().oa_clip_coef(sumsq_t.data_ptr(), float(max_norm), coef.data_ptr(), N.stream()), "oa_clip_coef")
    return coef


def scale_inplace(x: torch.Tensor, coef: torch.Tensor) -> torch.Tensor:
    if not x.is_cuda:
        x.mul_(float(coef[0]))
        return x
    _launch(N.require().oa_scale_inplace(dt(x), x.data_ptr(), x.numel(), coef.data_ptr(), N.stream()), "oa_scale_inplace")
    return x


# ---------------------------------------------------------------- attention
def _attn_ref(q, k, v, scale, causal):
    # q,k,v: [B, S, H, hd] fp32
    B, S, H, hd = q.shape
    qh, kh, vh = (t.permute(0, 2, 1, 3) for t in (q, k, v))
    s = torch.matmul(qh, kh.transpose(-1, -2)) * scale
    if causal:
        mask = torch.ones(S, S, dtype=torch.bool, device=q.device).tril()
        s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, -1)
    p = torch.softmax(s, -1)
    o = torch.matmul(p, vh).permute(0, 2, 1, 3)
    return o, lse


def flash_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, batch: int, seq: int, heads: int, head_dim: int, *,
              scale: Optional[float] = None, causal: bool = True):
    """q, k, v: [batch*seq, >= heads*head_dim] views (row stride free, e.g. slices of a packed QKV projection).

    Returns (o [batch*seq, heads*head_dim], lse [batch, heads, seq] fp32 natural-log).
    """
    scale = scale if scale is not None else 1.0 / math.sqrt(head_dim)
    D = heads * head_dim
    o = torch.empty((batch * seq, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((batch, heads, seq), dtype=torch.float32, device=q.device)
    if not q.is_cuda:
        qf, kf, vf = (t[:, :D].float().reshape(batch, seq, heads, head_dim) for t in (q, k, v))
        of, l = _attn_ref(qf, kf, vf, scale, causal)
        o.copy_(of.reshape(batch * seq, D))
        lse.copy_(l)
        return o, lse
    lib = N.require()
    if q.dtype == torch.bfloat16:
        assert q.stride(1) == 1 and k.stride(1) == 1 and v.stride(1) == 1 and k.stride(0) == v.stride(0)
        status = status_word(q.device)
        _launch(lib.oa_flash_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), batch, heads, seq,
                                 head_dim, q.stride(0), k.stride(0), o.stride(0), float(scale), int(causal),
                                 status.data_ptr(), N.stream()), "oa_flash_fwd")
        return o, lse
    assert q.dtype == torch.float32 and q.stride(0) == k.stride(0) == v.stride(0)
    _launch(lib.oa_attn_f32(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), batch, heads, seq, head_dim,
                            q.stride(0), o.stride(0), float(scale), int(causal), N.stream()), "oa_attn_f32")
    return o, lse


def flash_bwd(q, k, v, o, dout, lse, batch: int, seq: int, heads: int, head_dim: int, *, scale: Optional[float] = None,
              causal: bool = True, dqkv: Optional[torch.Tensor] = None):
    """Returns (dq, dk, dv) as [batch*seq, heads*head_dim] views.  With `dqkv` ([batch*seq, 3*heads*head_dim]) the three
    gradients are written side by side into it (the layout of a packed QKV projection output)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(head_dim)
    D = heads * head_dim
    if dqkv is None:
        dqkv = torch.empty((batch * seq, 3 * D), dtype=q.dtype, device=q.device)
    dq, dk, dv = dqkv[:, :D], dqkv[:, D:2 * D], dqkv[:, 2 * D:]
    if not q.is_cuda:
        with torch.enable_grad():
            qf, kf, vf = (t[:, :D].float().reshape(batch, seq, heads, head_dim).detach().requires_grad_(True) for t in (q, k, v))
            of, _ = _attn_ref(qf, kf, vf, scale, causal)
            gq, gk, gv = torch.autograd.grad(of, (qf, kf, vf), dout.float().reshape(batch, seq, heads, head_dim))
        dq.copy_(gq.reshape(batch * seq, D))
        dk.copy_(gk.reshape(batch * seq, D))
        dv.copy_(gv.reshape(batch * seq, D))
        return dq, dk, dv
    lib = N.require()
    if q.dtype == torch.bfloat16:
        status = status_word(q.device)
        sc = scratch(q.device, lib.oa_flash_bwd_scratch_bytes(batch, heads, seq, head_dim), "flash_bwd")
        _launch(lib.oa_flash_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), dout.data_ptr(), lse.data_ptr(),
                                 dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), batch, heads, seq, head_dim, q.stride(0),
                                 k.stride(0), o.stride(0), dq.stride(0), dk.stride(0), float(scale), int(causal),
                                 sc.data_ptr(), status.data_ptr(), N.stream()), "oa_flash_bwd", 3)
        return dq, dk, dv
    _launch(lib.oa_attn_f32_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), dout.data_ptr(), lse.data_ptr(),
                                dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), batch, heads, seq, head_dim, q.stride(0),
                                o.stride(0), dq.stride(0), float(scale), int(causal), N.stream()), "oa_attn_f32_bwd", 2)
    return dq, dk, dv


# ---------------------------------------------------------------- recurrent scans
def rnn_scan_fwd(gates_i: torch.Tensor, w_hh: torch.Tensor, b_hh: Optional[torch.Tensor], gates: int, h0: Optional[torch.Tensor] = None,
                 save: bool = True):
    """gates_i [B, S, gates*H] (input projection of all steps) -> (out [B,S,H], hprev [B,S,H] or None)."""
    B, S, GH = gates_i.shape
    H = GH // gates
    out = torch.empty((B, S, H), dtype=gates_i.dtype, device=gates_i.device)
    hprev = torch.empty_like(out) if save else None
    if not gates_i.is_cuda:
        h = h0.float().clone() if h0 is not None else torch.zeros(B, H)
        W = w_hh.float()
        bb = b_hh.float() if b_hh is not None else 0.0
        gi_all = gates_i.float()
        for t in range(S):
            gh = h @ W.t() + bb
            gi = gi_all[:, t]
            if hprev is not None:
                hprev[:, t] = h
            if gates == 3:
                r = torch.sigmoid(gi[:, :H] + gh[:, :H])
                z = torch.sigmoid(gi[:, H:2 * H] + gh[:, H:2 * H])
                n = torch.tanh(gi[:, 2 * H:] + r * gh[:, 2 * H:])
                h = (1 - z) * n + z * h
            else:
                h = torch.tanh(gi + gh)
            out[:, t] = h
        return out, hprev
    _launch(N.require().oa_rnn_scan_fwd(dt(gates_i), gates, gates_i.contiguous().data_ptr(), w_hh.contiguous().data_ptr(), N.ptr(b_hh),
                                        N.ptr(h0), out.data_ptr(), N.ptr(hprev), B, S, H, N.stream()), "oa_rnn_scan_fwd")
    return out, hprev


def rnn_scan_bwd(gates_i, w_hh, b_hh, hprev, dout, gates: int):
    """Returns (dgates_i [B,S,gates*H], dgates_h [B,S,gates*H], dh0 [B,H])."""
    B, S, GH = gates_i.shape
    H = GH // gates
    dgi = torch.empty_like(gates_i)
    dgh = torch.empty_like(gates_i)
    dh0 = torch.empty((B, H), dtype=gates_i.dtype, device=gates_i.device)
    if not gates_i.is_cuda:
        W = w_hh.float()
        bb = b_hh.float() if b_hh is not None else 0.0
        carry = torch.zeros(B, H)
        gi_all, hp_all, do_all = gates_i.float(), hprev.float(), dout.float()
        for t in range(S - 1, -1, -1):
            hp = hp_all[:, t]
            gh = hp @ W.t() + bb
            gi = gi_all[:, t]
            d = do_all[:, t] + carry
            if gates == 3:
                r = torch.sigmoid(gi[:, :H] + gh[:, :H])
                z = torch.sigmoid(gi[:, H:2 * H] + gh[:, H:2 * H])
                n = torch.tanh(gi[:, 2 * H:] + r * gh[:, 2 * H:])
                dn_pre = d * (1 - z) * (1 - n * n)
                dz_pre = d * (hp - n) * z * (1 - z)
                dr_pre = dn_pre * gh[:, 2 * H:] * r * (1 - r)
                gi_g = torch.cat([dr_pre, dz_pre, dn_pre], 1)
                gh_g = torch.cat([dr_pre, dz_pre, dn_pre * r], 1)
                carry = d * z + gh_g @ W
            else:
                hn = torch.tanh(gi + gh)
                gi_g = gh_g = d * (1 - hn * hn)
                carry = gh_g @ W
            dgi[:, t] = gi_g
            dgh[:, t] = gh_g
        dh0.copy_(carry)
        return dgi, dgh, dh0
    _launch(N.require().oa_rnn_scan_bwd(dt(gates_i), gates, gates_i.contiguous().data_ptr(), w_hh.contiguous().data_ptr(), N.ptr(b_hh),
                                        hprev.data_ptr(), dout.contiguous().data_ptr(), dgi.data_ptr(), dgh.data_ptr(), dh0.data_ptr(),
                                        B, S, H, N.stream()), "oa_rnn_scan_bwd")
    return dgi, dgh, dh0


# ---------------------------------------------------------------- KV-cache serving
def kv_append(k_src: torch.Tensor, v_src: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, batch: int, s_new: int,
              pos0: int, pos_dev: Optional[torch.Tensor] = None) -> None:
    """Copies new key / value rows ([batch*s_new, heads*head_dim] views, row stride allowed) into the caches
    [batch, heads, max_seq, head_dim] at positions pos0 .. pos0 + s_new."""
    _, heads, max_seq, hd = k_cache.shape
    if not k_cache.is_cuda:
        if pos_dev is not None:
            pos0 += int(pos_dev.item())
        for src, dst in ((k_src, k_cache), (v_src, v_cache)):
            dst[:, :, pos0:pos0 + s_new] = src.reshape(batch, s_new, heads, hd).permute(0, 2, 1, 3).to(dst.dtype)
        return
    assert k_src.stride(1) == 1 and k_src.stride(0) == v_src.stride(0) and k_cache.dtype == torch.bfloat16
    _launch(N.require().oa_kv_append(k_src.data_ptr(), v_src.data_ptr(), k_src.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), batch, s_new,
                                     heads, hd, pos0, max_seq, N.ptr(pos_dev), N.stream()), "oa_kv_append")


def decode_attn(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, length: int, scale: Optional[float] = None,
                pos_dev: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One query token per sequence, q [batch, heads*head_dim] (row stride allowed), against the first `length` cached
    positions; returns [batch, heads*head_dim]."""
    batch, heads, max_seq, hd = k_cache.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    if not q.is_cuda:
        if pos_dev is not None:
            length += int(pos_dev.item())
        qf = q.float().reshape(batch, heads, 1, hd)
        kf, vf = k_cache[:, :, :length].float(), v_cache[:, :, :length].float()
        p = torch.softmax((qf @ kf.transpose(-1, -2)) * scale, -1)
        return (p @ vf).reshape(batch, heads * hd).to(q.dtype)
    out = torch.empty((batch, heads * hd), dtype=q.dtype, device=q.device)
    assert q.stride(1) == 1 and q.dtype == torch.bfloat16
    lib = N.require()
    if hd in (64, 128) and k_cache.is_contiguous() and v_cache.is_contiguous() and os.environ.get("OA_DECODE_ATTN", "stream") == "stream":
        splits = decode_attn_splits(batch * heads, max_seq)
        part = scratch(q.device, lib.oa_decode_attn_stream_scratch_bytes(batch, heads, hd, splits), "decode_attn_partial")
        _launch(lib.oa_decode_attn_stream(q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), out.stride(0),
                                          batch, heads, hd, length, max_seq, float(scale), N.ptr(pos_dev), part.data_ptr(), splits,
                                          status_word(q.device).data_ptr(), N.stream()), "oa_decode_attn_stream", 2)
        return out
    _launch(lib.oa_decode_attn(q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), out.stride(0), batch,
                               heads, hd, length, max_seq, float(scale), N.ptr(pos_dev), N.stream()), "oa_decode_attn")
    return out


def decode_attn_splits(n_bh: int, max_seq: int, slots: int = 2 * 148) -> int:
    """How many pieces each (sequence, head) is cut into for the streamed decode kernel: the smallest count (up to 8) whose
    items fill the persistent CTAs' last round to 95 % while a piece keeps at least 256 positions; else the best filling."""
    best, best_eff = 1, 0.0
    for s in range(1, 9):
        if s > 1 and max_seq // s < 256:
            break
        waves = n_bh * s / slots
        eff = waves / math.ceil(waves)
        if eff >= 0.95:
            return s
        if eff > best_eff + 1e-9:
            best, best_eff = s, eff
    return best
