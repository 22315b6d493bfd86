"""Block quantisation (llama.cpp layouts): Q4_0 with separate scales, Q8_0 blocks, per-tensor int8.

Reference: Source/Public/Oa/Ml/FnMatrix.h:771-789 and Source/Public/Oa/Core/FnMatrix.h:86-94 (Quantize / Dequantize by
target type); kernels in csrc/kernels/quant.cu, CPU tensors run the same arithmetic in PyTorch.
"""
from __future__ import annotations

import torch

from .. import _native as N
from . import kernels as K

BLOCK = 32


def _run(op: int, src: torch.Tensor, scale, out: torch.Tensor, count: int) -> torch.Tensor:
    lib = N.require()
    K._launch(lib.oa_quantize(op, src.data_ptr(), N.ptr(scale), out.data_ptr(), count, N.stream()), f"oa_quantize[{op}]")
    return out


def _blocks(x: torch.Tensor) -> torch.Tensor:
    n = x.numel()
    pad = (-n) % BLOCK
    return torch.cat((x.reshape(-1), x.new_zeros(pad))).reshape(-1, BLOCK)


def _round(x: torch.Tensor) -> torch.Tensor:
    return torch.round(x)            # ties to even, as cvt.rni on the device


def q4_0_scale(x: torch.Tensor) -> torch.Tensor:
    x = x.reshape(-1).float().contiguous()
    nb = (x.numel() + BLOCK - 1) // BLOCK
    if x.is_cuda:
        return _run(0, x, None, torch.empty(nb, dtype=torch.float32, device=x.device), x.numel())
    s = _blocks(x).abs().max(1).values / 7.0
    return torch.where(s < 1e-6, torch.ones_like(s), s)


def q4_0_quantize(x: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    x = x.reshape(-1).float().contiguous()
    nb = (x.numel() + BLOCK - 1) // BLOCK
    if x.is_cuda:
        return _run(1, x, scale, torch.empty(nb * 16, dtype=torch.uint8, device=x.device), x.numel())
    b = _blocks(x)
    q = (_round(b / scale[:, None]).clamp(-7, 7) + 7).to(torch.uint8)
    n = x.numel()
    if n % BLOCK:
        q.reshape(-1)[n:] = 7
    return (q[:, 0::2] | (q[:, 1::2] << 4)).reshape(-1)


def q4_0_dequantize(packed: torch.Tensor, scale: torch.Tensor, count: int) -> torch.Tensor:
    if packed.is_cuda:
        return _run(2, packed.contiguous(), scale, torch.empty(count, dtype=torch.float32, device=packed.device), count)
    p = packed.reshape(-1, 16)
    q = torch.stack((p & 0xF, (p >> 4) & 0xF), 2).reshape(-1, BLOCK).float() - 7.0
    return (q * scale[:, None]).reshape(-1)[:count]


def q8_0_quantize(x: torch.Tensor) -> torch.Tensor:
    x = x.reshape(-1).float().contiguous()
    if x.numel() % BLOCK:
        raise ValueError("Q8_0 needs a multiple of 32 elements")
    nb = x.numel() // BLOCK
    if x.is_cuda:
        return _run(3, x, None, torch.empty(nb * 34, dtype=torch.uint8, device=x.device), x.numel())
    b = x.reshape(nb, BLOCK)
    d = b.abs().max(1).values / 127.0
    inv = torch.where(d != 0, 1.0 / d, torch.zeros_like(d))
    q = _round(b * inv[:, None]).clamp(-127, 127).to(torch.int8)
    out = torch.empty(nb, 34, dtype=torch.uint8)
    out[:, :2] = d.to(torch.float16).view(torch.uint8).reshape(nb, 2)
    out[:, 2:] = q.view(torch.uint8)
    return out.reshape(-1)


def q8_0_dequantize(blocks: torch.Tensor) -> torch.Tensor:
    nb = blocks.numel() // 34
    if blocks.is_cuda:
        return _run(4, blocks.contiguous(), None, torch.empty(nb * BLOCK, dtype=torch.float32, device=blocks.device), nb * BLOCK)
    b = blocks.reshape(nb, 34)
    d = b[:, :2].contiguous().view(torch.float16).float()
    return (b[:, 2:].contiguous().view(torch.int8).float() * d).reshape(-1)


def int8_quantize(x: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    x = x.reshape(-1).float().contiguous()
    if x.is_cuda:
        return _run(5, x, scale, torch.empty(x.numel(), dtype=torch.int8, device=x.device), x.numel())
    return _round(x / scale.reshape(-1)[0]).clamp(-127, 127).to(torch.int8)


def int8_dequantize(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    if q.is_cuda:
        return _run(6, q.contiguous(), scale, torch.empty(q.numel(), dtype=torch.float32, device=q.device), q.numel())
    return q.float() * scale.reshape(-1)[0]
