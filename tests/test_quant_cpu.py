"""Block quantisation on the CPU path: layouts and error bounds (the GPU test compares the kernels against this path)."""
import torch

from oa_b200.core import fn_matrix as F
from oa_b200.core.matrix import OaMatrix


def test_q4_0_roundtrip_and_layout():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(100, generator=g) * 3          # 3 full blocks + a ragged one
    x[32:64] = 0.0
    sc = F.ComputeScaleQ4_0(OaMatrix(x))
    assert sc.Tensor().shape == (4,) and sc.Tensor()[1] == 1.0
    assert torch.allclose(sc.Tensor()[0], x[:32].abs().max() / 7)
    q = F.QuantizeQ4_0(OaMatrix(x), sc)
    assert q.Tensor().dtype == torch.uint8 and q.Tensor().shape == (64,)
    lo, hi = q.Tensor()[0] & 0xF, q.Tensor()[0] >> 4
    assert lo == (x[0] / sc.Tensor()[0]).round().clamp(-7, 7) + 7 and hi == (x[1] / sc.Tensor()[0]).round().clamp(-7, 7) + 7
    y = F.DequantizeQ4_0(q, sc, 100).Tensor()
    assert y.shape == (100,) and (y - x).abs().max() <= sc.Tensor().max() * 0.5 + 1e-6 and y[32:64].abs().sum() == 0


def test_q8_0_and_int8_roundtrip():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(256, generator=g)
    blocks = F.QuantizeQ8_0(OaMatrix(x)).Tensor()
    assert blocks.shape == (8 * 34,)
    d0 = blocks[:2].view(torch.float16).float()
    assert abs(d0.item() - x[:32].abs().max().item() / 127) < 1e-3
    y = F.DequantizeQ8_0(OaMatrix(blocks)).Tensor()
    assert (y - x).abs().max() < 0.02
    s = OaMatrix(torch.tensor([x.abs().max().item() / 127]))
    q = F.QuantizeInt8(OaMatrix(x), s)
    assert q.Tensor().dtype == torch.int8 and q.Tensor().abs().max() == 127
    assert (F.DequantizeInt8(q, s).Tensor() - x).abs().max() <= s.Tensor().item() * 0.5 + 1e-6
