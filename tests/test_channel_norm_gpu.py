"""ChannelNorm kernels (fp32 and bf16 storage) against the fp32 tensor-expression path."""
import pytest
import torch

from oa_b200.core import fn_matrix as F

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("relu", [False, True])
def test_channel_norm_kernels(dtype, tol, relu):
    torch.manual_seed(0)
    B, C, L = 5, 96, 333
    x, w, b, g = torch.randn(B, C, L), torch.rand(C) + 0.5, torch.randn(C), torch.randn(B, C, L)
    q = lambda t: t.to(dtype).float()                       # the reference sees the same rounded inputs
    y_ref, mean, rstd = F._channel_norm_fwd(q(x), q(w), q(b), B, C, L, 1e-5, relu)
    dx_ref, dw_ref, db_ref = F._channel_norm_bwd(q(x), q(w), q(g), y_ref if relu else None, mean, rstd, B, C, L)
    d = lambda t: t.to(dtype).cuda()
    y, mean_g, rstd_g = F._channel_norm_fwd(d(x), d(w), d(b), B, C, L, 1e-5, relu)
    assert y.dtype == dtype and torch.allclose(y.float().cpu(), y_ref, atol=tol, rtol=tol)
    assert torch.allclose(mean_g.cpu(), mean, atol=1e-5) and torch.allclose(rstd_g.cpu(), rstd, atol=1e-4, rtol=1e-4)
    # backward on the GPU with the reference's forward output as the ReLU mask, so both sides gate the same elements
    dx, dw, db = F._channel_norm_bwd(d(x), d(w), d(g), y_ref.to(dtype).cuda() if relu else None, mean_g, rstd_g, B, C, L)
    assert torch.allclose(dx.float().cpu(), dx_ref, atol=tol, rtol=tol)
    assert torch.allclose(dw.cpu(), dw_ref, atol=tol * 30, rtol=tol) and torch.allclose(db.cpu(), db_ref, atol=tol * 30, rtol=tol)
