"""ChannelNorm and the 1-D convolution GEMM path on CPU tensors against torch.nn.functional."""
import torch


def test_channel_norm_and_conv1d_gemm_cpu():
    """ChannelNorm equals LayerNorm over the transposed tensor (values and gradients); Conv1dGemm equals conv1d."""
    import torch.nn.functional as TF
    from oa_b200.core import fn_matrix as F
    from oa_b200.ml.autograd import OaGradientTape
    torch.manual_seed(0)
    B, C, L = 3, 6, 10
    x0, w0, b0, g0 = torch.randn(B, C, L), torch.randn(C), torch.randn(C), torch.randn(B, C, L)
    for relu in (False, True):
        xr, wr, br = (t.clone().requires_grad_(True) for t in (x0, w0, b0))
        ref = TF.layer_norm(xr.transpose(1, 2), (C,), wr, br, 1e-5).transpose(1, 2)
        ref = torch.relu(ref) if relu else ref
        ref.backward(g0)
        x, w, b = (F.FromTensor(t.clone()).SetRequiresGrad(True) for t in (x0, w0, b0))
        with OaGradientTape() as tape:
            y = (F.ChannelNormRelu if relu else F.ChannelNorm)(x, w, b, B, C, L, 1e-5)
            tape.Backward(y, grad=g0)
        assert torch.allclose(y.Tensor(), ref, atol=1e-5)
        for got, want in ((x, xr), (w, wr), (b, br)):
            assert torch.allclose(got.GradMatrix().Tensor(), want.grad, atol=1e-4)
        dx, dw, db = (F.ChannelNormReluBwd(x, w, y, F.FromTensor(g0), B, C, L) if relu else F.ChannelNormBwd(x, w, F.FromTensor(g0), B, C, L))
        assert torch.allclose(dx.Tensor(), xr.grad, atol=1e-4) and torch.allclose(dw.Tensor(), wr.grad, atol=1e-4) and torch.allclose(db.Tensor(), br.grad, atol=1e-4)
    xc, wc, bc = torch.randn(2, 4, 17), torch.randn(5, 4, 3), torch.randn(5)
    for stride, pad, dil in ((1, 0, 1), (2, 1, 1), (1, 2, 2)):
        want = TF.conv1d(xc, wc, bc, stride, pad, dil)
        got = F.Conv1dGemm(F.FromTensor(xc), F.FromTensor(wc), F.FromTensor(bc), stride, pad, dil)
        assert torch.allclose(got.Tensor(), want, atol=1e-5)
        assert torch.allclose(F.Conv1dReluGemm(F.FromTensor(xc), F.FromTensor(wc), F.FromTensor(bc), stride, pad, dil).Tensor(), torch.relu(want), atol=1e-5)
        cols = F.Im2Col1d(F.FromTensor(xc), 3, stride, pad, dil)
        assert cols.Tensor().shape == (2 * want.shape[2], 12)
        back = F.Col2Im1d(cols, 2, 4, 17, 3, stride, pad, dil, want.shape[2])
        ones = F.Col2Im1d(F.FromTensor(torch.ones_like(cols.Tensor())), 2, 4, 17, 3, stride, pad, dil, want.shape[2])
        assert torch.allclose(back.Tensor(), xc * ones.Tensor(), atol=1e-5)          # every sample comes back once per window that covers it
