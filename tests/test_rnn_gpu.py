"""GRU / RNN scan kernels against the CPU statement of the recurrence (forward, backward, fp32 and bf16)."""
import pytest
import torch

from oa_b200.ops import kernels as K

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("gates", [1, 3])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 4e-2)])
@pytest.mark.parametrize("B,S,H", [(5, 7, 32), (64, 16, 64)])
def test_scan_fwd_bwd(gates, dtype, tol, B, S, H):
    torch.manual_seed(0)
    dev = "cuda"
    gi = (torch.randn(B, S, gates * H, device=dev)).to(dtype)
    w = (torch.randn(gates * H, H, device=dev) * 0.2).to(dtype)
    b = (torch.randn(gates * H, device=dev) * 0.1).to(dtype)
    out, hprev = K.rnn_scan_fwd(gi, w, b, gates)
    c = lambda t: t.cpu().float()
    outr, hprevr = K.rnn_scan_fwd(c(gi), c(w), c(b), gates)
    assert (c(out) - outr).abs().max().item() <= tol
    do = torch.randn(B, S, H, device=dev).to(dtype)
    got = K.rnn_scan_bwd(gi, w, b, hprev, do, gates)
    ref = K.rnn_scan_bwd(c(gi), c(w), c(b), hprevr, c(do), gates)
    for g, r, nm in zip(got, ref, ("dgi", "dgh", "dh0")):
        scale = r.abs().max().item() + 1e-6
        assert (c(g) - r).abs().max().item() <= tol * max(1.0, scale), nm
    torch.cuda.synchronize()
    K.check_status()
