"""Fused data-parallel step (reduce-scatter + AdamW + all-gather in one kernel) on ONE GPU: the ranks' arenas are
separate buffers of this process, the peer tables point at them, and the readiness flags are pre-set, so no kernel
ever waits on another kernel.  The result must equal averaging the gradients and running the plain AdamW kernel."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [1, 2, 4])
def test_dp_fused_step_matches_reference(world):
    from oa_b200 import _native as N
    from oa_b200.ops import kernels as K
    lib = N.require()
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    n = 8 * world * 1000
    w0 = torch.randn(n, device=dev).bfloat16()
    params = [w0.clone() for _ in range(world)]
    grads = [torch.randn(n, device=dev).bfloat16() for _ in range(world)]
    state = torch.tensor([1, 1e-2, 0.9, 0.999, 1e-8, 0.1, 1.0 / world, 0], dtype=torch.float32, device=dev)
    sn = n // world
    masters = [w0[r * sn:(r + 1) * sn].float() for r in range(world)]
    ms = [torch.zeros(sn, device=dev) for _ in range(world)]
    vs = [torch.zeros(sn, device=dev) for _ in range(world)]
    flags = torch.full((16,), 5, dtype=torch.int64, device=dev)      # every rank already signalled epoch 5
    epoch = torch.tensor([5, 0], dtype=torch.int64, device=dev)
    status = K.status_word(dev)
    gt = (ctypes.c_void_p * world)(*[g.data_ptr() for g in grads])
    pt = (ctypes.c_void_p * world)(*[p.data_ptr() for p in params])
    stream = torch.cuda.current_stream().cuda_stream
    for r in range(world):
        rc = lib.oa_dp_reduce_adam_gather(gt, pt, masters[r].data_ptr(), ms[r].data_ptr(), vs[r].data_ptr(), r * sn, sn,
                                          state.data_ptr(), None, 1, r, world, flags.data_ptr(), epoch.data_ptr(),
                                          status.data_ptr(), 0, stream)
        assert rc == 0
    torch.cuda.synchronize()
    K.check_status()
    # reference: average gradients in fp32, plain AdamW
    gsum = torch.stack([g.float() for g in grads]).sum(0)
    pref, mref, vref, master_ref = w0.clone(), torch.zeros(n, device=dev), torch.zeros(n, device=dev), w0.float()
    K.adam_step(pref, gsum, master_ref, mref, vref, state, decoupled=True)
    torch.cuda.synchronize()
    for r in range(world):
        assert torch.equal(params[r], params[0]), "all ranks must hold identical parameters after the push"
    assert (params[0].float() - pref.float()).abs().max().item() <= 2e-2
    got_master = torch.cat(masters)
    assert (got_master - master_ref).abs().max().item() <= 1e-5


def test_peer_wait_times_out_cleanly():
    """A wait on a flag that nobody sets must run out, report DeadlineExceeded through the status word and leave the
    context usable (bounded spin, no trap)."""
    from oa_b200 import _native as N
    from oa_b200.ops import kernels as K
    lib = N.require()
    dev = torch.device("cuda", 0)
    flags = torch.zeros(16, dtype=torch.int64, device=dev)
    epoch = torch.tensor([1, 0], dtype=torch.int64, device=dev)   # waits for epoch 1, flags stay 0
    status = K.status_word(dev)
    rc = lib.oa_peer_wait(flags.data_ptr(), epoch.data_ptr(), 2, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    with pytest.raises(N.OaKernelError):
        K.check_status()
    # context still usable
    x = torch.ones(1024, device=dev)
    assert K.unary("scale", x, 2.0).sum().item() == 2048.0
    K.check_status()
