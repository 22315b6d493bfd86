"""Tensor parallelism (Megatron column / row split with sequence-sharded activations) on fused compute+collective kernels.

The reference has no tensor parallelism (its OaCollective is host-staged and has no caller outside tests,
Source/Private/Oa/Runtime/Distributed/Collective.cpp:75-247), so this layer is new.  Between layers the activation is
sharded by rows (sequence parallel): rank r holds rows [r*M/W, (r+1)*M/W).  Two kernels carry all the traffic:

  all-gather -> GEMM   (column-parallel layer: QKV, gate/up, vocabulary head; backward of a row-parallel layer)
      communication CTAs of the GEMM kernel push this rank's rows into every rank's staging buffer over NVLink, block by
      block with a flag each; the tensor-core tiles of a block start as soon as its flag is up.
  GEMM -> reduce-scatter (row-parallel layer: attention out, FFN down; backward of a column-parallel layer)
      the epilogue stores each bf16 partial tile straight into its owner's staging slot and counts it in; the owner sums
      the `world` slots of its rows (+ residual) at the end of the same kernel.

Every call site owns its staging buffer, flags and a device-resident epoch, all carved from one peer-mapped arena, so the
kernels replay inside CUDA graphs.  The gathered input of a column-parallel layer stays in its staging buffer for the
weight-gradient GEMM of the backward pass (no re-gather).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from .. import _native as N
from ..core import fn_matrix as F
from ..core.matrix import OaMatrix
from ..ml import autograd as AG
from ..ml.module import OaModule
from ..ops import kernels as K
from .mesh import OaDeviceMesh

BM = 128


class OaTpArena:
    """One peer-mapped buffer of the same size on every rank with a bump allocator (offsets agree on all ranks)."""

    def __init__(self, mesh: OaDeviceMesh, nbytes: int):
        self.mesh = mesh
        self.buf = mesh.AllocSymmetric(nbytes)
        self.buf.tensor.zero_()
        self.used = 0
        self._last_site = None
        self._fence_ch = None
        torch.cuda.synchronize()
        if mesh.world > 1:
            dist.barrier(group=mesh.group)          # nobody pushes into a buffer that is still being zeroed

    def enter_site(self, site) -> None:
        """Orders two uses of one call site.  A peer may push the next use's rows into this rank's staging buffer as soon as
        it has finished its own kernel of this use, which only proves that this rank's PUSHES arrived, not that this rank
        has finished reading.  With another site's kernel in between the order holds by itself (that kernel completes on a
        peer only after this rank's kernel of it started, hence after this rank's earlier kernel ended); a site that
        runs twice in a row gets a ready/ack round over a channel first."""
        if self._last_site is site and self.mesh.world > 1:
            if self._fence_ch is None:
                self._fence_ch = self.mesh.NewChannel()
            self._fence_ch.Signal()
            self._fence_ch.Wait()
        self._last_site = site

    def take(self, nbytes: int) -> int:
        off = self.used
        self.used = (off + int(nbytes) + 1023) // 1024 * 1024
        if self.used > self.buf.nbytes:
            raise N.OaKernelError(f"tensor-parallel arena exhausted ({self.used} > {self.buf.nbytes} bytes)")
        return off


class _Site:
    def __init__(self, arena: OaTpArena, data_bytes: int, n_flags: int):
        self.arena, self.mesh = arena, arena.mesh
        self.data_off = arena.take(data_bytes)
        self.flag_off = arena.take(8 * n_flags)
        self.bufs = arena.buf.table(self.data_off)
        self.flags = arena.buf.table(self.flag_off)
        self.sync = torch.zeros(2, dtype=torch.int64, device=self.mesh.device)
        self.data_bytes = data_bytes

    def local(self, dtype, shape) -> torch.Tensor:
        n = 1
        for d in shape:
            n *= d
        return self.arena.buf.view(dtype, n, self.data_off).view(*shape)


class OaTpAgSite(_Site):
    """Call site of an all-gather -> GEMM over [M, K] activations."""

    def __init__(self, arena: OaTpArena, M: int, K_: int):
        W = arena.mesh.world
        if M % (BM * W):
            raise ValueError(f"tensor-parallel rows {M} must be a multiple of {BM * W}")
        super().__init__(arena, M * K_ * 2, M // BM)
        self.M, self.K = M, K_

    def gathered(self) -> torch.Tensor:
        return self.local(torch.bfloat16, (self.M, self.K))

    def own_rows(self) -> torch.Tensor:
        """This rank's rows of the staging buffer: an activation produced here needs no copy before the all-gather."""
        Ms = self.M // self.mesh.world
        return self.gathered()[self.mesh.rank * Ms:(self.mesh.rank + 1) * Ms]


class OaTpRsSite(_Site):
    """Call site of a GEMM -> reduce-scatter producing [M / W, N]."""

    def __init__(self, arena: OaTpArena, M: int, N_: int):
        W = arena.mesh.world
        if M % (BM * W):
            raise ValueError(f"tensor-parallel rows {M} must be a multiple of {BM * W}")
        super().__init__(arena, M * N_ * 2, M // (BM * W))
        self.M, self.N = M, N_


def ag_gemm(site: OaTpAgSite, x_shard: torch.Tensor, w: torch.Tensor, *, b_mn: bool = False, comm_ctas: int = 0) -> torch.Tensor:
    """allgather_rows(x_shard)[M, K] @ W^T -> [M, N] (W is [N, K], or [K, N] when b_mn).  One kernel."""
    m = site.mesh
    Nn = w.shape[1] if b_mn else w.shape[0]
    assert x_shard.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x_shard.is_contiguous() and w.is_contiguous()
    assert x_shard.shape == (site.M // m.world, site.K)
    out = torch.empty((site.M, Nn), dtype=torch.bfloat16, device=x_shard.device)
    stage = site.gathered()
    Ms = site.M // m.world
    own = stage[m.rank * Ms:(m.rank + 1) * Ms]
    if x_shard.data_ptr() != own.data_ptr():
        K.unary("copy", x_shard, out=own)      # a producer that writes into site.own_rows() directly skips this copy
    x_shard = own
    site.arena.enter_site(site)
    K._launch(N.require().oa_gemm_bf16_tp(1, stage.data_ptr(), w.data_ptr(), out.data_ptr(), site.M, Nn, site.K, site.K, w.shape[1], Nn,
                                          int(b_mn), None, 0, 0, 1.0, x_shard.data_ptr(), site.K, site.bufs, site.flags,
                                          site.sync.data_ptr(), m.world, m.rank, comm_ctas, K.status_word(m.device).data_ptr(),
                                          N.stream()), "oa_gemm_bf16_tp(all-gather)")
    return out


def gemm_rs(site: OaTpRsSite, a: torch.Tensor, w: torch.Tensor, *, b_mn: bool = False, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """reduce_scatter_rows(a[M, K] @ W^T) (+ residual) -> [M / W, N].  One kernel."""
    m = site.mesh
    Nn = w.shape[1] if b_mn else w.shape[0]
    Kk = a.shape[1]
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.is_contiguous() and w.is_contiguous()
    assert a.shape[0] == site.M and Nn == site.N
    out = torch.empty((site.M // m.world, Nn), dtype=torch.bfloat16, device=a.device)
    site.arena.enter_site(site)
    K._launch(N.require().oa_gemm_bf16_tp(2, a.data_ptr(), w.data_ptr(), out.data_ptr(), site.M, Nn, Kk, Kk, w.shape[1], Nn, int(b_mn),
                                          N.ptr(residual), Nn if residual is not None else 0, 0, 1.0, None, 0, site.bufs, site.flags,
                                          site.sync.data_ptr(), m.world, m.rank, 0, K.status_word(m.device).data_ptr(), N.stream()),
              "oa_gemm_bf16_tp(reduce-scatter)")
    return out


def _weight_grad(w: OaMatrix, g: torch.Tensor, x: torch.Tensor):
    """dW[N, K] = g[M, N]^T @ x[M, K] into the parameter's gradient sink."""
    if not w.RequiresGrad():
        return None
    tw = w.Tensor()
    buf, acc, direct = F._grad_out(w, tw.shape, tw.dtype, tw.device)
    K.gemm(g, x, a_mn=True, b_mn=True, out=buf, accumulate=acc)
    return None if direct else buf


def ColumnParallelLinear(x_shard: OaMatrix, w: OaMatrix, fwd: OaTpAgSite, bwd: OaTpRsSite, name: str = "TpColumnLinear") -> OaMatrix:
    """x_shard [M/W, K] (sequence shard), w [N_local, K] -> [M, N_local]."""
    F._ctx_add(name)
    tx, tw = F._c(x_shard.Tensor()), F._c(w.Tensor())
    out = OaMatrix(ag_gemm(fwd, tx, tw))

    def back(g):
        g = F._c(g)
        dw = _weight_grad(w, g, fwd.gathered())                         # before the reduce-scatter: see the module docstring
        dx = gemm_rs(bwd, g, tw, b_mn=True) if x_shard.RequiresGrad() else None
        return (dx, dw)

    return AG.attach(name, out, [x_shard, w], back)


def RowParallelLinear(a: OaMatrix, w: OaMatrix, fwd: OaTpRsSite, bwd: OaTpAgSite, residual: Optional[OaMatrix] = None,
                      name: str = "TpRowLinear") -> OaMatrix:
    """a [M, K_local], w [N, K_local] -> reduce-scattered [M/W, N] (+ residual [M/W, N])."""
    F._ctx_add(name)
    ta, tw = F._c(a.Tensor()), F._c(w.Tensor())
    tr = F._c(residual.Tensor()) if residual is not None else None
    out = OaMatrix(gemm_rs(fwd, ta, tw, residual=tr))

    def back(g):
        g = F._c(g)
        da = ag_gemm(bwd, g, tw, b_mn=True)                             # also leaves the gathered gradient in bwd's buffer
        dw = _weight_grad(w, bwd.gathered(), ta)
        return (da if a.RequiresGrad() else None, dw, g if residual is not None else None)

    return AG.attach(name, out, [a, w, residual], back)


# ------------------------------------------------------------------------------------------- vocabulary-parallel loss
def VocabParallelCrossEntropy(logits_local: OaMatrix, targets: OaMatrix, mesh: OaDeviceMesh, stats: "OaTpStats") -> OaMatrix:
    """Mean cross-entropy over [M, V/W] logit shards: each rank reduces its shard to (max, sum exp, target logit) per row,
    the three numbers are exchanged through peer memory, and every rank finishes loss and its own dlogits (in place)."""
    F._ctx_add("VocabParallelCrossEntropy")
    tl = F._c(logits_local.Tensor())
    M, Vl = tl.shape
    tg = targets.Tensor().reshape(-1).to(torch.int32)
    lib, st = N.require(), N.stream()
    W, r = mesh.world, mesh.rank
    loc = stats.local_rows(M)
    K._launch(lib.oa_vp_xent_stats(K.dt(tl), tl.data_ptr(), tg.data_ptr(), loc.data_ptr(), M, Vl, r * Vl, st), "oa_vp_xent_stats")
    K._launch(lib.oa_peer_push(stats.buf.ptr_array, stats.off + r * M * 12, loc.data_ptr(), M * 12, W, st), "oa_peer_push(stats)")
    stats.ch.Signal()
    stats.ch.Wait()
    row_loss = torch.empty(M, dtype=torch.float32, device=tl.device)
    need = AG.IsEnabled() and logits_local.RequiresGrad()
    all_stats = stats.buf.view(torch.float32, W * M * 3, stats.off)
    K._launch(lib.oa_vp_xent_finish(K.dt(tl), tl.data_ptr(), tg.data_ptr(), all_stats.data_ptr(), row_loss.data_ptr(), M, Vl, r * Vl, W,
                                    1.0 / M if need else 0.0, int(need), st), "oa_vp_xent_finish")
    out = OaMatrix(K.mean_f32(row_loss))

    def back(g):
        if getattr(g, "_oa_root_seed", False):
            return (tl, None)
        return (K.binary("mul", tl, g.reshape(1).to(tl.dtype)), None)

    return AG.attach("VocabParallelCrossEntropy", out, [logits_local, targets], back)


class OaTpStats:
    """Exchange buffer of the vocabulary-parallel loss: [W, M, 3] fp32 on every rank plus a ready channel."""

    def __init__(self, arena: OaTpArena, M: int):
        self.buf, self.M = arena.buf, M
        self.off = arena.take(arena.mesh.world * M * 12)
        self.ch = arena.mesh.NewChannel()
        self._loc = torch.empty(M * 3, dtype=torch.float32, device=arena.mesh.device)

    def local_rows(self, M: int) -> torch.Tensor:
        assert M == self.M
        return self._loc
