"""OaCollective: the collective verbs on a device mesh (Source/Public/Oa/Runtime/Collective.h:23-71).

The reference implements AllReduce / Broadcast / AllGather / Scatter / ReduceScatter on the host over mapped buffers, f32
only (Source/Private/Oa/Runtime/Distributed/Collective.cpp:75-247).  Here they are device collectives: on CUDA meshes the
data moves through a peer-mapped staging buffer with the push / reduce kernels of csrc/kernels/comm.cu and epoch flags
(one-shot algorithms: every rank publishes its contribution once, every rank reads what it needs), which is the right
shape for the small and medium messages these verbs are used for; the bulk paths of training have their own fused kernels
(parallel/dp.py, tp.py, ep.py).  `backend="nccl"` (or a CPU / gloo mesh) routes to torch.distributed instead, which is also
the baseline the fused paths are timed against.  AllToAll is added to the reference's five verbs."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from .. import _native as N
from ..ops import kernels as K
from .mesh import OaDeviceMesh, OaReduceOp

_TORCH_OP = {OaReduceOp.Sum: dist.ReduceOp.SUM, OaReduceOp.Max: dist.ReduceOp.MAX, OaReduceOp.Min: dist.ReduceOp.MIN}


class OaCollective:
    """Every verb moves only the bytes its definition needs over NVLink:
      AllGather / Broadcast   the owner pushes its block into its slot of every rank's staging buffer (posted stores);
      AllReduce / ReduceScatter  every rank stages its tensor locally, then pulls and reduces ONLY its own shard of every
                              peer's copy with the peer-reduce kernel (fp32 accumulation, fixed rank order); AllReduce then
                              pushes the reduced shard to every rank (reduce-scatter + all-gather, 2 (W-1)/W n bytes per
                              rank), or reduces the whole tensor in one pass when it is small or does not divide;
      Scatter / AllToAll      block j is pushed to rank j alone."""

    TwoPhaseBytes = 1 << 20        # AllReduce: below this one pass over all peers' copies beats two synchronisations

    def __init__(self, mesh: OaDeviceMesh, staging_bytes: int = 64 << 20, backend: str = "peer"):
        self.Mesh = mesh
        self.Peer = backend == "peer" and mesh.device.type == "cuda" and mesh.world > 1
        self.StagingBytes = int(staging_bytes)
        if self.Peer:
            self._buf = mesh.AllocSymmetric(self.StagingBytes)
            self._ready, self._done = mesh.NewChannel(), mesh.NewChannel()

    def _fits(self, t: torch.Tensor, copies: int, block_bytes: Optional[int] = None) -> bool:
        nb = t.numel() * t.element_size()
        return (self.Peer and t.dtype in (torch.float32, torch.bfloat16) and nb * copies <= self.StagingBytes
                and (block_bytes if block_bytes is not None else nb) % 16 == 0)

    # ---- building blocks
    def _push(self, src: torch.Tensor, dst_off_bytes: int, to: Optional[int] = None) -> None:
        """Stores `src` at byte offset `dst_off_bytes` of the staging buffer of every rank (or of rank `to` alone)."""
        m = self.Mesh
        if to is None:
            table, world = self._buf.ptr_array, m.world
        else:
            table, world = (ctypes.c_void_p * 1)(self._buf.peer_ptrs[to]), 1
        K._launch(N.require().oa_peer_push(table, dst_off_bytes, src.data_ptr(), src.numel() * src.element_size(), world, N.stream()),
                  "oa_peer_push")

    def _reduce(self, dtype: torch.dtype, out: torch.Tensor, lo: int, n: int, op: OaReduceOp) -> None:
        """out[i] = reduce over ranks of staging_r[lo + i] (elements of `dtype`), pulled over NVLink."""
        K._launch(N.require().oa_peer_reduce(K.dt(out), self._buf.ptr_array, out.data_ptr(), lo, n, self.Mesh.world, int(op), N.stream()),
                  "oa_peer_reduce")

    def _meet(self) -> None:
        self._ready.Signal()
        self._ready.Wait()

    def _release(self) -> None:
        self._done.Signal()        # nobody overwrites a staging buffer that a peer may still be reading
        self._done.Wait()

    # ---- verbs
    def AllGather(self, t: torch.Tensor) -> torch.Tensor:
        """[n, ...] on every rank -> [world * n, ...] (rank order)."""
        m, t = self.Mesh, t.contiguous()
        if not self._fits(t, m.world):
            out = torch.empty((m.world * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
            dist.all_gather_into_tensor(out, t, group=m.group)
            return out
        nb = t.numel() * t.element_size()
        self._push(t, m.rank * nb)
        self._meet()
        out = self._buf.view(t.dtype, m.world * t.numel()).clone().view((m.world * t.shape[0],) + tuple(t.shape[1:]))
        self._release()
        return out

    def AllReduce(self, t: torch.Tensor, op: OaReduceOp = OaReduceOp.Sum) -> torch.Tensor:
        m, t = self.Mesh, t.contiguous()
        n, nb = t.numel(), t.numel() * t.element_size()
        if not self._fits(t, 2):
            out = t.clone()
            dist.all_reduce(out, op=_TORCH_OP[op], group=m.group)
            return out
        self._buf.view(t.dtype, n).copy_(t.view(-1))            # local staging copy; peers read it after the meeting point
        self._meet()
        out = torch.empty_like(t)
        shard = n // m.world
        if nb >= self.TwoPhaseBytes and n % m.world == 0 and (shard * t.element_size()) % 16 == 0:
            red = torch.empty(shard, dtype=t.dtype, device=t.device)
            self._reduce(t.dtype, red, m.rank * shard, shard, op)            # reduce-scatter: my shard of every copy
            self._push(red, nb + m.rank * shard * t.element_size())          # all-gather into the second half of the buffer
            self._release()                                                  # (doubles as "all shards have landed")
            out.view(-1).copy_(self._buf.view(t.dtype, n, nb))
            self._meet()                                                     # the result region is read before anyone reuses it
            return out
        self._reduce(t.dtype, out.view(-1), 0, n, op)
        self._release()
        return out

    def ReduceScatter(self, t: torch.Tensor, op: OaReduceOp = OaReduceOp.Sum) -> torch.Tensor:
        """[world * n, ...] on every rank -> this rank's reduced [n, ...]."""
        m, t = self.Mesh, t.contiguous()
        n = t.shape[0] // m.world
        if not self._fits(t, 1):
            out = torch.empty((n,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
            dist.reduce_scatter_tensor(out, t, op=_TORCH_OP[op], group=m.group)
            return out
        self._buf.view(t.dtype, t.numel()).copy_(t.view(-1))
        self._meet()
        out = torch.empty((n,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        shard = t.numel() // m.world
        self._reduce(t.dtype, out.view(-1), m.rank * shard, shard, op)
        self._release()
        return out

    def Broadcast(self, t: torch.Tensor, root: int = 0) -> torch.Tensor:
        m, t = self.Mesh, t.contiguous()
        if not self._fits(t, 1):
            out = t.clone()
            dist.broadcast(out, src=dist.get_global_rank(m.group, root) if m.group is not None else root, group=m.group)
            return out
        if m.rank == root:
            self._push(t, 0)                                    # only the root's bytes travel
        self._meet()
        out = self._buf.view(t.dtype, t.numel()).clone().view(t.shape)
        self._release()
        return out

    def Scatter(self, t: Optional[torch.Tensor], root: int = 0, shape=None, dtype=None) -> torch.Tensor:
        """Root holds [world * n, ...]; rank r receives rows [r*n, (r+1)*n).  Non-root ranks pass shape / dtype of the input."""
        m = self.Mesh
        if t is None:
            t = torch.zeros(tuple(shape), dtype=dtype, device=m.device)
        t = t.contiguous()
        n = t.shape[0] // m.world
        blk = t.numel() // m.world
        if not self._fits(t, 1, blk * t.element_size()):
            full = self.Broadcast(t, root)
            return full[m.rank * n:(m.rank + 1) * n].clone()
        if m.rank == root:
            flat = t.view(-1)
            for r in range(m.world):
                self._push(flat[r * blk:(r + 1) * blk], 0, to=r)     # block r goes to rank r alone
        self._meet()
        out = self._buf.view(t.dtype, blk).clone().view((n,) + tuple(t.shape[1:]))
        self._release()
        return out

    def AllToAll(self, t: torch.Tensor) -> torch.Tensor:
        """[world * n, ...]: block j goes to rank j; the result's block i came from rank i."""
        m, t = self.Mesh, t.contiguous()
        blk = t.numel() // m.world
        if not self._fits(t, 1, blk * t.element_size()):
            out = torch.empty_like(t)
            dist.all_to_all_single(out, t, group=m.group)
            return out
        flat = t.view(-1)
        for j in range(m.world):
            self._push(flat[j * blk:(j + 1) * blk], m.rank * blk * t.element_size(), to=j)
        self._meet()
        out = self._buf.view(t.dtype, t.numel()).clone().view(t.shape)
        self._release()
        return out

    def Barrier(self) -> None:
        if self.Peer:
            self.Mesh.Barrier()
        elif self.Mesh.world > 1:
            dist.barrier(group=self.Mesh.group)
