"""OaCollective: the collective verbs on a device mesh (Source/Public/Oa/Runtime/Collective.h:23-71).

The reference implements AllReduce / Broadcast / AllGather / Scatter / ReduceScatter on the host over mapped buffers, f32
only (Source/Private/Oa/Runtime/Distributed/Collective.cpp:75-247).  Here they are device collectives: on CUDA meshes the
data moves through a peer-mapped staging buffer with the push / reduce kernels of csrc/kernels/comm.cu and epoch flags
(one-shot algorithms: every rank publishes its contribution once, every rank reads what it needs), which is the right
shape for the small and medium messages these verbs are used for; the bulk paths of training have their own fused kernels
(parallel/dp.py, tp.py, ep.py).  `backend="nccl"` (or a CPU / gloo mesh) routes to torch.distributed instead, which is also
the baseline the fused paths are timed against.  AllToAll is added to the reference's five verbs."""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .. import _native as N
from ..ops import kernels as K
from .mesh import OaDeviceMesh, OaReduceOp

_TORCH_OP = {OaReduceOp.Sum: dist.ReduceOp.SUM, OaReduceOp.Max: dist.ReduceOp.MAX, OaReduceOp.Min: dist.ReduceOp.MIN}


class OaCollective:
    def __init__(self, mesh: OaDeviceMesh, staging_bytes: int = 64 << 20, backend: str = "peer"):
        self.Mesh = mesh
        self.Peer = backend == "peer" and mesh.device.type == "cuda" and mesh.world > 1
        self.StagingBytes = int(staging_bytes)
        if self.Peer:
            self._buf = mesh.AllocSymmetric(self.StagingBytes)
            self._ready, self._done = mesh.NewChannel(), mesh.NewChannel()

    def _fits(self, t: torch.Tensor, copies: int) -> bool:
        return self.Peer and t.dtype in (torch.float32, torch.bfloat16) and t.numel() * t.element_size() * copies <= self.StagingBytes

    def _publish(self, t: torch.Tensor, slot_bytes: int) -> None:
        """Every rank writes `t` into slot `rank` of every rank's staging buffer, then all ranks meet."""
        m = self.Mesh
        K._launch(N.require().oa_peer_push(self._buf.ptr_array, m.rank * slot_bytes, t.data_ptr(), t.numel() * t.element_size(), m.world,
                                           N.stream()), "oa_peer_push")
        self._ready.Signal()
        self._ready.Wait()

    def _release(self) -> None:
        self._done.Signal()        # nobody overwrites a staging buffer that a peer may still be reading
        self._done.Wait()

    def AllGather(self, t: torch.Tensor) -> torch.Tensor:
        """[n, ...] on every rank -> [world * n, ...] (rank order)."""
        m, t = self.Mesh, t.contiguous()
        if not self._fits(t, m.world):
            out = torch.empty((m.world * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
            dist.all_gather_into_tensor(out, t, group=m.group)
            return out
        nb = t.numel() * t.element_size()
        self._publish(t, nb)
        out = self._buf.view(t.dtype, m.world * t.numel()).clone().view((m.world * t.shape[0],) + tuple(t.shape[1:]))
        self._release()
        return out

    def AllReduce(self, t: torch.Tensor, op: OaReduceOp = OaReduceOp.Sum) -> torch.Tensor:
        m, t = self.Mesh, t.contiguous()
        if not self._fits(t, m.world):
            out = t.clone()
            dist.all_reduce(out, op=_TORCH_OP[op], group=m.group)
            return out
        nb = t.numel() * t.element_size()
        self._publish(t, nb)
        slots = self._buf.view(t.dtype, m.world * t.numel()).view(m.world, -1).float()
        red = slots.sum(0) if op == OaReduceOp.Sum else (slots.max(0).values if op == OaReduceOp.Max else slots.min(0).values)
        out = red.to(t.dtype).view(t.shape)
        self._release()
        return out

    def ReduceScatter(self, t: torch.Tensor, op: OaReduceOp = OaReduceOp.Sum) -> torch.Tensor:
        """[world * n, ...] on every rank -> this rank's reduced [n, ...]."""
        m, t = self.Mesh, t.contiguous()
        n = t.shape[0] // m.world
        if not self._fits(t, m.world):
            out = torch.empty((n,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
            dist.reduce_scatter_tensor(out, t, op=_TORCH_OP[op], group=m.group)
            return out
        nb = t.numel() * t.element_size()
        self._publish(t, nb)
        slots = self._buf.view(t.dtype, m.world * t.numel()).view(m.world, m.world, -1)[:, m.rank].float()
        red = slots.sum(0) if op == OaReduceOp.Sum else (slots.max(0).values if op == OaReduceOp.Max else slots.min(0).values)
        out = red.to(t.dtype).view((n,) + tuple(t.shape[1:]))
        self._release()
        return out

    def Broadcast(self, t: torch.Tensor, root: int = 0) -> torch.Tensor:
        m, t = self.Mesh, t.contiguous()
        if not self._fits(t, m.world):
            out = t.clone()
            dist.broadcast(out, src=dist.get_global_rank(m.group, root) if m.group is not None else root, group=m.group)
            return out
        nb = t.numel() * t.element_size()
        self._publish(t, nb)
        out = self._buf.view(t.dtype, m.world * t.numel()).view(m.world, -1)[root].clone().view(t.shape)
        self._release()
        return out

    def Scatter(self, t: Optional[torch.Tensor], root: int = 0, shape=None, dtype=None) -> torch.Tensor:
        """Root holds [world * n, ...]; rank r receives rows [r*n, (r+1)*n).  Non-root ranks pass shape / dtype of the input."""
        m = self.Mesh
        if t is None:
            t = torch.zeros(tuple(shape), dtype=dtype, device=m.device)
        full = self.Broadcast(t, root)
        n = full.shape[0] // m.world
        return full[m.rank * n:(m.rank + 1) * n].clone()

    def AllToAll(self, t: torch.Tensor) -> torch.Tensor:
        """[world * n, ...]: block j goes to rank j; the result's block i came from rank i."""
        m, t = self.Mesh, t.contiguous()
        n = t.shape[0] // m.world
        if not self._fits(t, m.world):
            out = torch.empty_like(t)
            dist.all_to_all_single(out, t, group=m.group)
            return out
        nb = t.numel() * t.element_size()
        self._publish(t, nb)
        out = self._buf.view(t.dtype, m.world * t.numel()).view(m.world, m.world, -1)[:, m.rank].clone().view(t.shape)
        self._release()
        return out

    def Barrier(self) -> None:
        if self.Peer:
            self.Mesh.Barrier()
        elif self.Mesh.world > 1:
            dist.barrier(group=self.Mesh.group)
