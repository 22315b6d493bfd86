"""Expert parallelism: the MoE all-to-all dispatch and combine as peer-memory kernels fused with the routing.

The reference's MoE is single device (stacked expert tensors, GPU route plan, grouped GEMM; Nn/Moe/Moe.cpp:98-114),
so this layer is new.  Rank s owns experts [s*E/W, (s+1)*E/W) and keeps only their weights.  Per layer:
  forward   router + local plan -> push this rank's expert counts to every peer (flags) -> every rank derives the
            owner-side row of each of its routes -> DISPATCH: gather fused with the remote store, token rows are
            written straight into the owner's expert-major buffer over NVLink -> flags -> owner runs the two grouped
            tensor-core GEMMs over the rows that landed -> flags -> COMBINE: each rank pulls its result rows from the
            owners, weighted by the gates, fused with the residual add.
  backward  mirrored: gate-scaled output gradients are pushed to the owners, dgate is a pulled dot product, the
            owner computes dW and dX with grouped GEMMs, token gradients are pulled back.
Nothing is dropped and nothing can overflow: after the count exchange every rank holds the same [W, E] table, so every
rank knows, before any row moves, how many rows each owner receives.  The layout kernel reduces the table to two numbers
(rows this rank receives, rows of the busiest owner), the host reads them (one small copy and a stream synchronisation
per layer, what a dropless MoE pays everywhere), grows the peer-mapped buffers on all ranks alike when the busiest owner
needs more than they hold, and sizes the expert temporaries to exactly the rows that arrive.  Buffers holding rows are
per layer (they are saved for the backward pass); the gradient staging pair is shared by all layers.
Ordering of buffer reuse needs no extra round: a rank overwrites a peer's buffer only after a wait whose signal that
peer issued after its last read of the buffer (stream order), see the comments at the three rounds of each direction.
Dense parameters are data parallel (parallel/dp.py); expert gradients stay local and are scaled by 1/world.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from .. import _native as N
from ..ops import kernels as K
from ..ops import moe as M
from .mesh import OaDeviceMesh


class _LocalPlan:
    """Owner-side plan (duck-types ops.moe.Plan for the grouped GEMMs)."""
    __slots__ = ("counts", "offsets", "packed_token", "inverse", "max_rows", "experts", "k", "tokens", "counts_global")


def _round_up(n: int, m: int) -> int:
    return (int(n) + m - 1) // m * m


class _GradStaging:
    """The pair of gradient staging buffers of the backward pass, one for all layers (used one layer at a time)."""

    def __init__(self, mesh: OaDeviceMesh, d_model: int):
        self.mesh, self.D, self.cap = mesh, d_model, 0
        self.dpo = self.dpx = None

    def ensure(self, rows: int) -> None:
        if rows <= self.cap:
            return
        for old in (self.dpo, self.dpx):
            if old is not None:
                self.mesh.Release(old)
        self.cap = rows
        self.dpo = self.mesh.AllocSymmetric(rows * self.D * 2)
        self.dpx = self.mesh.AllocSymmetric(rows * self.D * 2)


class OaEpDispatcher:
    def __init__(self, mesh: OaDeviceMesh, num_experts: int, d_model: int, d_ff: int, tokens: int, k: int,
                 capacity_factor: float = 2.0, shared_bwd: Optional[_GradStaging] = None):
        self.mesh, self.E, self.D, self.F, self.T, self.k = mesh, num_experts, d_model, d_ff, tokens, k
        W = mesh.world
        assert num_experts % W == 0 and num_experts % 4 == 0
        self.E_loc = num_experts // W
        avg = tokens * k                                   # rows an owner receives when the load is uniform
        # `capacity_factor` only sets the FIRST size of the row buffers; they grow to what the routing asks for.  Twice the
        # mean by default: a growth is a collective reallocation (measured: a step that grows costs about twice a step that does not)
        self.cap = _round_up(int(avg * capacity_factor) + self.E_loc * M.SEG, M.SEG)
        self.Grown = 0                                     # how many times the buffers had to grow
        dev = mesh.device
        self.counts_all = mesh.AllocSymmetric(W * num_experts * 4)
        self.px = mesh.AllocSymmetric(self.cap * d_model * 2)          # dispatched token rows (saved for dW)
        self.po = mesh.AllocSymmetric(self.cap * d_model * 2)          # expert outputs (pulled by combine, and again by dgate)
        self.grads = shared_bwd if shared_bwd is not None else _GradStaging(mesh, d_model)
        self.grads.ensure(self.cap)
        self.ch = [mesh.NewChannel() for _ in range(5)]
        self.route_rank = torch.empty(tokens * k, dtype=torch.int32, device=dev)
        self.route_row = torch.empty(tokens * k, dtype=torch.int32, device=dev)
        self.loc_offsets = torch.zeros(self.E_loc + 1, dtype=torch.int32, device=dev)
        self.loc_counts = torch.zeros(self.E_loc, dtype=torch.int32, device=dev)
        self.counts_global = torch.zeros(num_experts, dtype=torch.int32, device=dev)
        self.need = torch.zeros(2, dtype=torch.int32, device=dev)
        self.need_host = torch.zeros(2, dtype=torch.int32).pin_memory() if dev.type == "cuda" else torch.zeros(2, dtype=torch.int32)
        self.LastRows = 0

    def shared_bwd(self) -> _GradStaging:
        return self.grads

    def _sync(self, i: int) -> None:
        self.ch[i].Signal()
        self.ch[i].Wait()

    def _view(self, buf, cols: int, rows: int) -> torch.Tensor:
        return buf.view(torch.bfloat16, rows * cols).view(rows, cols)

    def _size_for(self) -> int:
        """Reads {rows this rank receives, rows of the busiest owner} and grows the row buffers of every rank when the
        busiest owner needs more (the same decision everywhere: the table behind the two numbers is the same).  By now
        all peers have passed this layer's count exchange, so none of them still reads the buffers that are replaced."""
        self.need_host.copy_(self.need, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        rows, most = int(self.need_host[0]), int(self.need_host[1])
        if most > self.cap:
            self.cap = _round_up(most + most // 8, M.SEG)
            self.mesh.Release(self.px)
            self.mesh.Release(self.po)
            self.px = self.mesh.AllocSymmetric(self.cap * self.D * 2)
            self.po = self.mesh.AllocSymmetric(self.cap * self.D * 2)
            self.Grown += 1
        self.grads.ensure(self.cap)
        self.LastRows = rows
        return max(rows, M.SEG)

    def Forward(self, x: torch.Tensor, idx: torch.Tensor, w: torch.Tensor, wgu, bgu, wd, bd, base: Optional[torch.Tensor]):
        lib, m = N.require(), self.mesh
        st = N.stream()
        status = K.status_word(m.device)
        T, k = idx.shape
        Pl = M.plan(idx, self.E)
        # 1. counts -> every peer's table row `rank`
        K._launch(lib.oa_peer_push(self.counts_all.ptr_array, m.rank * self.E * 4, Pl.counts.data_ptr(), self.E * 4, m.world, st),
                  "oa_peer_push(counts)")
        self._sync(0)
        # 2. owner-side layout of my routes, and my own expert plan
        K._launch(lib.oa_ep_layout(self.counts_all.local_ptr, idx.data_ptr(), Pl.inverse.data_ptr(), Pl.offsets.data_ptr(),
                                   self.route_rank.data_ptr(), self.route_row.data_ptr(), self.loc_offsets.data_ptr(),
                                   self.loc_counts.data_ptr(), self.counts_global.data_ptr(), self.need.data_ptr(), T * k, self.E,
                                   m.world, m.rank, st), "oa_ep_layout")
        rows = self._size_for()
        # 3. dispatch: gather fused with the remote store
        K._launch(lib.oa_ep_push_rows(x.data_ptr(), self.px.ptr_array, self.route_rank.data_ptr(), self.route_row.data_ptr(), None,
                                      T * k, k, self.D, m.world, self.cap, status.data_ptr(), st), "oa_ep_push_rows(dispatch)")
        self._sync(1)
        px = self._view(self.px, self.D, rows)
        K._launch(lib.oa_ep_zero_pad(px.data_ptr(), self.loc_offsets.data_ptr(), self.loc_counts.data_ptr(), self.E_loc, self.D, st),
                  "oa_ep_zero_pad")
        P = _LocalPlan()
        P.counts, P.offsets, P.max_rows, P.experts, P.k, P.tokens = self.loc_counts, self.loc_offsets, rows, self.E_loc, k, T
        P.packed_token, P.inverse, P.counts_global = None, None, self.counts_global
        # 4. local experts on the rows that landed
        gu = M.grouped_linear(px, wgu, bgu, P)
        h = K.swiglu_fwd(gu)
        po = M.grouped_linear(h, wd, bd, P, out=self._view(self.po, self.D, rows))
        self._sync(2)
        # 5. combine: weighted pull of my routes' rows from their owners (+ residual)
        out = torch.empty((T, self.D), dtype=x.dtype, device=x.device)
        K._launch(lib.oa_ep_pull_rows(self.po.ptr_array, self.route_rank.data_ptr(), self.route_row.data_ptr(), w.data_ptr(),
                                      N.ptr(base), out.data_ptr(), T, k, self.D, m.world, st), "oa_ep_pull_rows(combine)")
        # routes are per layer state needed by backward: keep copies (the index buffers are reused by the next step only)
        return out, (P, px, gu, h, po, self.route_rank, self.route_row)

    def Backward(self, saved, g: torch.Tensor, w: torch.Tensor, wgu, bgu, wd, bd):
        from ..ml.nn.moe import _expert_grad
        lib, m = N.require(), self.mesh
        st = N.stream()
        status = K.status_word(m.device)
        P, px, gu, h, po, route_rank, route_row = saved
        T, k = P.tokens, P.k
        twgu, twd = wgu.Tensor(), wd.Tensor()
        # 1. dgate (pulled dot products) and gate-scaled output gradients pushed to the owners
        dgate = torch.empty((T, k), dtype=torch.float32, device=g.device)
        K._launch(lib.oa_ep_pull_dot(self.po.ptr_array, route_rank.data_ptr(), route_row.data_ptr(), g.data_ptr(), dgate.data_ptr(),
                                     T * k, k, self.D, m.world, st), "oa_ep_pull_dot")
        K._launch(lib.oa_ep_push_rows(g.data_ptr(), self.grads.dpo.ptr_array, route_rank.data_ptr(), route_row.data_ptr(), w.data_ptr(),
                                      T * k, k, self.D, m.world, self.grads.cap, status.data_ptr(), st), "oa_ep_push_rows(dcombine)")
        self._sync(3)
        dpo = self._view(self.grads.dpo, self.D, P.max_rows)
        K._launch(lib.oa_ep_zero_pad(dpo.data_ptr(), self.loc_offsets.data_ptr(), self.loc_counts.data_ptr(), self.E_loc, self.D, st),
                  "oa_ep_zero_pad")
        # 2. owner-side expert backward
        dh = M.grouped_linear(dpo, twd, None, P, b_mn=True)
        dwd = _expert_grad(wd, lambda o, a: M.grouped_weight_grad(dpo, h, P, out=o, accumulate=a), twd)
        dbd = M.grouped_bias_grad(dpo, P) if bd is not None and bd.RequiresGrad() else None
        dgu = K.swiglu_bwd(gu, dh)
        dpx = M.grouped_linear(dgu, twgu, None, P, b_mn=True, out=self._view(self.grads.dpx, self.D, P.max_rows))
        dwgu = _expert_grad(wgu, lambda o, a: M.grouped_weight_grad(dgu, px, P, out=o, accumulate=a), twgu)
        dbgu = M.grouped_bias_grad(dgu, P) if bgu is not None and bgu.RequiresGrad() else None
        self._sync(4)
        # 3. token gradients pulled back from the owners
        dx = torch.empty((T, self.D), dtype=g.dtype, device=g.device)
        K._launch(lib.oa_ep_pull_rows(self.grads.dpx.ptr_array, route_rank.data_ptr(), route_row.data_ptr(), None, None, dx.data_ptr(), T, k,
                                      self.D, m.world, st), "oa_ep_pull_rows(dgather)")
        # No round after the pull: the next writer of a peer's staging buffer (the next layer's push, the owner's next dX)
        # runs after a wait on a signal that this rank issues after this pull in stream order.
        return dx, dgate, dwgu, dbgu, dwd, dbd


class OaExpertParallel:
    """Shards the routed experts of every OaMoE layer of `model` over the mesh and installs the dispatchers."""

    def __init__(self, model, mesh: Optional[OaDeviceMesh] = None, tokens_per_rank: int = 0, capacity_factor: float = 2.0):
        from ..ml.nn.moe import OaMoE
        self.mesh = mesh or OaDeviceMesh()
        self.layers = []
        self._walk(model, OaMoE)
        W, r = self.mesh.world, self.mesh.rank
        shared = None
        for layer in self.layers:
            E = layer.NumExperts
            El = E // W
            for p in (layer.GateUpW, layer.GateUpB, layer.DownW, layer.DownB):
                if p is None:
                    continue
                full = p.Tensor()
                p._ep_full_shape = tuple(full.shape)
                p.Data._t = full[r * El:(r + 1) * El].clone()
            d = OaEpDispatcher(self.mesh, E, layer.DModel, layer.DFF, tokens_per_rank, layer.ExpertsPerToken, capacity_factor, shared)
            shared = d.shared_bwd()
            layer.Dispatcher = d

    def _walk(self, module, cls) -> None:
        if isinstance(module, cls):
            self.layers.append(module)
        for _, c in module.Children():
            self._walk(c, cls)

    def Growths(self) -> int:
        """How often any layer's row buffers had to be replaced by larger ones so far (each time is a collective reallocation)."""
        return sum(layer.Dispatcher.Grown for layer in self.layers)

    def ExpertParameters(self):
        out = []
        for layer in self.layers:
            out += [p for p in (layer.GateUpW, layer.GateUpB, layer.DownW, layer.DownB) if p is not None]
        return out

    def GatherExpertParameter(self, p) -> torch.Tensor:
        """Canonical unsharded [E, ...] tensor of a sharded expert parameter (for checkpoints)."""
        parts = [torch.empty_like(p.Tensor()) for _ in range(self.mesh.world)]
        dist.all_gather(parts, p.Tensor().contiguous(), group=self.mesh.group)
        return torch.cat(parts, 0)
