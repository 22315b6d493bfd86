"""Data parallelism (ZeRO-1 style) with the gradient reduce-scatter, the partitioned Adam update and the parameter
all-gather fused into one peer-memory kernel.

The reference has no data parallelism (its optimizers walk local parameters only, Optim/AdamW.cpp:116-131), so this
layer is new.  Plan:
  * the optimizer's flat parameter and gradient arenas are allocated as symmetric (IPC peer-mapped) buffers,
  * every rank owns a contiguous 1/world shard of the arena and keeps fp32 master / m / v for that shard only,
  * after backward each rank signals "gradients ready", then ONE kernel (csrc/kernels/comm.cu) waits for all
    ranks, pulls its shard of every rank's bf16 gradients over NVLink, sums in fp32, scales, applies AdamW to its
    master shard and pushes the bf16 result into every rank's parameter arena; a second signal / wait pair
    closes the step.  Gradients and parameters each cross NVLink once as bf16, nothing is staged.
  * `mode="nccl"` is the baseline the fused path is measured against: NCCL all-reduce of the gradient arena
    followed by the ordinary local optimizer step.
  * the bf16 arena is cut into buckets in parameter order.  Backward reaches the last parameters first, so the last bucket
    is complete first: as soon as the autograd tape reports that every parameter of a bucket has its final gradient, the
    bucket's kernel is queued on a second stream behind an event and runs UNDER the rest of the backward pass with a small
    CTA budget; the step itself then only joins that stream.  Gradient accumulation (`NoSync`) and gradient-norm clipping
    (the norm needs every gradient first) fall back to launching all buckets from `Step`.
Checkpoints stay in the canonical unsharded layout: optimizer moments are all-gathered on save and re-sharded
on load.
"""
from __future__ import annotations

import contextlib
import ctypes
import os
from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

from .. import _native as N
from ..core.types import OaStatus
from ..io.oam import OamModel, OamOptimizerState
from ..ops import kernels as K
from ..runtime import engine as RT
from .mesh import OaDeviceMesh


class _Bucket:
    """A slice [lo, hi) of a bf16 arena; every rank owns (hi - lo) / world consecutive elements of it."""
    __slots__ = ("arena", "lo", "hi", "sn", "state_off", "channel", "params", "pending", "launched")

    def __init__(self, arena: int, lo: int, hi: int, world: int, channel):
        self.arena, self.lo, self.hi = arena, lo, hi
        self.sn = (hi - lo) // world
        self.state_off = lo // world           # offset of this bucket's shard inside the rank's master / m / v
        self.channel = channel
        self.params: list = []                  # ids of the parameter matrices that overlap the slice
        self.pending = 0
        self.launched = False


class OaDataParallel:
    def __init__(self, model, optimizer, mode: str = "fused", mesh: Optional[OaDeviceMesh] = None, max_blocks: int = 0,
                 buckets: int = 8, overlap: Optional[bool] = None, overlap_blocks: int = 148):
        self.model, self.opt, self.mode = model, optimizer, mode
        self.mesh = mesh or OaDeviceMesh()
        self.world, self.rank = self.mesh.world, self.mesh.rank
        self.max_blocks = max_blocks
        self.overlap_blocks = overlap_blocks
        self._sym: dict[int, object] = {}
        self._summed: dict[int, torch.Tensor] = {}
        self._no_sync = False
        if mode == "fused":
            optimizer.SetArenaAllocator(self._alloc)
        optimizer._build()
        optimizer.SetGradScale(1.0 / self.world)
        self.arenas = optimizer.Arenas()
        # identical initial weights on every rank
        for a in self.arenas:
            dist.broadcast(a.flat, src=0, group=self.mesh.group)
        optimizer.ReduceMetric = self.ReduceMetric
        optimizer.IsPrimaryWriter = lambda: self.rank == 0
        if mode == "fused":
            self.ch_grads = self.mesh.NewChannel()
            self.ch_params = self.mesh.NewChannel()
            self.ch_norm = self.mesh.NewChannel()
            lib = N.require()
            self._norm_partial = torch.zeros(int(lib.oa_dp_sumsq_blocks()), dtype=torch.float32, device=self.mesh.device)
            self._norm_slots = self.mesh.AllocSymmetric(16 * 8)          # one 16-byte slot per rank
            self._norm_extra = torch.zeros(1, dtype=torch.float32, device=self.mesh.device)
            self._coef = torch.ones(2, dtype=torch.float32, device=self.mesh.device)
            self._shards = []
            self._buckets: list[_Bucket] = []
            self._by_param: dict[int, list] = {}
            q = 8 * self.world
            for i, a in enumerate(self.arenas):
                if a.dtype != torch.bfloat16:
                    # small fp32 arenas (biases, per-head scalars): replicated update - every rank sums all ranks' gradients
                    # with peer loads and applies the same AdamW step; no sharding, no all-gather
                    self._shards.append(None)
                    continue
                n = a.numel
                assert n % q == 0
                nb = max(1, min(int(buckets), n // (q * 1024) or 1))
                bounds = sorted({min(n, (n * k // nb + q - 1) // q * q) for k in range(nb + 1)})
                sn = n // self.world
                master = torch.empty(sn, dtype=torch.float32, device=a.device)
                for lo, hi in zip(bounds[:-1], bounds[1:]):
                    b = _Bucket(i, lo, hi, self.world, self.mesh.NewChannel())
                    master[b.state_off:b.state_off + b.sn].copy_(a.flat[lo + self.rank * b.sn: lo + (self.rank + 1) * b.sn])
                    for p, o in zip(a.params, a.offsets):
                        if o < hi and o + p.NumElements() > lo:
                            b.params.append(id(p.Data))
                            self._by_param.setdefault(id(p.Data), []).append(b)
                    self._buckets.append(b)
                m = torch.zeros(sn, dtype=torch.float32, device=a.device)
                v = torch.zeros(sn, dtype=torch.float32, device=a.device)
                self._shards.append((master, m, v))
                # the full-size optimizer state of the single-GPU path is not needed: free it
                a.master = None
                optimizer._m[i] = m
                optimizer._v[i] = v
            optimizer.Step = self._fused_step
            optimizer.SaveTo = self._save_to
            optimizer.LoadFrom = self._load_from
            # Measured on two B200s (350 M parameters): the sharded update after the backward pass costs less than the
            # single-GPU AdamW it replaces, and running the buckets under the backward pass slows the GEMMs by more than
            # it hides, so the overlap is opt-in (argument, or OA_DP_OVERLAP=1) rather than the default.
            if overlap is None:
                overlap = os.environ.get("OA_DP_OVERLAP", "0") == "1"
            self._overlap = bool(overlap) and self.world > 1
            self.overlap_blocks = int(os.environ.get("OA_DP_OVERLAP_BLOCKS", self.overlap_blocks))
            self._advanced = False
            if self._overlap:
                from ..ml import autograd as AG
                self._comm = torch.cuda.Stream(device=self.mesh.device)
                AG.SetLeafReadyHooks(self._on_backward_begin, self._on_leaf_ready)
        else:
            self._local_step = optimizer.Step
            optimizer.Step = self._nccl_step
        torch.cuda.synchronize()
        dist.barrier(group=self.mesh.group)

    # ---- allocation of the arenas in peer-mapped memory
    def _alloc(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        esz = torch.empty((), dtype=dtype).element_size()
        buf = self.mesh.AllocSymmetric(numel * esz)
        t = buf.view(dtype, numel)
        self._sym[t.data_ptr()] = buf
        return t

    # ---- steps
    def _clip_coef(self, replicated) -> Optional[torch.Tensor]:
        """Clip coefficient from the norm of the gradient summed over the ranks (every rank gets the same bits): each
        rank takes the sum of squares of its shard, the scalars are exchanged through peer memory."""
        opt = self.opt
        if opt._clip_norm is None:
            return None
        lib = N.require()
        ctx = RT.OaContext.GetDefault()
        for k, i in enumerate(replicated):
            K.sumsq(self._summed[i], self._norm_extra[0:1], accumulate=k > 0)
        first = True
        for b in self._buckets:
            a = self.arenas[b.arena]
            ctx.Add("DpShardSumSq")
            N.check(lib.oa_dp_shard_sumsq(self._sym[a.grad.data_ptr()].ptr_array, b.lo + self.rank * b.sn, b.sn, self.rank, self.world,
                                          self._norm_partial.data_ptr(), 0 if first else 1, N.stream()), "oa_dp_shard_sumsq")
            N.count_launch()
            first = False
        if first:
            self._norm_partial.zero_()
        N.check(lib.oa_dp_sumsq_publish(self._norm_partial.data_ptr(), self._norm_slots.ptr_array, self.rank, self.world, N.stream()),
                "oa_dp_sumsq_publish")
        N.count_launch()
        self.ch_norm.Signal()
        self.ch_norm.Wait()
        N.check(lib.oa_dp_clip_finalize(self._norm_slots.local_ptr, self.world, self._norm_extra.data_ptr() if replicated else None,
                                        float(opt._clip_norm) / max(opt.GradScale_, 1e-30), self._coef.data_ptr(), N.stream()),
                "oa_dp_clip_finalize")
        N.count_launch()
        return self._coef

    def _advance_once(self) -> None:
        if not self._advanced:
            RT.OaContext.GetDefault().Add("AdamwGraphAdvance")
            K.optim_advance(self.opt._state)
            self._advanced = True

    def _launch_bucket(self, b: _Bucket, coef, blocks: int) -> None:
        """Signals "my gradients of this bucket are final", then the fused kernel of the bucket on the CURRENT stream: it waits
        for every rank's signal, reduces this rank's shard over the peers, applies AdamW and pushes the new bf16 parameters."""
        opt, lib = self.opt, N.require()
        a = self.arenas[b.arena]
        master, m, v = self._shards[b.arena]
        RT.OaContext.GetDefault().Add("DpReduceScatterAdamAllGather")
        b.channel.Signal()
        gbuf, pbuf = self._sym[a.grad.data_ptr()], self._sym[a.flat.data_ptr()]
        o = b.state_off
        N.check(lib.oa_dp_reduce_adam_gather(gbuf.ptr_array, pbuf.ptr_array, master[o:].data_ptr(), m[o:].data_ptr(), v[o:].data_ptr(),
                                             b.lo + self.rank * b.sn, b.sn, opt._state.data_ptr(),
                                             coef.data_ptr() if coef is not None else None, int(opt.Decoupled), self.rank, self.world,
                                             b.channel.flags.local_ptr, b.channel.epoch.data_ptr(),
                                             K.status_word(self.mesh.device).data_ptr(), blocks, N.stream()), "oa_dp_reduce_adam_gather")
        N.count_launch()
        b.launched = True

    # -- overlap with the backward pass
    @contextlib.contextmanager
    def NoSync(self):
        """Backward passes inside this block only accumulate gradients (gradient accumulation): no bucket is reduced until
        a backward pass outside the block, or `Step`, does it."""
        prev, self._no_sync = self._no_sync, True
        try:
            yield
        finally:
            self._no_sync = prev

    def _on_backward_begin(self) -> None:
        live = self._overlap and not self._no_sync and self.opt._clip_norm is None
        self._bw_live = live
        if not live:
            return
        for b in self._buckets:
            b.pending, b.launched = len(b.params), False
        self._advanced = False
        self._forked = False

    def _on_leaf_ready(self, matrix) -> None:
        if not getattr(self, "_bw_live", False):
            return
        for b in self._by_param.get(id(matrix), ()):
            b.pending -= 1
            if b.pending == 0 and not b.launched:
                main = torch.cuda.current_stream()
                self._advance_once()                       # on the main stream, ahead of the first bucket of the step
                ev = torch.cuda.Event()
                ev.record(main)
                with torch.cuda.stream(self._comm):
                    self._comm.wait_event(ev)
                    self._launch_bucket(b, None, self.overlap_blocks)
                self._forked = True

    def _fused_step(self) -> None:
        opt = self.opt
        ctx = RT.OaContext.GetDefault()
        lib = N.require()
        self._advance_once()
        replicated = [i for i, sh in enumerate(self._shards) if sh is None]
        clip = opt._clip_norm is not None
        if replicated or clip:
            self.ch_grads.Signal()
            self.ch_grads.Wait()                       # every rank's gradients are complete
        for i in replicated:
            a = self.arenas[i]
            ctx.Add("DpPeerReduce")
            gbuf = self._sym[a.grad.data_ptr()]
            summed = self._summed.setdefault(i, torch.empty(a.numel, dtype=a.dtype, device=a.device))
            N.check(lib.oa_peer_reduce(K.dt(a.grad), gbuf.ptr_array, summed.data_ptr(), 0, a.numel, self.world, 0, N.stream()),
                    "oa_peer_reduce")
            N.count_launch()
        coef = self._clip_coef(replicated)
        for i in replicated:
            a = self.arenas[i]
            K.adam_step(a.flat, self._summed[i], a.master, opt._m[i], opt._v[i], opt._state, decoupled=opt.Decoupled, inv_clip=coef)
        # buckets that did not go out under the backward pass (no overlap, accumulation, clipping, unused parameters)
        for b in self._buckets:
            if not b.launched:
                self._launch_bucket(b, coef, self.max_blocks)
        if getattr(self, "_forked", False):            # join the communication stream
            ev = torch.cuda.Event()
            ev.record(self._comm)
            torch.cuda.current_stream().wait_event(ev)
            self._forked = False
        # parameters of every rank are complete once all ranks' pushes have landed
        self.ch_params.Signal()
        self.ch_params.Wait()
        for b in self._buckets:
            b.launched = False
        self._advanced = False
        opt.Step_ += 1

    def ReduceMetric(self, value: float) -> float:
        """Mean of a host scalar over the ranks: checkpoint decisions (is this the best loss so far?) must be the same on
        every rank, because saving gathers the sharded optimizer state with a collective."""
        t = torch.tensor([float(value)], dtype=torch.float64, device=self.mesh.device)
        dist.all_reduce(t, group=self.mesh.group)
        return float(t[0]) / self.world

    def _nccl_step(self) -> None:
        for a in self.arenas:
            dist.all_reduce(a.grad, group=self.mesh.group)
        self._local_step()

    # ---- checkpoints (canonical, unsharded)
    def _gather_full(self, arena_index: int, shard: torch.Tensor, numel: int) -> torch.Tensor:
        """Every rank's state shard -> the full-arena tensor (a rank's shard is the concatenation of its slice of every bucket)."""
        gathered = torch.empty(self.world * shard.numel(), dtype=shard.dtype, device=shard.device)
        dist.all_gather_into_tensor(gathered, shard.contiguous(), group=self.mesh.group)
        gathered = gathered.view(self.world, -1)
        full = torch.empty(numel, dtype=shard.dtype, device=shard.device)
        for b in self._buckets:
            if b.arena == arena_index:
                full[b.lo:b.hi].view(self.world, b.sn).copy_(gathered[:, b.state_off:b.state_off + b.sn])
        return full

    def _take_shard(self, arena_index: int, full: torch.Tensor, shard: torch.Tensor) -> None:
        for b in self._buckets:
            if b.arena == arena_index:
                shard[b.state_off:b.state_off + b.sn].copy_(full[b.lo + self.rank * b.sn: b.lo + (self.rank + 1) * b.sn])

    def _save_to(self, oam: OamModel) -> OaStatus:
        opt = self.opt
        RT.OaContext.GetDefault().Sync()
        st = OamOptimizerState()
        st.Type = opt.TypeName
        st.Lr, st.Beta1, st.Beta2, st.Eps, st.WeightDecay, st.Step = opt.Lr_, opt.Beta1_, opt.Beta2_, opt.Eps_, opt.WeightDecay_, opt.Step_
        ms, vs = [], []
        for i, (a, sh) in enumerate(zip(self.arenas, self._shards)):
            if sh is None:
                ms.append(a.gather(opt._m[i]))
                vs.append(a.gather(opt._v[i]))
                continue
            master, m, v = sh
            ms.append(a.gather(self._gather_full(i, m, a.numel)))
            vs.append(a.gather(self._gather_full(i, v, a.numel)))
        st.AdamM, st.AdamV = np.concatenate(ms), np.concatenate(vs)
        oam.SetOptimizer(st)
        return OaStatus.Ok()

    def _load_from(self, oam: OamModel) -> OaStatus:
        opt = self.opt
        stt = opt.ValidateLoad(oam)
        if not stt:
            return stt
        s = oam.GetOptimizer()
        opt.Lr_, opt.Beta1_, opt.Beta2_, opt.Eps_, opt.WeightDecay_, opt.Step_ = s.Lr, s.Beta1, s.Beta2, s.Eps, s.WeightDecay, s.Step
        pos_m = pos_v = 0
        for i, (a, sh) in enumerate(zip(self.arenas, self._shards)):
            full = torch.empty(a.numel, dtype=torch.float32, device=a.device)
            if sh is None:
                pos_m = a.scatter(opt._m[i], s.AdamM, pos_m)
                pos_v = a.scatter(opt._v[i], s.AdamV, pos_v)
                continue
            master, m, v = sh
            pos_m = a.scatter(full, s.AdamM, pos_m)
            self._take_shard(i, full, m)
            pos_v = a.scatter(full, s.AdamV, pos_v)
            self._take_shard(i, full, v)
            self._take_shard(i, a.flat.float(), master)      # masters are re-seeded from the loaded weights
        opt._state.copy_(torch.tensor([float(opt.Step_), opt.Lr_, opt.Beta1_, opt.Beta2_, opt.Eps_, opt.WeightDecay_,
                                       opt.GradScale_, 0.0], dtype=torch.float32))
        return OaStatus.Ok()

    def Close(self) -> None:
        if getattr(self, "_overlap", False):
            from ..ml import autograd as AG
            AG.SetLeafReadyHooks(None, None)
        self.mesh.Close()
