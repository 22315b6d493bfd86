"""OaUploadRing and OaPrefetcher: host -> device staging (Source/Public/Oa/Runtime/UploadRing.h:17-82, Prefetch.cpp).

The ring owns `slots` pinned host buffers and a copy stream.  `Upload(host_tensor)` copies into the next pinned slot,
issues an asynchronous copy to a device buffer on the copy stream and returns (device tensor, completion token); the slot
is reused only after its copy finished (the ring blocks on the slot's own event, never on the device).  The compute
stream waits on the token, not the host.  `OaPrefetcher` wraps a batch iterator and keeps `depth` batches in flight."""
from __future__ import annotations

from typing import Iterable, Iterator, List, Optional, Sequence

import torch


class OaCompletionToken:
    def __init__(self, event=None):
        self._ev = event

    def IsComplete(self) -> bool:
        return self._ev is None or self._ev.query()

    def Wait(self) -> None:
        if self._ev is not None:
            self._ev.synchronize()

    def WaitOnStream(self, stream=None) -> None:
        if self._ev is not None:
            (stream or torch.cuda.current_stream()).wait_event(self._ev)


class OaUploadRing:
    def __init__(self, slot_bytes: int = 16 << 20, slots: int = 4, device: Optional[torch.device] = None):
        self.Cuda = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
        self.Device = torch.device(device) if device is not None else (torch.device("cuda", torch.cuda.current_device()) if self.Cuda else torch.device("cpu"))
        self.SlotBytes, self.Slots = int(slot_bytes), int(slots)
        self._host = [torch.empty(self.SlotBytes, dtype=torch.uint8, pin_memory=self.Cuda) for _ in range(self.Slots)]
        self._events = [None] * self.Slots
        self._stream = torch.cuda.Stream(self.Device) if self.Cuda else None
        self._next = 0
        self._batch_host, self._batch_events, self._batch_next = [None, None], [None, None], 0
        self.BytesUploaded = 0

    def Upload(self, host: torch.Tensor, out: Optional[torch.Tensor] = None):
        """Returns (device tensor, OaCompletionToken)."""
        host = host.contiguous()
        nbytes = host.numel() * host.element_size()
        if nbytes > self.SlotBytes:
            raise ValueError(f"upload of {nbytes} bytes exceeds the ring's slot size {self.SlotBytes}")
        i = self._next
        self._next = (i + 1) % self.Slots
        if self._events[i] is not None:
            self._events[i].synchronize()                     # the slot's previous copy must have left the host buffer
        stage = self._host[i][:nbytes].view(host.dtype).view(host.shape)
        stage.copy_(host)
        self.BytesUploaded += nbytes
        if not self.Cuda:
            dst = out if out is not None else torch.empty_like(host)
            dst.copy_(stage)
            return dst, OaCompletionToken()
        dst = out if out is not None else torch.empty(host.shape, dtype=host.dtype, device=self.Device)
        ev = torch.cuda.Event()
        with torch.cuda.stream(self._stream):
            dst.copy_(stage, non_blocking=True)
            ev.record(self._stream)
        dst.record_stream(self._stream) if out is None else None
        self._events[i] = ev
        return dst, OaCompletionToken(ev)

    def UploadMany(self, hosts: Sequence[torch.Tensor]):
        """Uploads a batch of small host tensors with one packed copy per dtype: the tensors are concatenated into a
        pinned staging buffer (double-buffered, grow-only), cross the bus as a single transfer, and come back as views of
        one device allocation.  Returns (list of device tensors in input order, OaCompletionToken).  Many 4 KiB uploads
        cost one launch of the copy engine this way instead of one each."""
        if not hosts:
            return [], OaCompletionToken()
        groups = {}
        for i, h in enumerate(hosts):
            groups.setdefault(h.dtype, []).append(i)
        outs: List[Optional[torch.Tensor]] = [None] * len(hosts)
        ev = None
        for dt, ids in groups.items():
            flat = [hosts[i].reshape(-1) for i in ids]
            counts = [f.numel() for f in flat]
            total = sum(counts)
            nbytes = total * flat[0].element_size()
            stage = self._batch_stage(nbytes)[:nbytes].view(dt)
            torch.cat(flat, out=stage)
            self.BytesUploaded += nbytes
            if self.Cuda:
                dev = torch.empty(total, dtype=dt, device=self.Device)
                with torch.cuda.stream(self._stream):
                    dev.copy_(stage, non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(self._stream)
                dev.record_stream(self._stream)
                self._batch_events[self._batch_next ^ 1] = ev
            else:
                dev = stage.clone()
            for i, piece in zip(ids, dev.split_with_sizes(counts)):
                outs[i] = piece if hosts[i].dim() == 1 else piece.view(hosts[i].shape)
        return outs, OaCompletionToken(ev)

    def _batch_stage(self, nbytes: int) -> torch.Tensor:
        i = self._batch_next
        self._batch_next = i ^ 1
        if self._batch_events[i] is not None:
            self._batch_events[i].synchronize()               # the previous transfer out of this buffer has left the host
            self._batch_events[i] = None
        if self._batch_host[i] is None or self._batch_host[i].numel() < nbytes:
            cap = 1 << max(12, (nbytes - 1).bit_length())
            self._batch_host[i] = torch.empty(cap, dtype=torch.uint8, pin_memory=self.Cuda)
        return self._batch_host[i]

    def Synchronize(self) -> None:
        for ev in list(self._events) + list(self._batch_events):
            if ev is not None:
                ev.synchronize()


class OaPrefetcher:
    """Iterates `source` (tuples of host tensors) and yields tuples of device tensors, `depth` uploads ahead."""

    def __init__(self, source: Iterable, ring: OaUploadRing, depth: int = 2):
        self._it: Iterator = iter(source)
        self._ring, self._depth, self._q = ring, max(1, depth), []

    def _fill(self) -> None:
        while len(self._q) < self._depth:
            try:
                item = next(self._it)
            except StopIteration:
                return
            item = item if isinstance(item, (tuple, list)) else (item,)
            self._q.append([self._ring.Upload(t) for t in item])

    def __iter__(self):
        return self

    def __next__(self):
        self._fill()
        if not self._q:
            raise StopIteration
        ups = self._q.pop(0)
        for _, tok in ups:
            tok.WaitOnStream() if self._ring.Cuda else tok.Wait()
        self._fill()
        out = tuple(t for t, _ in ups)
        return out if len(out) > 1 else out[0]
