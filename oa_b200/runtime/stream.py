"""Streams, synchronisation tokens, one-shot dispatch, pre-allocated pools, the work-item queue, the static scheduler
and exported device memory.

Parity (paths inside the reference): Runtime/Stream.h:27-172 (OaVkStream), Runtime/Sync.h:9-108 (OaVkFence,
OaVkTimelineSemaphore, OaCompletionToken), Runtime/Dispatch.h + Dispatch.cpp:17-158 (OaVkDispatch),
Runtime/Pool.h:22-114 (OaVkInferencePool), Runtime/Persistent.h:11-58 (OaWorkQueue), Runtime/Scheduler.h:31-55
(OaScheduler), Runtime/ExternalMemory.h:17-122.

On this target a stream is a CUDA stream, a fence / timeline value is a recorded CUDA event, and exported memory is a
CUDA IPC handle.  Everything also works on a CPU engine, where work completes at submission.
"""
from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from ..core.types import OaStatus, OaStatusCode

OA_NODE_AUTO = 0xFFFFFFFF


def _cuda(device) -> bool:
    return torch.device(device).type == "cuda"


class OaFence:
    """Binary completion flag: `Signal(stream)` marks the point, `Wait` blocks the host until it passed."""

    def __init__(self, device="cpu", signaled: bool = False):
        self._device = torch.device(device)
        self._event = None
        self._signaled = signaled

    @staticmethod
    def Create(device="cpu", signaled: bool = False) -> "OaFence":
        return OaFence(device, signaled)

    def Signal(self, stream=None) -> None:
        if _cuda(self._device):
            self._event = torch.cuda.Event()
            self._event.record(stream if stream is not None else torch.cuda.current_stream(self._device))
        self._signaled = True

    def IsSignaled(self) -> bool:
        if not self._signaled:
            return False
        return self._event is None or self._event.query()

    def Wait(self, timeout_ns: Optional[int] = None) -> OaStatus:
        if not self._signaled:
            return OaStatus(OaStatusCode.FailedPrecondition, "fence was never signalled")
        if self._event is None:
            return OaStatus.Ok()
        if timeout_ns is None:
            self._event.synchronize()
            return OaStatus.Ok()
        deadline = time.monotonic_ns() + timeout_ns
        while not self._event.query():
            if time.monotonic_ns() > deadline:
                return OaStatus(OaStatusCode.DeadlineExceeded, "fence wait timed out")
            time.sleep(50e-6)
        return OaStatus.Ok()

    def Reset(self) -> None:
        self._event, self._signaled = None, False


class OaTimelineSemaphore:
    """Monotonic counter: work submitted with `Signal(value)` makes `Value()` reach `value` when it completes."""

    def __init__(self, device="cpu", initial: int = 0):
        self._device = torch.device(device)
        self._completed = initial
        self._pending: List[Tuple[int, object]] = []     # (value, event), ascending

    @staticmethod
    def Create(device="cpu", initial: int = 0) -> "OaTimelineSemaphore":
        return OaTimelineSemaphore(device, initial)

    def Signal(self, value: int, stream=None) -> OaStatus:
        last = self._pending[-1][0] if self._pending else self._completed
        if value <= last:
            return OaStatus(OaStatusCode.InvalidArgument, f"timeline value {value} does not advance past {last}")
        if _cuda(self._device):
            ev = torch.cuda.Event()
            ev.record(stream if stream is not None else torch.cuda.current_stream(self._device))
            self._pending.append((value, ev))
        else:
            self._completed = value
        return OaStatus.Ok()

    def _poll(self) -> None:
        while self._pending and self._pending[0][1].query():
            self._completed = self._pending.pop(0)[0]

    def Value(self) -> int:
        self._poll()
        return self._completed

    def LastSubmitted(self) -> int:
        return self._pending[-1][0] if self._pending else self._completed

    def Wait(self, value: int, timeout_ns: Optional[int] = None) -> OaStatus:
        if value > self.LastSubmitted():
            return OaStatus(OaStatusCode.FailedPrecondition, f"nothing submitted will signal {value}")
        deadline = None if timeout_ns is None else time.monotonic_ns() + timeout_ns
        while self.Value() < value:
            target = next(ev for v, ev in self._pending if v >= value)
            if deadline is None:
                target.synchronize()
            elif time.monotonic_ns() > deadline:
                return OaStatus(OaStatusCode.DeadlineExceeded, "timeline wait timed out")
            else:
                time.sleep(50e-6)
        return OaStatus.Ok()

    def WaitOn(self, value: int, stream) -> None:
        """Make `stream` wait (on the device) until `value` is reached."""
        for v, ev in self._pending:
            if v >= value:
                stream.wait_event(ev)
                return


@dataclass
class OaCompletionToken:
    """(semaphore, value) pair naming one submission."""
    Semaphore: Optional[OaTimelineSemaphore] = None
    Value: int = 0

    def IsValid(self) -> bool: return self.Semaphore is not None and self.Value > 0
    def IsComplete(self) -> bool: return self.IsValid() and self.Semaphore.Value() >= self.Value

    def Wait(self, timeout_ns: Optional[int] = None) -> OaStatus:
        if not self.IsValid():
            return OaStatus(OaStatusCode.InvalidArgument, "invalid completion token")
        return self.Semaphore.Wait(self.Value, timeout_ns)

    def IsSameCompletion(self, other: "OaCompletionToken") -> bool:
        return self.IsValid() and other.IsValid() and self.Semaphore is other.Semaphore and self.Value == other.Value


class OaStream:
    """Ordered queue of work with its own timeline: `Begin` ... record ... `Submit` -> token."""

    def __init__(self, device="cpu", priority: int = 0, name: str = "stream"):
        self._device = torch.device(device)
        self.Name = name
        self._cuda_stream = torch.cuda.Stream(device=self._device, priority=priority) if _cuda(self._device) else None
        self._timeline = OaTimelineSemaphore(self._device)
        self._recorded: List[Callable[[], None]] = []
        self._recording = False
        self._submissions = 0

    @staticmethod
    def Create(device="cpu", priority: int = 0, name: str = "stream") -> "OaStream":
        return OaStream(device, priority, name)

    def Handle(self):
        return self._cuda_stream

    def Timeline(self) -> OaTimelineSemaphore:
        return self._timeline

    def Begin(self) -> OaStatus:
        if self._recording:
            return OaStatus(OaStatusCode.FailedPrecondition, "stream is already recording")
        self._recording, self._recorded = True, []
        return OaStatus.Ok()

    def Record(self, fn: Callable[[], None]) -> None:
        """Queue a launch (any callable that enqueues work on the current stream)."""
        if not self._recording:
            raise RuntimeError("Record outside Begin / Submit")
        self._recorded.append(fn)

    def RecordCopyBuffer(self, dst: torch.Tensor, src: torch.Tensor) -> None:
        self.Record(lambda: dst.copy_(src, non_blocking=True))

    def RecordFillBuffer(self, dst: torch.Tensor, value) -> None:
        self.Record(lambda: dst.fill_(value))

    def _run(self, wait: Optional[OaCompletionToken]) -> OaCompletionToken:
        value = self._timeline.LastSubmitted() + 1
        if self._cuda_stream is not None:
            if wait is not None and wait.IsValid():
                wait.Semaphore.WaitOn(wait.Value, self._cuda_stream)
            with torch.cuda.stream(self._cuda_stream):
                for fn in self._recorded:
                    fn()
        else:
            if wait is not None and wait.IsValid():
                wait.Wait()
            for fn in self._recorded:
                fn()
        self._timeline.Signal(value, self._cuda_stream)
        self._recording, self._recorded = False, []
        self._submissions += 1
        return OaCompletionToken(self._timeline, value)

    def Submit(self) -> OaCompletionToken:
        if not self._recording:
            raise RuntimeError("Submit without Begin")
        return self._run(None)

    def SubmitWithDependency(self, wait: OaCompletionToken) -> OaCompletionToken:
        if not self._recording:
            raise RuntimeError("Submit without Begin")
        return self._run(wait)

    def SubmitAndWait(self) -> OaStatus:
        return self.Submit().Wait()

    def Synchronize(self) -> OaStatus:
        if self._cuda_stream is not None:
            self._cuda_stream.synchronize()
        return OaStatus.Ok()

    def SubmissionCount(self) -> int:
        return self._submissions


class OaStreamPool:
    """Round-robin pool of streams (the engine's compute / transfer queues)."""

    def __init__(self, device="cpu", count: int = 4, priority: int = 0):
        self._streams = [OaStream(device, priority, f"pool{i}") for i in range(max(1, count))]
        self._next = 0

    def Acquire(self) -> OaStream:
        s = self._streams[self._next % len(self._streams)]
        self._next += 1
        return s

    def Size(self) -> int: return len(self._streams)

    def SynchronizeAll(self) -> None:
        for s in self._streams:
            s.Synchronize()


class OaDispatch:
    """One-shot helpers: run a launch now, or batch several and flush them as one submission."""

    def __init__(self, stream: Optional[OaStream] = None, device="cpu"):
        self._stream = stream or OaStream(device, name="dispatch")
        self._batch: Optional[List[Callable[[], None]]] = None

    def Run(self, fn: Callable[[], None]) -> OaStatus:
        self._stream.Begin()
        self._stream.Record(fn)
        return self._stream.SubmitAndWait()

    def RunOn(self, stream: OaStream, fn: Callable[[], None]) -> OaCompletionToken:
        stream.Begin()
        stream.Record(fn)
        return stream.Submit()

    def BeginBatch(self) -> None:
        self._batch = []

    def Record(self, fn: Callable[[], None]) -> None:
        if self._batch is None:
            raise RuntimeError("Record outside BeginBatch / Flush")
        self._batch.append(fn)

    def Flush(self, wait: bool = True):
        if self._batch is None:
            raise RuntimeError("Flush without BeginBatch")
        self._stream.Begin()
        for fn in self._batch:
            self._stream.Record(fn)
        self._batch = None
        tok = self._stream.Submit()
        return tok.Wait() if wait else tok


# ------------------------------------------------------------------------------------------ pre-allocated pools
@dataclass
class OaInferencePoolConfig:
    NumLayers: int = 0
    ActivationSize: int = 0            # bytes per (layer, batch slot)
    MaxBatchSize: int = 1
    OutputRingBytes: int = 0
    OutputSlotBytes: int = 0           # 0: the ring is one slot
    PinWeights: bool = True


class OaInferencePool:
    """Everything a serving session needs, allocated once: per-layer activation slots for every batch slot, an output
    ring the host drains, and the pinned weight buffers.  After `Init` a decode step allocates nothing, which is what
    lets it replay as a CUDA graph."""

    def __init__(self):
        self._cfg: Optional[OaInferencePoolConfig] = None
        self._act: Optional[torch.Tensor] = None
        self._ring: Optional[torch.Tensor] = None
        self._weights: List[torch.Tensor] = []
        self._head = self._tail = 0

    def Init(self, device, config: OaInferencePoolConfig) -> OaStatus:
        if config.NumLayers <= 0 or config.ActivationSize <= 0 or config.MaxBatchSize <= 0:
            return OaStatus(OaStatusCode.InvalidArgument, "inference pool needs layers, an activation size and a batch size")
        slot = config.OutputSlotBytes or config.OutputRingBytes
        if config.OutputRingBytes and config.OutputRingBytes % slot:
            return OaStatus(OaStatusCode.InvalidArgument, "output ring is not a whole number of slots")
        self._cfg = config
        self._stride = (config.ActivationSize + 255) & ~255             # 256-byte aligned slots
        total = config.NumLayers * config.MaxBatchSize * self._stride
        raw = torch.empty(total + 256, dtype=torch.uint8, device=device)        # host allocations are only 64-byte aligned
        skew = (-raw.data_ptr()) % 256
        self._act = raw[skew:skew + total]
        self._ring = torch.empty(config.OutputRingBytes, dtype=torch.uint8, device=device) if config.OutputRingBytes else None
        self._slots = (config.OutputRingBytes // slot) if config.OutputRingBytes else 0
        self._slot_bytes = slot
        self._head = self._tail = 0
        return OaStatus.Ok()

    def Destroy(self) -> None:
        self._act = self._ring = self._cfg = None
        self._weights = []

    def IsValid(self) -> bool: return self._act is not None
    def TotalBytes(self) -> int:
        return (self._act.numel() if self._act is not None else 0) + (self._ring.numel() if self._ring is not None else 0)

    def GetActivation(self, layer: int, batch_slot: int, dtype: torch.dtype = torch.uint8) -> Optional[torch.Tensor]:
        c = self._cfg
        if c is None or not (0 <= layer < c.NumLayers and 0 <= batch_slot < c.MaxBatchSize):
            return None
        off = (layer * c.MaxBatchSize + batch_slot) * self._stride
        return self._act[off:off + c.ActivationSize].view(dtype)

    def NextOutputSlot(self) -> Optional[torch.Tensor]:
        """The next free slot of the output ring, or None while the consumer is a full ring behind."""
        if not self._slots or self._head - self._tail >= self._slots:
            return None
        i = self._head % self._slots
        self._head += 1
        return self._ring[i * self._slot_bytes:(i + 1) * self._slot_bytes]

    def ConsumeOutputSlot(self) -> None:
        if self._tail < self._head:
            self._tail += 1

    def PendingOutputs(self) -> int: return self._head - self._tail

    def PinWeights(self, weights: torch.Tensor) -> OaStatus:
        if self._cfg is None:
            return OaStatus(OaStatusCode.FailedPrecondition, "pool is not initialised")
        if self._cfg.PinWeights:
            self._weights.append(weights)          # held for the pool's lifetime
        return OaStatus.Ok()

    def ResetSession(self) -> None:
        self._head = self._tail = 0
        if self._act is not None:
            self._act.zero_()


# ------------------------------------------------------------------------------------------ work-item queue
@dataclass
class OaWorkItem:
    GroupsX: int = 0
    GroupsY: int = 0
    GroupsZ: int = 0
    PushOffset: int = 0


class OaWorkQueue:
    """Ring of work items + a push-constant arena.  The host enqueues items, `Flush` hands every pending item to the
    consumer in order on one stream submission (one launch per item, or one launch for the whole batch when the
    consumer takes the item table), and `Consumed` counts what has been handed over.  The consumer never polls a flag
    written by the host, so nothing on the device waits on the host."""

    def __init__(self, capacity: int, max_push_bytes: int = 4096, device="cpu",
                 consumer: Optional[Callable[[OaWorkItem, memoryview], None]] = None,
                 batch_consumer: Optional[Callable[[torch.Tensor, torch.Tensor], None]] = None):
        if capacity <= 0:
            raise ValueError("capacity must be positive")
        self.Capacity, self.Head = capacity, 0
        self._consumed = 0
        self._device = torch.device(device)
        self._items = torch.zeros(capacity, 4, dtype=torch.int32)               # host ring
        self._push = bytearray(max_push_bytes)
        self._consumer, self._batch_consumer = consumer, batch_consumer
        self._stream = OaStream(device, name="workqueue")

    @staticmethod
    def Create(capacity: int, max_push_bytes: int = 4096, device="cpu", **kw) -> "OaWorkQueue":
        return OaWorkQueue(capacity, max_push_bytes, device, **kw)

    def Enqueue(self, item: OaWorkItem) -> bool:
        if self.Head - self._consumed >= self.Capacity:
            return False
        if item.PushOffset < 0 or item.PushOffset >= max(1, len(self._push)):
            return False
        self._items[self.Head % self.Capacity] = torch.tensor([item.GroupsX, item.GroupsY, item.GroupsZ, item.PushOffset], dtype=torch.int32)
        self.Head += 1
        return True

    def WritePush(self, offset: int, data: bytes) -> None:
        if offset < 0 or offset + len(data) > len(self._push):
            raise ValueError("push data outside the arena")
        self._push[offset:offset + len(data)] = data

    def Pending(self) -> int: return self.Head - self._consumed
    def Consumed(self) -> int: return self._consumed

    def Flush(self) -> OaStatus:
        n = self.Pending()
        if n == 0:
            return OaStatus.Ok()
        order = [(self._consumed + i) % self.Capacity for i in range(n)]
        table = self._items[order]
        self._stream.Begin()
        if self._batch_consumer is not None:
            push = torch.frombuffer(bytearray(self._push), dtype=torch.uint8)
            dev_table, dev_push = table.to(self._device), push.to(self._device)
            self._stream.Record(lambda: self._batch_consumer(dev_table, dev_push))
        elif self._consumer is not None:
            view = memoryview(self._push)
            for row in table.tolist():
                item = OaWorkItem(*row)
                self._stream.Record(lambda item=item: self._consumer(item, view[item.PushOffset:]))
        st = self._stream.SubmitAndWait()
        self._consumed += n
        return st


# ------------------------------------------------------------------------------------------ static scheduler
class OaComputeClass(enum.IntEnum):
    Heavy = 0      # large matrix products, convolutions: primary device
    Light = 1      # norms, activations, reductions: may go to an auxiliary device
    Transfer = 2   # data movement
    Any = 3


def OaComputeClassName(c: OaComputeClass) -> str:
    return OaComputeClass(c).name


@dataclass
class OaDispatchHint:
    Class: OaComputeClass = OaComputeClass.Any
    PreferNode: int = OA_NODE_AUTO


class OaScheduler:
    """Static router over a list of device nodes (index 0 is the primary).  With SPMD ranks every process owns one
    GPU, so routing only matters for single-process multi-device tools; the policy is the reference's: Heavy and Any
    go to the primary, Light and Transfer to the first auxiliary device when there is one, an explicit node wins."""

    def __init__(self, num_nodes: int = 1):
        self.NumNodes = max(1, num_nodes)
        self.Routed: Dict[int, int] = {}

    @staticmethod
    def Create(mesh_or_count) -> "OaScheduler":
        n = mesh_or_count if isinstance(mesh_or_count, int) else mesh_or_count.NumDevices()
        return OaScheduler(n)

    def Route(self, hint) -> int:
        if isinstance(hint, OaComputeClass):
            hint = OaDispatchHint(hint)
        if hint.PreferNode != OA_NODE_AUTO:
            node = hint.PreferNode if 0 <= hint.PreferNode < self.NumNodes else 0
        elif hint.Class in (OaComputeClass.Light, OaComputeClass.Transfer) and self.NumNodes > 1:
            node = 1
        else:
            node = 0
        self.Routed[node] = self.Routed.get(node, 0) + 1
        return node


# ------------------------------------------------------------------------------------------ exported memory
@dataclass
class OaExternalMemoryHandle:
    """What travels to the importing process: the 64-byte CUDA IPC handle, the size and the exporting device."""
    Handle: bytes = b""
    Size: int = 0
    Device: int = 0

    def IsValid(self) -> bool: return len(self.Handle) == 64 and self.Size > 0

    def Pack(self) -> bytes:
        return self.Size.to_bytes(8, "little") + self.Device.to_bytes(4, "little") + self.Handle

    @staticmethod
    def Unpack(blob: bytes) -> "OaExternalMemoryHandle":
        if len(blob) != 76:
            raise ValueError("an exported-memory record is 76 bytes")
        return OaExternalMemoryHandle(blob[12:], int.from_bytes(blob[:8], "little"), int.from_bytes(blob[8:12], "little"))


class OaExternalMemory:
    """Export a device allocation to / import one from another process on the same machine (CUDA IPC).  The peer
    pointer tables of the symmetric buffers are built from the same primitive."""

    def __init__(self):
        self._ptr = 0
        self._size = 0
        self._owned = self._imported = False

    @staticmethod
    def _native():
        from .. import _native as N
        return N, N.require()

    @staticmethod
    def Allocate(nbytes: int) -> "OaExternalMemory":
        import ctypes
        N, lib = OaExternalMemory._native()
        m, p = OaExternalMemory(), ctypes.c_void_p()
        N.check(lib.oa_ipc_alloc(nbytes, ctypes.byref(p)), "oa_ipc_alloc")
        m._ptr, m._size, m._owned = p.value, nbytes, True
        return m

    def Export(self) -> OaExternalMemoryHandle:
        import ctypes
        N, lib = self._native()
        h = (ctypes.c_ubyte * 64)()
        N.check(lib.oa_ipc_get_handle(ctypes.c_void_p(self._ptr), h), "oa_ipc_get_handle")
        return OaExternalMemoryHandle(bytes(h), self._size, torch.cuda.current_device())

    @staticmethod
    def Import(handle: OaExternalMemoryHandle) -> "OaExternalMemory":
        import ctypes
        if not handle.IsValid():
            raise ValueError("invalid exported-memory handle")
        N, lib = OaExternalMemory._native()
        m, q = OaExternalMemory(), ctypes.c_void_p()
        h = (ctypes.c_ubyte * 64).from_buffer_copy(handle.Handle)
        N.check(lib.oa_ipc_open(h, ctypes.byref(q)), "oa_ipc_open")
        m._ptr, m._size, m._imported = q.value, handle.Size, True
        return m

    def Address(self) -> int: return self._ptr
    def Size(self) -> int: return self._size

    def Close(self) -> None:
        if not self._ptr:
            return
        _, lib = self._native()
        import ctypes
        if self._imported:
            lib.oa_ipc_close(ctypes.c_void_p(self._ptr))
        elif self._owned:
            lib.oa_ipc_free(ctypes.c_void_p(self._ptr))
        self._ptr = 0


# ------------------------------------------------------------------------------------------ hashing / signature pool
@dataclass
class OaPqcPoolConfig:
    MaxConcurrentSigns: int = 64
    MaxConcurrentHashes: int = 64
    NttSlotSize: int = 1024
    HashSlotSize: int = 200          # one Keccak state
    KeyCapacity: int = 64 << 10


class OaSecureBuffer:
    """A slice of the key arena that is overwritten with zeros when released."""

    def __init__(self, view: Optional[torch.Tensor]):
        self._v = view

    def IsValid(self) -> bool: return self._v is not None
    def Size(self) -> int: return 0 if self._v is None else self._v.numel()
    def Tensor(self) -> Optional[torch.Tensor]: return self._v

    def Release(self) -> None:
        if self._v is not None:
            self._v.zero_()
            self._v = None

    def __del__(self):
        self.Release()


class OaPqcPool:
    """Fixed slots for transform and hash states plus a bump arena for key material (Runtime/Pool.h:70-114): a batch of
    hashing or signing work takes its scratch from here instead of allocating.  Slot occupancy is a 64-bit bitmap per
    kind, as in the reference, so at most 64 slots of each kind exist."""

    def __init__(self):
        self._cfg: Optional[OaPqcPoolConfig] = None
        self._ntt = self._hash = self._key = None
        self._ntt_bits = self._hash_bits = 0
        self._key_off = 0

    def Init(self, device, config: Optional[OaPqcPoolConfig] = None) -> OaStatus:
        c = config or OaPqcPoolConfig()
        if not (0 < c.MaxConcurrentSigns <= 64 and 0 < c.MaxConcurrentHashes <= 64) or c.NttSlotSize <= 0 or c.HashSlotSize <= 0:
            return OaStatus(OaStatusCode.InvalidArgument, "between 1 and 64 slots of a positive size are required")
        self._cfg = c
        self._ntt = torch.zeros(c.MaxConcurrentSigns, c.NttSlotSize, dtype=torch.uint8, device=device)
        self._hash = torch.zeros(c.MaxConcurrentHashes, c.HashSlotSize, dtype=torch.uint8, device=device)
        self._key = torch.zeros(c.KeyCapacity, dtype=torch.uint8, device=device)
        self._ntt_bits = self._hash_bits = self._key_off = 0
        return OaStatus.Ok()

    def Destroy(self) -> None:
        if self._key is not None:
            self._key.zero_()
        self._ntt = self._hash = self._key = self._cfg = None

    @staticmethod
    def _take(bits: int, limit: int):
        for i in range(limit):
            if not (bits >> i) & 1:
                return i, bits | (1 << i)
        return -1, bits

    def AllocNttSlot(self) -> Optional[torch.Tensor]:
        if self._cfg is None:
            return None
        i, self._ntt_bits = self._take(self._ntt_bits, self._cfg.MaxConcurrentSigns)
        return None if i < 0 else self._ntt[i]

    def AllocHashSlot(self) -> Optional[torch.Tensor]:
        if self._cfg is None:
            return None
        i, self._hash_bits = self._take(self._hash_bits, self._cfg.MaxConcurrentHashes)
        return None if i < 0 else self._hash[i]

    def _slot_of(self, arena: torch.Tensor, slot: torch.Tensor) -> int:
        off = slot.data_ptr() - arena.data_ptr()
        stride = arena.shape[1]
        return off // stride if 0 <= off < arena.numel() and off % stride == 0 else -1

    def FreeNttSlot(self, slot: torch.Tensor) -> None:
        i = self._slot_of(self._ntt, slot)
        if i >= 0:
            self._ntt_bits &= ~(1 << i)

    def FreeHashSlot(self, slot: torch.Tensor) -> None:
        i = self._slot_of(self._hash, slot)
        if i >= 0:
            self._hash[i].zero_()
            self._hash_bits &= ~(1 << i)

    def AllocKeyBuffer(self, size: int) -> OaSecureBuffer:
        size_al = (size + 15) & ~15
        if self._key is None or size <= 0 or self._key_off + size_al > self._key.numel():
            return OaSecureBuffer(None)
        view = self._key[self._key_off:self._key_off + size]
        self._key_off += size_al
        return OaSecureBuffer(view)

    def NttSlotsUsed(self) -> int: return bin(self._ntt_bits).count("1")
    def HashSlotsUsed(self) -> int: return bin(self._hash_bits).count("1")
