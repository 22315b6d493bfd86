"""OaDeviceMesh: the ranks of one NVSwitch node, peer-mapped (symmetric) buffers, epoch-flag channels and the
device collectives.

Reference: Source/Public/Oa/Runtime/Topology.h:30-190 (OaDeviceMesh: devices, roles, links, CopyBuffer),
Source/Public/Oa/Runtime/Collective.h:23-71 (AllReduce / Broadcast / AllGather / Scatter / ReduceScatter over
f32 with Sum / Max / Min).  The reference stages collectives through host memory; here every rank is a process
that owns one GPU (`torch.distributed`, NCCL for bootstrap and as the baseline path), buffers are cudaMalloc'ed
by the kernel library and mapped into every peer with CUDA IPC, and kernels address `peer_ptr[r] + offset`
directly over NVLink.  Waits on peers are bounded on the device and surface as DeadlineExceeded on the host.
"""
from __future__ import annotations

import ctypes
import enum
from typing import Optional

import torch
import torch.distributed as dist

from .. import _native as N
from ..core.types import OaError, OaStatus, OaStatusCode
from ..ops import kernels as K


class OaInterconnect(enum.IntEnum):
    Unknown = 0
    PciE = 1
    NvLink = 2
    Xgmi = 3
    Host = 4


class OaReduceOp(enum.IntEnum):
    Sum = 0
    Max = 1
    Min = 2


class _CudaBuffer:
    """Exposes a raw device pointer through __cuda_array_interface__ so torch can alias it without copying."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class OaSymmetricBuffer:
    """A buffer of the same size on every rank; `peer_ptrs[r]` is rank r's buffer mapped into this process."""

    def __init__(self, mesh: "OaDeviceMesh", nbytes: int):
        lib = N.require()
        self.mesh = mesh
        self.nbytes = int(nbytes)
        p = ctypes.c_void_p()
        N.check(lib.oa_ipc_alloc(self.nbytes, ctypes.byref(p)), "oa_ipc_alloc")
        self.local_ptr = p.value
        self._opened: list[int] = []
        if mesh.world > 1:
            handle = ctypes.create_string_buffer(64)
            N.check(lib.oa_ipc_get_handle(self.local_ptr, handle), "oa_ipc_get_handle")
            handles = [None] * mesh.world
            dist.all_gather_object(handles, bytes(handle.raw), group=mesh.group)
            self.peer_ptrs = []
            for r, h in enumerate(handles):
                if r == mesh.rank:
                    self.peer_ptrs.append(self.local_ptr)
                else:
                    q = ctypes.c_void_p()
                    N.check(lib.oa_ipc_open(h, ctypes.byref(q)), f"oa_ipc_open(rank {r})")
                    self.peer_ptrs.append(q.value)
                    self._opened.append(q.value)
        else:
            self.peer_ptrs = [self.local_ptr]
        self.ptr_array = (ctypes.c_void_p * mesh.world)(*self.peer_ptrs)
        self.tensor = torch.as_tensor(_CudaBuffer(self.local_ptr, self.nbytes), device=mesh.device)

    def view(self, dtype: torch.dtype, numel: Optional[int] = None, byte_offset: int = 0) -> torch.Tensor:
        esz = torch.empty((), dtype=dtype).element_size()
        n = (self.nbytes - byte_offset) // esz if numel is None else numel
        return self.tensor[byte_offset: byte_offset + n * esz].view(dtype)

    def table(self, byte_offset: int = 0):
        """ctypes array of every rank's pointer advanced by `byte_offset` (kernel argument)."""
        return (ctypes.c_void_p * self.mesh.world)(*[p + byte_offset for p in self.peer_ptrs])

    def Close(self) -> None:
        lib = N.lib()
        if lib is None or self.local_ptr is None:
            return
        self.tensor = None
        for q in self._opened:
            lib.oa_ipc_close(q)
        self._opened = []
        lib.oa_ipc_free(self.local_ptr)
        self.local_ptr = None


class OaPeerChannel:
    """A ready/ack channel: one u64 slot per (receiver, sender) pair and a local epoch counter on the device."""

    def __init__(self, mesh: "OaDeviceMesh"):
        self.mesh = mesh
        self.flags = OaSymmetricBuffer(mesh, 8 * 16)     # 16 slots >= world
        self.epoch = torch.zeros(2, dtype=torch.int64, device=mesh.device)

    def Signal(self) -> None:
        m = self.mesh
        N.check(N.require().oa_peer_signal(self.flags.ptr_array, self.epoch.data_ptr(), m.rank, m.world, N.stream()), "oa_peer_signal")
        N.count_launch()

    def Wait(self) -> None:
        m = self.mesh
        N.check(N.require().oa_peer_wait(self.flags.local_ptr, self.epoch.data_ptr(), m.world, K.status_word(m.device).data_ptr(),
                                         N.stream()), "oa_peer_wait")
        N.count_launch()

    def Close(self) -> None:
        self.flags.Close()


class OaDeviceMesh:
    def __init__(self, group=None):
        if not dist.is_initialized():
            raise OaError(OaStatus.Error(OaStatusCode.FailedPrecondition, "torch.distributed is not initialised"))
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self._buffers: list = []
        self._channels: list = []
        self._barrier: Optional[OaPeerChannel] = None

    # ---- topology (Topology.h): one NVSwitch domain, uniform links
    def NumDevices(self) -> int:
        return self.world

    def LinkType(self, a: int, b: int) -> OaInterconnect:
        """What the driver says about the link between the devices of ranks a and b (one node: rank r runs on device r of
        the visible set): peer access with native atomics is NVLink / NVSwitch, peer access without them is PCIe, no peer
        access means staging through the host."""
        if self.device.type != "cuda":
            return OaInterconnect.Host
        if a == b:
            return OaInterconnect.Unknown
        n = torch.cuda.device_count()
        if a >= n or b >= n:
            return OaInterconnect.Unknown         # the other rank's device is not visible from this process
        out = (ctypes.c_int * 3)()
        if N.require().oa_p2p_attributes(int(a), int(b), out) != 0:
            return OaInterconnect.Unknown
        if not out[0]:
            return OaInterconnect.Host
        return OaInterconnect.NvLink if out[1] else OaInterconnect.PciE

    def CanAccessPeers(self) -> bool:
        if self.device.type != "cuda":
            return False
        me = self.device.index
        return all(torch.cuda.can_device_access_peer(me, d) for d in range(torch.cuda.device_count()) if d != me)

    # ---- allocation
    def AllocSymmetric(self, nbytes: int) -> OaSymmetricBuffer:
        b = OaSymmetricBuffer(self, (int(nbytes) + 255) // 256 * 256)
        self._buffers.append(b)
        return b

    def Release(self, buf: OaSymmetricBuffer) -> None:
        """Frees one symmetric buffer on every rank (a host collective: all ranks call it for the same buffer).  The caller
        has made sure that no kernel of any rank still touches it; the barrier keeps a rank from freeing memory that a
        peer still has mapped."""
        if buf in self._buffers:
            self._buffers.remove(buf)
        lib = N.lib()
        if lib is None or buf.local_ptr is None:
            return
        torch.cuda.synchronize()
        buf.tensor = None
        for q in buf._opened:
            lib.oa_ipc_close(q)
        buf._opened = []
        if dist.is_initialized() and self.world > 1:
            dist.barrier(group=self.group)
        lib.oa_ipc_free(buf.local_ptr)
        buf.local_ptr = None

    def NewChannel(self) -> OaPeerChannel:
        c = OaPeerChannel(self)
        self._channels.append(c)
        return c

    def SetPeerWaitMs(self, ms: int) -> None:
        """Upper bound of every device-side wait on a peer's flag (wall time).  Ranks drift apart by whole host phases (a
        data-loader stall, a checkpoint write): choose it above the longest such phase; a wait that runs out sets the kernel
        status word instead of hanging the stream."""
        N.check(N.require().oa_set_peer_wait_ms(int(ms)), "oa_set_peer_wait_ms")

    def Barrier(self) -> None:
        """Device-side barrier on the current stream: every rank signals, then waits for all (bounded)."""
        if self._barrier is None:
            self._barrier = self.NewChannel()
        self._barrier.Signal()
        self._barrier.Wait()

    def Close(self) -> None:
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        if dist.is_initialized() and self.world > 1:
            dist.barrier(group=self.group)
        for c in self._channels:
            c.Close()
        for b in self._buffers:
            b.Close()
        self._channels, self._buffers = [], []
