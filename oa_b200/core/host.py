"""Python faces of the native host primitives in `csrc/runtime/host.cpp`.

`OaSimd` (Source/Public/Oa/Core/Simd.h:17-29), the streaming copy and aligned allocation of Core/Memory.h:30-156,
`OaCpuTopology`, `OaChannel`, `OaTask` and `OaThreadPool` (Core/Thread.h:26-470).  The vector functions work in
place on fp32 numpy arrays or CPU torch tensors; the pool runs Python callables (through a C callback that takes
the GIL) as well as the native sharded copy / dot jobs that feed pinned upload buffers without the GIL.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence

import numpy as np
import torch

from ..io.oam import runtime_lib

_ready = False
_JOB = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p)


def _lib():
    global _ready
    L = runtime_lib()
    if _ready:
        return L
    vp, u64, i32, i64, f32 = ctypes.c_void_p, ctypes.c_uint64, ctypes.c_int, ctypes.c_int64, ctypes.c_float
    P = ctypes.POINTER
    sig = {
        "oa_simd_level": (i32, []), "oa_simd_dot_f32": (f32, [vp, vp, i64]),
        "oa_memcpy_nt": (vp, [vp, vp, ctypes.c_size_t]), "oa_mem_equal": (i32, [vp, vp, ctypes.c_size_t]),
        "oa_aligned_alloc": (vp, [ctypes.c_size_t, ctypes.c_size_t]), "oa_aligned_free": (None, [vp]),
        "oa_cpu_topology_detect": (vp, []), "oa_cpu_topology_destroy": (None, [vp]),
        "oa_cpu_topology_count": (i32, [vp, i32]), "oa_cpu_topology_core": (i32, [vp, i32, P(i32)]),
        "oa_spinlock_stress": (u64, [i32, i32]), "oa_rwlock_stress": (u64, [i32, i32, i32]),
        "oa_channel_create": (vp, [u64]), "oa_channel_destroy": (None, [vp]), "oa_channel_send": (i32, [vp, u64, i32]),
        "oa_channel_recv": (i32, [vp, P(u64), i32]), "oa_channel_close": (None, [vp]), "oa_channel_size": (u64, [vp]),
        "oa_pool_create": (vp, [i32, P(i32), i32]), "oa_pool_num_workers": (i32, [vp]), "oa_pool_executed": (u64, [vp]),
        "oa_pool_submit": (u64, [vp, _JOB, vp]), "oa_pool_wait": (i32, [vp, u64]), "oa_pool_shutdown": (None, [vp]),
        "oa_pool_destroy": (None, [vp]), "oa_pool_parallel_copy": (i32, [vp, vp, vp, u64, i32]),
        "oa_pool_parallel_dot": (ctypes.c_double, [vp, vp, vp, i64, i32]),
    }
    for op in ("scale", "add", "sub", "mul", "div", "neg"):
        sig[f"oa_simd_{op}_f32"] = (None, [vp, vp, f32, i64])
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype, fn.argtypes = res, args
    _ready = True
    return L


def _span(x, writable: bool = False):
    """(address, element count) of a contiguous fp32 numpy array or CPU tensor."""
    if isinstance(x, torch.Tensor):
        if x.device.type != "cpu" or x.dtype != torch.float32 or not x.is_contiguous():
            raise ValueError("expected a contiguous fp32 CPU tensor")
        return x.data_ptr(), x.numel()
    a = np.asarray(x)
    if a.dtype != np.float32 or not a.flags.c_contiguous or (writable and not a.flags.writeable):
        raise ValueError("expected a contiguous fp32 array")
    return a.ctypes.data, a.size


def _bytes_span(x):
    if isinstance(x, torch.Tensor):
        if x.device.type != "cpu" or not x.is_contiguous():
            raise ValueError("expected a contiguous CPU tensor")
        return x.data_ptr(), x.numel() * x.element_size()
    a = np.asarray(x)
    if not a.flags.c_contiguous:
        raise ValueError("expected a contiguous array")
    return a.ctypes.data, a.nbytes


class OaSimd:
    """In-place fp32 vector math on host memory."""

    @staticmethod
    def Level() -> int:
        """1 = baseline vectors, 2 = AVX2 + FMA."""
        return _lib().oa_simd_level()

    @staticmethod
    def DotF32(a, b) -> float:
        (pa, na), (pb, nb) = _span(a), _span(b)
        if na != nb:
            raise ValueError("length mismatch")
        return float(_lib().oa_simd_dot_f32(pa, pb, na))

    @staticmethod
    def _binary(name: str, a, b) -> None:
        (pa, na), (pb, nb) = _span(a, True), _span(b)
        if na != nb:
            raise ValueError("length mismatch")
        getattr(_lib(), name)(pa, pb, 0.0, na)

    @staticmethod
    def ScaleF32(a, scale: float) -> None:
        pa, na = _span(a, True)
        _lib().oa_simd_scale_f32(pa, None, float(scale), na)

    @staticmethod
    def NegF32(a) -> None:
        pa, na = _span(a, True)
        _lib().oa_simd_neg_f32(pa, None, 0.0, na)

    @staticmethod
    def AddF32(a, b) -> None: OaSimd._binary("oa_simd_add_f32", a, b)

    @staticmethod
    def SubF32(a, b) -> None: OaSimd._binary("oa_simd_sub_f32", a, b)

    @staticmethod
    def MulF32(a, b) -> None: OaSimd._binary("oa_simd_mul_f32", a, b)

    @staticmethod
    def DivF32(a, b) -> None: OaSimd._binary("oa_simd_div_f32", a, b)


def OaMemcpyNT(dst, src) -> None:
    """Copy `src` into `dst` (same byte size); large copies use streaming stores."""
    (pd, nd), (ps, ns) = _bytes_span(dst), _bytes_span(src)
    if nd != ns:
        raise ValueError("size mismatch")
    _lib().oa_memcpy_nt(pd, ps, nd)


def OaMemEqual(a, b) -> bool:
    (pa, na), (pb, nb) = _bytes_span(a), _bytes_span(b)
    return na == nb and bool(_lib().oa_mem_equal(pa, pb, na))


class OaAlignedBuffer:
    """Host allocation with a chosen alignment (default one cache line), exposed as a uint8 numpy array."""

    def __init__(self, size: int, alignment: int = 64):
        self._L = _lib()
        self._p = self._L.oa_aligned_alloc(size, alignment)
        if not self._p:
            raise MemoryError(f"aligned allocation of {size} bytes failed")
        self.Size, self.Alignment = size, alignment
        self.Array = np.ctypeslib.as_array((ctypes.c_uint8 * size).from_address(self._p))

    @property
    def Address(self) -> int: return self._p

    def __del__(self):
        if getattr(self, "_p", None):
            self.Array = None
            self._L.oa_aligned_free(self._p)
            self._p = None


@dataclass
class OaCoreInfo:
    Id: int = -1
    PackageId: int = 0
    NumaNode: int = 0
    MaxFreqKhz: int = 0
    CoreId: int = 0


class OaCpuTopology:
    """Cores this process may run on, with package / NUMA node / maximum frequency from sysfs."""

    def __init__(self):
        self.Cores: List[OaCoreInfo] = []
        self.NumPhysicalCores = self.NumLogicalCores = 0
        self.NumNumaNodes = self.NumPackages = 1

    @staticmethod
    def Detect() -> "OaCpuTopology":
        L = _lib()
        h = L.oa_cpu_topology_detect()
        t = OaCpuTopology()
        t.NumLogicalCores, t.NumPhysicalCores = L.oa_cpu_topology_count(h, 0), L.oa_cpu_topology_count(h, 1)
        t.NumNumaNodes, t.NumPackages = L.oa_cpu_topology_count(h, 2), L.oa_cpu_topology_count(h, 3)
        buf = (ctypes.c_int * 5)()
        for i in range(t.NumLogicalCores):
            L.oa_cpu_topology_core(h, i, buf)
            t.Cores.append(OaCoreInfo(buf[0], buf[1], buf[2], buf[3], buf[4]))
        L.oa_cpu_topology_destroy(h)
        return t

    def GetCoresOnNuma(self, node: int) -> List[int]:
        return [c.Id for c in self.Cores if c.NumaNode == node]

    def GetPcoreIds(self) -> List[int]:
        """Ids of the fastest cores (all of them on a homogeneous part)."""
        top = max((c.MaxFreqKhz for c in self.Cores), default=0)
        return [c.Id for c in self.Cores if c.MaxFreqKhz == top]

    def GetEcoreIds(self) -> List[int]:
        top = max((c.MaxFreqKhz for c in self.Cores), default=0)
        return [c.Id for c in self.Cores if c.MaxFreqKhz < top]

    def Print(self) -> None:
        print(f"cpu: {self.NumLogicalCores} logical / {self.NumPhysicalCores} physical cores, "
              f"{self.NumPackages} package(s), {self.NumNumaNodes} NUMA node(s)")


class OaChannel:
    """Bounded multi-producer multi-consumer queue of unsigned 64-bit values (ids, offsets, handles)."""

    def __init__(self, capacity: int = 64):
        self._L = _lib()
        self._h = self._L.oa_channel_create(capacity)

    def __del__(self):
        if getattr(self, "_h", None):
            self._L.oa_channel_destroy(self._h)
            self._h = None

    def Send(self, value: int) -> bool: return bool(self._L.oa_channel_send(self._h, value, 1))
    def TrySend(self, value: int) -> bool: return bool(self._L.oa_channel_send(self._h, value, 0))

    def Recv(self) -> Optional[int]:
        out = ctypes.c_uint64()
        return out.value if self._L.oa_channel_recv(self._h, ctypes.byref(out), 1) else None

    def TryRecv(self) -> Optional[int]:
        out = ctypes.c_uint64()
        return out.value if self._L.oa_channel_recv(self._h, ctypes.byref(out), 0) else None

    def Close(self) -> None: self._L.oa_channel_close(self._h)
    def Size(self) -> int: return self._L.oa_channel_size(self._h)


@dataclass
class OaThreadPoolConfig:
    NumWorkers: int = 0
    PinToCores: bool = True
    UseTopology: bool = True
    CoreIds: Sequence[int] = ()


class OaTask:
    """Handle of a submitted job; `Wait()` blocks and returns the job's value (or re-raises its exception)."""

    def __init__(self, pool: "OaThreadPool", task_id: int, box: dict, keep):
        self._pool, self._id, self._box, self._keep = pool, task_id, box, keep
        self._waited = False

    def Wait(self):
        if not self._waited:
            self._pool._L.oa_pool_wait(self._pool._h, self._id)
            self._waited, self._keep = True, None
        if "error" in self._box:
            raise self._box["error"]
        return self._box.get("value")

    def IsReady(self) -> bool:
        return self._waited or "value" in self._box or "error" in self._box


class OaThreadPool:
    def __init__(self, config: Optional[OaThreadPoolConfig] = None):
        cfg = config or OaThreadPoolConfig()
        self._L = _lib()
        ids = list(cfg.CoreIds)
        if cfg.PinToCores and not ids and cfg.UseTopology:
            ids = [c.Id for c in OaCpuTopology.Detect().Cores]
        n = cfg.NumWorkers or max(1, len(ids)) if cfg.PinToCores else cfg.NumWorkers
        arr = (ctypes.c_int * len(ids))(*ids) if (cfg.PinToCores and ids) else None
        self._h = self._L.oa_pool_create(int(n or 0), arr, len(ids) if arr is not None else 0)

    @staticmethod
    def Create(config: Optional[OaThreadPoolConfig] = None) -> "OaThreadPool":
        return OaThreadPool(config)

    def NumWorkers(self) -> int: return self._L.oa_pool_num_workers(self._h)
    def Executed(self) -> int: return self._L.oa_pool_executed(self._h)

    def SubmitTask(self, fn: Callable[[], object]) -> OaTask:
        box: dict = {}

        def run(_arg):
            try:
                box["value"] = fn()
                return 0
            except BaseException as e:   # delivered to the waiter
                box["error"] = e
                return 1

        cb = _JOB(run)
        tid = self._L.oa_pool_submit(self._h, cb, None)
        if tid == 0:
            raise RuntimeError("thread pool is shut down")
        return OaTask(self, tid, box, cb)

    def Submit(self, fn: Callable[[], object]) -> None:
        self._pending = [t for t in getattr(self, "_pending", []) if not t.IsReady()]
        self._pending.append(self.SubmitTask(fn))

    def ParallelCopy(self, dst, src, shards: int = 0) -> None:
        (pd, nd), (ps, ns) = _bytes_span(dst), _bytes_span(src)
        if nd != ns:
            raise ValueError("size mismatch")
        if self._L.oa_pool_parallel_copy(self._h, pd, ps, nd, shards) != 0:
            raise RuntimeError("parallel copy failed")

    def ParallelDot(self, a, b, shards: int = 0) -> float:
        (pa, na), (pb, nb) = _span(a), _span(b)
        if na != nb:
            raise ValueError("length mismatch")
        return float(self._L.oa_pool_parallel_dot(self._h, pa, pb, na, shards))

    def Shutdown(self) -> None:
        """Stops intake, drains queued jobs and joins every worker."""
        if self._h:
            self._L.oa_pool_shutdown(self._h)
            for t in getattr(self, "_pending", []):
                t._waited = True
            self._pending = []

    def __del__(self):
        if getattr(self, "_h", None):
            self._L.oa_pool_destroy(self._h)
            self._h = None


def SpinlockStress(threads: int = 4, iters: int = 20000) -> int:
    """Counter value after `threads` x `iters` increments under the native spinlock."""
    return _lib().oa_spinlock_stress(threads, iters)


def RwLockStress(readers: int = 3, writers: int = 2, iters: int = 5000) -> int:
    """Number of inconsistent observations under the native reader-writer lock (0 when it works)."""
    return _lib().oa_rwlock_stress(readers, writers, iters)
