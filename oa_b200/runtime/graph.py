"""Python faces of the native executor pieces in csrc/runtime: OaComputeGraph (hazards, levels, structural hash, alias
groups), OaDnnGraph / OaDnnPlanner (fusion partitions) and OaGemmPlanCache (launch plans, tuner samples, persistence)."""
from __future__ import annotations

import ctypes
import enum
from dataclasses import dataclass, field
from typing import Optional, Sequence

from ..core.types import OaStatus, OaStatusCode
from ..io.oam import runtime_lib

_ready = False


def _lib():
    global _ready
    L = runtime_lib()
    if _ready:
        return L
    vp, u64, u32, i32, cp = ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_int, ctypes.c_char_p
    P = ctypes.POINTER
    sig = {
        "oa_graph_create": (vp, []), "oa_graph_destroy": (None, [vp]), "oa_graph_clear": (None, [vp]),
        "oa_graph_add_node": (i32, [vp, cp, P(u64), P(u64), P(u32), i32, vp, i32, u32]), "oa_graph_num_nodes": (i32, [vp]),
        "oa_graph_hash": (u64, [vp]), "oa_graph_node_hash": (u64, [vp, i32]), "oa_graph_num_barriers": (i32, [vp]),
        "oa_graph_num_levels": (i32, [vp]), "oa_graph_node_level": (i32, [vp, i32]), "oa_graph_node_deps": (i32, [vp, i32, P(i32), i32]),
        "oa_graph_num_buffers": (i32, [vp]), "oa_graph_buffer_at": (None, [vp, i32, P(u64), P(u64), P(i32), P(i32), P(i32)]),
        "oa_graph_memory": (None, [vp, P(u64), P(u64)]), "oa_graph_node_kernel": (cp, [vp, i32]),
        "oa_dnn_create": (vp, []), "oa_dnn_destroy": (None, [vp]), "oa_dnn_error": (cp, [vp]),
        "oa_dnn_add_matrix": (i32, [vp, u32, i32, P(ctypes.c_int64), i32, i32, i32, i32]),
        "oa_dnn_add_op": (i32, [vp, i32, P(u32), i32, P(u32), i32, i32]), "oa_dnn_plan": (i32, [vp, i32]), "oa_dnn_hash": (u64, [vp]),
        "oa_dnn_num_partitions": (i32, [vp]), "oa_dnn_partition_engine": (i32, [vp, i32]),
        "oa_dnn_partition_ops": (i32, [vp, i32, P(u32), i32]), "oa_dnn_partition_saved": (i32, [vp, i32, P(u32), i32]),
        "oa_plan_cache_create": (vp, []), "oa_plan_cache_destroy": (None, [vp]),
        "oa_plan_cache_lookup": (i32, [vp] + [i32] * 7 + [P(i32), P(i32)]),
        "oa_plan_cache_record": (None, [vp] + [i32] * 9 + [ctypes.c_float]), "oa_plan_cache_set": (None, [vp] + [i32] * 9),
        "oa_plan_cache_size": (i32, [vp]), "oa_plan_cache_stats": (None, [vp, P(u64), P(u64)]),
        "oa_plan_cache_timing": (i32, [vp] + [i32] * 7 + [P(ctypes.c_float), P(ctypes.c_float), P(i32)]),
        "oa_plan_cache_save": (i32, [vp, cp]), "oa_plan_cache_load": (i32, [vp, cp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype, fn.argtypes = res, args
    _ready = True
    return L


class OaAccess(enum.IntFlag):
    Read = 1
    Write = 2
    ReadWrite = 3


class OaComputeGraph:
    def __init__(self):
        self._L = _lib()
        self._h = self._L.oa_graph_create()

    def __del__(self):
        if getattr(self, "_h", None):
            self._L.oa_graph_destroy(self._h)
            self._h = None

    def Clear(self) -> None:
        self._L.oa_graph_clear(self._h)

    def AddNode(self, kernel: str, buffers: Sequence[tuple], push: bytes = b"", queue: int = 0) -> int:
        """buffers: (id, bytes, access) triples; returns the node index."""
        n = len(buffers)
        ids = (ctypes.c_uint64 * max(n, 1))(*[int(b[0]) for b in buffers])
        sizes = (ctypes.c_uint64 * max(n, 1))(*[int(b[1]) for b in buffers])
        acc = (ctypes.c_uint32 * max(n, 1))(*[int(b[2]) for b in buffers])
        return self._L.oa_graph_add_node(self._h, kernel.encode(), ids, sizes, acc, n, push, len(push), queue)

    def NumNodes(self) -> int: return self._L.oa_graph_num_nodes(self._h)
    def Hash(self) -> int: return self._L.oa_graph_hash(self._h)
    def NodeHash(self, i: int) -> int: return self._L.oa_graph_node_hash(self._h, i)
    def NumBarriers(self) -> int: return self._L.oa_graph_num_barriers(self._h)
    def NumLevels(self) -> int: return self._L.oa_graph_num_levels(self._h)
    def NodeLevel(self, i: int) -> int: return self._L.oa_graph_node_level(self._h, i)
    def NodeKernel(self, i: int) -> str: return self._L.oa_graph_node_kernel(self._h, i).decode()

    def NodeDeps(self, i: int) -> list:
        buf = (ctypes.c_int * 64)()
        n = self._L.oa_graph_node_deps(self._h, i, buf, 64)
        return list(buf[:min(n, 64)])

    def Buffers(self) -> list:
        """[(id, bytes, first node, last node, alias group)] in order of first use."""
        out = []
        for k in range(self._L.oa_graph_num_buffers(self._h)):
            i, b = ctypes.c_uint64(), ctypes.c_uint64()
            f, l, g = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
            self._L.oa_graph_buffer_at(self._h, k, ctypes.byref(i), ctypes.byref(b), ctypes.byref(f), ctypes.byref(l), ctypes.byref(g))
            out.append((i.value, b.value, f.value, l.value, g.value))
        return out

    def Memory(self) -> tuple:
        """(bytes with one allocation per buffer, bytes with alias groups)."""
        a, b = ctypes.c_uint64(), ctypes.c_uint64()
        self._L.oa_graph_memory(self._h, ctypes.byref(a), ctypes.byref(b))
        return a.value, b.value

    def Report(self) -> dict:
        naive, aliased = self.Memory()
        return {"nodes": self.NumNodes(), "barriers": self.NumBarriers(), "levels": self.NumLevels(), "hash": f"{self.Hash():016x}",
                "bytes": naive, "bytes_aliased": aliased}


class OaDnnOpType(enum.IntEnum):
    Matmul = 0
    BiasAdd = 1
    Relu = 2
    Gelu = 3
    Silu = 4
    Multiply = 5
    Add = 6
    RmsNorm = 7
    FlashAttentionCausal = 8
    GroupedGemm = 9


class OaDnnEngineType(enum.IntEnum):
    Portable = 0
    BlasLtEpilogue = 1
    PackedQkv = 2
    GatedFfn = 3
    ResidualNorm = 4
    FlashAttention = 5
    GroupedMoe = 6
    AllGatherGemm = 7
    GemmReduceScatter = 8


@dataclass
class OaDnnPartition:
    Engine: OaDnnEngineType
    Ops: list
    SavedForBackward: list


@dataclass
class OaDnnPlan:
    Partitions: list = field(default_factory=list)
    GraphHash: int = 0
    PlannerAbi: int = 1


class OaDnnGraph:
    def __init__(self):
        self._L = _lib()
        self._h = self._L.oa_dnn_create()

    def __del__(self):
        if getattr(self, "_h", None):
            self._L.oa_dnn_destroy(self._h)
            self._h = None

    def _status(self, rc: int) -> OaStatus:
        return OaStatus.Ok() if rc == 0 else OaStatus.Error(OaStatusCode.InvalidArgument, self._L.oa_dnn_error(self._h).decode())

    def AddMatrix(self, ident: int, shape: Sequence[int], dtype: int = 0, external: bool = False, virtual: bool = False,
                  row_sharded: bool = False) -> OaStatus:
        sh = (ctypes.c_int64 * 4)(*(list(shape) + [0] * 4)[:4])
        return self._status(self._L.oa_dnn_add_matrix(self._h, ident, len(shape), sh, int(dtype), int(external), int(virtual), int(row_sharded)))

    def AddOp(self, op: OaDnnOpType, inputs: Sequence[int], outputs: Sequence[int], training: bool = True) -> OaStatus:
        i = (ctypes.c_uint32 * max(1, len(inputs)))(*inputs)
        o = (ctypes.c_uint32 * max(1, len(outputs)))(*outputs)
        return self._status(self._L.oa_dnn_add_op(self._h, int(op), i, len(inputs), o, len(outputs), int(training)))


class OaDnnPlanner:
    @staticmethod
    def Plan(graph: OaDnnGraph, allow_recompute: bool = True):
        """Returns (OaDnnPlan | None, OaStatus)."""
        L = graph._L
        if L.oa_dnn_plan(graph._h, int(allow_recompute)) != 0:
            return None, OaStatus.Error(OaStatusCode.InvalidArgument, L.oa_dnn_error(graph._h).decode())
        plan = OaDnnPlan(GraphHash=L.oa_dnn_hash(graph._h))
        buf = (ctypes.c_uint32 * 32)()
        for p in range(L.oa_dnn_num_partitions(graph._h)):
            n = L.oa_dnn_partition_ops(graph._h, p, buf, 32)
            ops = list(buf[:n])
            n = L.oa_dnn_partition_saved(graph._h, p, buf, 32)
            plan.Partitions.append(OaDnnPartition(OaDnnEngineType(L.oa_dnn_partition_engine(graph._h, p)), ops, list(buf[:n])))
        return plan, OaStatus.Ok()


class OaGemmPlanCache:
    """(M, N, K, layout, epilogue, role, world) -> (N tile, split-K) with tuner samples; persisted under var/."""

    def __init__(self):
        self._L = _lib()
        self._h = self._L.oa_plan_cache_create()

    def __del__(self):
        if getattr(self, "_h", None):
            self._L.oa_plan_cache_destroy(self._h)
            self._h = None

    def Lookup(self, M, N, K, layout=0, epilogue=0, role=0, world=1) -> Optional[tuple]:
        bn, sp = ctypes.c_int(), ctypes.c_int()
        if self._L.oa_plan_cache_lookup(self._h, M, N, K, layout, epilogue, role, world, ctypes.byref(bn), ctypes.byref(sp)):
            return bn.value, sp.value
        return None

    def Record(self, M, N, K, bn, splits, us, layout=0, epilogue=0, role=0, world=1) -> None:
        self._L.oa_plan_cache_record(self._h, M, N, K, layout, epilogue, role, world, bn, splits, float(us))

    def Set(self, M, N, K, bn, splits, layout=0, epilogue=0, role=0, world=1) -> None:
        self._L.oa_plan_cache_set(self._h, M, N, K, layout, epilogue, role, world, bn, splits)

    def Timing(self, M, N, K, layout=0, epilogue=0, role=0, world=1) -> Optional[tuple]:
        a, b, n = ctypes.c_float(), ctypes.c_float(), ctypes.c_int()
        if self._L.oa_plan_cache_timing(self._h, M, N, K, layout, epilogue, role, world, ctypes.byref(a), ctypes.byref(b), ctypes.byref(n)):
            return a.value, b.value, n.value
        return None

    def Size(self) -> int:
        return self._L.oa_plan_cache_size(self._h)

    def Stats(self) -> tuple:
        h, m = ctypes.c_uint64(), ctypes.c_uint64()
        self._L.oa_plan_cache_stats(self._h, ctypes.byref(h), ctypes.byref(m))
        return h.value, m.value

    def Save(self, path: str) -> OaStatus:
        return OaStatus.Ok() if self._L.oa_plan_cache_save(self._h, str(path).encode()) == 0 else OaStatus.Error(OaStatusCode.PermissionDenied, f"cannot write {path}")

    def Load(self, path: str) -> OaStatus:
        rc = self._L.oa_plan_cache_load(self._h, str(path).encode())
        if rc == 0:
            return OaStatus.Ok()
        return OaStatus.Error(OaStatusCode.NotFound if rc == 1 else OaStatusCode.DataLoss, f"plan cache {path}: {'missing' if rc == 1 else 'corrupt'}")
