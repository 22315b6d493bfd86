"""Python faces of `csrc/runtime/semantic.cpp` and `csrc/runtime/session.cpp`.

* `OaSemanticGraph` / `OaAnalyzeSemanticLowering` / `OaValidateSemanticLowering`
  (Source/Public/Oa/Runtime/SemanticGraph.h:10-198): operations and values with contracts, attributes and autograd
  provenance, and the direct / decomposed / fused classification against the launches that implement them.
* `OaExecutionSession` (Source/Private/Oa/Runtime/ExecutionSession.h:22-177): the stable resource frame (temporaries
  handed out by ordinal so that a captured CUDA graph sees the same addresses on every step), reusable graphs and
  the hazards between graphs of an asynchronous batch.
* `OaExecutionPlan` (Source/Private/Oa/Runtime/ExecutionPlan.{h,cpp}): what was compiled, kept to decide whether
  a newly recorded graph may replay it.
"""
from __future__ import annotations

import ctypes
import json
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Union

import torch

from ..core.types import OaStatus, OaStatusCode
from ..io.oam import runtime_lib

_ready = False


def _lib():
    global _ready
    L = runtime_lib()
    if _ready:
        return L
    vp, u64, u32, i32, i64, cp = ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_int, ctypes.c_int64, ctypes.c_char_p
    P = ctypes.POINTER
    sig = {
        "oa_sem_create": (vp, []), "oa_sem_destroy": (None, [vp]), "oa_sem_reset": (None, [vp]), "oa_sem_error": (cp, [vp]),
        "oa_sem_num_values": (i32, [vp]), "oa_sem_num_ops": (i32, [vp]), "oa_sem_num_autograd": (i32, [vp]),
        "oa_sem_add_value": (i32, [vp, cp, i32, i32, P(i64), i32, i32, i32]),
        "oa_sem_add_op": (i32, [vp, cp, u64, i32, i32, P(u32), i32, P(u32), i32, P(u32), i32, u64]),
        "oa_sem_op_set_attr": (i32, [vp, u32, cp, cp]), "oa_sem_op_add_alias": (i32, [vp, u32, u32, u32]),
        "oa_sem_op_set_backward_of": (i32, [vp, u32, u32, u64]), "oa_sem_attach_autograd": (i32, [vp, u32, u32, u64]),
        "oa_sem_complete_autograd": (i32, [vp, u32, u64, u32, u32]), "oa_sem_validate": (i32, [vp]),
        "oa_sem_copy_from": (i32, [vp, vp]), "oa_sem_value_info": (i32, [vp, u32, P(i64), P(i64)]),
        "oa_sem_value_name": (cp, [vp, u32]), "oa_sem_op_name": (cp, [vp, u32]), "oa_sem_op_info": (i32, [vp, u32, P(i64)]),
        "oa_sem_analyze_lowering": (i32, [vp, P(u32), P(u32), i32, P(u32), P(u32)]), "oa_sem_report_json": (cp, [vp, cp]),
        "oa_session_create": (vp, []), "oa_session_destroy": (None, [vp]), "oa_session_begin_frame": (i32, [vp]),
        "oa_session_request": (i32, [vp, u64, P(i32), P(u64)]), "oa_session_end_frame": (i32, [vp]), "oa_session_trim": (i32, [vp]),
        "oa_session_stat": (u64, [vp, i32]), "oa_session_slot_generation": (u32, [vp, u32]),
        "oa_session_park_graph": (None, [vp, u64]), "oa_session_take_graph": (i32, [vp, u64]),
        "oa_session_batch_begin": (i32, [vp]), "oa_session_batch_add": (i32, [vp, P(u64), P(u32), i32, P(i32), i32]),
        "oa_session_batch_end": (i32, [vp, u64]),
        "oa_plan_create": (vp, [vp, vp]), "oa_plan_destroy": (None, [vp]), "oa_plan_hash": (u64, [vp]), "oa_plan_num_nodes": (i32, [vp]),
        "oa_plan_replays": (u64, [vp]), "oa_plan_first_mismatch": (i32, [vp, vp]), "oa_plan_note_replay": (u64, [vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype, fn.argtypes = res, args
    _ready = True
    return L


def _u32(xs: Sequence[int]):
    return (ctypes.c_uint32 * max(1, len(xs)))(*xs)


@dataclass
class OaSemanticValueDesc:
    Id: int
    Name: str
    Kind: int
    Shape: List[int]
    Dtype: int
    External: bool
    Virtual: bool
    Producer: Optional[int]


@dataclass
class OaSemanticOperationDesc:
    Id: int
    Name: str
    ContractHash: int
    Differentiation: int
    Lowering: int
    NumInputs: int
    NumOutputs: int
    BackwardOf: Optional[int]
    BackwardSequence: int
    NumMutated: int


class OaSemanticGraph:
    def __init__(self):
        self._L = _lib()
        self._h = self._L.oa_sem_create()

    def __del__(self):
        if getattr(self, "_h", None):
            self._L.oa_sem_destroy(self._h)
            self._h = None

    def _status(self, rc: int) -> OaStatus:
        return OaStatus.Ok() if rc >= 0 else OaStatus(OaStatusCode.InvalidArgument, self._L.oa_sem_error(self._h).decode())

    def LastError(self) -> str: return self._L.oa_sem_error(self._h).decode()
    def Reset(self) -> None: self._L.oa_sem_reset(self._h)
    def ValueCount(self) -> int: return self._L.oa_sem_num_values(self._h)
    def OperationCount(self) -> int: return self._L.oa_sem_num_ops(self._h)
    def AutogradCount(self) -> int: return self._L.oa_sem_num_autograd(self._h)

    def AddValue(self, name: str, shape: Sequence[int] = (), dtype: int = 0, kind: int = 0, external: bool = False,
                 virtual: bool = False) -> int:
        """Returns the value id; raises ValueError on a bad description."""
        arr = (ctypes.c_int64 * max(1, len(shape)))(*shape)
        v = self._L.oa_sem_add_value(self._h, name.encode(), kind, len(shape), arr, int(dtype), int(external), int(virtual))
        if v < 0:
            raise ValueError(self.LastError())
        return v

    def AddOperation(self, contract, inputs: Sequence[int], outputs: Sequence[int], control: Sequence[int] = (),
                     attributes: Optional[Dict[str, object]] = None) -> int:
        """`contract` is an operation contract (Name, Hash, Differentiation, Lowering, MutatedInputMask) or a bare name."""
        if isinstance(contract, str):
            name, h, diff, low, mask = contract, 0, 0, 0, 0
        else:
            name, h, diff, low = contract.Name, int(contract.Hash), int(contract.Differentiation), int(contract.Lowering)
            mask = int(getattr(contract, "MutatedInputMask", 0))
        op = self._L.oa_sem_add_op(self._h, name.encode(), h, diff, low, _u32(inputs), len(inputs), _u32(outputs), len(outputs),
                                   _u32(control), len(control), mask)
        if op < 0:
            raise ValueError(self.LastError())
        for k, v in (attributes or {}).items():
            self._L.oa_sem_op_set_attr(self._h, op, k.encode(), str(v).encode())
        return op

    def AddAlias(self, op: int, output: int, input: int) -> OaStatus:
        return self._status(self._L.oa_sem_op_add_alias(self._h, op, output, input))

    def AttachAutograd(self, forward_op: int, output_index: int, sequence: int) -> OaStatus:
        return self._status(self._L.oa_sem_attach_autograd(self._h, forward_op, output_index, sequence))

    def CompleteAutograd(self, forward_op: int, sequence: int, backward_first: int, backward_count: int) -> OaStatus:
        return self._status(self._L.oa_sem_complete_autograd(self._h, forward_op, sequence, backward_first, backward_count))

    def Validate(self) -> OaStatus:
        return self._status(self._L.oa_sem_validate(self._h))

    def CopyFrom(self, other: "OaSemanticGraph") -> OaStatus:
        return self._status(self._L.oa_sem_copy_from(self._h, other._h))

    def FindValue(self, v: int) -> Optional[OaSemanticValueDesc]:
        info, shape = (ctypes.c_int64 * 6)(), (ctypes.c_int64 * 8)()
        if self._L.oa_sem_value_info(self._h, v, info, shape) != 0:
            return None
        return OaSemanticValueDesc(v, self._L.oa_sem_value_name(self._h, v).decode(), info[1], list(shape[:info[3]]), info[2],
                                   bool(info[4]), bool(info[5]), None if info[0] < 0 else int(info[0]))

    def Values(self) -> List[OaSemanticValueDesc]:
        return [self.FindValue(i) for i in range(self.ValueCount())]

    def Operation(self, op: int) -> Optional[OaSemanticOperationDesc]:
        info = (ctypes.c_int64 * 8)()
        if self._L.oa_sem_op_info(self._h, op, info) != 0:
            return None
        return OaSemanticOperationDesc(op, self._L.oa_sem_op_name(self._h, op).decode(), info[0] & (2 ** 64 - 1), info[1], info[2],
                                       info[3], info[4], None if info[5] < 0 else int(info[5]), info[6], info[7])

    def Operations(self) -> List[OaSemanticOperationDesc]:
        return [self.Operation(i) for i in range(self.OperationCount())]

    def DebugReportJson(self, name: str = "") -> str:
        return self._L.oa_sem_report_json(self._h, name.encode()).decode()

    def DebugReport(self, name: str = "") -> dict:
        return json.loads(self.DebugReportJson(name))


@dataclass
class OaSemanticLoweringAnalysis:
    ExecutableNodeCounts: List[int]
    SchemaOwnedNodeCount: int
    CompatibilityNodeCount: int
    DirectOperationCount: int
    DecomposedOperationCount: int
    FusedOperationCount: int
    FusedNodeCount: int
    MaximumNodesPerOperation: int
    MaximumOperationsPerNode: int

    def OperationCount(self) -> int: return len(self.ExecutableNodeCounts)
    def ExecutableNodeCount(self, op: int) -> int: return self.ExecutableNodeCounts[op] if 0 <= op < len(self.ExecutableNodeCounts) else 0


def OaAnalyzeSemanticLowering(semantic: OaSemanticGraph, node_operations: Sequence[Sequence[int]]) -> OaSemanticLoweringAnalysis:
    """`node_operations[n]` lists the semantic operations that executable node n implements (empty = a launch recorded
    outside any contract).  Raises ValueError when the two graphs do not cover each other."""
    L = _lib()
    flat = [o for ops in node_operations for o in ops]
    offs = [0]
    for ops in node_operations:
        offs.append(offs[-1] + len(ops))
    out, per = (ctypes.c_uint32 * 8)(), (ctypes.c_uint32 * max(1, semantic.OperationCount()))()
    if L.oa_sem_analyze_lowering(semantic._h, _u32(flat), _u32(offs), len(node_operations), out, per) != 0:
        raise ValueError(semantic.LastError())
    return OaSemanticLoweringAnalysis(list(per[:semantic.OperationCount()]), *[int(x) for x in out])


def OaValidateSemanticLowering(semantic: OaSemanticGraph, node_operations: Sequence[Sequence[int]]) -> OaStatus:
    st = semantic.Validate()
    if not st.IsOk():
        return st
    try:
        OaAnalyzeSemanticLowering(semantic, node_operations)
    except ValueError as e:
        return OaStatus(OaStatusCode.InvalidArgument, str(e))
    return OaStatus.Ok()


class OaExecutionSession:
    """Stable resource frame + reusable graphs + batch hazards.  Temporaries are uint8 tensors on `device`; the n-th
    `Temp` of a frame returns the same storage as the n-th `Temp` of the frame before whenever it fits."""

    def __init__(self, device: Union[str, torch.device] = "cpu"):
        self._L = _lib()
        self._h = self._L.oa_session_create()
        self._device = torch.device(device)
        self._slots: List[torch.Tensor] = []

    def __del__(self):
        if getattr(self, "_h", None):
            self._L.oa_session_destroy(self._h)
            self._h = None

    def BeginFrame(self) -> None:
        if self._L.oa_session_begin_frame(self._h) != 0:
            raise RuntimeError("a frame is already open")

    def Temp(self, shape: Sequence[int], dtype: torch.dtype = torch.float32) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        reused, cap = ctypes.c_int(), ctypes.c_uint64()
        ord_ = self._L.oa_session_request(self._h, nbytes, ctypes.byref(reused), ctypes.byref(cap))
        if ord_ < 0:
            raise RuntimeError("Temp outside BeginFrame / EndFrame")
        if not reused.value:
            block = torch.empty(cap.value, dtype=torch.uint8, device=self._device)
            if ord_ < len(self._slots):
                self._slots[ord_] = block
            else:
                self._slots.append(block)
        return self._slots[ord_][:nbytes].view(dtype).view(*shape)

    def EndFrame(self) -> bool:
        """True when every temporary of the frame kept its address (the step may be captured / replayed)."""
        rc = self._L.oa_session_end_frame(self._h)
        if rc < 0:
            raise RuntimeError("no open frame")
        return rc == 1

    def Trim(self) -> int:
        dropped = self._L.oa_session_trim(self._h)
        if dropped:
            del self._slots[len(self._slots) - dropped:]
        return dropped

    def FrameCount(self) -> int: return self._L.oa_session_stat(self._h, 0)
    def StableFrameCount(self) -> int: return self._L.oa_session_stat(self._h, 1)
    def SlotCount(self) -> int: return self._L.oa_session_stat(self._h, 2)
    def BytesHeld(self) -> int: return self._L.oa_session_stat(self._h, 3)
    def SlotGeneration(self, ordinal: int) -> int: return self._L.oa_session_slot_generation(self._h, ordinal)

    def ParkGraph(self, structural_hash: int) -> None: self._L.oa_session_park_graph(self._h, structural_hash)
    def TakeGraph(self, structural_hash: int) -> bool: return bool(self._L.oa_session_take_graph(self._h, structural_hash))
    def ReuseStats(self) -> tuple: return self._L.oa_session_stat(self._h, 4), self._L.oa_session_stat(self._h, 5)

    def BeginAsyncBatch(self) -> None:
        if self._L.oa_session_batch_begin(self._h) != 0:
            raise RuntimeError("a batch is already open")

    def AddToBatch(self, buffers: Sequence[tuple]) -> List[int]:
        """`buffers` = (buffer id, access) pairs with access 1 read, 2 write, 3 both.  Returns the indices of the
        earlier graphs of the batch this one must wait for."""
        ids = (ctypes.c_uint64 * max(1, len(buffers)))(*[b for b, _ in buffers])
        acc = (ctypes.c_uint32 * max(1, len(buffers)))(*[int(a) for _, a in buffers])
        deps = (ctypes.c_int * 64)()
        n = self._L.oa_session_batch_add(self._h, ids, acc, len(buffers), deps, 64)
        if n < 0:
            raise RuntimeError("no open batch")
        return list(deps[:min(n, 64)])

    def SubmitBatch(self, event_id: int = 0) -> int:
        n = self._L.oa_session_batch_end(self._h, event_id)
        if n < 0:
            raise RuntimeError("no open batch")
        return n

    def PendingEvent(self) -> int: return self._L.oa_session_stat(self._h, 6)


class OaExecutionPlan:
    """Immutable record of a compiled graph (structural hash and per-node hashes)."""

    def __init__(self, graph, session: Optional[OaExecutionSession] = None):
        self._L = _lib()
        self._h = self._L.oa_plan_create(graph._h, session._h if session is not None else None)

    def __del__(self):
        if getattr(self, "_h", None):
            self._L.oa_plan_destroy(self._h)
            self._h = None

    def Hash(self) -> int: return self._L.oa_plan_hash(self._h)
    def NodeCount(self) -> int: return self._L.oa_plan_num_nodes(self._h)
    def ReplayCount(self) -> int: return self._L.oa_plan_replays(self._h)
    def Matches(self, graph) -> bool: return self._L.oa_plan_first_mismatch(self._h, graph._h) < 0
    def FirstMismatch(self, graph) -> int: return self._L.oa_plan_first_mismatch(self._h, graph._h)
    def NoteReplay(self) -> int: return self._L.oa_plan_note_replay(self._h)
