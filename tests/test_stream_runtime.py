"""Streams, fences, timeline tokens, dispatch, inference pool, work queue, scheduler (CPU engine semantics;
the CUDA variants of the same calls run in the gpu-marked test at the end)."""
import pytest
import torch

from oa_b200.runtime.stream import (OA_NODE_AUTO, OaCompletionToken, OaComputeClass, OaComputeClassName, OaDispatch, OaDispatchHint,
                                    OaExternalMemoryHandle, OaFence, OaInferencePool, OaInferencePoolConfig, OaScheduler, OaStream,
                                    OaStreamPool, OaTimelineSemaphore, OaWorkItem, OaWorkQueue)


def _exercise_stream(device):
    s = OaStream.Create(device, name="t")
    a = torch.zeros(1024, device=device)
    b = torch.empty(1024, device=device)
    assert s.Begin().IsOk() and not s.Begin().IsOk()
    s.RecordFillBuffer(a, 3.0)
    s.RecordCopyBuffer(b, a)
    t1 = s.Submit()
    s.Begin()
    s.Record(lambda: b.mul_(2))
    t2 = s.SubmitWithDependency(t1)
    assert t2.Wait().IsOk() and t1.IsComplete() and t2.IsComplete() and not t1.IsSameCompletion(t2)
    assert torch.all(b == 6.0).item() and s.SubmissionCount() == 2 and s.Timeline().Value() == 2
    other = OaStream(device, name="u")
    other.Begin()
    other.Record(lambda: b.add_(1))
    assert other.SubmitWithDependency(t2).Wait().IsOk() and torch.all(b == 7.0).item()
    with pytest.raises(RuntimeError):
        s.Submit()
    assert not OaCompletionToken().Wait().IsOk()
    f = OaFence.Create(device)
    assert not f.IsSignaled() and not f.Wait().IsOk()
    f.Signal(s.Handle())
    assert f.Wait(timeout_ns=5_000_000_000).IsOk() and f.IsSignaled()
    f.Reset()
    assert not f.IsSignaled()
    d = OaDispatch(device=device)
    assert d.Run(lambda: a.fill_(9.0)).IsOk()
    d.BeginBatch(); d.Record(lambda: a.add_(1)); d.Record(lambda: a.mul_(2))
    assert d.Flush().IsOk() and torch.all(a == 20.0).item()
    pool = OaStreamPool(device, 2)
    assert pool.Acquire() is not pool.Acquire() and pool.Size() == 2
    pool.SynchronizeAll()


def test_stream_fence_dispatch_cpu():
    _exercise_stream("cpu")


@pytest.mark.gpu
def test_stream_fence_dispatch_cuda():
    _exercise_stream("cuda")


def test_timeline_rules():
    t = OaTimelineSemaphore.Create()
    assert t.Signal(1).IsOk() and not t.Signal(1).IsOk() and t.Signal(5).IsOk() and t.Value() == 5
    assert t.Wait(5).IsOk() and not t.Wait(6).IsOk()


def test_inference_pool():
    p = OaInferencePool()
    assert not p.Init("cpu", OaInferencePoolConfig()).IsOk()
    cfg = OaInferencePoolConfig(NumLayers=3, ActivationSize=1000, MaxBatchSize=2, OutputRingBytes=64, OutputSlotBytes=16)
    assert p.Init("cpu", cfg).IsOk() and p.IsValid() and p.TotalBytes() == 3 * 2 * 1024 + 64
    a, b = p.GetActivation(2, 1), p.GetActivation(0, 0, torch.float16)
    assert a.numel() == 1000 and b.numel() == 500 and a.data_ptr() % 256 == 0 and p.GetActivation(3, 0) is None
    slots = [p.NextOutputSlot() for _ in range(5)]
    assert all(s is not None and s.numel() == 16 for s in slots[:4]) and slots[4] is None and p.PendingOutputs() == 4
    p.ConsumeOutputSlot()
    assert p.NextOutputSlot().data_ptr() == slots[0].data_ptr()
    w = torch.ones(4)
    assert p.PinWeights(w).IsOk()
    p.ResetSession()
    assert p.PendingOutputs() == 0
    p.Destroy()
    assert not p.IsValid()


def test_work_queue_in_order_and_capacity():
    seen = []
    q = OaWorkQueue.Create(3, 64, consumer=lambda item, push: seen.append((item.GroupsX, bytes(push[:2]))))
    q.WritePush(8, b"hi")
    assert q.Enqueue(OaWorkItem(1, 1, 1, 8)) and q.Enqueue(OaWorkItem(2, 1, 1, 8)) and q.Enqueue(OaWorkItem(3, 1, 1, 0))
    assert not q.Enqueue(OaWorkItem(4)) and q.Pending() == 3 and not q.Enqueue(OaWorkItem(1, 1, 1, 64))
    assert q.Flush().IsOk() and q.Consumed() == 3 and [s[0] for s in seen] == [1, 2, 3] and seen[0][1] == b"hi"
    assert q.Enqueue(OaWorkItem(5)) and q.Flush().IsOk() and seen[-1][0] == 5 and q.Flush().IsOk()
    with pytest.raises(ValueError):
        q.WritePush(60, b"too long")
    tables = []
    qb = OaWorkQueue(4, 16, batch_consumer=lambda table, push: tables.append((table.clone(), push.numel())))
    qb.Enqueue(OaWorkItem(7, 2, 1, 0)); qb.Enqueue(OaWorkItem(8, 2, 1, 4)); qb.Flush()
    assert tables[0][0].tolist() == [[7, 2, 1, 0], [8, 2, 1, 4]] and tables[0][1] == 16


def test_scheduler_policy():
    s = OaScheduler.Create(2)
    assert s.Route(OaComputeClass.Heavy) == 0 and s.Route(OaComputeClass.Any) == 0
    assert s.Route(OaComputeClass.Light) == 1 and s.Route(OaDispatchHint(OaComputeClass.Transfer)) == 1
    assert s.Route(OaDispatchHint(OaComputeClass.Light, PreferNode=0)) == 0 and s.Routed == {0: 3, 1: 2}
    assert OaScheduler(1).Route(OaComputeClass.Light) == 0 and OaComputeClassName(OaComputeClass.Transfer) == "Transfer"
    assert OaDispatchHint().PreferNode == OA_NODE_AUTO


def test_external_memory_handle_record():
    h = OaExternalMemoryHandle(bytes(range(64)), 4096, 3)
    assert h.IsValid() and OaExternalMemoryHandle.Unpack(h.Pack()) == h and not OaExternalMemoryHandle().IsValid()
    with pytest.raises(ValueError):
        OaExternalMemoryHandle.Unpack(b"short")


def test_precision_policy():
    from oa_b200.core.types import OaPrecision
    from oa_b200.ml.precision import (OaLoadStoreStrideBytes, OaLookupPrecision, OaPipelineNameIsF32Variant, OaPrecisionDtype,
                                      OaPrecisionTag)
    assert OaLookupPrecision("AdamwMixed") == OaPrecisionTag.Mixed and OaLookupPrecision("rmsnorm_fwd_kernel") == OaPrecisionTag.Bf16
    assert OaPrecisionDtype(OaPrecisionTag.Bf16, OaPrecision.BF16) == 1 and OaPrecisionDtype(OaPrecisionTag.Mixed, OaPrecision.BF16) == 0
    assert OaPrecisionDtype(OaPrecisionTag.Bf16, OaPrecision.FP32) == 0
    assert OaLoadStoreStrideBytes(OaPrecisionTag.Bf16, OaPrecision.BF16) == 2 and OaLoadStoreStrideBytes(OaPrecisionTag.Fp32, OaPrecision.BF16) == 4
    assert OaPipelineNameIsF32Variant("Gemm_f32") and not OaPipelineNameIsF32Variant("f32") and not OaPipelineNameIsF32Variant("Gemm_bf16")


def test_pqc_pool_slots_and_secure_buffers():
    from oa_b200.runtime.stream import OaPqcPool, OaPqcPoolConfig
    pool = OaPqcPool()
    assert pool.AllocNttSlot() is None and not pool.Init("cpu", OaPqcPoolConfig(MaxConcurrentSigns=65)).IsOk()
    assert pool.Init("cpu", OaPqcPoolConfig(MaxConcurrentSigns=2, MaxConcurrentHashes=3, KeyCapacity=64)).IsOk()
    a, b = pool.AllocNttSlot(), pool.AllocNttSlot()
    assert a.numel() == 1024 and a.data_ptr() != b.data_ptr() and pool.AllocNttSlot() is None and pool.NttSlotsUsed() == 2
    pool.FreeNttSlot(a)
    assert pool.NttSlotsUsed() == 1 and pool.AllocNttSlot().data_ptr() == a.data_ptr()
    h = pool.AllocHashSlot(); h.fill_(7)
    pool.FreeHashSlot(h)
    assert pool.HashSlotsUsed() == 0 and int(pool.AllocHashSlot().sum()) == 0         # a freed state is wiped
    k1, k2 = pool.AllocKeyBuffer(20), pool.AllocKeyBuffer(30)
    assert k1.IsValid() and k1.Size() == 20 and k2.Tensor().data_ptr() - k1.Tensor().data_ptr() == 32 and not pool.AllocKeyBuffer(10).IsValid()
    view = k1.Tensor(); view.fill_(9); k1.Release()
    assert int(view.sum()) == 0 and not k1.IsValid()
    pool.Destroy()
    assert pool.AllocHashSlot() is None
