"""Native host primitives (vector math, streaming copy, topology, channel, pool) against numpy."""
import threading

import numpy as np
import pytest
import torch

from oa_b200.core.host import (OaAlignedBuffer, OaChannel, OaCpuTopology, OaMemcpyNT, OaMemEqual, OaSimd, OaThreadPool,
                               OaThreadPoolConfig, RwLockStress, SpinlockStress)


def test_simd_matches_numpy():
    rng = np.random.default_rng(0)
    for n in (1, 7, 8, 33, 1000, 4099):
        a = rng.standard_normal(n).astype(np.float32)
        b = (rng.standard_normal(n).astype(np.float32) + 3.0)
        assert OaSimd.DotF32(a, b) == pytest.approx(float(np.dot(a.astype(np.float64), b)), rel=1e-4, abs=1e-3)
        for name, ref in (("AddF32", a + b), ("SubF32", a - b), ("MulF32", a * b), ("DivF32", a / b)):
            x = a.copy()
            getattr(OaSimd, name)(x, b)
            np.testing.assert_allclose(x, ref, rtol=1e-6)
        x = a.copy(); OaSimd.ScaleF32(x, 0.5); np.testing.assert_array_equal(x, a * np.float32(0.5))
        x = a.copy(); OaSimd.NegF32(x); np.testing.assert_array_equal(x, -a)
    t = torch.ones(19)
    OaSimd.AddF32(t, torch.full((19,), 2.0))
    assert torch.equal(t, torch.full((19,), 3.0))
    assert OaSimd.Level() in (1, 2)
    with pytest.raises(ValueError):
        OaSimd.AddF32(np.zeros(3, np.float32), np.zeros(4, np.float32))


def test_streaming_copy_and_aligned_buffer():
    src = np.random.default_rng(1).integers(0, 255, size=(1 << 20) + 13, dtype=np.uint8)
    buf = OaAlignedBuffer(src.nbytes + 64, alignment=256)
    assert buf.Address % 256 == 0
    for shift in (0, 1, 31):          # unaligned destinations take the head / tail paths
        dst = buf.Array[shift:shift + src.nbytes]
        dst[:] = 0
        OaMemcpyNT(dst, src)
        assert OaMemEqual(dst, src)
    dst[5] ^= 1
    assert not OaMemEqual(dst, src)


def test_topology():
    t = OaCpuTopology.Detect()
    assert t.NumLogicalCores >= 1 and 1 <= t.NumPhysicalCores <= t.NumLogicalCores
    assert len(t.Cores) == t.NumLogicalCores and t.NumNumaNodes >= 1 and t.NumPackages >= 1
    assert sorted(t.GetPcoreIds() + t.GetEcoreIds()) == sorted(c.Id for c in t.Cores)
    assert set(t.GetCoresOnNuma(t.Cores[0].NumaNode)) <= {c.Id for c in t.Cores}


def test_locks():
    assert SpinlockStress(4, 5000) == 20000
    assert RwLockStress(3, 2, 2000) == 0


def test_channel_blocking_and_close():
    ch = OaChannel(2)
    assert ch.TrySend(1) and ch.TrySend(2) and not ch.TrySend(3)
    got = []
    th = threading.Thread(target=lambda: [got.append(ch.Recv()) for _ in range(4)])
    th.start()
    assert ch.Send(3) and ch.Send(4)
    th.join(10)
    assert got == [1, 2, 3, 4]
    ch.Send(9)
    ch.Close()
    assert not ch.Send(10)
    assert ch.Recv() == 9 and ch.Recv() is None and ch.TryRecv() is None


def test_pool_tasks_and_native_jobs():
    pool = OaThreadPool(OaThreadPoolConfig(NumWorkers=3, PinToCores=False))
    assert pool.NumWorkers() == 3
    tasks = [pool.SubmitTask(lambda i=i: i * i) for i in range(16)]
    assert [t.Wait() for t in tasks] == [i * i for i in range(16)]
    bad = pool.SubmitTask(lambda: 1 / 0)
    with pytest.raises(ZeroDivisionError):
        bad.Wait()
    src = torch.randn(3 * (1 << 18) + 5)
    dst = torch.empty_like(src)
    pool.ParallelCopy(dst, src, shards=5)
    assert torch.equal(dst, src)
    a, b = np.random.default_rng(2).standard_normal((2, 100003)).astype(np.float32)
    assert pool.ParallelDot(a, b, shards=4) == pytest.approx(float(np.dot(a.astype(np.float64), b)), rel=1e-4, abs=1e-2)
    done = []
    pool.Submit(lambda: done.append(1))
    pool.Shutdown()
    assert done == [1] and pool.Executed() >= 18
    with pytest.raises(RuntimeError):
        pool.SubmitTask(lambda: 0)


def test_pinned_pool():
    pool = OaThreadPool.Create(OaThreadPoolConfig(NumWorkers=2))
    assert pool.SubmitTask(lambda: 7).Wait() == 7
    pool.Shutdown()
