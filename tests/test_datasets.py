"""Datasets, index utilities and the native asynchronous reader, on files written by the test."""
import math
import os
import struct

import numpy as np
import pytest
import torch

from oa_b200.core.matrix import OaMatrix
from oa_b200.core.types import OaStatusCode
from oa_b200.data.datasets import (OaAsyncReader, OaDsDailyDialog, OaDsHumanMl3d, OaDsMnist, OaDsSharded, OaDsSubset,
                                   OaDsTinyShakespeare, OaFnDataset, OaHumanMl3dEvaluateMotion, OaHumanMl3dMpjpeCm,
                                   OaHumanMl3dRecoverWorldJoints, OaReadFileParallel)


def test_async_reader(tmp_path):
    data = np.random.default_rng(0).integers(0, 256, size=3_000_017, dtype=np.uint8)
    p = tmp_path / "blob.bin"
    data.tofile(p)
    r = OaAsyncReader(str(p), queue_depth=2)
    assert r.IsValid() and r.FileSize() == data.size
    a, b, c = torch.empty(1000, dtype=torch.uint8), torch.empty(500, dtype=torch.int32), torch.empty(10, dtype=torch.uint8)
    assert r.SubmitRead(a, 5).IsOk() and r.SubmitRead(b, 1_000_000).IsOk()
    assert r.SubmitRead(c, 0).code == OaStatusCode.ResourceExhausted
    assert r.WaitCompletions(2) == 2 and r.InFlight() == 0
    assert np.array_equal(a.numpy(), data[5:1005]) and np.array_equal(b.numpy().view(np.uint8), data[1_000_000:1_002_000])
    assert r.SubmitRead(c, data.size - 5).code == OaStatusCode.OutOfRange
    assert r.SubmitRead(c, data.size - 10).IsOk() and r.WaitCompletions() == 1 and np.array_equal(c.numpy(), data[-10:])
    r.Close()
    assert not OaAsyncReader(str(tmp_path / "missing")).IsValid()
    whole = OaReadFileParallel(str(p), chunk_bytes=256 << 10, queue_depth=3)
    assert np.array_equal(whole.numpy(), data)


def _write_idx(path, arr):
    with open(path, "wb") as f:
        f.write(struct.pack(">HBB", 0, 8, arr.ndim) + struct.pack(">" + "I" * arr.ndim, *arr.shape) + arr.tobytes())


def test_mnist(tmp_path):
    rng = np.random.default_rng(1)
    imgs, lbls = rng.integers(0, 256, size=(50, 28, 28), dtype=np.uint8), rng.integers(0, 10, size=(50,), dtype=np.uint8)
    _write_idx(tmp_path / "train-images-idx3-ubyte", imgs)
    _write_idx(tmp_path / "train-labels-idx1-ubyte", lbls)
    ds = OaDsMnist(str(tmp_path), "train", batch_size=16, shuffle=True)
    assert ds.Size() == 50 and ds.NumBatches() == 3 and ds.InputSize() == 784
    s = ds.GetSample(7)
    assert np.array_equal(s.X.Tensor().numpy(), imgs[7].reshape(-1)) and int(s.Y.Tensor()[0]) == lbls[7]
    seen = []
    while (b := ds.NextBatch()) is not None:
        x, y = b
        assert x.Tensor().shape == (16, 784) and y.Tensor().shape == (16,)
        for row, lab in zip(x.Tensor().numpy(), y.Tensor().numpy()):
            k = next(i for i in range(50) if np.array_equal(imgs[i].reshape(-1), row))
            assert lbls[k] == lab
            seen.append(k)
    assert len(set(seen)) == 48
    ds.Reset()
    assert ds.NextBatch() is not None
    with pytest.raises(FileNotFoundError):
        OaDsMnist(str(tmp_path), "test")


def test_text_datasets_and_subset(tmp_path):
    text = b"A: hello there\nB: hi\n\nA: how are you\nB: fine\n\n\nA: bye\n"
    p = tmp_path / "dialog.txt"
    p.write_bytes(text)
    dd = OaDsDailyDialog(str(p), batch_size=4, context_len=8, shuffle=False)
    assert dd.NumChars() == len(text) and dd.NumConversations() == 3 and dd.Size() == len(text) - 8
    s = dd.GetSample(3)
    assert bytes(s.X.Tensor().numpy()) == text[3:11] and int(s.Y.Tensor()[0]) == text[11] and dd.GetItem(10 ** 6).IsEmpty()
    x, y = dd.NextBatch()
    assert bytes(x.Tensor()[2].numpy()) == text[2:10] and int(y.Tensor()[2]) == text[10]
    ts = OaDsTinyShakespeare(str(p), batch_size=5, context_len=4)
    assert ts.NumBatches() == (len(text) - 4) // 5 and ts.ContextLen() == 4
    sub = OaDsSubset(ts, [5, 1])
    assert sub.Size() == 2 and bytes(sub.GetItem(1).Tensor().numpy()) == text[1:5] and sub.Parent() is ts
    with pytest.raises(IndexError):
        OaDsSubset(ts, [10 ** 6])


def test_sharded(tmp_path):
    for k, n in enumerate((100, 37, 64)):
        (tmp_path / f"shard{k}.bin").write_bytes(bytes((k * 50 + i) % 256 for i in range(n)))
    ds = OaDsSharded(str(tmp_path), 16)
    assert ds.NumShards() == 3 and ds.TotalBytes() == 201 and ds.Size() == 6 + 2 + 4 and ds.ShardBytes(1) == 37
    assert ds.GetItem(6).Tensor().tolist() == [(50 + i) % 256 for i in range(16)]
    assert ds.GetItem(11).Tensor().tolist() == [(100 + 48 + i) % 256 for i in range(16)]
    seq, state = ds.SampleSequence(123)
    assert len(seq) == 16 and state != 123


def test_fn_dataset():
    idx = list(range(100))
    OaFnDataset.Shuffle(idx, 7)
    again = list(range(100)); OaFnDataset.Shuffle(again, 7)
    assert idx == again and sorted(idx) == list(range(100)) and idx != list(range(100))
    sp = OaFnDataset.RandomSplit(100)
    assert (len(sp.Train), len(sp.Val), len(sp.Test)) == (80, 10, 10) and sorted(sp.Train + sp.Val + sp.Test) == list(range(100))
    from oa_b200.data.dataset import OaDataset
    b = OaFnDataset.Collate([OaDataset.Sample(OaMatrix(torch.ones(3) * i), OaMatrix(torch.tensor([i]))) for i in range(4)])
    assert b.X.Tensor().shape == (4, 3) and b.Y.Tensor().view(-1).tolist() == [0, 1, 2, 3]
    img = OaMatrix(torch.rand(2, 3, 4, 4))
    ref = (img.Tensor().clone() - torch.tensor([0.5, 0.4, 0.3]).view(1, 3, 1, 1)) / torch.tensor([0.2, 0.3, 0.4]).view(1, 3, 1, 1)
    assert OaFnDataset.Normalize(img, [0.5, 0.4, 0.3], [0.2, 0.3, 0.4]).IsOk() and torch.allclose(img.Tensor(), ref)
    assert not OaFnDataset.Normalize(img, [0, 0, 0], [1, 0, 1]).IsOk()
    m = OaMatrix(torch.tensor([2.0, 4.0, 6.0]))
    assert OaFnDataset.ScaleToRange(m, -1, 1).IsOk() and torch.allclose(m.Tensor(), torch.tensor([-1.0, 0.0, 1.0]))
    assert OaFnDataset.Cast(m, torch.int32).Tensor().dtype == torch.int32


def _recover_loop(f, frames, feat_dim=263):
    """Frame-by-frame statement of the recovery with explicit quaternion rotation."""
    joints = (feat_dim + 1) // 12
    f = np.asarray(f, np.float64).reshape(frames, feat_dim)
    def rot(a, v):                         # quaternion (x, y, z, w) = (0, -sin a, 0, cos a)
        q = np.array([0.0, -math.sin(a), 0.0]); w = math.cos(a)
        t = 2.0 * np.cross(q, v)
        return v + w * t + np.cross(q, t)
    yaw = np.zeros(frames)
    for t in range(1, frames):
        yaw[t] = yaw[t - 1] + f[t - 1, 0]
    root = np.zeros((frames, 3))
    for t in range(frames):
        d = np.array([f[t - 1, 1], 0.0, f[t - 1, 2]]) if t > 0 else np.zeros(3)
        root[t] = rot(yaw[t], d) + (root[t - 1] if t > 0 else 0)
    root[:, 1] = f[:, 3]
    out = np.zeros((frames, joints, 3))
    for t in range(frames):
        out[t, 0] = root[t]
        for j in range(joints - 1):
            w = rot(yaw[t], f[t, 4 + 3 * j: 7 + 3 * j])
            out[t, j + 1] = [w[0] + root[t, 0], w[1], w[2] + root[t, 2]]
    return out


def test_humanml3d(tmp_path):
    rng = np.random.default_rng(3)
    feats = (rng.standard_normal((12, 263)) * 0.2).astype(np.float32)
    world = OaHumanMl3dRecoverWorldJoints(feats, 12)
    assert world.shape == (12, 22, 3)
    np.testing.assert_allclose(world.numpy(), _recover_loop(feats, 12), atol=1e-5)
    assert OaHumanMl3dRecoverWorldJoints(feats, 12, 100).numel() == 0
    same = OaHumanMl3dEvaluateMotion(feats, feats, 12)
    assert same.Ok and same.MpjpeCm == 0 and same.VelocityErrorCmPerFrame == 0 and same.ContactAccuracy == 1.0
    shifted = feats.copy(); shifted[:, 3] += 0.1          # root 10 cm higher: only the root joint moves
    m = OaHumanMl3dEvaluateMotion(shifted, feats, 12)
    assert m.MpjpeCm == pytest.approx(10.0 / 22, rel=1e-4) and m.VelocityErrorCmPerFrame == pytest.approx(0, abs=1e-4)
    assert OaHumanMl3dMpjpeCm(world, world + 0.01) == pytest.approx(math.sqrt(3.0), rel=1e-5)
    os.makedirs(tmp_path / "new_joint_vecs"); os.makedirs(tmp_path / "texts")
    np.save(tmp_path / "Mean.npy", np.zeros(263, np.float32)); np.save(tmp_path / "Std.npy", np.full(263, 2.0, np.float32))
    (tmp_path / "train.txt").write_text("000001\n000002\nmissing\n")
    np.save(tmp_path / "new_joint_vecs" / "000001.npy", feats); np.save(tmp_path / "new_joint_vecs" / "000002.npy", feats[:5])
    (tmp_path / "texts" / "000001.txt").write_text("a person walks#a/DET person/NOUN walk/VERB#0.0#0.0\nthen sits#x#1.5#3.0\n")
    ds = OaDsHumanMl3d(str(tmp_path))
    assert ds.Ok() and ds.NumClips() == 2 and ds.TotalFrames() == 17 and ds.NumJoints() == 22 and ds.ClipId(1) == "000002"
    caps = ds.ClipCaptions(0)
    assert ds.ClipText(0) == "a person walks" and not caps[0].HasRange and caps[1].HasRange and caps[1].EndSec == 3.0
    assert torch.allclose(ds.GetItem(0).Tensor(), torch.from_numpy(feats) / 2) and ds.ClipText(1) == ""
    assert torch.allclose(ds.Denormalize(ds.GetItem(1).Tensor()), torch.from_numpy(feats[:5]))
    assert not OaDsHumanMl3d(str(tmp_path), "val").Ok()
