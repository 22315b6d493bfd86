""".oad archives, SafeTensors transfer, configuration, datasets / loader, the upload ring, OaMlTraining with gradient
accumulation, and the collective verbs on a two-process gloo mesh (CPU)."""
import json
import os
import struct
import subprocess
import sys

import pytest
import torch

from oa_b200.core import fn_matrix as F
from oa_b200.core.matrix import OaMatrix
from oa_b200.data import OaByteDataset, OaDataLoader, OaDataLoaderConfig, OaOadTokenDataset
from oa_b200.io import oad as OAD
from oa_b200.io import safetensors as ST
from oa_b200.ml import config as C
from oa_b200.ml.nn.layers import OaLinear, OaSequential, OaRelu
from oa_b200.runtime.upload import OaPrefetcher, OaUploadRing

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_oad_round_trip_and_rejection(tmp_path):
    p = str(tmp_path / "d.oad")
    assert OAD.OaOadWriteFile(p, b"train-bytes" * 10, b"val", b"")
    raw = open(p, "rb").read()
    assert len(raw) == 64 + 110 + 3 and OAD.OaOadProbeMagic(raw) and raw[:4] == b"OAD1"
    f = OAD.OaOadFile()
    assert f.TryOpen(p) and bytes(f.TrainSpan()) == b"train-bytes" * 10 and bytes(f.ValSpan()) == b"val" and len(f.TestSpan()) == 0
    f.Close()
    bad = bytearray(raw)
    struct.pack_into("<Q", bad, 20, 10 ** 9)              # train size beyond the file
    open(p, "wb").write(bytes(bad))
    assert not OAD.OaOadFile().TryOpen(p)
    open(p, "wb").write(b"nope")
    assert not OAD.OaOadFile().TryOpen(p)


def test_datasets_and_loader(tmp_path):
    p = str(tmp_path / "d.oad")
    OAD.OaOadWriteFile(p, bytes(range(256)) * 4, b"", b"")
    ds = OaOadTokenDataset(p, 16)
    assert ds.Size() == (1024 - 1) // 16
    s = ds.GetSample(3)
    assert torch.equal(s.X.Tensor()[1:], s.Y.Tensor()[:-1])
    cfg = OaDataLoaderConfig(BatchSize=8, Shuffle=True, Seed=5, DropLast=True, NumWorkers=2)
    a = [b.X.Tensor().clone() for b in OaDataLoader(ds, cfg)]
    b = [b.X.Tensor().clone() for b in OaDataLoader(ds, cfg)]
    assert len(a) == ds.Size() // 8 and all(torch.equal(x, y) for x, y in zip(a, b))      # same seed, same order
    assert a[0].shape == (8, 16)
    txt = tmp_path / "t.bin"
    txt.write_bytes(b"abcdefghij" * 10)
    bd = OaByteDataset(str(txt), 32)
    assert bd.Size() == 3 and bd.TotalBytes() == 100 and bd[0].Tensor()[0].item() == ord("a")


def test_safetensors_transfer(tmp_path):
    F.SetRngSeed(0)
    src = OaSequential(OaLinear(4, 6), OaRelu(), OaLinear(6, 2))
    tensors = {f"model.layers.{n.Name}": n.Param.Tensor().clone() for n in src.AllNamedParameterPtrs()}
    p = str(tmp_path / "m.safetensors")
    assert ST.OaSafeTensorWrite(p, tensors, {"format": "pt"})
    r = ST.OaSafeTensorReader()
    assert r.Open(p) and r.Metadata["format"] == "pt" and len(r.Names()) == 4
    r.Close()
    F.SetRngSeed(1)
    dst = OaSequential(OaLinear(4, 6), OaRelu(), OaLinear(6, 2))
    tw = ST.OaTransferWeights([ST.OaTransferRule(r"^model\.layers\.", "")])
    info, st = tw.Inspect(p)
    assert st and info["model.layers.0.weight"][1] == [6, 4]
    rep, st = tw.LoadInto(dst, p)
    assert st and rep.Ok() and len(rep.Loaded) == 4
    assert tw.Verify(dst, p)[1]
    # a wrong shape fails before anything is copied
    other = OaSequential(OaLinear(4, 5), OaRelu(), OaLinear(5, 2))
    before = [q.Tensor().clone() for q in other.AllParameterPtrs()]
    rep, st = tw.LoadInto(other, p)
    assert not st and rep.ShapeMismatch and all(torch.equal(q.Tensor(), b) for q, b in zip(other.AllParameterPtrs(), before))
    # corrupt header: offsets outside the file
    raw = bytearray(open(p, "rb").read())
    n = struct.unpack_from("<Q", raw, 0)[0]
    hdr = json.loads(bytes(raw[8:8 + n]))
    hdr["model.layers.0.weight"]["data_offsets"] = [0, 10 ** 9]
    hj = json.dumps(hdr).encode()
    open(p, "wb").write(struct.pack("<Q", len(hj)) + hj + bytes(raw[8 + n:]))
    assert not ST.OaSafeTensorReader().Open(p)


def test_config_yaml_and_budget():
    y = """
optimizer: {lr: 0.001, weight_decay: 0.1, scheduler: cosine, warmup_steps: 10}
training: {batch_size: 8, total_steps: 100, precision: fp32, grad_accum_steps: 4, phases: [{id: warm, steps: 10, lr: 0.01}]}
"""
    o, t = C.OaLoadOptimizerYaml(y), C.OaLoadTrainBaseYaml(y)
    assert o.Lr == pytest.approx(1e-3) and o.WeightDecay == pytest.approx(0.1) and o.Beta1 == pytest.approx(0.9)
    assert t.BatchSize == 8 and t.GradAccumSteps == 4 and t.Precision.name == "FP32" and t.UsesPhases() and t.Phases[0].Lr == 0.01
    sched = o.MakeScheduler(100)
    assert sched.GetLr(10) == pytest.approx(1e-3) and sched.GetLr(100) < 2e-5
    r = C.OaComputeVRAMBudget(1_000_000_000, 1 << 20, C.OaVRAMBudgetConfig(PreferredBatchSize=64, PreferredSeqLen=4096), available_bytes=80 << 30)
    assert r.FitsInVRAM and r.ModelBytes == 20_000_000_000 and (r.BatchSize < 64 or r.SeqLen < 4096)
    tiny = C.OaComputeVRAMBudget(10 ** 11, 4096, available_bytes=80 << 30)
    assert not tiny.FitsInVRAM


def test_upload_ring_and_prefetcher():
    ring = OaUploadRing(slot_bytes=1 << 16, slots=2, device="cpu")
    batches = [(torch.full((4, 8), i, dtype=torch.int32), torch.full((4,), -i, dtype=torch.int32)) for i in range(5)]
    got = list(OaPrefetcher(batches, ring, depth=2))
    assert len(got) == 5 and all(torch.equal(g[0], b[0]) and torch.equal(g[1], b[1]) for g, b in zip(got, batches))
    assert ring.BytesUploaded == 5 * (4 * 8 * 4 + 4 * 4)
    with pytest.raises(ValueError):
        ring.Upload(torch.zeros(1 << 20))
    # batched form: mixed dtypes and shapes, one packed transfer per dtype, staging buffers reused across calls
    hosts = [torch.randn(5), torch.arange(6).reshape(2, 3), torch.randn(2, 2), torch.arange(3)]
    for _ in range(3):
        outs, tok = ring.UploadMany(hosts)
        tok.Wait()
        assert all(o.dtype == h.dtype and o.shape == h.shape and torch.equal(o, h) for o, h in zip(outs, hosts))
    assert ring.UploadMany([])[0] == []


def test_ml_training_with_gradient_accumulation():
    from oa_b200.ml import fn_loss as L
    from oa_b200.ml.ml_training import OaMlTraining, OaMlTrainingConfig
    from oa_b200.ml.optim import OaSGD
    torch.manual_seed(0)
    xs, ys = torch.randn(8, 4), torch.randn(8, 2)

    def run(accum, bs):
        F.SetRngSeed(0)
        net = OaLinear(4, 2)
        opt = OaSGD(net.AllParameterPtrs(), 0.1)
        it = iter(range(10 ** 6))

        def nxt():
            i = next(it) % (8 // bs)
            return OaMatrix(xs[i * bs:(i + 1) * bs]), OaMatrix(ys[i * bs:(i + 1) * bs])

        t = OaMlTraining(net, opt, OaMlTrainingConfig(Steps=3, BatchSize=bs * accum, GradAccumSteps=accum, ProgressBar=False, Summary=False))
        assert t.Run(nxt, lambda x, y: L.Mse(net.Forward(x), y))
        return net.Weight.Tensor().clone()

    assert (run(1, 8) - run(4, 2)).abs().max().item() < 1e-5      # four micro-batches of 2 == one batch of 8


def test_collective_verbs_on_a_gloo_mesh(tmp_path):
    script = tmp_path / "coll.py"
    script.write_text(f"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, {ROOT!r})
dist.init_process_group("gloo")
from oa_b200.parallel.mesh import OaDeviceMesh, OaReduceOp
from oa_b200.parallel.collective import OaCollective
m = OaDeviceMesh(); c = OaCollective(m); r, W = m.rank, m.world
t = torch.arange(4, dtype=torch.float32) + 10 * r
assert torch.equal(c.AllReduce(t), torch.arange(4.) * W + 10 * sum(range(W)))
assert torch.equal(c.AllReduce(t, OaReduceOp.Max), torch.arange(4.) + 10 * (W - 1))
assert torch.equal(c.AllGather(t.reshape(1, 4)), torch.stack([torch.arange(4.) + 10 * k for k in range(W)]))
assert torch.equal(c.Broadcast(t, 1), torch.arange(4.) + 10)
full = torch.arange(W * 2, dtype=torch.float32).reshape(W, 2) + 100 * r
assert torch.equal(c.ReduceScatter(full), (torch.arange(W * 2.).reshape(W, 2)[r:r+1] * W + 100 * sum(range(W))))
a2a = c.AllToAll(full)
assert torch.equal(a2a, torch.stack([torch.arange(W * 2.).reshape(W, 2)[r] + 100 * k for k in range(W)]))
sc = c.Scatter(torch.arange(W * 3.).reshape(W, 3) if r == 0 else None, 0, shape=(W, 3), dtype=torch.float32)
assert torch.equal(sc, torch.arange(W * 3.).reshape(W, 3)[r:r+1])
c.Barrier()
if r == 0: print("COLL_OK")
dist.destroy_process_group()
""")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29591", str(script)], capture_output=True, text=True, timeout=240, cwd=ROOT,
                       env=dict(os.environ, OA_DEVICE="cpu", CUDA_VISIBLE_DEVICES=""))
    assert r.returncode == 0 and "COLL_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
