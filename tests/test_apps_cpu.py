"""modelctl / datasetctl command functions on temporary files."""
import os

import torch

from oa_b200.apps import datasetctl, modelctl
from oa_b200.io.oam import OamModel
from oa_b200.io.safetensors import OaSafeTensorWrite


def run(fn, *args):
    lines = []
    rc = fn(*args, out=lines.append)
    return rc, "\n".join(lines)


def test_modelctl_commands(tmp_path):
    st = str(tmp_path / "w.safetensors")
    tensors = {"layer.0.weight": torch.randn(4, 8), "layer.0.bias": torch.randn(4), "emb": torch.randn(16, 8).bfloat16()}
    assert OaSafeTensorWrite(st, tensors).IsOk()
    rc, text = run(modelctl.CmdInspect, st)
    assert rc == 0 and "layer.0.weight" in text and "3 tensors" in text
    oam = str(tmp_path / "m.oam")
    rc, text = run(modelctl.CmdImport, st, "auto", "raw", oam, "preserve", True)
    assert rc == 0 and "imported 3 tensors" in text and "checksums valid" in text
    assert run(modelctl.CmdImport, st, "auto", "raw", oam, "bf16", False)[0] == 1         # raw keeps dtypes
    assert run(modelctl.CmdImport, st, "gguf", "raw", oam, "preserve", False)[0] == 1
    rc, text = run(modelctl.CmdInfo, oam)
    assert rc == 0 and "raw" in text and "3 tensors" in text and "BFloat16" in text
    rc, text = run(modelctl.CmdDump, oam)
    assert rc == 0 and "CHECKSUM MISMATCH" not in text and "section 0" in text
    m, _ = OamModel.Load(oam)
    assert torch.equal(m.FindWeight("emb").ToTorch(), tensors["emb"])
    # a second file with one tensor changed: compare reports it, list finds both
    other = str(tmp_path / "sub" / "n.oam")
    os.makedirs(os.path.dirname(other))
    m2 = OamModel()
    for k, v in tensors.items():
        m2.AddWeight(k, v + 1 if k == "layer.0.bias" else v)
    m2.SetConfig("raw")
    assert m2.Save(other).IsOk()
    assert run(modelctl.CmdCompare, oam, oam)[0] == 0
    rc, text = run(modelctl.CmdCompare, oam, other)
    assert rc == 2 and "layer.0.bias" in text and "1 difference" in text
    rc, text = run(modelctl.CmdList, str(tmp_path))
    assert rc == 0 and "2 model(s)" in text
    # corruption: flip a payload byte -> verify fails at load, dump names the section
    data = bytearray(open(oam, "rb").read())
    data[-5] ^= 0xFF
    bad = str(tmp_path / "bad.oam")
    open(bad, "wb").write(bytes(data))
    assert run(modelctl.CmdVerify, bad)[0] == 1
    assert "CHECKSUM MISMATCH" in run(modelctl.CmdDump, bad)[1]
    nan = OamModel()
    nan.AddWeight("w", torch.tensor([1.0, float("nan")]))
    nan.SetConfig("raw")
    nanp = str(tmp_path / "nan.oam")
    assert nan.Save(nanp).IsOk() and run(modelctl.CmdVerify, nanp)[0] == 1
    assert modelctl.main(["info", oam]) == 0 and modelctl.main(["validate", oam, "--reference", other]) == 2


def test_datasetctl_round_trip(tmp_path):
    tr, va = tmp_path / "train.txt", tmp_path / "val.txt"
    tr.write_bytes(b"hello world " * 100)
    va.write_bytes(b"validation")
    oad = str(tmp_path / "d.oad")
    rc, text = run(datasetctl.CmdPack, oad, str(tr), str(va), "")
    assert rc == 0 and "wrote" in text
    rc, text = run(datasetctl.CmdInfo, oad)
    assert rc == 0 and "Train:" in text and "1.20 KB" in text
    out = tmp_path / "out"
    assert run(datasetctl.CmdUnpack, oad, str(out))[0] == 0
    assert (out / "train.txt").read_bytes() == tr.read_bytes() and (out / "val.txt").read_bytes() == b"validation" and not (out / "test.txt").exists()
    assert run(datasetctl.CmdInfo, str(tr))[0] == 1 and run(datasetctl.CmdPack, oad, str(tmp_path / "missing"), "", "")[0] == 1
    assert datasetctl.main(["info", oad]) == 0
