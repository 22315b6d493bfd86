"""datasetctl: pack, inspect and unpack `.oad` dataset archives (train / val / test byte splits).

    python -m oa_b200.apps.datasetctl pack -o out.oad --train train.txt [--val val.txt] [--test test.txt]
    python -m oa_b200.apps.datasetctl info path.oad
    python -m oa_b200.apps.datasetctl unpack path.oad -o outdir

Reference: Apps/Ml/util/datasetctl.cpp.
"""
from __future__ import annotations

import argparse
import os
import sys

from ..io.oad import OaOadFile, OaOadWriteFile
from .modelctl import FormatBytes


def _read(path: str) -> bytes:
    if not path:
        return b""
    with open(path, "rb") as f:
        return f.read()


def CmdPack(out_path: str, train: str, val: str, test: str, out=print) -> int:
    try:
        parts = [_read(train), _read(val), _read(test)]
    except OSError as e:
        out(f"Error: {e}")
        return 1
    if not parts[0]:
        out("Error: the train split is empty")
        return 1
    st = OaOadWriteFile(out_path, *parts)
    if not st.IsOk():
        out(f"Error: {st.message}")
        return 1
    out(f"  wrote {out_path}: train {FormatBytes(len(parts[0]))}, val {FormatBytes(len(parts[1]))}, test {FormatBytes(len(parts[2]))}")
    return 0


def CmdInfo(path: str, out=print) -> int:
    f = OaOadFile()
    if not f.TryOpen(path):
        out(f"Error: not a valid .oad v1 file: {path}")
        return 1
    h = f.Header()
    out(f"  File:     {path}")
    out(f"  Size:     {FormatBytes(os.path.getsize(path))}")
    out(f"  Version:  {h.VersionMajor}.{h.VersionMinor}  flags=0x{h.Flags:x}")
    for name, off, n in (("Train", h.TrainOffset, h.TrainBytes), ("Val", h.ValOffset, h.ValBytes), ("Test", h.TestOffset, h.TestBytes)):
        out(f"  {name + ':':<9} {FormatBytes(n):>12} at offset {off}")
    f.Close()
    return 0


def CmdUnpack(path: str, outdir: str, out=print) -> int:
    f = OaOadFile()
    if not f.TryOpen(path):
        out(f"Error: not a valid .oad v1 file: {path}")
        return 1
    os.makedirs(outdir, exist_ok=True)
    for name, span in (("train.txt", f.TrainSpan()), ("val.txt", f.ValSpan()), ("test.txt", f.TestSpan())):
        if len(span):
            with open(os.path.join(outdir, name), "wb") as g:
                g.write(bytes(span))
            out(f"  {os.path.join(outdir, name)}: {FormatBytes(len(span))}")
    f.Close()
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="datasetctl", description="Pack, inspect and unpack .oad dataset archives")
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("pack")
    p.add_argument("-o", "--out", required=True)
    p.add_argument("--train", required=True)
    p.add_argument("--val", default="")
    p.add_argument("--test", default="")
    sub.add_parser("info").add_argument("path")
    u = sub.add_parser("unpack")
    u.add_argument("path")
    u.add_argument("-o", "--out", required=True)
    a = ap.parse_args(argv)
    if a.cmd == "pack": return CmdPack(a.out, a.train, a.val, a.test)
    if a.cmd == "info": return CmdInfo(a.path)
    return CmdUnpack(a.path, a.out)


if __name__ == "__main__":
    sys.exit(main())
