"""dsgen3danimctl: data pipeline of the skeletal-motion data sets (Apps/Ml/Gen3dAnim/dsgen3danimctl.cpp of the reference).

    python -m oa_b200.apps.dsgen3danimctl clean --in clip.usda [--save clip.3danim] [--usda c.usda] [--fbx c.fbx]
    python -m oa_b200.apps.dsgen3danimctl strip --in clip.usda | --dir folder
    python -m oa_b200.apps.dsgen3danimctl pack  --in folder --out set.usda [--val NAME ...] [--test NAME ...]
    python -m oa_b200.apps.dsgen3danimctl info  --dataset set.usda [--context 32]
    python -m oa_b200.apps.dsgen3danimctl bake  --dataset set.usda --out set.3dset [--root-delta]

clean   put a retargeted UE clip onto the clean canonical body: joints outside the skeleton (IK, weapon, corrective, twist)
        are dropped, a Y-up stage is turned Z-up, the result is packed to canonical channels and can be saved as `.3danim`,
        re-written as `.usda`, or exported as ASCII FBX
strip   delete the junk joints of source clips in place, the kept joints' samples untouched
pack    combine clips into ONE `.usda` data set (one Skeleton, one SkelAnimation per clip); the split of a clip is chosen by
        its name (`--val`, `--test` substrings), everything else trains
info    per-clip split / frames / seconds, window counts for a context length, per-channel statistic ranges
bake    the whole data set as one self-contained binary: header, per-channel mean / std, per-clip (name, split, frames),
        then the packed frames (`--root-delta` stores the root translation as per-frame deltas)
Everything runs on the CPU.
"""
from __future__ import annotations

import argparse
import json
import struct
import sys
from pathlib import Path
from typing import List

import torch

from ..core.types import OaError
from ..extensions import anim as A
from ..extensions import rig as R

JUNK_PREFIXES = ("ik_", "weapon", "center_of_mass", "interaction", "attach")
JUNK_PARTS = ("_twist_", "_corrective", "_bck_", "_fwd_", "_in_", "_out_")


def is_junk(leaf: str) -> bool:
    return leaf.startswith(JUNK_PREFIXES) or any(p in leaf for p in JUNK_PARTS)


def to_z_up(clip: A.OaUsdSkelClip) -> A.OaUsdSkelClip:
    """Y-up stage -> Z-up: rotate the ROOT joint's samples by +90 degrees about X (children are local, they do not change)."""
    if clip.UpAxis == 2:
        return clip
    rx = torch.tensor(R.EulerXyzDegToQuat((90.0, 0.0, 0.0)))
    m = R.QuatToMatrixT(rx)
    roots = [i for i, p in enumerate(clip.JointPaths) if "/" not in p]
    for i in roots:
        clip.Translations[:, i] = clip.Translations[:, i] @ m.t()
        clip.Rotations[:, i] = R.MatrixToQuatT(m @ R.QuatToMatrixT(clip.Rotations[:, i]))
    clip.UpAxis = 2
    return clip


def strip_clip(clip: A.OaUsdSkelClip) -> A.OaUsdSkelClip:
    keep = [i for i, p in enumerate(clip.JointPaths) if not any(is_junk(part) for part in p.split("/"))]
    pick = lambda t: None if t is None else t[keep]
    return A.OaUsdSkelClip([clip.JointPaths[i] for i in keep], pick(clip.BindTransforms), pick(clip.RestTransforms), clip.FrameCount, clip.Fps,
                           clip.UpAxis, clip.Translations[:, keep].clone(), clip.Rotations[:, keep].clone())


def clean_clip(clip: A.OaUsdSkelClip, sk: R.OaSkeleton) -> A.OaPoseClip:
    return A.OaPosePack.Pack(to_z_up(strip_clip(clip)), sk)


def split_of(name: str, val: List[str], test: List[str]) -> str:
    if any(s and s in name for s in test):
        return "test"
    if any(s and s in name for s in val):
        return "val"
    return "train"


def cmd_clean(a) -> int:
    sk = R.OaSkeletonById(a.skeleton)
    pose = clean_clip(A.OaUsd.ReadUsda(a.inp), sk)
    print(f"clean: {pose.FrameCount} frames x {pose.PoseDim} channels at {pose.Fps:g} fps on {sk.Name}")
    if a.save:
        st = pose.Write3dAnim(a.save)
        if not st.IsOk():
            print(st.message, file=sys.stderr)
            return 1
    if a.usda or a.fbx:
        clip = A.OaPosePack.Unpack(pose, sk)
        for path, fn in ((a.usda, lambda p: A.OaUsd.WriteUsda(p, clip)), (a.fbx, lambda p: A.OaFbxWriter.Write(p, sk, clip))):
            if path:
                st = fn(path)
                if not st.IsOk():
                    print(st.message, file=sys.stderr)
                    return 1
    return 0


def cmd_strip(a) -> int:
    files = [Path(a.inp)] if a.inp else sorted(Path(a.dir).glob("*.usda"))
    for f in files:
        clips = A.OaUsd.ReadUsdaMulti(f)
        before = clips[0].Clip.JointCount()
        for c in clips:
            c.Clip = strip_clip(c.Clip)
        st = A.OaUsd.WriteUsdaMulti(f, clips)
        if not st.IsOk():
            print(st.message, file=sys.stderr)
            return 1
        print(f"strip: {f.name}: {before} -> {clips[0].Clip.JointCount()} joints")
    return 0


def cmd_pack(a) -> int:
    sk = R.OaSkeletonById(a.skeleton)
    files = sorted(Path(a.inp).rglob("*.usda")) if a.inp else [Path(line.strip()) for line in Path(a.clips).read_text().splitlines() if line.strip()]
    named = []
    for f in files:
        for c in A.OaUsd.ReadUsdaMulti(f):
            name = f.stem if c.Name in ("anim", "clip") else c.Name
            canon = A.OaPosePack.Unpack(clean_clip(c.Clip, sk), sk)          # every clip on the same canonical joint list
            named.append(A.OaUsdNamedClip(name, split_of(name, a.val, a.test), canon))
    if not named:
        print("pack: no clips found", file=sys.stderr)
        return 1
    st = A.OaUsd.WriteUsdaMulti(a.out, named)
    if not st.IsOk():
        print(st.message, file=sys.stderr)
        return 1
    counts = {s: sum(c.Split == s for c in named) for s in ("train", "val", "test")}
    print(f"pack: {len(named)} clips -> {a.out} ({counts})")
    return 0


def dataset_table(path, sk: R.OaSkeleton, context: int):
    rows, frames = [], []
    for c in A.OaUsd.ReadUsdaMulti(path):
        pose = A.OaPosePack.Pack(c.Clip, sk)
        rows.append({"name": c.Name, "split": c.Split, "frames": pose.FrameCount, "seconds": round(pose.FrameCount / pose.Fps, 3),
                     "windows": max(0, pose.FrameCount - context + 1)})
        frames.append((c, pose))
    return rows, frames


def cmd_info(a) -> int:
    sk = R.OaSkeletonById(a.skeleton)
    rows, frames = dataset_table(a.dataset, sk, a.context)
    allf = torch.cat([p.Samples for _, p in frames], 0)
    mean, std = allf.mean(0), allf.std(0, unbiased=False)
    report = {"skeleton": sk.Name, "pose_dim": sk.PoseDim(), "clips": rows, "context": a.context, "total_frames": int(allf.shape[0]),
              "windows": {s: sum(r["windows"] for r in rows if r["split"] == s) for s in ("train", "val", "test")},
              "mean_range": [float(mean.min()), float(mean.max())], "std_range": [float(std.min()), float(std.max())]}
    print(json.dumps(report, indent=1))
    return 0


BAKE_MAGIC = b"3DST"


def cmd_bake(a) -> int:
    sk = R.OaSkeletonById(a.skeleton)
    _, frames = dataset_table(a.dataset, sk, 1)
    mats = []
    for _, p in frames:
        x = p.Samples.clone()
        if a.root_delta:                                   # root translation as per-frame deltas (first frame: zero)
            x[1:, 0:3] = p.Samples[1:, 0:3] - p.Samples[:-1, 0:3]
            x[0, 0:3] = 0
        mats.append(x)
    allf = torch.cat(mats, 0)
    mean, std = allf.mean(0), allf.std(0, unbiased=False).clamp_min(1e-6)
    with open(a.out, "wb") as f:
        f.write(struct.pack("<4sIIIIfI", BAKE_MAGIC, 1, int(a.root_delta), len(frames), sk.PoseDim(), frames[0][1].Fps, sk.SkeletonId))
        f.write(mean.numpy().astype("<f4").tobytes())
        f.write(std.numpy().astype("<f4").tobytes())
        for (c, p), x in zip(frames, mats):
            name = c.Name.encode()[:63]
            f.write(struct.pack("<64sBI", name, {"train": 0, "val": 1, "test": 2}[c.Split], p.FrameCount))
        for x in mats:
            f.write(x.numpy().astype("<f4").tobytes())
    print(f"bake: {len(frames)} clips, {allf.shape[0]} frames x {sk.PoseDim()} channels -> {a.out}")
    return 0


def read_bake(path):
    """(header dict, mean, std, [(name, split, frames tensor)]) of a baked data set."""
    blob = Path(path).read_bytes()
    magic, ver, delta, n, dim, fps, sid = struct.unpack_from("<4sIIIIfI", blob)
    if magic != BAKE_MAGIC or ver != 1:
        raise OaError(A.OaStatus.Error(A.OaStatusCode.InvalidArgument, f"{path}: not a baked motion data set"))
    import numpy as np
    off = struct.calcsize("<4sIIIIfI")
    mean = torch.from_numpy(np.frombuffer(blob, "<f4", dim, off).copy())
    std = torch.from_numpy(np.frombuffer(blob, "<f4", dim, off + 4 * dim).copy())
    off += 8 * dim
    meta = []
    for _ in range(n):
        name, split, fr = struct.unpack_from("<64sBI", blob, off)
        off += struct.calcsize("<64sBI")
        meta.append((name.rstrip(b"\0").decode(), ("train", "val", "test")[split], fr))
    clips = []
    for name, split, fr in meta:
        clips.append((name, split, torch.from_numpy(np.frombuffer(blob, "<f4", fr * dim, off).copy()).reshape(fr, dim)))
        off += 4 * fr * dim
    return {"root_delta": bool(delta), "clips": n, "pose_dim": dim, "fps": fps, "skeleton_id": sid}, mean, std, clips


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="dsgen3danimctl", description="skeletal-motion data set pipeline: clean -> strip -> pack -> info -> bake")
    ap.add_argument("--skeleton", type=int, default=0, help="0 MetaHuman body, 1 HumanIK, 2 HumanML3D")
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("clean")
    p.add_argument("--in", dest="inp", required=True)
    p.add_argument("--save")
    p.add_argument("--usda")
    p.add_argument("--fbx")
    p = sub.add_parser("strip")
    p.add_argument("--in", dest="inp")
    p.add_argument("--dir")
    p = sub.add_parser("pack")
    p.add_argument("--in", dest="inp")
    p.add_argument("--clips")
    p.add_argument("--out", required=True)
    p.add_argument("--val", action="append", default=[])
    p.add_argument("--test", action="append", default=[])
    p = sub.add_parser("info")
    p.add_argument("--dataset", required=True)
    p.add_argument("--context", type=int, default=32)
    p = sub.add_parser("bake")
    p.add_argument("--dataset", required=True)
    p.add_argument("--out", required=True)
    p.add_argument("--root-delta", action="store_true")
    a = ap.parse_args(argv)
    if a.cmd == "strip" and not (a.inp or a.dir):
        ap.error("strip needs --in or --dir")
    if a.cmd == "pack" and not (a.inp or a.clips):
        ap.error("pack needs --in or --clips")
    try:
        return {"clean": cmd_clean, "strip": cmd_strip, "pack": cmd_pack, "info": cmd_info, "bake": cmd_bake}[a.cmd](a)
    except OaError as e:
        print(f"dsgen3danimctl: {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
