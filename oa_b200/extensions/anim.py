"""Skeletal-motion containers and converters: OaPoseClip (`.3danim`), OaUsdSkelClip with a minimal `.usda` UsdSkel writer /
reader, OaPosePack (clip <-> packed canonical channels), an ASCII FBX writer, and the rest-relative retarget.

Reference: Extensions/Public/Anim/{PoseClip,PosePack,Usd,FbxWriter}.h, Extensions/Public/Retarget/Retarget.h and their
sources under Extensions/Private.  Formats kept: `.3danim` = magic "3DAN", version, flags, frame count, pose dimension, fps,
skeleton id, then row-major f32[frames * pose_dim]; canonical channels in joint order (translate xyz when live, then 6-D
rotation = first two columns of the local rotation, or one hinge angle about the rest orient's Z), soft foot contacts
trailing (height band 6 cm, speed threshold 40 cm/s, value = height term x speed term).  The converters work on tensors
over all frames at once.
"""
from __future__ import annotations

import math
import re
import struct
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Optional, Sequence

import torch

from ..core.types import OaError, OaStatus, OaStatusCode
from . import rig as R

MAGIC = b"3DAN"
_HEAD = struct.Struct("<4sIIIIfI")       # magic, version, flags, frames, pose_dim, fps, skeleton_id


def _fail(code, msg):
    raise OaError(OaStatus.Error(code, msg))


# ----------------------------------------------------------------------------------------------------------- pose clip
@dataclass
class OaPoseClip:
    FormatVersion = 1
    Version: int = 1
    Flags: int = 0
    FrameCount: int = 0
    PoseDim: int = 0
    Fps: float = 30.0
    SkeletonId: int = 0
    Samples: torch.Tensor = field(default_factory=lambda: torch.zeros(0, 0))        # [FrameCount, PoseDim] float32

    def IsValid(self) -> bool:
        return (self.FrameCount > 0 and self.PoseDim > 0 and self.Fps > 0 and tuple(self.Samples.shape) == (self.FrameCount, self.PoseDim)
                and bool(torch.isfinite(self.Samples).all()))

    def ValueCount(self) -> int:
        return self.FrameCount * self.PoseDim

    @staticmethod
    def Create(frames: int, pose_dim: int, fps: float, skeleton_id: int, samples, flags: int = 0) -> "OaPoseClip":
        t = torch.as_tensor(samples, dtype=torch.float32).reshape(-1)
        if frames <= 0 or pose_dim <= 0 or fps <= 0 or t.numel() != frames * pose_dim:
            _fail(OaStatusCode.InvalidArgument, f"OaPoseClip.Create: {t.numel()} samples for {frames} frames x {pose_dim} channels at {fps} fps")
        return OaPoseClip(1, flags, frames, pose_dim, float(fps), skeleton_id, t.reshape(frames, pose_dim).clone())

    def Write3dAnim(self, path) -> OaStatus:
        if not self.IsValid():
            return OaStatus.Error(OaStatusCode.InvalidArgument, "Write3dAnim: invalid clip")
        try:
            with open(path, "wb") as f:
                f.write(_HEAD.pack(MAGIC, self.Version, self.Flags, self.FrameCount, self.PoseDim, self.Fps, self.SkeletonId))
                f.write(self.Samples.contiguous().cpu().numpy().astype("<f4").tobytes())
        except OSError as e:
            return OaStatus.Error(OaStatusCode.PermissionDenied, f"cannot write {path}: {e}")
        return OaStatus.Ok()

    @staticmethod
    def Read3dAnim(path) -> "OaPoseClip":
        try:
            blob = Path(path).read_bytes()
        except OSError as e:
            _fail(OaStatusCode.NotFound, f"cannot read {path}: {e}")
        if len(blob) < _HEAD.size:
            _fail(OaStatusCode.DataLoss, f"{path}: shorter than the .3danim header")
        magic, ver, flags, frames, dim, fps, sid = _HEAD.unpack_from(blob)
        if magic != MAGIC:
            _fail(OaStatusCode.InvalidArgument, f"{path}: not a .3danim file")
        if ver != OaPoseClip.FormatVersion:
            _fail(OaStatusCode.InvalidArgument, f"{path}: .3danim version {ver}, expected {OaPoseClip.FormatVersion}")
        need = frames * dim * 4
        if frames == 0 or dim == 0 or len(blob) - _HEAD.size != need:
            _fail(OaStatusCode.DataLoss, f"{path}: payload of {len(blob) - _HEAD.size} bytes, header promises {need}")
        import numpy as np
        data = torch.from_numpy(np.frombuffer(blob, dtype="<f4", offset=_HEAD.size).copy()).reshape(frames, dim)
        return OaPoseClip(ver, flags, frames, dim, fps, sid, data)

    def WriteTxt(self, path) -> OaStatus:
        try:
            with open(path, "w") as f:
                f.write(f"# 3danim frames={self.FrameCount} pose_dim={self.PoseDim} fps={self.Fps:g} skeleton_id={self.SkeletonId}\n")
                for row in self.Samples.tolist():
                    f.write(" ".join(f"{v:.6f}" for v in row) + "\n")
        except OSError as e:
            return OaStatus.Error(OaStatusCode.PermissionDenied, f"cannot write {path}: {e}")
        return OaStatus.Ok()


# ------------------------------------------------------------------------------------------------------- USD skel clip
@dataclass
class OaUsdSkelClip:
    JointPaths: List[str] = field(default_factory=list)                 # "root/pelvis/spine_01"
    BindTransforms: Optional[torch.Tensor] = None                       # [J, 4, 4] world bind, row-vector
    RestTransforms: Optional[torch.Tensor] = None                       # [J, 4, 4] local rest, row-vector
    FrameCount: int = 0
    Fps: float = 30.0
    UpAxis: int = 2
    Translations: torch.Tensor = field(default_factory=lambda: torch.zeros(0, 0, 3))    # [F, J, 3]
    Rotations: torch.Tensor = field(default_factory=lambda: torch.zeros(0, 0, 4))       # [F, J, 4] (x, y, z, w)

    def JointCount(self) -> int:
        return len(self.JointPaths)

    def IsValid(self) -> bool:
        J, F = self.JointCount(), self.FrameCount
        return J > 0 and F > 0 and self.Fps > 0 and tuple(self.Translations.shape) == (F, J, 3) and tuple(self.Rotations.shape) == (F, J, 4)

    def LeafNames(self) -> List[str]:
        return [p.rsplit("/", 1)[-1] for p in self.JointPaths]


@dataclass
class OaUsdNamedClip:
    Name: str = "clip"
    Split: str = "train"
    Clip: OaUsdSkelClip = field(default_factory=OaUsdSkelClip)


def SkeletonJointPaths(sk: R.OaSkeleton) -> List[str]:
    paths: List[str] = []
    for j in sk.Joints:
        paths.append(j.Name if j.ParentIndex < 0 else paths[j.ParentIndex] + "/" + j.Name)
    return paths


def _rest_matrices(sk: R.OaSkeleton):
    rest = torch.tensor([R.TrsMatrix((1, 1, 1), j.Rest.OrientedRotation(), j.Rest.Translate) for j in sk.Joints], dtype=torch.float32)
    bind = []
    for i, j in enumerate(sk.Joints):
        bind.append(rest[i] if j.ParentIndex < 0 else rest[i] @ bind[j.ParentIndex])       # row-vector: child . parent
    return torch.stack(bind), rest


def RestClip(sk: R.OaSkeleton, frames: int = 1, fps: float = 30.0) -> OaUsdSkelClip:
    """A clip that holds the skeleton at rest (bind / rest matrices filled): the canvas animations are written onto."""
    bind, rest = _rest_matrices(sk)
    tr = torch.tensor([j.Rest.Translate for j in sk.Joints], dtype=torch.float32).expand(frames, -1, -1).clone()
    ro = torch.tensor([j.Rest.OrientedRotation() for j in sk.Joints], dtype=torch.float32).expand(frames, -1, -1).clone()
    return OaUsdSkelClip(SkeletonJointPaths(sk), bind, rest, frames, fps, 2, tr, ro)


class OaUsd:
    """Minimal `.usda` UsdSkel writer / reader: SkelRoot -> Skeleton (joints, bind, rest) -> SkelAnimation prims with
    translations and rotations as timeSamples.  Not a composition engine."""

    @staticmethod
    def _mat(m) -> str:
        return "( " + ", ".join("(" + ", ".join(f"{v:.7g}" for v in row) + ")" for row in m.tolist()) + " )"

    @staticmethod
    def _anim(name: str, split: str, clip: OaUsdSkelClip, joints_decl: str) -> List[str]:
        out = [f'    def SkelAnimation "{name}" (', f'        customData = {{ dictionary oa = {{ string split = "{split}" }} }}', "    )", "    {",
               f"        uniform token[] joints = {joints_decl}", "        float3[] translations.timeSamples = {"]
        for f in range(clip.FrameCount):
            out.append(f"            {f}: [" + ", ".join("(%.7g, %.7g, %.7g)" % tuple(v) for v in clip.Translations[f].tolist()) + "],")
        out += ["        }", "        quatf[] rotations.timeSamples = {"]
        for f in range(clip.FrameCount):                                    # USD quatf order is (w, x, y, z)
            out.append(f"            {f}: [" + ", ".join("(%.7g, %.7g, %.7g, %.7g)" % (q[3], q[0], q[1], q[2]) for q in clip.Rotations[f].tolist()) + "],")
        out += ["        }", "        half3[] scales = [" + ", ".join("(1, 1, 1)" for _ in clip.JointPaths) + "]", "    }"]
        return out

    @staticmethod
    def WriteUsdaMulti(path, clips: Sequence[OaUsdNamedClip], default_prim: str = "rig") -> OaStatus:
        if not clips or not all(c.Clip.IsValid() for c in clips):
            return OaStatus.Error(OaStatusCode.InvalidArgument, "WriteUsda: invalid clip")
        first = clips[0].Clip
        if any(c.Clip.JointPaths != first.JointPaths for c in clips):
            return OaStatus.Error(OaStatusCode.InvalidArgument, "WriteUsdaMulti: the clips do not share one joint list")
        joints = "[" + ", ".join(f'"{p}"' for p in first.JointPaths) + "]"
        frames = max(c.Clip.FrameCount for c in clips)
        up = "Z" if first.UpAxis == 2 else "Y"
        lines = ["#usda 1.0", "(", f'    defaultPrim = "{default_prim}"', f"    endTimeCode = {frames - 1}", "    startTimeCode = 0",
                 f"    timeCodesPerSecond = {first.Fps:g}", f"    framesPerSecond = {first.Fps:g}", "    metersPerUnit = 0.01", f'    upAxis = "{up}"', ")", "",
                 f'def SkelRoot "{default_prim}"', "{", '    def Skeleton "skeleton" (', '        prepend apiSchemas = ["SkelBindingAPI"]', "    )", "    {",
                 f"        uniform token[] joints = {joints}"]
        if first.BindTransforms is not None:
            lines.append("        uniform matrix4d[] bindTransforms = [" + ", ".join(OaUsd._mat(m) for m in first.BindTransforms) + "]")
        if first.RestTransforms is not None:
            lines.append("        uniform matrix4d[] restTransforms = [" + ", ".join(OaUsd._mat(m) for m in first.RestTransforms) + "]")
        lines.append(f'        rel skel:animationSource = </{default_prim}/{clips[0].Name}>')
        lines.append("    }")
        for c in clips:
            lines += OaUsd._anim(c.Name, c.Split, c.Clip, joints)
        lines.append("}")
        try:
            Path(path).write_text("\n".join(lines) + "\n")
        except OSError as e:
            return OaStatus.Error(OaStatusCode.PermissionDenied, f"cannot write {path}: {e}")
        return OaStatus.Ok()

    @staticmethod
    def WriteUsda(path, clip: OaUsdSkelClip, default_prim: str = "rig") -> OaStatus:
        return OaUsd.WriteUsdaMulti(path, [OaUsdNamedClip("anim", "train", clip)], default_prim)

    @staticmethod
    def _tuples(text: str, width: int) -> torch.Tensor:
        nums = [float(x) for x in re.findall(r"[-+]?(?:\d+\.?\d*|\.\d+)(?:[eE][-+]?\d+)?", text)]
        if len(nums) % width:
            _fail(OaStatusCode.DataLoss, "usda: a tuple array does not divide into its tuple width")
        return torch.tensor(nums, dtype=torch.float32).reshape(-1, width)

    @staticmethod
    def _samples(block: str, attr: str, width: int, joints: int) -> torch.Tensor:
        m = re.search(re.escape(attr) + r"\.timeSamples\s*=\s*\{(.*?)\n\s*\}", block, flags=re.S)
        if not m:
            _fail(OaStatusCode.DataLoss, f"usda: no {attr}.timeSamples")
        frames = []
        for fm in re.finditer(r"(-?\d+(?:\.\d+)?)\s*:\s*\[(.*?)\]\s*,?", m.group(1), flags=re.S):
            t = OaUsd._tuples(fm.group(2), width)
            if t.shape[0] != joints:
                _fail(OaStatusCode.DataLoss, f"usda: a time sample of {attr} holds {t.shape[0]} values for {joints} joints")
            frames.append((float(fm.group(1)), t))
        frames.sort(key=lambda x: x[0])
        return torch.stack([t for _, t in frames])

    @staticmethod
    def ReadUsdaMulti(path) -> List[OaUsdNamedClip]:
        try:
            text = Path(path).read_text()
        except OSError as e:
            _fail(OaStatusCode.NotFound, f"cannot read {path}: {e}")
        if not text.lstrip().startswith("#usda"):
            _fail(OaStatusCode.InvalidArgument, f"{path}: not a .usda text file")
        fps = re.search(r"timeCodesPerSecond\s*=\s*([\d.]+)", text)
        up = re.search(r'upAxis\s*=\s*"([YZ])"', text)
        sk = re.search(r'def Skeleton\s+"[^"]*".*?\n    \}', text, flags=re.S)
        jm = re.search(r"uniform token\[\] joints\s*=\s*\[(.*?)\]", sk.group(0) if sk else text, flags=re.S)
        if not jm:
            _fail(OaStatusCode.DataLoss, f"{path}: no joints array")
        joints = re.findall(r'"([^"]+)"', jm.group(1))
        bind = rest = None
        if sk:
            for attr in ("bindTransforms", "restTransforms"):
                mm = re.search(attr + r"\s*=\s*\[(.*?)\]\s*\n", sk.group(0), flags=re.S)
                if mm:
                    t = OaUsd._tuples(mm.group(1), 16).reshape(-1, 4, 4)
                    if t.shape[0] == len(joints):
                        bind, rest = (t, rest) if attr == "bindTransforms" else (bind, t)
        out = []
        for am in re.finditer(r'def SkelAnimation\s+"([^"]+)"(.*?)\n    \}', text, flags=re.S):
            block = am.group(2)
            split = re.search(r'string split\s*=\s*"([^"]+)"', block)
            tr = OaUsd._samples(block, "translations", 3, len(joints))
            ro = OaUsd._samples(block, "rotations", 4, len(joints))
            ro = torch.cat([ro[..., 1:4], ro[..., 0:1]], -1)               # (w, x, y, z) on disk -> (x, y, z, w)
            if tr.shape[0] != ro.shape[0]:
                _fail(OaStatusCode.DataLoss, f"{path}: translations and rotations of {am.group(1)} differ in frame count")
            clip = OaUsdSkelClip(list(joints), bind, rest, tr.shape[0], float(fps.group(1)) if fps else 30.0, 2 if (up is None or up.group(1) == "Z") else 1, tr, ro)
            out.append(OaUsdNamedClip(am.group(1), split.group(1) if split else "train", clip))
        if not out:
            _fail(OaStatusCode.DataLoss, f"{path}: no SkelAnimation prim")
        return out

    @staticmethod
    def ReadUsda(path) -> OaUsdSkelClip:
        return OaUsd.ReadUsdaMulti(path)[0].Clip


# ------------------------------------------------------------------------------------------------------------ pose pack
HEIGHT_BAND_CM = 6.0
SPEED_THRESHOLD_CM_S = 40.0


def _match_joints(clip: OaUsdSkelClip, sk: R.OaSkeleton) -> List[int]:
    leaf = {n: i for i, n in enumerate(clip.LeafNames())}
    idx = []
    for j in sk.Joints:
        if j.Name not in leaf:
            _fail(OaStatusCode.InvalidArgument, f"OaPosePack: the clip has no joint named {j.Name!r}")
        idx.append(leaf[j.Name])
    return idx


def _world_positions(sk: R.OaSkeleton, rot: torch.Tensor, trans: torch.Tensor) -> torch.Tensor:
    """rot [F, J, 3, 3] full local rotations, trans [F, J, 3] local offsets -> world positions [F, J, 3]."""
    wpos, wrot = [None] * sk.JointCount(), [None] * sk.JointCount()
    for i, j in enumerate(sk.Joints):
        if j.ParentIndex < 0:
            wpos[i], wrot[i] = trans[:, i], rot[:, i]
        else:
            p = j.ParentIndex
            wpos[i] = wpos[p] + (wrot[p] @ trans[:, i, :, None]).squeeze(-1)
            wrot[i] = wrot[p] @ rot[:, i]
    return torch.stack(wpos, 1)


class OaPosePack:
    @staticmethod
    def Pack(clip: OaUsdSkelClip, sk: R.OaSkeleton) -> OaPoseClip:
        """USD SkelAnimation clip -> packed canonical channels (quat -> 6-D or hinge angle, live translations, contacts from
        forward kinematics on foot height and horizontal speed)."""
        if not clip.IsValid() or not sk.IsValid():
            _fail(OaStatusCode.InvalidArgument, "OaPosePack.Pack: invalid clip or skeleton")
        idx = _match_joints(clip, sk)
        F, D = clip.FrameCount, sk.PoseDim()
        quat = clip.Rotations[:, idx].float()
        trans = clip.Translations[:, idx].float().clone()
        rest = torch.tensor([j.Rest.Translate for j in sk.Joints], dtype=torch.float32)
        live = torch.tensor([j.HasTranslate for j in sk.Joints])
        trans[:, ~live] = rest[~live]                                  # locked translate channels stay at rest
        rot = R.QuatToMatrixT(quat)
        out = torch.zeros(F, D)
        for s, j in enumerate(sk.Joints):
            c = sk.ChannelOffset(s)
            if j.HasTranslate:
                out[:, c:c + 3] = trans[:, s]
                c += 3
            if j.RotDof == 3:
                out[:, c:c + 6] = R.Rot6dFromMatrix(rot[:, s])
            elif j.RotDof == 1:                                        # angle about the rest orient's local Z
                o = j.Rest.JointOrient
                conj = torch.tensor([-o[0], -o[1], -o[2], o[3]])
                q = quat[:, s]
                dz = conj[3] * q[:, 2] + conj[0] * q[:, 1] - conj[1] * q[:, 0] + conj[2] * q[:, 3]
                dw = conj[3] * q[:, 3] - conj[0] * q[:, 0] - conj[1] * q[:, 1] - conj[2] * q[:, 2]
                out[:, c] = 2.0 * torch.atan2(dz, dw)
        C = len(sk.ContactJoints)
        if C:
            up = clip.UpAxis
            h0, h1 = [a for a in (0, 1, 2) if a != up]
            w = _world_positions(sk, rot, trans)[:, sk.ContactJoints]          # [F, C, 3]
            floor = w[..., up].min()
            prev = torch.cat([w[:1], w[:-1]], 0)
            nxt = torch.cat([w[1:], w[-1:]], 0)
            dt = torch.full((F, 1), 2.0 / clip.Fps)
            dt[0] = dt[-1] = 1.0 / clip.Fps
            speed = torch.sqrt((nxt[..., h0] - prev[..., h0]) ** 2 + (nxt[..., h1] - prev[..., h1]) ** 2) / dt.clamp_min(1e-6)
            height_term = (1.0 - (w[..., up] - floor) / HEIGHT_BAND_CM).clamp(0, 1)
            speed_term = (1.0 - speed / SPEED_THRESHOLD_CM_S).clamp(0, 1)
            out[:, sk.ContactOffset():] = height_term * speed_term
        return OaPoseClip.Create(F, D, clip.Fps, sk.SkeletonId, out)

    @staticmethod
    def Unpack(pose: OaPoseClip, sk: R.OaSkeleton) -> OaUsdSkelClip:
        """Packed channels -> USD clip (6-D -> quat, hinge angle -> rest orient x spin about Z, locked translations from the
        rest pose, bind / rest matrices from the skeleton, contacts dropped)."""
        if not pose.IsValid() or not sk.IsValid():
            _fail(OaStatusCode.InvalidArgument, "OaPosePack.Unpack: invalid clip or skeleton")
        if pose.PoseDim != sk.PoseDim():
            _fail(OaStatusCode.InvalidArgument, f"OaPosePack.Unpack: pose dimension {pose.PoseDim} != skeleton channel budget {sk.PoseDim()}")
        F = pose.FrameCount
        clip = RestClip(sk, F, pose.Fps)
        x = pose.Samples.float()
        for s, j in enumerate(sk.Joints):
            c = sk.ChannelOffset(s)
            if j.HasTranslate:
                clip.Translations[:, s] = x[:, c:c + 3]
                c += 3
            if j.RotDof == 3:
                clip.Rotations[:, s] = R.MatrixToQuatT(R.MatrixFromRot6d(x[:, c:c + 6]))
            elif j.RotDof == 1:
                h = x[:, c] * 0.5
                ox, oy, oz, ow = j.Rest.JointOrient
                sz, cz = torch.sin(h), torch.cos(h)                    # rest orient (x) (0, 0, sin, cos)
                clip.Rotations[:, s] = torch.stack([ox * cz + oy * sz, oy * cz - ox * sz, oz * cz + ow * sz, ow * cz - oz * sz], -1)
        return clip


# -------------------------------------------------------------------------------------------------------------- retarget
class OaRetarget:
    @staticmethod
    def RetargetClip(src: R.OaSkeleton, dst: R.OaSkeleton, clip: OaPoseClip, src_ref: R.OaRefPose, dst_ref: R.OaRefPose) -> OaPoseClip:
        """Rest-relative rotation transfer: every joint's rotation relative to the SOURCE reference pose is re-applied on top
        of the DESTINATION reference (q_dst = ref_dst (x) conj(ref_src) (x) q_src).  Source and destination share the channel
        layout; root translation, hinge angles' layout and contacts pass through."""
        if src.JointCount() != dst.JointCount() or src.PoseDim() != dst.PoseDim() or clip.PoseDim != src.PoseDim():
            _fail(OaStatusCode.InvalidArgument, "OaRetarget: source and destination must share the channel layout of the clip")
        usd = OaPosePack.Unpack(clip, src)
        q = usd.Rotations.clone()
        for s, (js, jd) in enumerate(zip(src.Joints, dst.Joints)):
            if js.RotDof != jd.RotDof or js.HasTranslate != jd.HasTranslate:
                _fail(OaStatusCode.InvalidArgument, f"OaRetarget: joint {s} has different channels in the two skeletons")
            delta = R.QuatMul(dst_ref.OrientOf(jd.Name), R.QuatConjugate(src_ref.OrientOf(js.Name)))
            d = torch.tensor(delta, dtype=torch.float32)
            a = q[:, s]
            q[:, s] = torch.stack([d[3] * a[:, 0] + d[0] * a[:, 3] + d[1] * a[:, 2] - d[2] * a[:, 1],
                                   d[3] * a[:, 1] - d[0] * a[:, 2] + d[1] * a[:, 3] + d[2] * a[:, 0],
                                   d[3] * a[:, 2] + d[0] * a[:, 1] - d[1] * a[:, 0] + d[2] * a[:, 3],
                                   d[3] * a[:, 3] - d[0] * a[:, 0] - d[1] * a[:, 1] - d[2] * a[:, 2]], -1)
        out = RestClip(dst, clip.FrameCount, clip.Fps)
        out.Rotations = q
        live = [s for s, j in enumerate(dst.Joints) if j.HasTranslate]
        out.Translations[:, live] = usd.Translations[:, live]
        packed = OaPosePack.Pack(out, dst)
        C = len(dst.ContactJoints)
        if C:
            packed.Samples[:, dst.ContactOffset():] = clip.Samples[:, src.ContactOffset():]
        return packed


# -------------------------------------------------------------------------------------------------------------- FBX
class OaFbxWriter:
    """ASCII FBX 7.4 writer for one skeleton and one take: LimbNode models with their rest transforms, parent connections,
    and per-joint translation / Euler rotation curves (Extensions/Public/Anim/FbxWriter.h)."""
    TICKS_PER_SECOND = 46186158000

    @staticmethod
    def _euler_xyz_deg(m: torch.Tensor) -> torch.Tensor:
        """[..., 3, 3] column-vector rotations -> XYZ Euler degrees (X applied first): R = Rz Ry Rx."""
        sy = (-m[..., 2, 0]).clamp(-1, 1)
        y = torch.asin(sy)
        x = torch.atan2(m[..., 2, 1], m[..., 2, 2])
        z = torch.atan2(m[..., 1, 0], m[..., 0, 0])
        return torch.rad2deg(torch.stack([x, y, z], -1))

    @staticmethod
    def Write(path, sk: R.OaSkeleton, clip: Optional[OaUsdSkelClip] = None, take: str = "Take 001") -> OaStatus:
        if not sk.IsValid() or (clip is not None and not clip.IsValid()):
            return OaStatus.Error(OaStatusCode.InvalidArgument, "OaFbxWriter: invalid skeleton or clip")
        idx = _match_joints(clip, sk) if clip is not None else None
        J = sk.JointCount()
        uid = lambda k, base: base + k
        L = ["; FBX 7.4.0 project file", "FBXHeaderExtension:  {", "\tFBXHeaderVersion: 1003", "\tFBXVersion: 7400", '\tCreator: "oa_b200"', "}",
             "GlobalSettings:  {", "\tVersion: 1000", "\tProperties70:  {", '\t\tP: "UpAxis", "int", "Integer", "",2', '\t\tP: "UpAxisSign", "int", "Integer", "",1',
             '\t\tP: "FrontAxis", "int", "Integer", "",1', '\t\tP: "CoordAxis", "int", "Integer", "",0', '\t\tP: "UnitScaleFactor", "double", "Number", "",1', "\t}", "}",
             "Objects:  {"]
        rest_e = OaFbxWriter._euler_xyz_deg(R.QuatToMatrixT(torch.tensor([j.Rest.OrientedRotation() for j in sk.Joints], dtype=torch.float32)))
        for k, j in enumerate(sk.Joints):
            t, e = j.Rest.Translate, rest_e[k].tolist()
            L += [f'\tNodeAttribute: {uid(k, 200000)}, "NodeAttribute::{j.Name}", "LimbNode" {{', '\t\tTypeFlags: "Skeleton"', "\t}",
                  f'\tModel: {uid(k, 100000)}, "Model::{j.Name}", "LimbNode" {{', "\t\tVersion: 232", "\t\tProperties70:  {",
                  f'\t\t\tP: "Lcl Translation", "Lcl Translation", "", "A",{t[0]:.6f},{t[1]:.6f},{t[2]:.6f}',
                  f'\t\t\tP: "Lcl Rotation", "Lcl Rotation", "", "A",{e[0]:.6f},{e[1]:.6f},{e[2]:.6f}', "\t\t}", "\t}"]
        conns = []
        for k, j in enumerate(sk.Joints):
            conns.append(f'\tC: "OO",{uid(k, 200000)},{uid(k, 100000)}')
            conns.append(f'\tC: "OO",{uid(k, 100000)},{uid(j.ParentIndex, 100000) if j.ParentIndex >= 0 else 0}')
        if clip is not None:
            F = clip.FrameCount
            times = ",".join(str(int(round(f / clip.Fps * OaFbxWriter.TICKS_PER_SECOND))) for f in range(F))
            eul = OaFbxWriter._euler_xyz_deg(R.QuatToMatrixT(clip.Rotations[:, idx].float()))
            tr = clip.Translations[:, idx].float()
            L += [f'\tAnimationStack: 300000, "AnimStack::{take}", "" {{', "\t}", '\tAnimationLayer: 300001, "AnimLayer::BaseLayer", "" {', "\t}"]
            conns.append('\tC: "OO",300001,300000')
            cid = 400000
            for k in range(J):
                for prop, data in (("T", tr[:, k]), ("R", eul[:, k])):
                    node = cid
                    cid += 1
                    L += [f'\tAnimationCurveNode: {node}, "AnimCurveNode::{prop}", "" {{', "\t}"]
                    conns.append(f'\tC: "OO",{node},300001')
                    conns.append(f'\tC: "OP",{node},{uid(k, 100000)}, "Lcl {"Translation" if prop == "T" else "Rotation"}"')
                    for a, axis in enumerate("XYZ"):
                        vals = ",".join(f"{v:.6f}" for v in data[:, a].tolist())
                        L += [f'\tAnimationCurve: {cid}, "AnimCurve::", "" {{', f"\t\tKeyVer: 4008", f"\t\tKeyTime: *{F} {{", f"\t\t\ta: {times}", "\t\t}",
                              f"\t\tKeyValueFloat: *{F} {{", f"\t\t\ta: {vals}", "\t\t}", "\t}"]
                        conns.append(f'\tC: "OP",{cid},{node}, "d|{axis}"')
                        cid += 1
        L += ["}", "Connections:  {"] + conns + ["}"]
        if clip is not None:
            stop = int(round((clip.FrameCount - 1) / clip.Fps * OaFbxWriter.TICKS_PER_SECOND))
            L += ["Takes:  {", f'\tCurrent: "{take}"', f'\tTake: "{take}" {{', f"\t\tLocalTime: 0,{stop}", f"\t\tReferenceTime: 0,{stop}", "\t}", "}"]
        try:
            Path(path).write_text("\n".join(L) + "\n")
        except OSError as e:
            return OaStatus.Error(OaStatusCode.PermissionDenied, f"cannot write {path}: {e}")
        return OaStatus.Ok()
