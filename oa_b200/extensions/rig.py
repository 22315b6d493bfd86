"""3-D animation stack of the extensions: transforms and joints, skeletons, reference poses, forward kinematics.

Reference: Extensions/Public/Core/{Transform,Joint}.h, Extensions/Public/Rig/Skeleton.h, Extensions/Public/Retarget/HumanIk.h
(OaTransform / OaJoint with Maya-style joint orients, OaSkeleton with per-joint channel specs and the canonical pose
dimension, the HumanIK characterization as the retarget hub, the HumanML3D 22-joint body).

Conventions, as in the reference: quaternions are (x, y, z, w); `QuatMul(a, b)` applies b first, then a; a joint's
effective rotation is `JointOrient (x) Rotate`; world position = parent world + parent world rotation applied to the local
offset; units are centimetres, Z up.  Joint names and hierarchies are the public ones of the UE mannequin, of the HumanIK
characterization and of the HumanML3D kinematic chain.  The rest offsets in this file are this build's own proportions of
a 175 cm figure (segment fractions after Drillis & Contini), not the reference's asset tables; masses are Dempster-style
fractions of 80 kg.  Batched forward kinematics runs on tensors (any device), one step per hierarchy depth.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..core.types import OaError, OaStatus, OaStatusCode

Quat = Tuple[float, float, float, float]
Vec3 = Tuple[float, float, float]
IDENTITY: Quat = (0.0, 0.0, 0.0, 1.0)


# ------------------------------------------------------------------------------------------------- quaternion helpers
def QuatMul(a: Quat, b: Quat) -> Quat:
    """Hamilton product a (x) b: the rotation that applies b first, then a."""
    ax, ay, az, aw = a
    bx, by, bz, bw = b
    return (aw * bx + ax * bw + ay * bz - az * by,
            aw * by - ax * bz + ay * bw + az * bx,
            aw * bz + ax * by - ay * bx + az * bw,
            aw * bw - ax * bx - ay * by - az * bz)


def QuatNormalize(q: Quat) -> Quat:
    n = math.sqrt(sum(c * c for c in q))
    return IDENTITY if n < 1e-12 else tuple(c / n for c in q)


def QuatConjugate(q: Quat) -> Quat:
    return (-q[0], -q[1], -q[2], q[3])


def QuatRotate(q: Quat, v: Vec3) -> Vec3:
    x, y, z, w = q
    vx, vy, vz = v
    tx, ty, tz = 2 * (y * vz - z * vy), 2 * (z * vx - x * vz), 2 * (x * vy - y * vx)
    return (vx + w * tx + (y * tz - z * ty), vy + w * ty + (z * tx - x * tz), vz + w * tz + (x * ty - y * tx))


def EulerXyzDegToQuat(deg: Vec3) -> Quat:
    """Maya-style XYZ Euler angles in degrees: X is applied first, then Y, then Z."""
    hx, hy, hz = (math.radians(d) * 0.5 for d in deg)
    qx = (math.sin(hx), 0.0, 0.0, math.cos(hx))
    qy = (0.0, math.sin(hy), 0.0, math.cos(hy))
    qz = (0.0, 0.0, math.sin(hz), math.cos(hz))
    return QuatNormalize(QuatMul(qz, QuatMul(qy, qx)))


def QuatToMatrix(q: Quat) -> List[List[float]]:
    """Column-vector rotation matrix (p' = R p)."""
    x, y, z, w = QuatNormalize(q)
    return [[1 - 2 * (y * y + z * z), 2 * (x * y - z * w), 2 * (x * z + y * w)],
            [2 * (x * y + z * w), 1 - 2 * (x * x + z * z), 2 * (y * z - x * w)],
            [2 * (x * z - y * w), 2 * (y * z + x * w), 1 - 2 * (x * x + y * y)]]


def TrsMatrix(scale: Vec3, rot: Quat, trans: Vec3) -> List[List[float]]:
    """Row-vector S.R.T matrix (p' = p M, translation in row 3): the 3 x 3 block is the transpose of QuatToMatrix."""
    r = QuatToMatrix(rot)
    m = [[r[c][rw] * scale[rw] for c in range(3)] + [0.0] for rw in range(3)]
    m.append([trans[0], trans[1], trans[2], 1.0])
    return m


def TransformPoint(m: List[List[float]], p: Vec3) -> Vec3:
    return tuple(p[0] * m[0][c] + p[1] * m[1][c] + p[2] * m[2][c] + m[3][c] for c in range(3))


# --------------------------------------------------------------------------------------------------- transform, joint
@dataclass
class OaTransform:
    Translate: Vec3 = (0.0, 0.0, 0.0)
    Rotate: Quat = IDENTITY
    Scale: Vec3 = (1.0, 1.0, 1.0)

    def OrientedRotation(self) -> Quat:
        return self.Rotate

    def LocalMatrix(self) -> List[List[float]]:
        return TrsMatrix(self.Scale, self.OrientedRotation(), self.Translate)


@dataclass
class OaJoint(OaTransform):
    """A transform with a fixed rest orientation against which `Rotate` is a delta (Maya joint orient)."""
    JointOrient: Quat = IDENTITY

    def OrientedRotation(self) -> Quat:
        return QuatMul(self.JointOrient, self.Rotate)

    def OffsetParentMatrix(self) -> List[List[float]]:
        return TrsMatrix((1.0, 1.0, 1.0), self.JointOrient, (0.0, 0.0, 0.0))


@dataclass
class OaSkelJoint:
    Name: str = ""
    ParentIndex: int = -1
    HumanIkId: int = 0
    Mass: float = 0.0
    Rest: OaJoint = field(default_factory=OaJoint)
    HasTranslate: bool = False          # live translate channel (root and pelvis only)
    RotDof: int = 3                     # 3 = full rotation (6-D), 1 = hinge angle, 0 = locked

    def Length(self) -> float:
        return math.sqrt(sum(c * c for c in self.Rest.Translate))

    def ChannelCount(self) -> int:
        return (3 if self.HasTranslate else 0) + (6 if self.RotDof == 3 else (1 if self.RotDof == 1 else 0))


# ------------------------------------------------------------------------------------------------------------ skeleton
@dataclass
class OaSkeleton:
    FormatVersion = 2
    Name: str = "metahuman_body"
    SkeletonId: int = 0
    Joints: List[OaSkelJoint] = field(default_factory=list)
    ContactJoints: List[int] = field(default_factory=list)

    def JointCount(self) -> int:
        return len(self.Joints)

    def PoseDim(self) -> int:
        return sum(j.ChannelCount() for j in self.Joints) + len(self.ContactJoints)

    def ChannelOffset(self, joint: int) -> int:
        return sum(j.ChannelCount() for j in self.Joints[:max(0, min(joint, len(self.Joints)))])

    def ContactOffset(self) -> int:
        return self.ChannelOffset(self.JointCount())

    def IndexOf(self, name: str) -> int:
        for i, j in enumerate(self.Joints):
            if j.Name == name:
                return i
        return -1

    def IndexOfHumanIk(self, hik_id: int) -> int:
        for i, j in enumerate(self.Joints):
            if j.HumanIkId == hik_id and hik_id != 0:
                return i
        return -1

    def RestWorldRotation(self, joint: int) -> Quat:
        chain = []
        k = joint
        while k >= 0:
            chain.append(k)
            k = self.Joints[k].ParentIndex
        q = IDENTITY
        for k in reversed(chain):
            q = QuatMul(q, self.Joints[k].Rest.OrientedRotation())
        return QuatNormalize(q)

    def RestWorld(self, joint: int) -> Vec3:
        """Bind-pose world position by forward kinematics over the rest joints (orientation-aware)."""
        chain = []
        k = joint
        while k >= 0:
            chain.append(k)
            k = self.Joints[k].ParentIndex
        pos, rot = (0.0, 0.0, 0.0), IDENTITY
        for k in reversed(chain):
            j = self.Joints[k]
            off = QuatRotate(rot, j.Rest.Translate)
            pos = (pos[0] + off[0], pos[1] + off[1], pos[2] + off[2])
            rot = QuatMul(rot, j.Rest.OrientedRotation())
        return pos

    def IsValid(self) -> bool:
        if not self.Joints or self.Joints[0].ParentIndex != -1:
            return False
        names = set()
        for i, j in enumerate(self.Joints):
            if not j.Name or j.Name in names or j.RotDof not in (0, 1, 3):
                return False
            names.add(j.Name)
            if i > 0 and not (0 <= j.ParentIndex < i):
                return False
        return all(0 <= c < len(self.Joints) for c in self.ContactJoints)

    def Depths(self) -> List[int]:
        d = [0] * len(self.Joints)
        for i, j in enumerate(self.Joints):
            d[i] = 0 if j.ParentIndex < 0 else d[j.ParentIndex] + 1
        return d

    def TotalMass(self) -> float:
        return sum(j.Mass for j in self.Joints)

    # ---- `.skel` JSON
    def ToDict(self) -> dict:
        return {"format_version": self.FormatVersion, "name": self.Name, "skeleton_id": self.SkeletonId,
                "contact_joints": list(self.ContactJoints),
                "joints": [{"name": j.Name, "parent": j.ParentIndex, "humanik_id": j.HumanIkId, "mass": j.Mass,
                            "translate": list(j.Rest.Translate), "joint_orient": list(j.Rest.JointOrient),
                            "has_translate": j.HasTranslate, "rot_dof": j.RotDof} for j in self.Joints]}

    def WriteSkel(self, path) -> OaStatus:
        try:
            with open(path, "w") as f:
                json.dump(self.ToDict(), f, indent=1)
        except OSError as e:
            return OaStatus.Error(OaStatusCode.PermissionDenied, f"cannot write {path}: {e}")
        return OaStatus.Ok()

    @staticmethod
    def ReadSkel(path) -> "OaSkeleton":
        try:
            with open(path) as f:
                d = json.load(f)
        except (OSError, ValueError) as e:
            raise OaError(OaStatus.Error(OaStatusCode.NotFound, f"cannot read skeleton {path}: {e}"))
        if int(d.get("format_version", 0)) != OaSkeleton.FormatVersion:
            raise OaError(OaStatus.Error(OaStatusCode.InvalidArgument, f"{path}: skeleton format version {d.get('format_version')}, expected 2"))
        sk = OaSkeleton(d.get("name", ""), int(d.get("skeleton_id", 0)), [], [int(c) for c in d.get("contact_joints", [])])
        for j in d.get("joints", []):
            sk.Joints.append(OaSkelJoint(j["name"], int(j["parent"]), int(j.get("humanik_id", 0)), float(j.get("mass", 0.0)),
                                         OaJoint(Translate=tuple(j["translate"]), JointOrient=tuple(j.get("joint_orient", IDENTITY))),
                                         bool(j.get("has_translate", False)), int(j.get("rot_dof", 3))))
        if not sk.IsValid():
            raise OaError(OaStatus.Error(OaStatusCode.InvalidArgument, f"{path}: not a valid skeleton (hierarchy order, names or channel specs)"))
        return sk


# ------------------------------------------------------------------------------------------------- HumanIK hub, builders
@dataclass
class OaHumanIkSlot:
    Slot: str
    Id: int
    Node: str


# The 25 core body slots of the HumanIK characterization and the UE bones they bind to (ids are the HumanIK node ids).
_HIK = [("Reference", 0, "root"), ("Hips", 1, "pelvis"), ("LeftUpLeg", 2, "thigh_l"), ("LeftLeg", 3, "calf_l"), ("LeftFoot", 4, "foot_l"),
        ("RightUpLeg", 5, "thigh_r"), ("RightLeg", 6, "calf_r"), ("RightFoot", 7, "foot_r"), ("Spine", 8, "spine_01"),
        ("LeftArm", 9, "upperarm_l"), ("LeftForeArm", 10, "lowerarm_l"), ("LeftHand", 11, "hand_l"), ("RightArm", 12, "upperarm_r"),
        ("RightForeArm", 13, "lowerarm_r"), ("RightHand", 14, "hand_r"), ("Head", 15, "head"), ("LeftToeBase", 16, "ball_l"),
        ("RightToeBase", 17, "ball_r"), ("LeftShoulder", 18, "clavicle_l"), ("RightShoulder", 19, "clavicle_r"), ("Neck", 20, "neck_01"),
        ("Spine1", 23, "spine_02"), ("Spine2", 24, "spine_03"), ("Spine3", 25, "spine_04"), ("Spine4", 26, "spine_05")]


def OaHumanIkCharacterization() -> List[OaHumanIkSlot]:
    return [OaHumanIkSlot(*s) for s in _HIK]


_HIK_BY_NODE = {node: hid for _, hid, node in _HIK}
H = 175.0            # stature of the figure the offsets are derived from (cm)


def _j(name, parent, offset, mass=0.0, translate=False, dof=3, orient=IDENTITY) -> tuple:
    return (name, parent, offset, mass, translate, dof, orient)


def _build(name: str, sid: int, rows: Sequence[tuple], contacts: Sequence[str]) -> OaSkeleton:
    sk = OaSkeleton(name, sid, [], [])
    index: Dict[str, int] = {}
    for nm, parent, off, mass, tr, dof, orient in rows:
        p = -1 if parent is None else index[parent]
        index[nm] = len(sk.Joints)
        sk.Joints.append(OaSkelJoint(nm, p, _HIK_BY_NODE.get(nm, 0), mass, OaJoint(Translate=tuple(float(c) for c in off), JointOrient=orient), tr, dof))
    sk.ContactJoints = [index[c] for c in contacts]
    assert sk.IsValid(), name
    return sk


def _metahuman_rows() -> List[tuple]:
    rows = [_j("root", None, (0, 0, 0), 0.0, True), _j("pelvis", "root", (0, 0, 0.53 * H), 11.2, True),
            _j("spine_01", "pelvis", (0, 0, 0.03 * H), 4.0), _j("spine_02", "spine_01", (0, 0, 0.035 * H), 5.0),
            _j("spine_03", "spine_02", (0, 0, 0.05 * H), 6.0), _j("spine_04", "spine_03", (0, 0, 0.05 * H), 7.0),
            _j("spine_05", "spine_04", (0, 0, 0.06 * H), 6.4), _j("neck_01", "spine_05", (0, 0, 0.045 * H), 0.8),
            _j("neck_02", "neck_01", (0, 0, 0.025 * H), 0.6), _j("head", "neck_02", (0, 0, 0.03 * H), 5.1)]
    for s, sign in (("l", 1.0), ("r", -1.0)):
        rows += [_j(f"clavicle_{s}", "spine_05", (sign * 0.015 * H, 0, 0.02 * H), 1.0),
                 _j(f"upperarm_{s}", f"clavicle_{s}", (sign * 0.09 * H, 0, 0), 2.2),
                 _j(f"lowerarm_{s}", f"upperarm_{s}", (sign * 0.16 * H, 0, 0), 1.3, False, 1),        # elbow: hinge
                 _j(f"hand_{s}", f"lowerarm_{s}", (sign * 0.145 * H, 0, 0), 0.5)]
        rows.append(_j(f"thumb_01_{s}", f"hand_{s}", (sign * 0.015 * H, 0.012 * H, 0), 0.01))
        rows.append(_j(f"thumb_02_{s}", f"thumb_01_{s}", (sign * 0.02 * H, 0, 0), 0.01))
        rows.append(_j(f"thumb_03_{s}", f"thumb_02_{s}", (sign * 0.016 * H, 0, 0), 0.01, False, 1))
        for k, fgr in enumerate(("index", "middle", "ring", "pinky")):
            y = (0.009 - 0.006 * k) * H
            rows.append(_j(f"{fgr}_metacarpal_{s}", f"hand_{s}", (sign * 0.02 * H, y, 0), 0.01))
            rows.append(_j(f"{fgr}_01_{s}", f"{fgr}_metacarpal_{s}", (sign * 0.03 * H, 0, 0), 0.01))
            rows.append(_j(f"{fgr}_02_{s}", f"{fgr}_01_{s}", (sign * 0.022 * H, 0, 0), 0.01, False, 1))
            rows.append(_j(f"{fgr}_03_{s}", f"{fgr}_02_{s}", (sign * 0.014 * H, 0, 0), 0.01, False, 1))
    for s, sign in (("l", 1.0), ("r", -1.0)):
        rows += [_j(f"thigh_{s}", "pelvis", (sign * 0.055 * H, 0, -0.01 * H), 8.0),
                 _j(f"calf_{s}", f"thigh_{s}", (0, 0, -0.245 * H), 3.7, False, 1),                    # knee: hinge
                 _j(f"foot_{s}", f"calf_{s}", (0, 0, -0.246 * H), 1.1),
                 _j(f"ball_{s}", f"foot_{s}", (0, 0.08 * H, -0.03 * H), 0.1)]
    return rows


_cache: Dict[str, OaSkeleton] = {}


def OaSkMetaHuman() -> OaSkeleton:
    """The clean 64-joint UE body (SkeletonId 0): spine, neck, head, arms with all fingers, legs to the ball of the foot."""
    if "mh" not in _cache:
        _cache["mh"] = _build("metahuman_body", 0, _metahuman_rows(), ("foot_l", "foot_r"))
    return _cache["mh"]


OaMetaHumanBodySkeleton = OaSkMetaHuman


def OaSkHumanIk() -> OaSkeleton:
    """The HumanIK characterization rig (SkeletonId 1): the 25 core slots bound to their UE bones, the retarget hub."""
    if "hik" not in _cache:
        keep = {node for _, _, node in _HIK}
        rows = [r for r in _metahuman_rows() if r[0] in keep]
        # neck_02 is not a HumanIK slot: the head hangs on neck_01 with the summed offset
        fixed = []
        for r in rows:
            if r[0] == "head":
                r = _j("head", "neck_01", (0, 0, 0.055 * H), r[3])
            fixed.append(r)
        _cache["hik"] = _build("humanik", 1, fixed, ("foot_l", "foot_r"))
    return _cache["hik"]


# HumanML3D / SMPL 22-joint body in the order of the 263-dimensional feature vector (t2m kinematic chain), Y up in the data
# sets; offsets here are expressed Z up like the rest of the stack.
_HML_NAMES = ["pelvis", "left_hip", "right_hip", "spine1", "left_knee", "right_knee", "spine2", "left_ankle", "right_ankle", "spine3",
              "left_foot", "right_foot", "neck", "left_collar", "right_collar", "head", "left_shoulder", "right_shoulder", "left_elbow",
              "right_elbow", "left_wrist", "right_wrist"]
_HML_PARENTS = [-1, 0, 0, 0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 9, 9, 12, 13, 14, 16, 17, 18, 19]
_HML_HIK = {"pelvis": 1, "left_hip": 2, "right_hip": 5, "spine1": 8, "left_knee": 3, "right_knee": 6, "spine2": 23, "left_ankle": 4,
            "right_ankle": 7, "spine3": 24, "left_foot": 16, "right_foot": 17, "neck": 20, "left_collar": 18, "right_collar": 19, "head": 15,
            "left_shoulder": 9, "right_shoulder": 12, "left_elbow": 10, "right_elbow": 13, "left_wrist": 11, "right_wrist": 14}


def OaSkHumanMl3d() -> OaSkeleton:
    """The HumanML3D / SMPL 22-joint body (SkeletonId 2); joint order = the data sets' `new_joints` arrays."""
    if "hml" in _cache:
        return _cache["hml"]
    off = {"pelvis": (0, 0, 0.53 * H), "left_hip": (0.04 * H, 0, -0.05 * H), "right_hip": (-0.04 * H, 0, -0.05 * H), "spine1": (0, 0, 0.07 * H),
           "left_knee": (0, 0, -0.22 * H), "right_knee": (0, 0, -0.22 * H), "spine2": (0, 0, 0.08 * H), "left_ankle": (0, 0, -0.24 * H),
           "right_ankle": (0, 0, -0.24 * H), "spine3": (0, 0, 0.03 * H), "left_foot": (0, 0.07 * H, -0.03 * H), "right_foot": (0, 0.07 * H, -0.03 * H),
           "neck": (0, 0, 0.12 * H), "left_collar": (0.045 * H, 0, 0.07 * H), "right_collar": (-0.045 * H, 0, 0.07 * H), "head": (0, 0, 0.05 * H),
           "left_shoulder": (0.07 * H, 0, 0.01 * H), "right_shoulder": (-0.07 * H, 0, 0.01 * H), "left_elbow": (0.15 * H, 0, 0),
           "right_elbow": (-0.15 * H, 0, 0), "left_wrist": (0.145 * H, 0, 0), "right_wrist": (-0.145 * H, 0, 0)}
    sk = OaSkeleton("humanml3d", 2, [], [])
    for i, nm in enumerate(_HML_NAMES):
        sk.Joints.append(OaSkelJoint(nm, _HML_PARENTS[i], _HML_HIK.get(nm, 0), 80.0 / 22, OaJoint(Translate=tuple(float(c) for c in off[nm])),
                                     i == 0, 3))
    sk.ContactJoints = [sk.IndexOf("left_ankle"), sk.IndexOf("right_ankle"), sk.IndexOf("left_foot"), sk.IndexOf("right_foot")]
    assert sk.IsValid()
    _cache["hml"] = sk
    return sk


def OaSkeletonById(skeleton_id: int) -> OaSkeleton:
    for b in (OaSkMetaHuman, OaSkHumanIk, OaSkHumanMl3d):
        if b().SkeletonId == skeleton_id:
            return b()
    raise OaError(OaStatus.Error(OaStatusCode.NotFound, f"no built-in skeleton has id {skeleton_id}"))


# ------------------------------------------------------------------------------------------------------ reference poses
@dataclass
class OaRefJoint:
    Name: str
    LocalOrient: Quat = IDENTITY
    LocalTrans: Vec3 = (0.0, 0.0, 0.0)


@dataclass
class OaRefPose:
    Joints: List[OaRefJoint] = field(default_factory=list)

    def OrientOf(self, name: str) -> Quat:
        for j in self.Joints:
            if j.Name == name:
                return j.LocalOrient
        return IDENTITY


def OaRefPoseFor(skeleton: OaSkeleton, kind: str = "tpose") -> OaRefPose:
    """Reference pose of a skeleton: `tpose` is its rest; `apose` lowers the upper arms by 45 degrees about the forward axis
    (the usual A-pose of a mannequin), everything else at rest."""
    if kind not in ("tpose", "apose"):
        raise ValueError("pose kind must be 'tpose' or 'apose'")
    out = OaRefPose()
    for j in skeleton.Joints:
        q = j.Rest.OrientedRotation()
        if kind == "apose" and j.HumanIkId in (9, 12):
            sign = 1.0 if j.HumanIkId == 9 else -1.0
            q = QuatMul(q, EulerXyzDegToQuat((0.0, sign * 45.0, 0.0)))
        out.Joints.append(OaRefJoint(j.Name, QuatNormalize(q), j.Rest.Translate))
    return out


# --------------------------------------------------------------------------------------- tensors: rotations, kinematics
def QuatToMatrixT(q: torch.Tensor) -> torch.Tensor:
    """[..., 4] (x, y, z, w) -> [..., 3, 3] column-vector rotation matrices."""
    q = q / q.norm(dim=-1, keepdim=True).clamp_min(1e-12)
    x, y, z, w = q.unbind(-1)
    m = torch.stack([1 - 2 * (y * y + z * z), 2 * (x * y - z * w), 2 * (x * z + y * w),
                     2 * (x * y + z * w), 1 - 2 * (x * x + z * z), 2 * (y * z - x * w),
                     2 * (x * z - y * w), 2 * (y * z + x * w), 1 - 2 * (x * x + y * y)], -1)
    return m.reshape(*q.shape[:-1], 3, 3)


def MatrixToQuatT(m: torch.Tensor) -> torch.Tensor:
    """[..., 3, 3] -> [..., 4] (x, y, z, w), w >= 0; branch-free (largest of the four candidates per element)."""
    m00, m11, m22 = m[..., 0, 0], m[..., 1, 1], m[..., 2, 2]
    c = torch.stack([1 + m00 - m11 - m22, 1 - m00 + m11 - m22, 1 - m00 - m11 + m22, 1 + m00 + m11 + m22], -1).clamp_min(0)
    k = c.argmax(-1, keepdim=True)
    s = 2 * torch.sqrt(c.gather(-1, k).clamp_min(1e-12)).squeeze(-1)
    xy, xz, yz = m[..., 0, 1] + m[..., 1, 0], m[..., 0, 2] + m[..., 2, 0], m[..., 1, 2] + m[..., 2, 1]
    wx, wy, wz = m[..., 2, 1] - m[..., 1, 2], m[..., 0, 2] - m[..., 2, 0], m[..., 1, 0] - m[..., 0, 1]
    cand = torch.stack([torch.stack([s / 4, xy / s, xz / s, wx / s], -1), torch.stack([xy / s, s / 4, yz / s, wy / s], -1),
                        torch.stack([xz / s, yz / s, s / 4, wz / s], -1), torch.stack([wx / s, wy / s, wz / s, s / 4], -1)], -2)
    q = cand.gather(-2, k.unsqueeze(-1).expand(*k.shape[:-1], 1, 4)).squeeze(-2)
    q = torch.where(q[..., 3:4] < 0, -q, q)
    return q / q.norm(dim=-1, keepdim=True).clamp_min(1e-12)


def Rot6dFromMatrix(m: torch.Tensor) -> torch.Tensor:
    """First two columns of the rotation, flattened: [..., 6]."""
    return torch.cat([m[..., :, 0], m[..., :, 1]], -1)


def MatrixFromRot6d(r: torch.Tensor) -> torch.Tensor:
    """Gram-Schmidt on the two stored columns; the third is their cross product."""
    a, b = r[..., 0:3], r[..., 3:6]
    x = a / a.norm(dim=-1, keepdim=True).clamp_min(1e-12)
    b = b - (x * b).sum(-1, keepdim=True) * x
    y = b / b.norm(dim=-1, keepdim=True).clamp_min(1e-12)
    z = torch.cross(x, y, dim=-1)
    return torch.stack([x, y, z], -1)


def ForwardKinematics(skeleton: OaSkeleton, local_rot: torch.Tensor, root_trans: Optional[torch.Tensor] = None,
                      translations: Optional[Dict[int, torch.Tensor]] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Batched forward kinematics.  `local_rot` [..., J, 3, 3] are the ANIMATED local rotations (the delta against each
    joint's rest orient); `root_trans` [..., 3] replaces joint 0's rest offset; `translations` maps further joints with a
    live translate channel to their [..., 3] values.  Returns (world positions [..., J, 3], world rotations [..., J, 3, 3]).
    One step per hierarchy depth; runs wherever the tensors live."""
    J = skeleton.JointCount()
    assert local_rot.shape[-3] == J
    dev, dt = local_rot.device, local_rot.dtype
    orient = QuatToMatrixT(torch.tensor([j.Rest.JointOrient for j in skeleton.Joints], device=dev, dtype=dt))
    rest = torch.tensor([j.Rest.Translate for j in skeleton.Joints], device=dev, dtype=dt)
    eff = orient @ local_rot                                        # JointOrient (x) Rotate per joint
    lead = local_rot.shape[:-3]
    offs = rest.expand(*lead, J, 3).clone()
    if root_trans is not None:
        offs[..., 0, :] = root_trans
    for k, v in (translations or {}).items():
        offs[..., k, :] = v
    wpos = [None] * J
    wrot = [None] * J
    for i, j in enumerate(skeleton.Joints):                        # parents precede children
        if j.ParentIndex < 0:
            wpos[i], wrot[i] = offs[..., i, :], eff[..., i, :, :]
        else:
            p = j.ParentIndex
            wpos[i] = wpos[p] + (wrot[p] @ offs[..., i, :, None]).squeeze(-1)
            wrot[i] = wrot[p] @ eff[..., i, :, :]
    return torch.stack(wpos, -2), torch.stack(wrot, -3)
