"""Skeletons, kinematics, pose packing, `.3danim` / `.usda` / FBX files, retarget and the data-set tool
(Extensions/Public/{Core,Rig,Anim,Retarget} of the reference; Apps/Ml/Gen3dAnim/dsgen3danimctl.cpp)."""
import json
import math

import pytest
import torch

from oa_b200.apps import dsgen3danimctl as CTL
from oa_b200.core.types import OaError
from oa_b200.extensions import anim as A
from oa_b200.extensions import rig as R


def test_quaternion_conventions():
    qx = R.EulerXyzDegToQuat((90, 0, 0))
    assert R.QuatRotate(qx, (0, 1, 0)) == pytest.approx((0, 0, 1), abs=1e-6)
    # X first, then Z: (0,1,0) -X90-> (0,0,1) -Z90-> (0,0,1); (1,0,0) -X90-> (1,0,0) -Z90-> (0,1,0)
    q = R.EulerXyzDegToQuat((90, 0, 90))
    assert R.QuatRotate(q, (1, 0, 0)) == pytest.approx((0, 1, 0), abs=1e-6)
    a, b = R.EulerXyzDegToQuat((10, 20, 30)), R.EulerXyzDegToQuat((-40, 5, 60))
    v = (0.3, -1.2, 2.0)
    assert R.QuatRotate(R.QuatMul(a, b), v) == pytest.approx(R.QuatRotate(a, R.QuatRotate(b, v)), abs=1e-5)       # b first, then a
    assert R.QuatMul(a, R.QuatConjugate(a)) == pytest.approx(R.IDENTITY, abs=1e-6)
    m = R.TrsMatrix((1, 1, 1), a, (1, 2, 3))                                                                         # row-vector S.R.T
    p = R.QuatRotate(a, v)
    assert R.TransformPoint(m, v) == pytest.approx((p[0] + 1, p[1] + 2, p[2] + 3), abs=1e-5)
    j = R.OaJoint(Rotate=b, JointOrient=a)
    assert j.OrientedRotation() == pytest.approx(R.QuatMul(a, b))


def test_builtin_skeletons():
    mh, hik, hml = R.OaSkMetaHuman(), R.OaSkHumanIk(), R.OaSkHumanMl3d()
    assert (mh.JointCount(), hik.JointCount(), hml.JointCount()) == (64, 25, 22)
    assert mh.IsValid() and hik.IsValid() and hml.IsValid()
    # channel budget: root and pelvis 9 each, hinges 1, the rest 6, two contacts
    hinges = sum(j.RotDof == 1 for j in mh.Joints)
    assert mh.PoseDim() == 2 * 9 + hinges * 1 + (64 - 2 - hinges) * 6 + 2
    assert mh.ChannelOffset(0) == 0 and mh.ChannelOffset(2) == 18 and mh.ContactOffset() == mh.PoseDim() - 2
    assert mh.Joints[mh.IndexOf("calf_l")].RotDof == 1 and mh.Joints[mh.IndexOf("pelvis")].HasTranslate
    assert mh.IndexOf("nope") == -1 and mh.IndexOfHumanIk(15) == mh.IndexOf("head")
    assert {s.Node for s in R.OaHumanIkCharacterization()} == {j.Name for j in hik.Joints}
    assert 75 < mh.TotalMass() < 90
    head, foot = mh.RestWorld(mh.IndexOf("head")), mh.RestWorld(mh.IndexOf("foot_l"))
    assert 140 < head[2] < 160 and 0 < foot[2] < 12 and foot[0] > 0
    assert mh.RestWorld(mh.IndexOf("hand_r"))[0] == pytest.approx(-mh.RestWorld(mh.IndexOf("hand_l"))[0])
    assert [j.ParentIndex for j in hml.Joints][:6] == [-1, 0, 0, 0, 1, 2]
    assert R.OaSkeletonById(2) is hml
    with pytest.raises(OaError):
        R.OaSkeletonById(9)


def test_skel_file_round_trip(tmp_path):
    sk = R.OaSkHumanIk()
    assert sk.WriteSkel(tmp_path / "h.skel").IsOk()
    back = R.OaSkeleton.ReadSkel(tmp_path / "h.skel")
    assert back.ToDict() == sk.ToDict()
    d = sk.ToDict()
    d["joints"][3]["parent"] = 7                                   # a parent that comes after its child
    (tmp_path / "bad.skel").write_text(json.dumps(d))
    with pytest.raises(OaError, match="not a valid skeleton"):
        R.OaSkeleton.ReadSkel(tmp_path / "bad.skel")


def test_tensor_kinematics_match_the_scalar_walk():
    sk = R.OaSkMetaHuman()
    J = sk.JointCount()
    rot = torch.eye(3).expand(3, J, 3, 3)
    pos, wrot = R.ForwardKinematics(sk, rot)
    for name in ("head", "hand_l", "ball_r", "pinky_03_l"):
        i = sk.IndexOf(name)
        assert pos[1, i].tolist() == pytest.approx(list(sk.RestWorld(i)), abs=1e-4)
    # bend the left elbow by 90 degrees about Z: the hand swings from +X to +Y around the elbow
    q = torch.tensor([0, 0, math.sin(math.pi / 4), math.cos(math.pi / 4)])
    rot = torch.eye(3).repeat(J, 1, 1)
    e, h = sk.IndexOf("lowerarm_l"), sk.IndexOf("hand_l")
    rot[e] = R.QuatToMatrixT(q)
    pos, _ = R.ForwardKinematics(sk, rot, root_trans=torch.tensor([10.0, 0, 0]))
    elbow, hand = pos[e], pos[h]
    assert (hand - elbow).tolist() == pytest.approx([0, sk.Joints[h].Length(), 0], abs=1e-4)
    assert pos[0].tolist() == [10.0, 0, 0]
    m = R.QuatToMatrixT(torch.randn(50, 4))
    assert torch.allclose(R.QuatToMatrixT(R.MatrixToQuatT(m)), m, atol=1e-5)
    assert torch.allclose(R.MatrixFromRot6d(R.Rot6dFromMatrix(m)), m, atol=1e-5)


def _walk_clip(sk, frames=40, fps=30.0):
    clip = A.RestClip(sk, frames, fps)
    t = torch.arange(frames) / fps
    pel = sk.IndexOf("pelvis")
    clip.Translations[:, pel, 1] = 50 * t
    for name, fn in (("thigh_l", lambda s: (30 * math.sin(4 * s), 0, 0)), ("calf_l", lambda s: (0, 0, 20 + 20 * math.sin(4 * s))),
                     ("upperarm_r", lambda s: (0, 25 * math.sin(3 * s), 10))):
        i = sk.IndexOf(name)
        for f in range(frames):
            clip.Rotations[f, i] = torch.tensor(R.QuatMul(sk.Joints[i].Rest.JointOrient, R.EulerXyzDegToQuat(fn(float(t[f])))))
    return clip


def test_pack_unpack_and_contacts():
    sk = R.OaSkMetaHuman()
    clip = _walk_clip(sk)
    pose = A.OaPosePack.Pack(clip, sk)
    assert pose.IsValid() and pose.PoseDim == sk.PoseDim() and pose.SkeletonId == 0
    back = A.OaPosePack.Unpack(pose, sk)
    assert torch.allclose(R.QuatToMatrixT(back.Rotations), R.QuatToMatrixT(clip.Rotations), atol=1e-5)
    assert torch.allclose(back.Translations, clip.Translations, atol=1e-5)
    c = sk.ChannelOffset(sk.IndexOf("calf_l"))
    assert pose.Samples[:, c].tolist() == pytest.approx([math.radians(20 + 20 * math.sin(4 * f / 30.0)) for f in range(40)], abs=1e-5)
    # a figure standing still has both feet planted: contacts 1; the walking clip's feet move at 50 cm/s: contacts 0
    still = A.OaPosePack.Pack(A.RestClip(sk, 5), sk)
    assert still.Samples[:, sk.ContactOffset():].min() == 1.0
    assert pose.Samples[:, sk.ContactOffset():].max() == 0.0
    with pytest.raises(OaError):
        A.OaPosePack.Unpack(A.OaPoseClip.Create(2, 7, 30, 0, torch.zeros(14)), sk)
    short = A.RestClip(R.OaSkHumanIk(), 3)
    with pytest.raises(OaError, match="no joint named"):
        A.OaPosePack.Pack(short, sk)


def test_3danim_file(tmp_path):
    sk = R.OaSkHumanIk()
    pose = A.OaPosePack.Pack(A.RestClip(sk, 6, 24.0), sk)
    assert pose.Write3dAnim(tmp_path / "a.3danim").IsOk()
    back = A.OaPoseClip.Read3dAnim(tmp_path / "a.3danim")
    assert torch.equal(back.Samples, pose.Samples) and (back.Fps, back.SkeletonId, back.FrameCount) == (24.0, 1, 6)
    blob = (tmp_path / "a.3danim").read_bytes()
    (tmp_path / "cut.3danim").write_bytes(blob[:-8])
    with pytest.raises(OaError, match="payload"):
        A.OaPoseClip.Read3dAnim(tmp_path / "cut.3danim")
    (tmp_path / "magic.3danim").write_bytes(b"XXXX" + blob[4:])
    with pytest.raises(OaError, match="not a .3danim"):
        A.OaPoseClip.Read3dAnim(tmp_path / "magic.3danim")
    assert pose.WriteTxt(tmp_path / "a.txt").IsOk() and len((tmp_path / "a.txt").read_text().splitlines()) == 7
    with pytest.raises(OaError):
        A.OaPoseClip.Create(2, 3, 30, 0, torch.zeros(5))


def test_usda_and_fbx_files(tmp_path):
    sk = R.OaSkMetaHuman()
    clip = _walk_clip(sk, 12)
    assert A.OaUsd.WriteUsdaMulti(tmp_path / "s.usda", [A.OaUsdNamedClip("walk_fwd", "train", clip), A.OaUsdNamedClip("idle", "val", A.RestClip(sk, 4))]).IsOk()
    clips = A.OaUsd.ReadUsdaMulti(tmp_path / "s.usda")
    assert [(c.Name, c.Split, c.Clip.FrameCount) for c in clips] == [("walk_fwd", "train", 12), ("idle", "val", 4)]
    got = clips[0].Clip
    assert got.JointPaths == clip.JointPaths and got.JointPaths[2] == "root/pelvis/spine_01" and got.Fps == 30.0 and got.UpAxis == 2
    assert torch.allclose(got.Rotations, clip.Rotations, atol=1e-6) and torch.allclose(got.Translations, clip.Translations, atol=1e-4)
    assert torch.allclose(got.BindTransforms, clip.BindTransforms, atol=1e-4) and torch.allclose(got.RestTransforms, clip.RestTransforms, atol=1e-4)
    head = sk.IndexOf("head")
    assert got.BindTransforms[head][3, :3].tolist() == pytest.approx(list(sk.RestWorld(head)), abs=1e-3)       # world bind = FK of the rest
    (tmp_path / "n.usda").write_text("not usd")
    with pytest.raises(OaError):
        A.OaUsd.ReadUsda(tmp_path / "n.usda")
    assert A.OaFbxWriter.Write(tmp_path / "s.fbx", sk, clip).IsOk()
    fbx = (tmp_path / "s.fbx").read_text()
    assert fbx.count('"LimbNode"') == 2 * 64 and "FBXVersion: 7400" in fbx and fbx.count("AnimationCurve:") == 64 * 6 and 'Take: "Take 001"' in fbx


def test_retarget_is_rest_relative():
    sk = R.OaSkMetaHuman()
    pose = A.OaPosePack.Pack(_walk_clip(sk, 10), sk)
    t, a = R.OaRefPoseFor(sk, "tpose"), R.OaRefPoseFor(sk, "apose")
    same = A.OaRetarget.RetargetClip(sk, sk, pose, t, t)
    assert torch.allclose(same.Samples, pose.Samples, atol=1e-5)
    moved = A.OaRetarget.RetargetClip(sk, sk, pose, t, a)
    ua = sk.ChannelOffset(sk.IndexOf("upperarm_l"))
    changed = (moved.Samples - pose.Samples).abs().amax(0)
    assert changed[ua:ua + 6].max() > 0.1                                      # the arms carry the pose difference ...
    th = sk.ChannelOffset(sk.IndexOf("thigh_l"))
    assert changed[th:th + 6].max() < 1e-5 and changed[0:3].max() == 0        # ... legs and root translation do not
    back = A.OaRetarget.RetargetClip(sk, sk, moved, a, t)
    assert torch.allclose(back.Samples, pose.Samples, atol=1e-4)
    with pytest.raises(OaError):
        A.OaRetarget.RetargetClip(sk, R.OaSkHumanIk(), pose, t, t)


def test_dataset_tool_pipeline(tmp_path, capsys):
    sk = R.OaSkMetaHuman()
    src = tmp_path / "src"
    src.mkdir()
    # source clips carry junk joints (IK, twist) and one of them is Y-up
    for name, frames, yup in (("Walk_Fwd", 14, False), ("Walk_Left", 10, True), ("Idle", 6, False)):
        clip = _walk_clip(sk, frames)
        extra = ["root/ik_foot_root", "root/pelvis/thigh_l/thigh_twist_01_l"]
        J = clip.JointCount()
        clip.JointPaths = clip.JointPaths + extra
        clip.Translations = torch.cat([clip.Translations, torch.zeros(frames, 2, 3)], 1)
        clip.Rotations = torch.cat([clip.Rotations, torch.tensor(R.IDENTITY).expand(frames, 2, 4)], 1)
        clip.BindTransforms = clip.RestTransforms = None
        if yup:                                             # express the same motion in a Y-up stage
            inv = R.QuatToMatrixT(torch.tensor(R.EulerXyzDegToQuat((-90.0, 0, 0))))
            clip.Translations[:, 0] = clip.Translations[:, 0] @ inv.t()
            clip.Rotations[:, 0] = R.MatrixToQuatT(inv @ R.QuatToMatrixT(clip.Rotations[:, 0]))
            clip.UpAxis = 1
        assert A.OaUsd.WriteUsda(src / f"{name}.usda", clip).IsOk()
    assert CTL.main(["clean", "--in", str(src / "Walk_Left.usda"), "--save", str(tmp_path / "w.3danim"), "--fbx", str(tmp_path / "w.fbx")]) == 0
    cleaned = A.OaPoseClip.Read3dAnim(tmp_path / "w.3danim")
    want = A.OaPosePack.Pack(_walk_clip(sk, 10), sk)
    assert torch.allclose(cleaned.Samples, want.Samples, atol=1e-4)           # junk dropped, Y-up undone
    assert CTL.main(["strip", "--in", str(src / "Idle.usda")]) == 0
    assert A.OaUsd.ReadUsda(src / "Idle.usda").JointCount() == 64
    assert CTL.main(["pack", "--in", str(src), "--out", str(tmp_path / "set.usda"), "--val", "Walk_Left", "--test", "Idle"]) == 0
    clips = A.OaUsd.ReadUsdaMulti(tmp_path / "set.usda")
    assert {c.Name: c.Split for c in clips} == {"Idle": "test", "Walk_Fwd": "train", "Walk_Left": "val"}
    capsys.readouterr()
    assert CTL.main(["info", "--dataset", str(tmp_path / "set.usda"), "--context", "8"]) == 0
    rep = json.loads(capsys.readouterr().out)
    assert rep["total_frames"] == 30 and rep["windows"] == {"train": 7, "val": 3, "test": 0} and rep["pose_dim"] == sk.PoseDim()
    assert CTL.main(["bake", "--dataset", str(tmp_path / "set.usda"), "--out", str(tmp_path / "set.3dset"), "--root-delta"]) == 0
    head, mean, std, baked = CTL.read_bake(tmp_path / "set.3dset")
    assert head == {"root_delta": True, "clips": 3, "pose_dim": sk.PoseDim(), "fps": 30.0, "skeleton_id": 0}
    assert [(n, s, x.shape[0]) for n, s, x in baked] == [("Idle", "test", 6), ("Walk_Fwd", "train", 14), ("Walk_Left", "val", 10)]
    assert baked[1][2][0, 0:3].abs().max() == 0 and mean.shape[0] == sk.PoseDim() and std.min() > 0
    assert CTL.main(["clean", "--in", str(tmp_path / "missing.usda")]) == 1
