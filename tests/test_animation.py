"""Curves (scalar and batched), easing, time codes and the timeline."""
import math

import pytest
import torch

from oa_b200.animation import (OaCurveColor, OaCurveFloat, OaCurveQuat, OaCurveVec3, OaEasing, OaFrameRate, OaKeyInterpolation, OaKeyframeTrack,
                               OaTimeCode, OaTimeDirection, OaTimeTransform, OaTimeline, OaTimelineState)


def test_track_keeps_keys_sorted():
    tr = OaKeyframeTrack(1)
    for t in (2.0, 0.0, 1.0, 1.0):
        tr.AddKeyframe(t, t * 10)
    assert [tr.GetKeyframe(i).Time for i in range(tr.GetKeyframeCount())] == [0.0, 1.0, 2.0]
    assert tr.FindKeyframeAt(-1) == -1 and tr.FindKeyframeAt(1.5) == 1 and tr.FindKeyframeAt(9) == 2
    tr.RemoveKeyframe(0)
    assert tr.GetKeyframeCount() == 2
    with pytest.raises(ValueError):
        tr.AddKeyframe(0, (1, 2))


def test_float_and_vector_curves():
    c = OaCurveFloat()
    c.AddKeyframe(0, 0.0); c.AddKeyframe(1, 10.0, OaKeyInterpolation.Stepped); c.AddKeyframe(2, 20.0); c.AddKeyframe(4, 0.0)
    assert c.Evaluate(-5) == 0.0 and c.Evaluate(0.25) == 2.5 and c.Evaluate(1.5) == 10.0 and c.Evaluate(3) == 10.0 and c.Evaluate(99) == 0.0
    assert c.Derivative(0.5) == pytest.approx(10.0, rel=1e-3) and c.Derivative(3) == pytest.approx(-10.0, rel=1e-3)
    times = torch.linspace(-1, 5, 61)
    batch = c.EvaluateBatch(times)[:, 0]
    assert torch.allclose(batch, torch.tensor([c.Evaluate(float(t)) for t in times]))
    v = OaCurveVec3()
    v.AddKeyframe(0, (0, 0, 0)); v.AddKeyframe(2, (2, 4, -6))
    assert v.Evaluate(1) == (1.0, 2.0, -3.0) and v.Derivative(1) == pytest.approx((1.0, 2.0, -3.0), rel=1e-3)
    # Catmull-Rom passes through its keys and reproduces a straight line exactly
    k = OaCurveFloat()
    for t in range(5):
        k.AddKeyframe(t, 3.0 * t + 1, OaKeyInterpolation.Cubic)
    assert all(k.Evaluate(x) == pytest.approx(3 * x + 1, abs=1e-5) for x in (1.0, 1.3, 2.5, 2.99))
    col = OaCurveColor()
    col.AddKeyframe(0, (0, 0, 0, 1)); col.AddKeyframe(1, (2, 1, 0.5, 1))
    assert col.Evaluate(1) == (1.0, 1.0, 0.5, 1.0)
    assert OaCurveFloat().EvaluateBatch(torch.zeros(3)).shape == (3, 1)


def test_quaternion_curve_is_a_constant_speed_rotation():
    q = OaCurveQuat()
    half = math.sqrt(0.5)
    q.AddKeyframe(0, (0, 0, 0, 1)); q.AddKeyframe(1, (0, half, 0, half)); q.AddKeyframe(2, (0, -1, 0, 0))      # 0, 90, 180 (negated) degrees about y
    for t, deg in ((0.5, 45), (1.0, 90), (1.5, 135)):
        x, y, z, w = q.Evaluate(t)
        assert (x, z) == (0.0, 0.0) and math.degrees(2 * math.atan2(abs(y), abs(w))) == pytest.approx(deg, abs=1e-3)
        assert x * x + y * y + z * z + w * w == pytest.approx(1.0, abs=1e-6)


def test_easing_end_points_and_shapes():
    names = [n for n in dir(OaEasing) if n[0].isupper()]
    assert len(names) == 15
    for n in names:
        f = getattr(OaEasing, n)
        assert f(0.0) == pytest.approx(0.0, abs=1e-9) and f(1.0) == pytest.approx(1.0, abs=1e-9), n
    assert OaEasing.EaseInQuad(0.5) == 0.25 and OaEasing.EaseOutQuad(0.5) == 0.75 and OaEasing.EaseInOutCubic(0.5) == 0.5
    assert OaEasing.EaseOutBounce(0.5) == pytest.approx(0.765625) and OaEasing.EaseOutElastic(0.1) > 1.0


def test_time_code_and_transform():
    ntsc = OaFrameRate(30000, 1001)
    assert OaTimeCode.FromFrames(30, ntsc).Seconds == pytest.approx(1.001) and OaTimeCode(1.001).ToFrames(ntsc) == 30
    assert OaTimeCode(3725.5).ToSmpte(OaFrameRate(24)) == "01:02:05:12" and OaFrameRate(25).FrameDuration() == 0.04
    tf = OaTimeTransform(Offset=OaTimeCode(2.0), Scale=2.0, TrimStart=OaTimeCode(1.0), TrimEnd=OaTimeCode(5.0))
    local = tf.ToLocal(OaTimeCode(3.0))
    assert local.Seconds == 2.0 and tf.ToParent(local).Seconds == 3.0 and tf.IsInTrim(local) and not tf.IsInTrim(OaTimeCode(0.5))
    assert tf.ApplyTrim(OaTimeCode(9.0)).Seconds == 5.0 and tf.ApplyTrim(OaTimeCode(0.0)).Seconds == 1.0
    assert OaTimeTransform.WithScale(0.0).ToParent(OaTimeCode(4.0)).Seconds == 0.0


def test_timeline_playback():
    tl = OaTimeline(2.0, OaFrameRate(10))
    tl.Update(1.0)
    assert tl.GetTime().Seconds == 0.0                       # not playing
    tl.Play(); tl.Update(0.55)
    assert tl.GetFrame() == 5 and tl.GetState() == OaTimelineState.Playing
    tl.Pause(); tl.Update(1.0)
    assert tl.GetTime().Seconds == pytest.approx(0.55)
    tl.Play(); tl.Update(5.0)
    assert tl.GetTime().Seconds == 2.0 and tl.GetState() == OaTimelineState.Stopped
    tl.SetLooping(True); tl.Seek(OaTimeCode(1.5)); tl.Play(); tl.Update(1.0)
    assert tl.GetTime().Seconds == pytest.approx(0.5)
    tl.SetDirection(OaTimeDirection.Reverse); tl.Update(0.75)
    assert tl.GetTime().Seconds == pytest.approx(1.75)
    tl.SetDirection(OaTimeDirection.PingPong); tl.SeekFrame(15); tl.SetSpeed(2.0); tl.Update(0.5)
    assert tl.GetTime().Seconds == pytest.approx(1.5)        # 1.5 -> 2.0 -> back to 1.5
    tl.Stop()
    assert tl.GetTime().Seconds == 0.0 and tl.GetState() == OaTimelineState.Stopped
