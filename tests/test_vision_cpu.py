"""OaFnImage / OaFnDetection on CPU tensors: the tensor-expression path checked against scipy.ndimage, closed forms and
hand-worked cases (the model is the reference's Test/Vision/Image/Kernel/TestVision50Ops.cpp: every operation, small inputs)."""
import math

import numpy as np
import pytest
import scipy.ndimage as ndi
import torch

from oa_b200.core.matrix import OaMatrix
from oa_b200.vision import fn_detection as D
from oa_b200.vision import fn_image as I
from oa_b200.vision import OaBorderMode as B
from oa_b200.vision import OaInterpolationMode as Interp

SCIPY_MODE = {B.Constant: "constant", B.Replicate: "nearest", B.Reflect: "reflect", B.Reflect101: "mirror", B.Wrap: "wrap"}


def img(n=2, c=3, h=9, w=11, seed=0):
    g = torch.Generator().manual_seed(seed)
    return OaMatrix(torch.rand(n, c, h, w, generator=g))


def per_plane(t, fn):
    out = np.empty_like(t.numpy())
    for n in range(t.shape[0]):
        for c in range(t.shape[1]):
            out[n, c] = fn(t[n, c].numpy())
    return torch.from_numpy(out)


def test_pointwise_operations():
    x = img()
    t = x.Tensor()
    assert torch.equal(I.ThresholdBinary(x, 0.5, 2.0).Tensor(), torch.where(t > 0.5, 2.0, 0.0))
    assert torch.equal(I.ThresholdBinaryInv(x, 0.5).Tensor(), torch.where(t > 0.5, 0.0, 1.0))
    assert torch.equal(I.ThresholdTruncate(x, 0.4).Tensor(), t.clamp_max(0.4))
    assert torch.equal(I.ThresholdToZero(x, 0.4).Tensor(), torch.where(t > 0.4, t, torch.zeros_like(t)))
    assert torch.equal(I.ThresholdToZeroInv(x, 0.4).Tensor(), torch.where(t > 0.4, torch.zeros_like(t), t))
    assert torch.equal(I.InRange(x, 0.2, 0.6, 3.0).Tensor(), torch.where((t >= 0.2) & (t <= 0.6), 3.0, 0.0))
    assert torch.equal(I.Clamp(x, 0.2, 0.6).Tensor(), t.clamp(0.2, 0.6))
    assert torch.allclose(I.Invert(x).Tensor(), 1 - t)
    assert torch.allclose(I.BrightnessContrast(x, 0.1, 1.5).Tensor(), t * 1.5 + 0.1)
    assert torch.allclose(I.GammaContrast(x, 2.2, 0.9).Tensor(), t.pow(2.2) * 0.9)
    assert torch.allclose(I.Solarize(x, 0.5).Tensor(), torch.where(t >= 0.5, 1 - t, t))
    post = I.Posterize(OaMatrix(torch.tensor([0.0, 0.24, 0.25, 0.5, 0.76, 1.0]).reshape(1, 1, 1, 6)), 3).Tensor().reshape(-1)
    assert torch.equal(post, torch.tensor([0.0, 0.0, 0.5, 0.5, 1.0, 1.0]))          # ties round up
    assert I.Clamp(x, 1.0, 0.0) is x and I.GammaContrast(x, -1.0) is x and I.Posterize(x, 1) is x   # invalid -> input unchanged


def test_channel_and_blend_operations():
    x = img(c=4)
    t = x.Tensor()
    gray = I.Grayscale(x).Tensor()
    assert gray.shape == (2, 1, 9, 11) and torch.allclose(gray[:, 0], 0.2126 * t[:, 0] + 0.7152 * t[:, 1] + 0.0722 * t[:, 2], atol=1e-6)
    assert torch.equal(I.ChannelReorder(x, 2, 1, 0, 3).Tensor(), t[:, [2, 1, 0, 3]])
    T = torch.tensor([[0.5, 0.1, 0.0, 0.2], [0.0, 1.0, 0.0, 0.0], [0.3, 0.3, 0.3, -0.1]])
    tw = I.ColorTwist(x, OaMatrix(T)).Tensor()
    assert torch.allclose(tw[:, :3], torch.einsum("cj,njhw->nchw", T[:, :3], t[:, :3]) + T[:, 3].reshape(1, 3, 1, 1), atol=1e-6)
    assert torch.equal(tw[:, 3], t[:, 3])
    prm = I.OaNormalizationParams()
    nm = I.Normalize(img(), prm).Tensor()
    assert torch.allclose(nm, (img().Tensor() - torch.tensor(prm.Mean).reshape(1, 3, 1, 1)) / torch.tensor(prm.Std).reshape(1, 3, 1, 1), atol=1e-5)
    y = img(c=4, seed=1)
    assert torch.allclose(I.AlphaBlend(x, y, 0.3).Tensor(), t * 0.7 + y.Tensor() * 0.3)
    m = OaMatrix((torch.rand(2, 1, 9, 11) * 1.4 - 0.2))
    mc = m.Tensor().clamp(0, 1)
    assert torch.allclose(I.Composite(x, y, m).Tensor(), t * (1 - mc) + y.Tensor() * mc)
    er = I.Erase(x, 2, 1, 4, 3, 9.0).Tensor()
    assert bool((er[:, :, 1:4, 2:6] == 9).all()) and torch.equal(er[:, :, 4:], t[:, :, 4:]) and torch.equal(er[:, :, :, :2], t[:, :, :, :2])
    lab = OaMatrix(torch.randint(-1, 4, (2, 9, 11), dtype=torch.int32))
    pal = OaMatrix(torch.rand(3, 3))
    ov = I.SegmentationOverlay(x, lab, pal, 0.25).Tensor()
    for (n, yy, xx) in [(0, 0, 0), (1, 4, 7), (1, 8, 10)]:
        l = int(lab.Tensor()[n, yy, xx])
        want = t[n, :3, yy, xx] * 0.75 + pal.Tensor()[l] * 0.25 if 0 <= l < 3 else t[n, :3, yy, xx]
        assert torch.allclose(ov[n, :3, yy, xx], want, atol=1e-6)
    assert torch.equal(ov[:, 3], t[:, 3])


def test_noise_is_deterministic_and_has_the_requested_moments():
    x = OaMatrix(torch.full((1, 1, 256, 256), 0.5))
    a, b, c = (I.GaussianNoise(x, 0.1, 0.2, Seed=s).Tensor() for s in (7, 7, 8))
    assert torch.equal(a, b) and not torch.equal(a, c)
    d = a - 0.5
    assert abs(float(d.mean()) - 0.1) < 5e-3 and abs(float(d.std()) - 0.2) < 5e-3
    sp = I.SaltPepperNoise(x, 0.1, 1.0, 0.0, Seed=3).Tensor()
    assert abs(float((sp == 1).float().mean()) - 0.05) < 5e-3 and abs(float((sp == 0).float().mean()) - 0.05) < 5e-3
    assert float(((sp != 0) & (sp != 1) & (sp != 0.5)).sum()) == 0


@pytest.mark.parametrize("border", list(SCIPY_MODE))
def test_filters_match_scipy_for_every_border_rule(border):
    x = img(h=8, w=10)
    t = x.Tensor()
    mode = SCIPY_MODE[border]
    k = torch.rand(3, 5)
    got = I.Convolve2d(x, OaMatrix(k), border, 0.25).Tensor()
    assert torch.allclose(got, per_plane(t, lambda p: ndi.correlate(p, k.numpy(), mode=mode, cval=0.25)), atol=1e-5)
    kx, ky = torch.rand(5), torch.rand(3)
    got = I.SeparableConvolve2d(x, OaMatrix(kx), OaMatrix(ky), border, 0.25).Tensor()
    want = per_plane(t, lambda p: ndi.correlate(p, np.outer(ky.numpy(), kx.numpy()), mode=mode, cval=0.25))
    assert torch.allclose(got, want, atol=1e-5)
    assert torch.allclose(I.AverageBlur(x, 5, 3, border).Tensor(), per_plane(t, lambda p: ndi.uniform_filter(p, (3, 5), mode=mode)), atol=1e-5)
    assert torch.allclose(I.Erode(x, 3, 5, border, 0.25).Tensor(), per_plane(t, lambda p: ndi.minimum_filter(p, (5, 3), mode=mode, cval=0.25)))
    assert torch.allclose(I.Dilate(x, 3, 5, border, 0.25).Tensor(), per_plane(t, lambda p: ndi.maximum_filter(p, (5, 3), mode=mode, cval=0.25)))
    assert torch.allclose(I.MedianBlur(x, 3, border).Tensor(), per_plane(t, lambda p: ndi.median_filter(p, 3, mode=mode)))
    assert torch.allclose(I.Pad(x, 2, 3, 1, 4, border, 0.25).Tensor(),
                          torch.from_numpy(np.pad(t.numpy(), ((0, 0), (0, 0), (1, 4), (2, 3)),
                                                  mode={"constant": "constant", "nearest": "edge", "reflect": "symmetric", "mirror": "reflect",
                                                        "wrap": "wrap"}[mode], **({"constant_values": 0.25} if mode == "constant" else {}))))


def test_derived_filters():
    x = img(h=12, w=12)
    t = x.Tensor()
    sob = per_plane(t, lambda p: ndi.correlate(p, np.array([[-1, 0, 1], [-2, 0, 2], [-1, 0, 1]], np.float32), mode="mirror"))
    assert torch.allclose(I.Sobel(x, 1, 0).Tensor(), sob, atol=1e-5)
    sch = per_plane(t, lambda p: ndi.correlate(p, np.array([[-3, -10, -3], [0, 0, 0], [3, 10, 3]], np.float32), mode="mirror"))
    assert torch.allclose(I.Scharr(x, 0, 1).Tensor(), sch, atol=1e-5)
    lap = per_plane(t, lambda p: ndi.correlate(p, np.array([[0, 1, 0], [1, -4, 1], [0, 1, 0]], np.float32), mode="mirror"))
    assert torch.allclose(I.Laplacian(x).Tensor(), lap, atol=1e-5)
    assert torch.allclose(I.Sharpen(x, 0.5).Tensor(), t - 0.5 * lap, atol=1e-5)
    g = I.GaussianBlur(x, 1.0).Tensor()
    assert torch.allclose(g, per_plane(t, lambda p: ndi.gaussian_filter(p, 1.0, mode="nearest", truncate=3.0)), atol=1e-5)
    assert torch.allclose(I.UnsharpMask(x, 1.0, 0.7).Tensor(), t + 0.7 * (t - g), atol=1e-5)
    er, di = I.Erode(x).Tensor(), I.Dilate(x).Tensor()
    assert torch.equal(I.MorphologyGradient(x).Tensor(), di - er)
    op = I.MorphologyOpen(x).Tensor()
    assert torch.equal(op, I.Dilate(OaMatrix(er)).Tensor()) and torch.equal(I.MorphologyTopHat(x).Tensor(), t - op)
    cl = I.MorphologyClose(x).Tensor()
    assert torch.equal(cl, I.Erode(OaMatrix(di)).Tensor()) and torch.equal(I.MorphologyBlackHat(x).Tensor(), cl - t)
    # bilateral with a huge colour sigma degenerates to a Gaussian-weighted mean; adaptive thresholds against local means
    w = np.exp(-(np.arange(-2, 3)[:, None] ** 2 + np.arange(-2, 3)[None] ** 2) / 2.0).astype(np.float32)
    gm = per_plane(t, lambda p: ndi.correlate(p, w / w.sum(), mode="mirror"))
    assert torch.allclose(I.BilateralFilter(x, 5, 1e4, 1.0).Tensor(), gm, atol=1e-5)
    bl = I.BilateralFilter(x, 5, 0.05, 1.0).Tensor()
    assert float((bl - t).abs().mean()) < float((gm - t).abs().mean())          # edge preserving: closer to the input
    mean5 = per_plane(t, lambda p: ndi.uniform_filter(p, 5, mode="mirror"))
    assert torch.equal(I.AdaptiveThresholdMean(x, 5, 0.02, 2.0).Tensor(), torch.where(t > mean5 - 0.02, 2.0, 0.0))
    assert torch.equal(I.AdaptiveThresholdGaussian(x, 5, 0.0, 1.0, 1.0).Tensor(), torch.where(t > gm, 1.0, 0.0))


def test_geometry():
    x = img(h=6, w=8)
    t = x.Tensor()
    assert torch.equal(I.Crop(x, 2, 1, 4, 3).Tensor(), t[:, :, 1:4, 2:6])
    assert torch.equal(I.CenterCrop(x, 4, 2).Tensor(), t[:, :, 2:4, 2:6])
    assert torch.equal(I.Flip(x, True, False).Tensor(), t.flip(3)) and torch.equal(I.Flip(x, True, True).Tensor(), t.flip(2, 3))
    r90 = I.Rotate(x, 90).Tensor()
    assert r90.shape == (2, 3, 8, 6) and float(r90[0, 0, 0, 0]) == float(t[0, 0, 5, 0]) and float(r90[0, 0, 0, 5]) == float(t[0, 0, 0, 0])
    assert torch.equal(I.Rotate(OaMatrix(r90), 270).Tensor(), t) and torch.equal(I.Rotate(x, 180).Tensor(), t.flip(2, 3))
    assert I.Crop(x, 6, 0, 4, 3) is x and I.Rotate(x, 45) is x
    # resize: nearest by integer factors is an index pick, bilinear matches align_corners=False interpolation (edges clamped)
    assert torch.equal(I.Resize(x, 4, 3, Interp.Nearest).Tensor(), t[:, :, ::2, ::2])
    up = I.Resize(x, 16, 12).Tensor()
    assert torch.allclose(up, torch.nn.functional.interpolate(t, size=(12, 16), mode="bilinear", align_corners=False), atol=1e-6)
    prm = I.OaNormalizationParams((0.5, 0.4, 0.3), (0.2, 0.3, 0.4))
    rn = I.ResizeNormalize(x, 16, 12, prm).Tensor()
    assert torch.allclose(rn, (up - torch.tensor(prm.Mean).reshape(1, 3, 1, 1)) / torch.tensor(prm.Std).reshape(1, 3, 1, 1), atol=1e-5)
    assert [m.Tensor().shape[-1] for m in I.ResizeBatch([x, x], 5, 5)] == [5, 5]
    # warps: identity, integer translation with a constant border, remap equal to the affine map it was built from
    eye = OaMatrix(torch.tensor([[1.0, 0, 0], [0, 1.0, 0]]))
    assert torch.allclose(I.WarpAffine(x, eye, 8, 6).Tensor(), t)
    sh = I.WarpAffine(x, OaMatrix(torch.tensor([[1.0, 0, 2], [0, 1.0, -1]])), 8, 6, Interp.Nearest, B.Constant, -1.0).Tensor()
    assert torch.equal(sh[:, :, 1:, :6], t[:, :, :5, 2:]) and bool((sh[:, :, 0] == -1).all()) and bool((sh[:, :, :, 6:] == -1).all())
    A = torch.tensor([[0.9, 0.2, 0.3], [-0.1, 1.1, 0.4]])
    ys, xs = torch.meshgrid(torch.arange(6.0), torch.arange(8.0), indexing="ij")
    mp = torch.stack([A[0, 0] * xs + A[0, 1] * ys + A[0, 2], A[1, 0] * xs + A[1, 1] * ys + A[1, 2]])[None]
    wa = I.WarpAffine(x, OaMatrix(A), 8, 6, Interp.Bilinear, B.Reflect101).Tensor()
    assert torch.allclose(I.Remap(x, OaMatrix(mp), Interp.Bilinear, B.Reflect101).Tensor(), wa, atol=1e-6)
    Hm = torch.tensor([[0.9, 0.2, 0.3], [-0.1, 1.1, 0.4], [0.0, 0.0, 1.0]])
    assert torch.allclose(I.WarpPerspective(x, OaMatrix(Hm), 8, 6, Interp.Bilinear, B.Reflect101).Tensor(), wa, atol=1e-6)
    Hp = torch.tensor([[1.0, 0, 0], [0, 1.0, 0], [0.01, 0.0, 1.0]])
    wp = I.WarpPerspective(x, OaMatrix(Hp), 8, 6, Interp.Nearest, B.Replicate).Tensor()
    sx = torch.floor(xs / (0.01 * xs + 1) + 0.5).long()
    assert torch.equal(wp, t[:, :, ys.long(), sx])


def test_semantic_image_overloads():
    t = torch.rand(5, 7, 3)
    im = I.OaImage(OaMatrix(t), I.OaImageLayout.Hwc, I.OaImageFormat.Rgb)
    assert im.Validate() and (im.Width(), im.Height(), im.Channels(), im.BatchSize()) == (7, 5, 3, 1)
    bgr = I.ConvertColor(im, I.OaImageFormat.Bgr)
    assert bgr.Format() == I.OaImageFormat.Bgr and torch.equal(bgr.AsMatrix().Tensor(), t[..., [2, 1, 0]])
    gray = I.ConvertColor(bgr, I.OaImageFormat.Gray)
    assert gray.AsMatrix().Tensor().shape == (5, 7, 1)
    assert torch.allclose(gray.AsMatrix().Tensor()[..., 0], 0.2126 * t[..., 0] + 0.7152 * t[..., 1] + 0.0722 * t[..., 2], atol=1e-6)
    rgba = I.ConvertColor(gray, I.OaImageFormat.Rgba).AsMatrix().Tensor()
    assert rgba.shape == (5, 7, 4) and torch.equal(rgba[..., 0], rgba[..., 2]) and bool((rgba[..., 3] == 1).all())
    small = I.Resize(im, 4, 3)
    assert small.AsMatrix().Tensor().shape == (3, 4, 3) and small.Layout() == I.OaImageLayout.Hwc
    assert I.BrightnessContrast(im, 0.1, 2.0).AsMatrix().Tensor().allclose(t * 2 + 0.1)
    assert not I.OaImage(OaMatrix(t), I.OaImageLayout.Hwc, I.OaImageFormat.Rgba).Validate()


def test_detection_post_processing():
    boxes = torch.tensor([[10, 10, 10, 10], [11, 10, 10, 10], [30, 30, 8, 8], [10.5, 10, 10, 10], [30, 31, 8, 8]], dtype=torch.float32)
    iou = D.BoxIou(OaMatrix(boxes), OaMatrix(boxes)).Tensor()
    assert torch.allclose(iou.diag(), torch.ones(5)) and abs(float(iou[0, 1]) - 9 / 11) < 1e-6 and float(iou[0, 2]) == 0
    scores = torch.tensor([0.9, 0.8, 0.7, 0.95, 0.7])
    classes = torch.tensor([0, 0, 1, 1, 1], dtype=torch.int32)
    r = D.Nms(OaMatrix(boxes), OaMatrix(scores), OaMatrix(classes), D.OaNmsConfig(IouThreshold=0.5))
    assert r.IsValid() and r.Indices.Tensor().tolist() == [3, 0, 2, -1, -1] and int(r.Count.Tensor()) == 3    # tie 2 vs 4 -> lower row
    r = D.Nms(OaMatrix(boxes), OaMatrix(scores), OaMatrix(classes), D.OaNmsConfig(IouThreshold=0.5, ClassAgnostic=True, ScoreThreshold=0.75))
    assert r.Indices.Tensor().tolist() == [3, -1, -1, -1, -1]
    r = D.Nms(OaMatrix(boxes), OaMatrix(scores), OaMatrix(classes), D.OaNmsConfig(IouThreshold=0.5, MaxDetections=2))
    assert int(r.Count.Tensor()) == 2
    pred = torch.tensor([0, 1, 2, 2, 1, 5, 0], dtype=torch.int32)
    targ = torch.tensor([0, 1, 1, 2, 1, 0, -1], dtype=torch.int32)
    conf = D.ConfusionMatrix(OaMatrix(pred), OaMatrix(targ), 3).Tensor()
    assert conf.tolist() == [[1, 0, 0], [0, 2, 1], [0, 0, 1]]
    seg = D.EvaluateSegmentation(OaMatrix(pred), OaMatrix(targ), 3)
    per = seg.PerClass.Tensor()
    assert torch.allclose(per[1], torch.tensor([1.0, 2 / 3, 0.8, 2 / 3]), atol=1e-6) and torch.allclose(per[2], torch.tensor([0.5, 1.0, 2 / 3, 0.5]), atol=1e-6)
    assert abs(float(seg.MeanIou.Tensor()) - (1 + 2 / 3 + 0.5) / 3) < 1e-6 and abs(float(seg.PixelAccuracy.Tensor()) - 0.8) < 1e-6
    pm = torch.tensor([1, 1, 0, 0, 1, 0], dtype=torch.uint8)
    tm = torch.tensor([1, 0, 0, 1, 1, 0], dtype=torch.uint8)
    assert D.BinaryMaskCounts(OaMatrix(pm), OaMatrix(tm)).Tensor().tolist() == [2, 1, 1, 2]


def test_detection_evaluation_hand_worked():
    # one class, one image, two targets; predictions by score: hit, miss, hit -> precision 1, 1/2, 2/3; recall 1/2, 1/2, 1
    tb = torch.tensor([[10, 10, 10, 10], [40, 40, 10, 10]], dtype=torch.float32)
    pb = torch.tensor([[10, 10, 10, 10], [70, 70, 10, 10], [41, 40, 10, 10]], dtype=torch.float32)
    ps = torch.tensor([0.9, 0.8, 0.7])
    z = lambda n: OaMatrix(torch.zeros(n, dtype=torch.int32))
    res = D.Evaluate(OaMatrix(pb), OaMatrix(ps), z(3), z(3), OaMatrix(tb), z(2), z(2), OaMatrix(torch.tensor([0.5, 0.95])), 2, 0.75)
    assert res.IsValid()
    # threshold 0.5: AP = (51 * 1 + 50 * 2/3) / 101; counts at score >= 0.75: 1 hit, 1 miss, 1 target left
    ap = (51 * 1.0 + 50 * (2 / 3)) / 101
    assert abs(float(res.PerClass.Tensor()[0, 0, 3]) - ap) < 1e-5
    assert res.Counts.Tensor()[0, 0].tolist() == [1, 1, 1]
    assert torch.allclose(res.PerClass.Tensor()[0, 0, :3], torch.tensor([0.5, 0.5, 0.5]), atol=1e-6)
    # threshold 0.95: the third prediction (IoU 9/11) no longer matches: curve (1, .5), (.5, .5), (1/3, .5) -> AP = 51/101
    assert abs(float(res.PerClass.Tensor()[1, 0, 3]) - 51 / 101) < 1e-5
    # class 1 has no targets: AP 0 and excluded from the mean
    assert float(res.PerClass.Tensor()[0, 1, 3]) == 0
    assert torch.allclose(res.MeanAveragePrecisionByThreshold.Tensor(), torch.tensor([ap, 51 / 101]), atol=1e-5)
    assert abs(float(res.MeanAveragePrecision.Tensor()) - (ap + 51 / 101) / 2) < 1e-5


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("shape", [((5, 7), (11, 4)), ((8, 8), (3, 16)), ((6, 9), (6, 9)), ((1, 4), (5, 1))])
def test_resize_backward_is_the_adjoint_of_resize(mode, shape):
    """<Resize(x), g> == <x, ResizeBwd(g)> for random x, g, and the tape delivers the same gradient."""
    from oa_b200.ml import autograd as AG
    (H, W), (Ho, Wo) = shape
    gen = torch.Generator().manual_seed(H * 100 + Wo)
    x = torch.randn(2, 3, H, W, generator=gen)
    g = torch.randn(2, 3, Ho, Wo, generator=gen)
    from oa_b200.core import fn_matrix as F
    FI = I
    y = FI.Resize(OaMatrix(x), Wo, Ho, mode).Tensor()
    bwd = (FI.ResizeBilinearBwd if mode else FI.ResizeNearestBwd)(OaMatrix(g), H, W).Tensor()
    assert bwd.shape == x.shape and torch.allclose((y * g).sum(), (x * bwd).sum(), rtol=1e-4, atol=1e-4)
    xm = OaMatrix(x.clone())
    xm.SetRequiresGrad(True)
    with AG.OaGradientTape() as tape:
        out = FI.Resize(xm, Wo, Ho, mode)
        loss = F.Sum(F.Mul(out, OaMatrix(g)))
    tape.Backward(loss)
    assert torch.allclose(xm.GradMatrix().Tensor(), bwd, atol=1e-5)
