"""The image and detection kernels against the tensor-expression path of the same functions on CPU (plain PyTorch fp32)."""
import pytest
import torch

from oa_b200.core.matrix import OaMatrix
from oa_b200.vision import fn_detection as D
from oa_b200.vision import fn_image as I
from oa_b200.vision import OaBorderMode as B
from oa_b200.vision import OaInterpolationMode as Interp

pytestmark = pytest.mark.gpu


def both(fn, *mats, atol=1e-5, exact=False):
    """Runs fn on CPU matrices and on their CUDA copies and compares the results."""
    cpu = fn(*mats)
    gpu = fn(*[OaMatrix(m.Tensor().cuda()) if isinstance(m, OaMatrix) else m for m in mats])
    a, b = cpu.Tensor(), gpu.Tensor().cpu()
    assert a.shape == b.shape and a.dtype == b.dtype
    if exact:
        assert torch.equal(a, b)
    else:
        assert torch.allclose(a, b, atol=atol, rtol=1e-5), float((a - b).abs().max())
    return gpu


def img(n=2, c=3, h=70, w=45, seed=0):
    g = torch.Generator().manual_seed(seed)
    return OaMatrix(torch.rand(n, c, h, w, generator=g))


def test_pointwise_channel_blend_noise_kernels():
    x, y = img(c=4), img(c=4, seed=1)
    for fn in (lambda m: I.ThresholdBinary(m, 0.5, 2.0), lambda m: I.ThresholdBinaryInv(m, 0.5), lambda m: I.ThresholdTruncate(m, 0.4),
               lambda m: I.ThresholdToZero(m, 0.4), lambda m: I.ThresholdToZeroInv(m, 0.4), lambda m: I.InRange(m, 0.2, 0.6, 3.0),
               lambda m: I.Clamp(m, 0.2, 0.6), lambda m: I.Invert(m), lambda m: I.BrightnessContrast(m, 0.1, 1.5),
               lambda m: I.GammaContrast(m, 2.2, 0.9), lambda m: I.Solarize(m), lambda m: I.Posterize(m, 5)):
        both(fn, x)
    both(lambda m: I.Invert(m), img(n=1, c=1, h=7, w=3))                           # scalar (not 16-byte multiple) path
    both(I.Grayscale, x)
    both(lambda m: I.ChannelReorder(m, 2, 1, 0, 3), x, exact=True)
    both(lambda m, t: I.ColorTwist(m, t), x, OaMatrix(torch.rand(3, 4)))
    both(lambda m: I.Normalize(m, I.OaNormalizationParams()), img())
    both(lambda a, b: I.AlphaBlend(a, b, 0.3), x, y)
    both(I.Composite, x, y, OaMatrix(torch.rand(2, 1, 70, 45) * 1.4 - 0.2))
    both(I.Composite, x, y, OaMatrix(torch.rand(2, 4, 70, 45)))
    both(lambda m: I.Erase(m, 5, 60, 100, 100, 0.5), x, exact=True)                 # rectangle clipped by the image
    both(lambda m, l, p: I.SegmentationOverlay(m, l, p, 0.25), x, OaMatrix(torch.randint(-1, 5, (2, 70, 45), dtype=torch.int32)),
         OaMatrix(torch.rand(4, 3)))
    both(lambda m: I.GaussianNoise(m, 0.1, 0.2, Seed=(5 << 32) | 7), x, atol=2e-5)  # same counter-based stream on both devices
    both(lambda m: I.SaltPepperNoise(m, 0.2, 1.0, 0.0, Seed=11), x, exact=True)


@pytest.mark.parametrize("border", list(B))
def test_tile_filters_every_border(border):
    x = img()
    both(lambda m, k: I.Convolve2d(m, k, border, 0.25), x, OaMatrix(torch.rand(7, 5)))
    both(lambda m, kx, ky: I.SeparableConvolve2d(m, kx, ky, border, 0.25), x, OaMatrix(torch.rand(9)), OaMatrix(torch.rand(3)))
    both(lambda m: I.AverageBlur(m, 5, 3, border), x)
    both(lambda m: I.Erode(m, 3, 7, border, 0.25), x, exact=True)
    both(lambda m: I.Dilate(m, 5, 3, border, 0.25), x, exact=True)
    both(lambda m: I.MedianBlur(m, 5, border), x, exact=True)
    both(lambda m: I.BilateralFilter(m, 5, 0.1, 1.5, border), x)
    both(lambda m: I.Pad(m, 3, 50, 80, 2, border, 0.25), x, exact=True)             # padding wider than the image: several reflections


def test_large_radius_and_derived_filters():
    x = img(n=1, c=2, h=33, w=100)
    both(lambda m: I.GaussianBlur(m, 5.0), x)                                       # radius 15: the widest halo
    both(lambda m, k: I.Convolve2d(m, k), x, OaMatrix(torch.rand(31, 31) / 961))
    both(lambda m: I.MedianBlur(m, 15), x, exact=True)
    both(lambda m: I.MedianBlur(m, 3), OaMatrix(torch.randn(1, 1, 40, 40) * 10), exact=True)   # negative values: order-preserving keys
    for fn in (I.Sobel, lambda m: I.Scharr(m, 0, 1), I.Laplacian, lambda m: I.Sharpen(m, 0.5), lambda m: I.UnsharpMask(m, 1.0, 0.7),
               I.MorphologyOpen, I.MorphologyClose, I.MorphologyGradient, I.MorphologyTopHat, I.MorphologyBlackHat):
        both(fn, x)
    # thresholds compare against a filtered value: allow a handful of pixels that sit within rounding of the threshold
    for fn in (lambda m: I.AdaptiveThresholdMean(m, 11, 0.01), lambda m: I.AdaptiveThresholdGaussian(m, 11)):
        cpu = fn(x).Tensor()
        gpu = fn(OaMatrix(x.Tensor().cuda())).Tensor().cpu()
        assert float((cpu != gpu).float().mean()) < 1e-3


def test_geometry_kernels():
    x = img()
    both(lambda m: I.Crop(m, 3, 10, 30, 50), x, exact=True)
    both(lambda m: I.CenterCrop(m, 21, 33), x, exact=True)
    both(lambda m: I.Flip(m, True, True), x, exact=True)
    for deg in (90, 180, 270):
        both(lambda m: I.Rotate(m, deg), x, exact=True)
    both(lambda m: I.Resize(m, 20, 31, Interp.Nearest), x, exact=True)
    both(lambda m: I.Resize(m, 97, 131, Interp.Nearest), x, exact=True)
    both(lambda m: I.Resize(m, 97, 131), x)
    both(lambda m: I.Resize(m, 20, 31), x)
    both(lambda m: I.ResizeNormalize(m, 64, 64, I.OaNormalizationParams()), x)
    A = OaMatrix(torch.tensor([[0.9, 0.2, -3.0], [-0.1, 1.1, 4.0]]))
    Hm = OaMatrix(torch.tensor([[0.9, 0.2, -3.0], [-0.1, 1.1, 4.0], [0.001, 0.002, 1.0]]))
    for border in B:
        both(lambda m, t: I.WarpAffine(m, t, 50, 60, Interp.Bilinear, border, 0.5), x, A, atol=2e-4)
        both(lambda m, t: I.WarpPerspective(m, t, 50, 60, Interp.Bilinear, border, 0.5), x, Hm, atol=2e-4)
        # nearest picks a pixel: a coordinate that lands within rounding of a half-integer may pick the neighbour
        for fn, t in ((I.WarpAffine, A), (I.WarpPerspective, Hm)):
            cpu = fn(x, t, 50, 60, Interp.Nearest, border, 0.5).Tensor()
            gpu = fn(OaMatrix(x.Tensor().cuda()), OaMatrix(t.Tensor().cuda()), 50, 60, Interp.Nearest, border, 0.5).Tensor().cpu()
            assert float((cpu != gpu).float().mean()) < 2e-3
    ys, xs = torch.meshgrid(torch.arange(40.0), torch.arange(30.0), indexing="ij")
    mp = torch.stack([xs * 1.5 - 2.25, ys * 1.75 + 0.5])[None]
    both(lambda m, p: I.Remap(m, p, Interp.Bilinear, B.Reflect), x, OaMatrix(mp), atol=1e-4)
    both(lambda m, p: I.Remap(m, p, Interp.Nearest, B.Wrap), x, OaMatrix(mp.repeat(2, 1, 1, 1) + 0.25), exact=True)


def test_detection_kernels():
    g = torch.Generator().manual_seed(3)
    n = 3000
    boxes = torch.cat([torch.rand(n, 2, generator=g) * 100, torch.rand(n, 2, generator=g) * 20 + 1], 1)
    scores = (torch.rand(n, generator=g) * 50).round() / 50                       # many ties
    scores[5] = float("nan")
    classes = torch.randint(0, 4, (n,), generator=g, dtype=torch.int32)
    both(D.BoxIou, OaMatrix(boxes[:300]), OaMatrix(boxes[300:700]), atol=1e-6)
    for cfg in (D.OaNmsConfig(), D.OaNmsConfig(0.3, 0.5, 40, True), D.OaNmsConfig(0.6, 0.0, 5000)):
        cpu = D.Nms(OaMatrix(boxes), OaMatrix(scores), OaMatrix(classes), cfg)
        gpu = D.Nms(OaMatrix(boxes.cuda()), OaMatrix(scores.cuda()), OaMatrix(classes.cuda()), cfg)
        assert torch.equal(cpu.Indices.Tensor(), gpu.Indices.Tensor().cpu()) and int(cpu.Count.Tensor()) == int(gpu.Count.Tensor())
    pred = torch.randint(-1, 7, (100000,), generator=g, dtype=torch.int32)
    targ = torch.randint(-1, 7, (100000,), generator=g, dtype=torch.int32)
    both(lambda p, t: D.ConfusionMatrix(p, t, 6), OaMatrix(pred), OaMatrix(targ), exact=True)
    sc, sg = D.EvaluateSegmentation(OaMatrix(pred), OaMatrix(targ), 6), D.EvaluateSegmentation(OaMatrix(pred.cuda()), OaMatrix(targ.cuda()), 6)
    for a, b in ((sc.PerClass, sg.PerClass), (sc.MeanIou, sg.MeanIou), (sc.PixelAccuracy, sg.PixelAccuracy)):
        assert torch.allclose(a.Tensor(), b.Tensor().cpu(), atol=1e-6)
    both(D.BinaryMaskCounts, OaMatrix((pred > 2).to(torch.uint8)), OaMatrix((targ > 3).to(torch.uint8)), exact=True)
    # dataset evaluation: 3 images, 3 classes, jittered copies of the targets plus clutter
    G, P = 60, 150
    tb = torch.cat([torch.rand(G, 2, generator=g) * 100, torch.rand(G, 2, generator=g) * 20 + 5], 1)
    tc = torch.randint(0, 3, (G,), generator=g, dtype=torch.int32)
    ti = torch.randint(0, 3, (G,), generator=g, dtype=torch.int32)
    src = torch.randint(0, G, (P,), generator=g)
    pb = tb[src] + torch.randn(P, 4, generator=g) * 2.0
    pc, pi = tc[src].clone(), ti[src].clone()
    pc[::7] = (pc[::7] + 1) % 3
    ps = (torch.rand(P, generator=g) * 20).round() / 20
    thr = torch.tensor([0.3, 0.5, 0.75, float("nan")])
    args = (pb, ps, pc, pi, tb, tc, ti, thr)
    rc = D.Evaluate(*[OaMatrix(a) for a in args], 4, 0.4)
    rg = D.Evaluate(*[OaMatrix(a.cuda()) for a in args], 4, 0.4)
    assert torch.equal(rc.Counts.Tensor(), rg.Counts.Tensor().cpu())
    assert torch.allclose(rc.PerClass.Tensor(), rg.PerClass.Tensor().cpu(), atol=1e-5)
    assert torch.allclose(rc.MeanAveragePrecisionByThreshold.Tensor(), rg.MeanAveragePrecisionByThreshold.Tensor().cpu(), atol=1e-5)
    assert torch.allclose(rc.MeanAveragePrecision.Tensor(), rg.MeanAveragePrecision.Tensor().cpu(), atol=1e-5)
    assert float(rc.MeanAveragePrecision.Tensor()) > 0.1


@pytest.mark.parametrize("mode", [0, 1])
def test_resize_backward_kernel(mode):
    """The gather kernel against the dense axis-matrix formulation on CPU, up- and down-scaling, odd sizes."""
    fn = I.ResizeBilinearBwd if mode else I.ResizeNearestBwd
    for (H, W), (Ho, Wo) in (((70, 45), (33, 101)), ((16, 16), (64, 64)), ((64, 48), (7, 5)), ((5, 9), (5, 9)), ((1, 3), (4, 1))):
        g = OaMatrix(torch.randn(2, 3, Ho, Wo, generator=torch.Generator().manual_seed(H + Wo)))
        both(lambda m: fn(m, H, W), g, atol=2e-4)
