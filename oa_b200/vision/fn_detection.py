"""OaFnDetection: detection post-processing and evaluation that stays on the device.

Reference: Source/Public/Oa/Vision/FnDetection.h:8-125 (BoxIou, Nms, ConfusionMatrix, BinaryMaskCounts, Evaluate,
EvaluateSegmentation) and the shaders under Source/Private/Oa/Vision/Shader/Compute/Postprocess.  Boxes are fp32
centre-x / centre-y / width / height.  The GPU path is `detection.cu`; the CPU path evaluates the same definitions with
plain loops and tensor expressions and is the oracle of the GPU tests.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import _native as N
from ..core.matrix import OaMatrix
from ..ops import kernels as K


@dataclass
class OaNmsConfig:
    IouThreshold: float = 0.45
    ScoreThreshold: float = 0.0
    MaxDetections: int = 100
    ClassAgnostic: bool = False


@dataclass
class OaNmsResult:
    Indices: Optional[OaMatrix] = None      # int32 [N]: selected rows first, -1 after
    Count: Optional[OaMatrix] = None        # uint32-valued [1] (stored as int32), device resident

    def IsValid(self) -> bool:
        return self.Indices is not None and self.Count is not None


@dataclass
class OaDetectionMetricsResult:
    Counts: Optional[OaMatrix] = None                            # [T,C,3] true positive, false positive, false negative
    PerClass: Optional[OaMatrix] = None                          # [T,C,4] precision, recall, F1, 101-point AP
    MeanAveragePrecisionByThreshold: Optional[OaMatrix] = None   # [T]
    MeanAveragePrecision: Optional[OaMatrix] = None              # [1]

    def IsValid(self) -> bool:
        return None not in (self.Counts, self.PerClass, self.MeanAveragePrecisionByThreshold, self.MeanAveragePrecision)


@dataclass
class OaSegmentationMetricsResult:
    Confusion: Optional[OaMatrix] = None     # [C,C], rows = target
    PerClass: Optional[OaMatrix] = None      # [C,4] precision, recall, F1 / Dice, IoU
    MeanIou: Optional[OaMatrix] = None
    PixelAccuracy: Optional[OaMatrix] = None

    def IsValid(self) -> bool:
        return None not in (self.Confusion, self.PerClass, self.MeanIou, self.PixelAccuracy)


def _t(m) -> torch.Tensor:
    return m.Tensor() if isinstance(m, OaMatrix) else m


def _boxes(m, rows: Optional[int] = None) -> Optional[torch.Tensor]:
    t = _t(m)
    if t.dim() != 2 or t.shape[1] != 4 or t.dtype != torch.float32 or (rows is not None and t.shape[0] != rows):
        return None
    return t.contiguous()


def _vec(m, dtype, rows: int) -> Optional[torch.Tensor]:
    t = _t(m)
    if t.dtype != dtype or t.numel() != rows:
        return None
    return t.reshape(-1).contiguous()


def _iou_cpu(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    aw, ah, bw, bh = a[:, 2].clamp_min(0), a[:, 3].clamp_min(0), b[:, 2].clamp_min(0), b[:, 3].clamp_min(0)
    ix = (torch.minimum((a[:, 0] + aw * 0.5)[:, None], (b[:, 0] + bw * 0.5)[None]) -
          torch.maximum((a[:, 0] - aw * 0.5)[:, None], (b[:, 0] - bw * 0.5)[None])).clamp_min(0)
    iy = (torch.minimum((a[:, 1] + ah * 0.5)[:, None], (b[:, 1] + bh * 0.5)[None]) -
          torch.maximum((a[:, 1] - ah * 0.5)[:, None], (b[:, 1] - bh * 0.5)[None])).clamp_min(0)
    inter = ix * iy
    union = (aw * ah)[:, None] + (bw * bh)[None] - inter
    return torch.where(union > 0, inter / union.clamp_min(1e-30), torch.zeros_like(inter))


def BoxIou(A: OaMatrix, B: OaMatrix) -> Optional[OaMatrix]:
    a, b = _boxes(A), _boxes(B)
    if a is None or b is None:
        return None
    if not a.is_cuda:
        return OaMatrix(_iou_cpu(a, b))
    out = torch.empty((a.shape[0], b.shape[0]), dtype=torch.float32, device=a.device)
    K._launch(N.require().oa_det_box_iou(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.shape[0], b.shape[0], N.stream()), "oa_det_box_iou")
    return OaMatrix(out)


def Nms(Boxes: OaMatrix, Scores: OaMatrix, Classes: OaMatrix, Config: Optional[OaNmsConfig] = None) -> OaNmsResult:
    """Greedy class-aware suppression: repeatedly keep the best remaining box (ties: lower row) and drop the boxes of its
    class (any class when ClassAgnostic) whose IoU with it reaches IouThreshold.  Fixed-shape result, no host round trip."""
    cfg = Config or OaNmsConfig()
    boxes = _boxes(Boxes)
    if boxes is None or cfg.MaxDetections <= 0:
        return OaNmsResult()
    n = boxes.shape[0]
    scores, classes = _vec(Scores, torch.float32, n), _vec(Classes, torch.int32, n)
    if scores is None or classes is None:
        return OaNmsResult()
    indices = torch.full((n,), -1, dtype=torch.int32, device=boxes.device)
    count = torch.zeros(1, dtype=torch.int32, device=boxes.device)
    if n == 0:
        return OaNmsResult(OaMatrix(indices), OaMatrix(count))
    if boxes.is_cuda:
        alive = K.scratch(boxes.device, n, "nms_alive")
        K._launch(N.require().oa_det_nms(boxes.data_ptr(), scores.data_ptr(), classes.data_ptr(), n, float(cfg.IouThreshold),
                                         float(cfg.ScoreThreshold), int(cfg.MaxDetections), int(cfg.ClassAgnostic), indices.data_ptr(),
                                         count.data_ptr(), alive.data_ptr(), N.stream()), "oa_det_nms")
        return OaNmsResult(OaMatrix(indices), OaMatrix(count))
    iou = _iou_cpu(boxes, boxes)
    alive = (~torch.isnan(scores)) & (scores >= cfg.ScoreThreshold)
    picked = []
    while len(picked) < min(cfg.MaxDetections, n) and bool(alive.any()):
        masked = torch.where(alive, scores, torch.full_like(scores, float("-inf")))
        best = int(torch.nonzero(alive & (masked == masked.max()))[0])
        picked.append(best)
        same = torch.ones(n, dtype=torch.bool) if cfg.ClassAgnostic else classes == classes[best]
        alive = alive & ~(same & (iou[best] >= cfg.IouThreshold))
        alive[best] = False
    indices[:len(picked)] = torch.tensor(picked, dtype=torch.int32)
    count[0] = len(picked)
    return OaNmsResult(OaMatrix(indices), OaMatrix(count))


def ConfusionMatrix(Predicted: OaMatrix, Target: OaMatrix, ClassCount: int) -> Optional[OaMatrix]:
    """[C,C] counts, rows = target class, columns = predicted class; labels outside [0, C) are skipped."""
    p, t = _t(Predicted), _t(Target)
    if ClassCount <= 0 or p.dtype != torch.int32 or t.dtype != torch.int32 or p.numel() != t.numel():
        return None
    p, t = p.reshape(-1).contiguous(), t.reshape(-1).contiguous()
    out = torch.zeros((ClassCount, ClassCount), dtype=torch.int32, device=p.device)
    if p.is_cuda:
        K._launch(N.require().oa_det_confusion(p.data_ptr(), t.data_ptr(), p.numel(), ClassCount, out.data_ptr(), N.stream()), "oa_det_confusion")
        return OaMatrix(out)
    ok = (p >= 0) & (p < ClassCount) & (t >= 0) & (t < ClassCount)
    lin = (t[ok].long() * ClassCount + p[ok].long())
    out.reshape(-1).copy_(torch.bincount(lin, minlength=ClassCount * ClassCount).to(torch.int32))
    return OaMatrix(out)


def BinaryMaskCounts(Predicted: OaMatrix, Target: OaMatrix) -> Optional[OaMatrix]:
    """[4] = true positive, false positive, false negative, true negative over equally shaped uint8 masks."""
    p, t = _t(Predicted), _t(Target)
    if p.dtype != torch.uint8 or t.dtype != torch.uint8 or p.shape != t.shape:
        return None
    p, t = p.reshape(-1).contiguous(), t.reshape(-1).contiguous()
    out = torch.zeros(4, dtype=torch.int32, device=p.device)
    if p.is_cuda:
        K._launch(N.require().oa_det_binary_counts(p.data_ptr(), t.data_ptr(), p.numel(), out.data_ptr(), N.stream()), "oa_det_binary_counts")
        return OaMatrix(out)
    pb, tb = p != 0, t != 0
    out.copy_(torch.tensor([int((pb & tb).sum()), int((pb & ~tb).sum()), int((~pb & tb).sum()), int((~pb & ~tb).sum())], dtype=torch.int32))
    return OaMatrix(out)


def EvaluateSegmentation(Predicted: OaMatrix, Target: OaMatrix, ClassCount: int) -> OaSegmentationMetricsResult:
    conf = ConfusionMatrix(Predicted, Target, ClassCount)
    if conf is None:
        return OaSegmentationMetricsResult()
    c = conf.Tensor()
    per = torch.zeros((ClassCount, 4), dtype=torch.float32, device=c.device)
    miou = torch.zeros(1, dtype=torch.float32, device=c.device)
    acc = torch.zeros(1, dtype=torch.float32, device=c.device)
    if c.is_cuda:
        K._launch(N.require().oa_det_segmentation_metrics(c.data_ptr(), ClassCount, per.data_ptr(), miou.data_ptr(), acc.data_ptr(),
                                                          N.stream()), "oa_det_segmentation_metrics")
        return OaSegmentationMetricsResult(conf, OaMatrix(per), OaMatrix(miou), OaMatrix(acc))
    cf = c.float()
    tp, tt, pt = cf.diag(), cf.sum(1), cf.sum(0)
    union = tt + pt - tp
    z = torch.zeros_like(tp)
    precision = torch.where(pt > 0, tp / pt.clamp_min(1), z)
    recall = torch.where(tt > 0, tp / tt.clamp_min(1), z)
    f1 = torch.where(precision + recall > 0, 2 * precision * recall / (precision + recall).clamp_min(1e-30), z)
    iou = torch.where(union > 0, tp / union.clamp_min(1), z)
    per.copy_(torch.stack([precision, recall, f1, iou], 1))
    valid = int((union > 0).sum())
    miou[0] = float(iou[union > 0].sum()) / valid if valid else 0.0
    acc[0] = float(tp.sum() / tt.sum()) if float(tt.sum()) > 0 else 0.0
    return OaSegmentationMetricsResult(conf, OaMatrix(per), OaMatrix(miou), OaMatrix(acc))


def Evaluate(PredictedBoxes: OaMatrix, PredictedScores: OaMatrix, PredictedClasses: OaMatrix, PredictedImageIds: OaMatrix,
             TargetBoxes: OaMatrix, TargetClasses: OaMatrix, TargetImageIds: OaMatrix, IouThresholds: OaMatrix, ClassCount: int,
             ScoreThreshold: float = 0.0) -> OaDetectionMetricsResult:
    """Dataset-level detection metrics.  Per (IoU threshold, class): predictions in descending score order are matched greedily
    to the unmatched target of the same class and image with the highest IoU; a match needs IoU >= threshold.  The precision /
    recall curve over ranks gives the 101-point interpolated AP; counts and precision / recall / F1 use the predictions whose
    score reaches ScoreThreshold.  mAP averages classes that have targets."""
    pb, tb = _boxes(PredictedBoxes), _boxes(TargetBoxes)
    thr = _t(IouThresholds)
    if pb is None or tb is None or ClassCount <= 0 or thr.dtype != torch.float32 or thr.numel() == 0:
        return OaDetectionMetricsResult()
    P, G, T = pb.shape[0], tb.shape[0], thr.numel()
    ps, pc, pi = _vec(PredictedScores, torch.float32, P), _vec(PredictedClasses, torch.int32, P), _vec(PredictedImageIds, torch.int32, P)
    tc, tim = _vec(TargetClasses, torch.int32, G), _vec(TargetImageIds, torch.int32, G)
    if None in (ps, pc, pi, tc, tim):
        return OaDetectionMetricsResult()
    thr = thr.reshape(-1).contiguous()
    dev = pb.device
    counts = torch.zeros((T, ClassCount, 3), dtype=torch.int32, device=dev)
    metrics = torch.zeros((T, ClassCount, 4), dtype=torch.float32, device=dev)
    map_t = torch.zeros(T, dtype=torch.float32, device=dev)
    mean = torch.zeros(1, dtype=torch.float32, device=dev)
    # descending score, ties by ascending row (a stable sort of the negated scores); NaN scores sort last and are skipped
    order = torch.sort(torch.where(torch.isnan(ps), torch.full_like(ps, float("inf")), -ps), stable=True).indices.to(torch.int32)
    if pb.is_cuda:
        matched = K.scratch(dev, max(1, T * ClassCount * G), "det_matched")
        curve = K.scratch(dev, max(1, T * ClassCount * P * 2) * 4, "det_curve")
        K._launch(N.require().oa_det_evaluate(pb.data_ptr(), ps.data_ptr(), pc.data_ptr(), pi.data_ptr(), order.data_ptr(), P, tb.data_ptr(),
                                              tc.data_ptr(), tim.data_ptr(), G, thr.data_ptr(), T, ClassCount, float(ScoreThreshold),
                                              matched.data_ptr(), curve.data_ptr(), counts.data_ptr(), metrics.data_ptr(), map_t.data_ptr(),
                                              mean.data_ptr(), N.stream()), "oa_det_evaluate", 2)
        return OaDetectionMetricsResult(OaMatrix(counts), OaMatrix(metrics), OaMatrix(map_t), OaMatrix(mean))
    iou = _iou_cpu(pb, tb) if P and G else torch.zeros((P, G))
    f32 = lambda v: float(torch.tensor(v, dtype=torch.float32))
    total, valid_t = 0.0, 0
    for ti in range(T):
        th = float(thr[ti])
        th_ok = th == th and 0.0 <= th <= 1.0
        cls_sum, cls_valid = 0.0, 0
        for c in range(ClassCount):
            targets = int((tc == c).sum())
            used = [False] * G
            tp = fp = etp = efp = 0
            curve = []
            for p in order.tolist():
                s = float(ps[p])
                if int(pc[p]) != c or s != s:
                    continue
                best, best_iou = -1, -1.0
                for g in range(G):
                    if used[g] or int(tc[g]) != c or int(tim[g]) != int(pi[p]):
                        continue
                    v = float(iou[p, g])
                    if v > best_iou:
                        best, best_iou = g, v
                hit = best >= 0 and th_ok and best_iou >= th
                if hit:
                    used[best] = True
                    tp += 1
                else:
                    fp += 1
                if s >= ScoreThreshold:
                    etp, efp = etp + int(hit), efp + int(not hit)
                curve.append((f32(tp / (tp + fp)), f32(tp / targets) if targets else 0.0))
            fn = max(targets - etp, 0)
            precision = f32(etp / (etp + efp)) if etp + efp else 0.0
            recall = f32(etp / targets) if targets else 0.0
            f1 = f32(2 * precision * recall / (precision + recall)) if precision + recall > 0 else 0.0
            ap = 0.0
            if targets:
                acc = torch.zeros((), dtype=torch.float32)
                for rp in range(101):
                    need = f32(rp * f32(0.01))
                    acc = acc + max([pr for pr, rc in curve if f32(rc + 1e-7) >= need], default=0.0)
                ap = float(acc / 101.0)
                cls_sum, cls_valid = cls_sum + ap, cls_valid + 1
            counts[ti, c] = torch.tensor([etp, efp, fn], dtype=torch.int32)
            metrics[ti, c] = torch.tensor([precision, recall, f1, ap])
        m = cls_sum / cls_valid if cls_valid else 0.0
        map_t[ti] = m
        if cls_valid:
            total, valid_t = total + m, valid_t + 1
    mean[0] = total / valid_t if valid_t else 0.0
    return OaDetectionMetricsResult(OaMatrix(counts), OaMatrix(metrics), OaMatrix(map_t), OaMatrix(mean))


EvaluateDetections = Evaluate
