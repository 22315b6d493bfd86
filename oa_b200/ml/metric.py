"""Metrics (Source/Public/Oa/Ml/Metric.h:30-177): OaMetric, OaMetricLoss, OaMetricAccuracy, OaFnMetric."""
from __future__ import annotations

import torch

from ..core.matrix import OaMatrix
from ..ops import kernels as K


class OaFnMetric:
    @staticmethod
    def ScalarLoss(loss: OaMatrix) -> float:
        return loss.Item()

    @staticmethod
    def Accuracy(logits: OaMatrix, targets: OaMatrix) -> float:
        """Fraction of rows whose argmax equals the target."""
        l2 = logits.Tensor().reshape(-1, logits.Size(-1))
        pred = K.row_reduce("argmax", l2 if l2.is_contiguous() else K.contiguous(l2))
        tg = targets.Tensor().reshape(-1).to(torch.int32)
        return float((pred == tg).float().mean().item())


class OaMetric:
    def __init__(self, name: str = "metric"):
        self.Name = name
        self.Reset()

    def Reset(self) -> None:
        self._sum, self._count, self._last = 0.0, 0, 0.0

    def Update(self, value: float, weight: int = 1) -> None:
        self._sum += float(value) * weight
        self._count += weight
        self._last = float(value)

    def Value(self) -> float:
        return self._sum / self._count if self._count else 0.0

    def Last(self) -> float:
        return self._last

    def Count(self) -> int:
        return self._count

    Result = Value


class OaMetricLoss(OaMetric):
    def __init__(self, name: str = "loss"):
        super().__init__(name)


class OaMetricAccuracy(OaMetric):
    def __init__(self):
        super().__init__("accuracy")

    def UpdateFrom(self, logits: OaMatrix, targets: OaMatrix) -> None:
        self.Update(OaFnMetric.Accuracy(logits, targets), targets.NumElements())
