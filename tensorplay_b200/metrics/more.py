"""Nominal association, operating-point, multi-task and spectral image metrics, permutation-invariant
training loss, and the task dispatchers of the curve metrics."""
from __future__ import annotations

import itertools
import math
from typing import Callable, Dict, Optional

import torch
from torch import Tensor

from . import Metric
from .classification import (BinaryPrecisionRecallCurve, BinaryROC, MulticlassAUROC, MulticlassAveragePrecision,
                             MulticlassConfusionMatrix, MultilabelAUROC, MultilabelAveragePrecision, _Scores)


# ----------------------------------------------------------------------------- nominal association
class _Contingency(MulticlassConfusionMatrix):
    """Contingency table of two categorical variables with ``num_classes`` levels each."""

    def _table(self):
        m = self.matrix.double()
        m = m[m.sum(1) > 0][:, m.sum(0) > 0]
        return m, m.sum()

    def _chi2(self):
        m, n = self._table()
        exp = m.sum(1, keepdim=True) * m.sum(0, keepdim=True) / n
        return ((m - exp) ** 2 / exp).sum(), n, m.shape


class CramersV(_Contingency):
    def __init__(self, num_classes: int, bias_correction: bool = False, **kw) -> None:
        super().__init__(num_classes)
        self.bias_correction = bias_correction

    def compute(self) -> Tensor:
        chi2, n, (r, c) = self._chi2()
        phi2 = chi2 / n
        if self.bias_correction:
            phi2 = (phi2 - (r - 1) * (c - 1) / (n - 1)).clamp(min=0)
            r, c = r - (r - 1) ** 2 / (n - 1), c - (c - 1) ** 2 / (n - 1)
        return torch.sqrt(phi2 / max(1e-12, float(min(r - 1, c - 1)))).float()


class TschuprowsT(_Contingency):
    def compute(self) -> Tensor:
        chi2, n, (r, c) = self._chi2()
        return torch.sqrt(chi2 / n / max(1e-12, math.sqrt((r - 1) * (c - 1)))).float()


class PearsonsContingencyCoefficient(_Contingency):
    def compute(self) -> Tensor:
        chi2, n, _ = self._chi2()
        return torch.sqrt(chi2 / (chi2 + n)).float()


class TheilsU(_Contingency):
    """Uncertainty coefficient ``U(target | preds) = (H(t) - H(t | p)) / H(t)`` (asymmetric)."""

    def compute(self) -> Tensor:
        m, n = self._table()
        p = m / n
        pt, pp = p.sum(1), p.sum(0)
        h_t = -(pt * torch.log(pt.clamp(min=1e-300))).sum()
        cond = -(p * (torch.log(p.clamp(min=1e-300)) - torch.log(pp.clamp(min=1e-300))[None, :])).sum()
        return ((h_t - cond) / h_t.clamp(min=1e-300)).float()


class FleissKappa(Metric):
    """Agreement of several raters: ``update`` takes ``[subjects, categories]`` counts of ratings."""

    def __init__(self, **kw) -> None:
        super().__init__()
        self.rows = []

    def reset(self) -> None:
        self.rows = []

    def update(self, counts: Tensor) -> None:
        self.rows.append(counts.detach().double())

    def compute(self) -> Tensor:
        m = torch.cat(self.rows)
        n = m.sum(1)[0]
        p_j = m.sum(0) / m.sum()
        p_i = ((m * m).sum(1) - n) / (n * (n - 1))
        pe = (p_j * p_j).sum()
        return ((p_i.mean() - pe) / (1 - pe).clamp(min=1e-12)).float()


# ----------------------------------------------------------------------------- operating points
class _AtFixed(_Scores):
    def __init__(self, min_value: float, **kw) -> None:
        super().__init__()
        self.min_value = min_value

    def _curves(self):
        p, t = self._all()
        fpr, tpr, thr = BinaryROC.compute(self)
        prec, rec, thr_pr = BinaryPrecisionRecallCurve.compute(self)
        return fpr, tpr, thr, prec, rec, thr_pr

    @staticmethod
    def _best(value: Tensor, constraint: Tensor, minimum: float, thresholds: Tensor):
        ok = constraint >= minimum
        if not bool(ok.any()):
            return torch.zeros(()), torch.tensor(1e6)
        v = torch.where(ok, value, torch.full_like(value, -1.0))
        i = int(v.argmax())
        return value[i].float(), thresholds[min(i, thresholds.numel() - 1)].float()


class BinaryPrecisionAtFixedRecall(_AtFixed):
    def compute(self):
        _, _, _, prec, rec, thr = self._curves()
        return self._best(prec, rec, self.min_value, thr)


class BinaryRecallAtFixedPrecision(_AtFixed):
    def compute(self):
        _, _, _, prec, rec, thr = self._curves()
        return self._best(rec, prec, self.min_value, thr)


class BinarySensitivityAtSpecificity(_AtFixed):
    def compute(self):
        fpr, tpr, thr, *_ = self._curves()
        return self._best(tpr, 1 - fpr, self.min_value, thr)


class BinarySpecificityAtSensitivity(_AtFixed):
    def compute(self):
        fpr, tpr, thr, *_ = self._curves()
        return self._best(1 - fpr, tpr, self.min_value, thr)


PrecisionAtFixedRecall, RecallAtFixedPrecision = BinaryPrecisionAtFixedRecall, BinaryRecallAtFixedPrecision
SensitivityAtSpecificity, SpecificityAtSensitivity = BinarySensitivityAtSpecificity, BinarySpecificityAtSensitivity


class CriticalSuccessIndex(Metric):
    """Threat score ``tp / (tp + fn + fp)`` of events defined by ``value >= threshold``."""

    def __init__(self, threshold: float, **kw) -> None:
        super().__init__()
        self.threshold = threshold
        for n in ("hit", "miss", "false"):
            self.add_state(n, torch.zeros((), dtype=torch.float64))

    def update(self, preds: Tensor, target: Tensor) -> None:
        self._to(preds.device)
        p, t = preds >= self.threshold, target >= self.threshold
        self.hit += (p & t).sum()
        self.miss += (~p & t).sum()
        self.false += (p & ~t).sum()

    def compute(self) -> Tensor:
        return (self.hit / (self.hit + self.miss + self.false).clamp(min=1)).float()


def _dispatch(binary, multiclass, multilabel):
    def make(task: str = "binary", **kw):
        return {"binary": binary, "multiclass": multiclass, "multilabel": multilabel}[task](**kw)
    return make


class _PerClassCurve(_Scores):
    curve = None

    def __init__(self, num_classes: int = None, num_labels: int = None, **kw) -> None:
        super().__init__()
        self.C, self.multilabel = num_classes or num_labels, num_labels is not None

    def compute(self):
        p, t = self._all()
        p = p.reshape(-1, self.C)
        out = []
        for c in range(self.C):
            m = type(self).curve()
            m.update(p[:, c], t.reshape(-1, self.C)[:, c] if self.multilabel else (t.reshape(-1) == c).long())
            out.append(m.compute())
        return out


MulticlassROC = type("MulticlassROC", (_PerClassCurve,), {"curve": BinaryROC})
MultilabelROC = type("MultilabelROC", (_PerClassCurve,), {"curve": BinaryROC})
MulticlassPrecisionRecallCurve = type("MulticlassPrecisionRecallCurve", (_PerClassCurve,), {"curve": BinaryPrecisionRecallCurve})
MultilabelPrecisionRecallCurve = type("MultilabelPrecisionRecallCurve", (_PerClassCurve,), {"curve": BinaryPrecisionRecallCurve})
ROC = _dispatch(BinaryROC, MulticlassROC, MultilabelROC)
PrecisionRecallCurve = _dispatch(BinaryPrecisionRecallCurve, MulticlassPrecisionRecallCurve, MultilabelPrecisionRecallCurve)


# ----------------------------------------------------------------------------- wrappers, audio, spectral image
class MultitaskWrapper(Metric):
    """Dictionary of metrics fed with dictionaries of predictions and targets keyed by task."""

    def __init__(self, task_metrics: Dict[str, Metric]) -> None:
        super().__init__()
        self.task_metrics = dict(task_metrics)

    def update(self, preds: Dict[str, Tensor], target: Dict[str, Tensor]) -> None:
        for k, m in self.task_metrics.items():
            m.update(preds[k], target[k])

    def compute(self):
        return {k: m.compute() for k, m in self.task_metrics.items()}

    def reset(self) -> None:
        for m in self.task_metrics.values():
            m.reset()

    def sync(self, group=None) -> None:
        for m in self.task_metrics.values():
            m.sync(group)


class PermutationInvariantTraining(Metric):
    """Best value of a pairwise metric over the assignments of estimated to reference sources
    (``[batch, sources, time]``); ``eval_func`` "max" or "min"."""

    def __init__(self, metric_func: Callable[[Tensor, Tensor], Tensor], eval_func: str = "max", **kw) -> None:
        super().__init__()
        self.fn, self.eval_func = metric_func, eval_func
        self.add_state("total", torch.zeros((), dtype=torch.float64))
        self.add_state("n", torch.zeros((), dtype=torch.float64))

    def update(self, preds: Tensor, target: Tensor) -> None:
        self._to(preds.device)
        s = preds.shape[1]
        pair = torch.stack([torch.stack([self.fn(preds[:, i], target[:, j]) for j in range(s)], -1) for i in range(s)], -2)
        vals = torch.stack([pair[:, list(range(s)), list(perm)].mean(-1) for perm in itertools.permutations(range(s))], -1)
        best = vals.max(-1).values if self.eval_func == "max" else vals.min(-1).values
        self.total += best.double().sum()
        self.n += best.numel()

    def compute(self) -> Tensor:
        return (self.total / self.n.clamp(min=1)).float()


class _ImageMean(Metric):
    def __init__(self, **kw) -> None:
        super().__init__()
        self.add_state("total", torch.zeros((), dtype=torch.float64))
        self.add_state("n", torch.zeros((), dtype=torch.float64))

    def _value(self, p: Tensor, t: Tensor) -> Tensor:
        raise NotImplementedError

    def update(self, preds: Tensor, target: Tensor) -> None:
        self._to(preds.device)
        v = self._value(preds.double(), target.double())
        self.total += v.sum()
        self.n += v.numel()

    def compute(self) -> Tensor:
        return (self.total / self.n.clamp(min=1)).float()


class SpectralAngleMapper(_ImageMean):
    """Mean angle (radians) between the spectra (channel vectors) of corresponding pixels."""

    def _value(self, p, t):
        cos = (p * t).sum(1) / (p.norm(dim=1) * t.norm(dim=1)).clamp(min=1e-30)
        return torch.acos(cos.clamp(-1, 1)).flatten(1).mean(-1)


class ErrorRelativeGlobalDimensionlessSynthesis(_ImageMean):
    """ERGAS: ``100 * ratio * sqrt(mean_bands(RMSE_b^2 / mean_b^2))``."""

    def __init__(self, ratio: float = 4.0, **kw) -> None:
        super().__init__()
        self.ratio = ratio

    def _value(self, p, t):
        rmse2 = ((p - t) ** 2).flatten(2).mean(-1)
        mean2 = t.flatten(2).mean(-1) ** 2
        return 100 * self.ratio * torch.sqrt((rmse2 / mean2.clamp(min=1e-30)).mean(-1))


class RelativeAverageSpectralError(_ImageMean):
    """RASE: ``100 / mean * sqrt(mean_bands(RMSE_b^2))`` over whole images."""

    def _value(self, p, t):
        rmse2 = ((p - t) ** 2).flatten(2).mean(-1)
        return 100 / t.flatten(1).mean(-1).clamp(min=1e-30) * torch.sqrt(rmse2.mean(-1))


class RootMeanSquaredErrorUsingSlidingWindow(_ImageMean):
    def __init__(self, window_size: int = 8, **kw) -> None:
        super().__init__()
        self.w = window_size

    def _value(self, p, t):
        mse = torch.nn.functional.avg_pool2d((p - t) ** 2, self.w, stride=1)
        return torch.sqrt(mse).flatten(1).mean(-1)


__all__ = sorted(n for n in globals() if n[0].isupper() and n not in ("Metric", "Tensor", "Optional", "Callable", "Dict"))
