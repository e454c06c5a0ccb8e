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


# ----------------------------------------------------------------------------- further classification / retrieval
def HingeLoss(task: str = "binary", **kw):
    from .classification import BinaryHingeLoss, MulticlassHingeLoss
    return {"binary": BinaryHingeLoss, "multiclass": MulticlassHingeLoss}[task](**kw)


class MultilabelMatthewsCorrCoef(Metric):
    """Matthews correlation of the 2 x 2 table pooled over all labels (``preds`` thresholded)."""

    def __init__(self, num_labels: int, threshold: float = 0.5, **kw) -> None:
        super().__init__()
        self.threshold = threshold
        self.add_state("table", torch.zeros(2, 2, dtype=torch.float64))

    def update(self, preds: Tensor, target: Tensor) -> None:
        self._to(preds.device)
        p = (preds >= self.threshold).reshape(-1) if preds.is_floating_point() else preds.reshape(-1).bool()
        t = target.reshape(-1).bool()
        for a in (0, 1):
            for b in (0, 1):
                self.table[a, b] += ((t == bool(a)) & (p == bool(b))).sum()

    def compute(self) -> Tensor:
        (tn, fp), (fn, tp) = self.table.tolist()
        den = math.sqrt((tp + fp) * (tp + fn) * (tn + fp) * (tn + fn))
        return torch.tensor((tp * tn - fp * fn) / den if den else 0.0)


def _interp(x: Tensor, xp: Tensor, fp: Tensor) -> Tensor:
    i = torch.searchsorted(xp, x).clamp(1, xp.numel() - 1)
    x0, x1, y0, y1 = xp[i - 1], xp[i], fp[i - 1], fp[i]
    w = torch.where(x1 > x0, (x - x0) / (x1 - x0).clamp(min=1e-300), torch.zeros_like(x))
    return y0 + w * (y1 - y0)


class BinaryLogAUC(_Scores):
    """Area under the ROC curve over ``log10(fpr)`` within ``fpr_range``, divided by the width of the
    range in decades (1.0 = perfect, about 0.0215 for a random classifier over (0.001, 0.1))."""

    def __init__(self, fpr_range=(0.001, 0.1), **kw) -> None:
        super().__init__()
        self.fpr_range = fpr_range

    def compute(self) -> Tensor:
        fpr, tpr, _ = BinaryROC.compute(self)
        fpr, tpr = fpr.double(), tpr.double()
        lo, hi = self.fpr_range
        bounds = torch.tensor([lo, hi], dtype=torch.float64)
        tb = _interp(bounds, fpr, tpr)
        keep = (fpr > lo) & (fpr < hi)
        x = torch.log10(torch.cat((bounds[:1], fpr[keep], bounds[1:])))
        y = torch.cat((tb[:1], tpr[keep], tb[1:]))
        return (torch.trapezoid(y, x) / (math.log10(hi) - math.log10(lo))).float()


LogAUC = _dispatch(BinaryLogAUC, None, None)


class RetrievalPrecisionRecallCurve(Metric):
    """Precision and recall at every cut-off ``k = 1 .. max_k``, averaged over the queries."""

    def __init__(self, max_k: Optional[int] = None, adaptive_k: bool = False, **kw) -> None:
        super().__init__()
        self.max_k, self.adaptive_k = max_k, adaptive_k
        self.p, self.t, self.q = [], [], []

    def reset(self) -> None:
        self.p, self.t, self.q = [], [], []

    def update(self, preds: Tensor, target: Tensor, indexes: Tensor) -> None:
        self.p.append(preds.detach().reshape(-1))
        self.t.append(target.detach().reshape(-1))
        self.q.append(indexes.detach().reshape(-1))

    def compute(self):
        p, t, q = torch.cat(self.p), torch.cat(self.t), torch.cat(self.q)
        groups = [q == qi for qi in q.unique().tolist()]
        max_k = self.max_k or max(int(m.sum()) for m in groups)
        ks = torch.arange(1, max_k + 1, dtype=torch.float64)
        precs, recs = [], []
        for m in groups:
            rel = t[m][torch.argsort(p[m], descending=True)].double()
            n = rel.numel()
            hits = torch.cumsum(torch.cat((rel, torch.zeros(max(0, max_k - n), dtype=torch.float64)))[:max_k], 0)
            denom = ks.clamp(max=n) if self.adaptive_k else ks
            precs.append(hits / denom)
            recs.append(hits / rel.sum() if rel.sum() > 0 else torch.zeros_like(hits))
        return torch.stack(precs).mean(0).float(), torch.stack(recs).mean(0).float(), ks.long()


class RetrievalRecallAtFixedPrecision(RetrievalPrecisionRecallCurve):
    """Highest recall among the cut-offs whose precision reaches ``min_precision``, and its ``k``."""

    def __init__(self, min_precision: float = 0.0, max_k: Optional[int] = None, adaptive_k: bool = False, **kw) -> None:
        super().__init__(max_k, adaptive_k)
        self.min_precision = min_precision

    def compute(self):
        prec, rec, ks = super().compute()
        ok = prec >= self.min_precision
        if not bool(ok.any()):
            return torch.zeros(()), ks[-1]
        i = int(torch.where(ok, rec, torch.full_like(rec, -1.0)).argmax())
        return rec[i], ks[i]


# ----------------------------------------------------------------------------- audio
def signal_distortion_ratio(preds: Tensor, target: Tensor, filter_length: int = 512, zero_mean: bool = False,
                            load_diag: Optional[float] = None) -> Tensor:
    """SDR of BSS-eval: the reference may be distorted by any FIR filter of ``filter_length`` taps;
    the optimal filter comes from the Toeplitz normal equations (auto- and cross-correlation by FFT)."""
    p, t = preds.double(), target.double()
    if zero_mean:
        p, t = p - p.mean(-1, keepdim=True), t - t.mean(-1, keepdim=True)
    t = t / t.norm(dim=-1, keepdim=True).clamp(min=1e-12)
    p = p / p.norm(dim=-1, keepdim=True).clamp(min=1e-12)
    n = 1 << (t.shape[-1] + filter_length - 1).bit_length()
    tf, pf = torch.fft.rfft(t, n), torch.fft.rfft(p, n)
    acf = torch.fft.irfft(tf.abs() ** 2, n)[..., :filter_length]
    xcorr = torch.fft.irfft(tf.conj() * pf, n)[..., :filter_length]
    if load_diag is not None:
        acf[..., 0] += load_diag
    idx = (torch.arange(filter_length)[:, None] - torch.arange(filter_length)[None, :]).abs()
    sol = torch.linalg.solve(acf[..., idx], xcorr.unsqueeze(-1)).squeeze(-1)
    coh = (xcorr * sol).sum(-1)
    return (10 * torch.log10(coh / (1 - coh).clamp(min=1e-30))).float()


class SignalDistortionRatio(_ImageMean):
    def __init__(self, filter_length: int = 512, zero_mean: bool = False, load_diag: Optional[float] = None, **kw) -> None:
        super().__init__()
        self.kw = dict(filter_length=filter_length, zero_mean=zero_mean, load_diag=load_diag)

    def _value(self, p, t):
        return signal_distortion_ratio(p, t, **self.kw).double()


class SourceAggregatedSignalDistortionRatio(_ImageMean):
    """``10 log10(sum_s |t_s|^2 / sum_s |t_s - p_s|^2)`` over the sources of a mixture
    (``[..., sources, time]``); ``scale_invariant`` rescales the targets by one common factor first."""

    def __init__(self, scale_invariant: bool = True, zero_mean: bool = False, **kw) -> None:
        super().__init__()
        self.scale_invariant, self.zero_mean = scale_invariant, zero_mean

    def _value(self, p, t):
        if self.zero_mean:
            p, t = p - p.mean(-1, keepdim=True), t - t.mean(-1, keepdim=True)
        if self.scale_invariant:
            alpha = ((p * t).sum((-1, -2), keepdim=True) + 1e-12) / ((t * t).sum((-1, -2), keepdim=True) + 1e-12)
            t = alpha * t
        return 10 * torch.log10(((t * t).sum((-1, -2)) + 1e-12) / (((t - p) ** 2).sum((-1, -2)) + 1e-12))


# ----------------------------------------------------------------------------- image
class MultiScaleStructuralSimilarityIndexMeasure(_ImageMean):
    """MS-SSIM: the contrast-structure term at five dyadic scales and the full SSIM at the coarsest,
    combined with the exponents of Wang et al. (2003)."""

    def __init__(self, data_range: float = 1.0, kernel_size: int = 11, sigma: float = 1.5,
                 betas=(0.0448, 0.2856, 0.3001, 0.2363, 0.1333), k1: float = 0.01, k2: float = 0.03, **kw) -> None:
        super().__init__()
        self.args = (data_range, kernel_size, sigma, k1, k2)
        self.betas = betas

    def _value(self, p, t):
        from .domains import _gaussian_window
        data_range, ks, sigma, k1, k2 = self.args
        c1, c2 = (k1 * data_range) ** 2, (k2 * data_range) ** 2
        ch = p.shape[1]
        w = _gaussian_window(ks, sigma, ch, p.device, p.dtype)
        conv = lambda x: torch.nn.functional.conv2d(x, w, groups=ch)   # noqa: E731
        out = torch.ones(p.shape[0], dtype=p.dtype)
        for i, beta in enumerate(self.betas):
            mp, mt = conv(p), conv(t)
            vp, vt, cov = conv(p * p) - mp * mp, conv(t * t) - mt * mt, conv(p * t) - mp * mt
            cs = (2 * cov + c2) / (vp + vt + c2)
            if i == len(self.betas) - 1:
                term = (((2 * mp * mt + c1) / (mp * mp + mt * mt + c1)) * cs).flatten(1).mean(-1)
            else:
                term = cs.flatten(1).mean(-1)
                p, t = torch.nn.functional.avg_pool2d(p, 2), torch.nn.functional.avg_pool2d(t, 2)
            out = out * term.clamp(min=0) ** beta
        return out


def _uqi_pair(a: Tensor, b: Tensor, window: int = 7) -> Tensor:
    from .domains import ssim
    return ssim(a, b, kernel_size=window, sigma=1.5, k1=1e-8, k2=1e-8)


class SpectralDistortionIndex(_ImageMean):
    """D_lambda of the QNR protocol: how much the inter-band quality indices change between the
    low-resolution multispectral image (``target``) and the fused image (``preds``)."""

    def __init__(self, p: int = 1, **kw) -> None:
        super().__init__()
        self.p = p

    def _value(self, fused, ms):
        L = fused.shape[1]
        acc = torch.zeros(fused.shape[0], dtype=fused.dtype)
        for a in range(L):
            for b in range(a + 1, L):
                d = _uqi_pair(ms[:, a:a + 1], ms[:, b:b + 1]) - _uqi_pair(fused[:, a:a + 1], fused[:, b:b + 1])
                acc += 2 * d.abs() ** self.p
        return (acc / (L * (L - 1))) ** (1.0 / self.p)


class SpatialDistortionIndex(Metric):
    """D_s of the QNR protocol; ``target`` is a dict with ``ms`` (low-resolution multispectral),
    ``pan`` (panchromatic at the fused resolution) and optionally ``pan_lr`` (else ``pan`` is
    average-pooled to the size of ``ms``)."""

    def __init__(self, norm_order: int = 1, window_size: int = 7, **kw) -> None:
        super().__init__()
        self.q, self.window = norm_order, window_size
        self.add_state("total", torch.zeros((), dtype=torch.float64))
        self.add_state("n", torch.zeros((), dtype=torch.float64))

    def update(self, preds: Tensor, target: Dict[str, Tensor]) -> None:
        fused, ms, pan = preds.double(), target["ms"].double(), target["pan"].double()
        pan_lr = target.get("pan_lr")
        pan_lr = pan_lr.double() if pan_lr is not None else torch.nn.functional.adaptive_avg_pool2d(pan, ms.shape[-2:])
        L = fused.shape[1]
        acc = torch.zeros(fused.shape[0], dtype=torch.float64)
        for l in range(L):
            d = _uqi_pair(fused[:, l:l + 1], pan[:, l:l + 1] if pan.shape[1] > 1 else pan, self.window) \
                - _uqi_pair(ms[:, l:l + 1], pan_lr[:, l:l + 1] if pan_lr.shape[1] > 1 else pan_lr, self.window)
            acc += d.abs() ** self.q
        v = (acc / L) ** (1.0 / self.q)
        self.total += v.sum()
        self.n += v.numel()

    def compute(self) -> Tensor:
        return (self.total / self.n.clamp(min=1)).float()


class LipVertexError(Metric):
    """Mean over frames of the largest squared L2 error among the lip vertices
    (``[frames, vertices, 3]`` inputs, ``mouth_map`` = indices of the lip vertices)."""

    def __init__(self, mouth_map, **kw) -> None:
        super().__init__()
        self.mouth_map = list(mouth_map)
        self.add_state("total", torch.zeros((), dtype=torch.float64))
        self.add_state("n", torch.zeros((), dtype=torch.float64))

    def update(self, vertices_pred: Tensor, vertices_gt: Tensor) -> None:
        self._to(vertices_pred.device)
        f = min(vertices_pred.shape[0], vertices_gt.shape[0])
        d = ((vertices_pred[:f, self.mouth_map] - vertices_gt[:f, self.mouth_map]).double() ** 2).sum(-1)
        self.total += d.max(-1).values.sum()
        self.n += f

    def compute(self) -> Tensor:
        return (self.total / self.n.clamp(min=1)).float()


# ----------------------------------------------------------------------------- per-class forms and matrices
def _per_class(binary_cls, name: str):
    """Multiclass (one class against the rest) and multilabel forms of a binary score metric: the
    binary metric per column; tuples of (value, threshold) come back as two stacked tensors."""

    class _PerClass(_Scores):
        def __init__(self, num_classes: int = None, num_labels: int = None, average: Optional[str] = None, **kw) -> None:
            super().__init__()
            self.C, self.multilabel, self.average, self.kw = num_classes or num_labels, num_labels is not None, average, kw

        def compute(self):
            p, t = self._all()
            p = p.reshape(-1, self.C)
            out = []
            for c in range(self.C):
                m = binary_cls(**self.kw)
                m.update(p[:, c], t.reshape(-1, self.C)[:, c] if self.multilabel else (t.reshape(-1) == c).long())
                out.append(m.compute())
            if isinstance(out[0], tuple):
                return tuple(torch.stack([o[i] for o in out]) for i in range(len(out[0])))
            vals = torch.stack(out)
            return vals.mean() if self.average == "macro" else vals
    _PerClass.__name__ = _PerClass.__qualname__ = name
    return _PerClass


for _stem, _cls in (("PrecisionAtFixedRecall", BinaryPrecisionAtFixedRecall), ("RecallAtFixedPrecision", BinaryRecallAtFixedPrecision),
                    ("SensitivityAtSpecificity", BinarySensitivityAtSpecificity),
                    ("SpecificityAtSensitivity", BinarySpecificityAtSensitivity), ("LogAUC", BinaryLogAUC)):
    for _kind in ("Multiclass", "Multilabel"):
        globals()[_kind + _stem] = _per_class(_cls, _kind + _stem)
LogAUC = _dispatch(BinaryLogAUC, globals()["MulticlassLogAUC"], globals()["MultilabelLogAUC"])
PrecisionAtFixedRecall = _dispatch(BinaryPrecisionAtFixedRecall, globals()["MulticlassPrecisionAtFixedRecall"],
                                   globals()["MultilabelPrecisionAtFixedRecall"])
RecallAtFixedPrecision = _dispatch(BinaryRecallAtFixedPrecision, globals()["MulticlassRecallAtFixedPrecision"],
                                   globals()["MultilabelRecallAtFixedPrecision"])
SensitivityAtSpecificity = _dispatch(BinarySensitivityAtSpecificity, globals()["MulticlassSensitivityAtSpecificity"],
                                     globals()["MultilabelSensitivityAtSpecificity"])
SpecificityAtSensitivity = _dispatch(BinarySpecificityAtSensitivity, globals()["MulticlassSpecificityAtSensitivity"],
                                     globals()["MultilabelSpecificityAtSensitivity"])


class MulticlassExactMatch(Metric):
    """Fraction of samples all of whose positions are classified right (``[N, ...]`` labels or
    ``[N, C, ...]`` scores); ``multidim_average="samplewise"`` returns the 0/1 value per sample."""

    def __init__(self, num_classes: int = None, multidim_average: str = "global", ignore_index: Optional[int] = None, **kw) -> None:
        super().__init__()
        self.samplewise, self.ignore_index = multidim_average == "samplewise", ignore_index
        self.rows = []

    def reset(self) -> None:
        self.rows = []

    def update(self, preds: Tensor, target: Tensor) -> None:
        p = preds.argmax(1) if preds.dim() == target.dim() + 1 else preds
        ok = p == target
        if self.ignore_index is not None:
            ok = ok | (target == self.ignore_index)
        self.rows.append(ok.reshape(ok.shape[0], -1).all(-1).detach().cpu())

    def compute(self) -> Tensor:
        v = torch.cat(self.rows).float()
        return v if self.samplewise else v.mean()


class MultilabelExactMatch(MulticlassExactMatch):
    def __init__(self, num_labels: int = None, threshold: float = 0.5, multidim_average: str = "global", **kw) -> None:
        super().__init__(multidim_average=multidim_average)
        self.threshold = threshold

    def update(self, preds: Tensor, target: Tensor) -> None:
        p = (preds >= self.threshold).long() if preds.is_floating_point() else preds
        self.rows.append((p == target).reshape(p.shape[0], -1).all(-1).detach().cpu())


def _association_matrix(cls):
    def fn(matrix: Tensor, **kw) -> Tensor:
        """Pairwise association of the columns of a ``[samples, variables]`` matrix of category codes."""
        n = matrix.shape[1]
        levels = int(matrix.max()) + 1
        out = torch.ones(n, n)
        for i in range(n):
            for j in range(n):
                if i == j or (j < i and cls is not TheilsU):
                    out[i, j] = out[j, i] if j < i else 1.0
                    continue
                m = cls(levels, **kw)
                m.update(matrix[:, i], matrix[:, j])
                out[i, j] = m.compute()
        return out
    return fn


cramers_v_matrix = _association_matrix(CramersV)
tschuprows_t_matrix = _association_matrix(TschuprowsT)
pearsons_contingency_coefficient_matrix = _association_matrix(PearsonsContingencyCoefficient)
theils_u_matrix = _association_matrix(TheilsU)


def pit_permutate(preds: Tensor, perm: Tensor) -> Tensor:
    """Reorder the sources of ``preds`` (``[batch, sources, ...]``) by the permutation of each sample."""
    return torch.stack([p[q] for p, q in zip(preds, perm)])


__all__ = sorted(n for n in globals() if n[0].isupper() and n not in ("Metric", "Tensor", "Optional", "Callable", "Dict")) + ["cramers_v_matrix", "tschuprows_t_matrix", "pearsons_contingency_coefficient_matrix", "theils_u_matrix",
           "pit_permutate", "signal_distortion_ratio"]


# the reference has a package at this path: deeper module names resolve to views of the pack
__path__: list = []


def __getattr__(name):
    """Names of this domain that live in another file of the pack (task wrappers, shared bases)."""
    if name.startswith("__"):
        raise AttributeError(name)
    import importlib
    pkg = importlib.import_module(__name__.rsplit(".", 1)[0])
    if name in pkg.__dict__:
        return pkg.__dict__[name]
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
