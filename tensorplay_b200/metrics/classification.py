"""Task-specific classification metrics (binary / multiclass / multilabel variants of the
stat-score family, curves, kappa / Matthews, hinge loss), built on per-class counts of true and false
positives and negatives that are summed across updates and ranks."""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from . import Metric


def _binarize(preds: Tensor, threshold: float) -> Tensor:
    if preds.is_floating_point():
        if preds.min() < 0 or preds.max() > 1:
            preds = torch.sigmoid(preds)           # logits
        return (preds > threshold).long()
    return preds.long()


class _Counts(Metric):
    """tp / fp / tn / fn per class (``C`` = 1 for binary, classes for multiclass, labels for multilabel)."""

    task = "binary"

    def __init__(self, num_classes: int = 2, num_labels: Optional[int] = None, threshold: float = 0.5,
                 average: Optional[str] = None, top_k: int = 1, ignore_index: Optional[int] = None, **kw) -> None:
        super().__init__()
        self.C = 1 if self.task == "binary" else (num_labels or num_classes if self.task == "multilabel" else num_classes)
        self.threshold, self.top_k, self.ignore_index = threshold, top_k, ignore_index
        self.average = average if average is not None else ("micro" if self.task == "binary" else "macro")
        for n in ("tp", "fp", "tn", "fn"):
            self.add_state(n, torch.zeros(self.C, dtype=torch.long))

    def update(self, preds: Tensor, target: Tensor) -> None:
        self._to(target.device)
        if self.task == "multiclass":
            t = target.reshape(-1)
            if preds.is_floating_point() and preds.dim() == target.dim() + 1:
                p2 = preds.reshape(-1, preds.shape[-1])
                hit = p2.topk(self.top_k, -1).indices if self.top_k > 1 else p2.argmax(-1, keepdim=True)
                # with top-k the prediction counts as the target class when the target is among the k
                p = torch.where((hit == t[:, None]).any(-1), t, hit[:, 0])
            else:
                p = preds.reshape(-1).long()
            if self.ignore_index is not None:
                keep = t != self.ignore_index
                p, t = p[keep], t[keep]
            oh_p = torch.nn.functional.one_hot(p, self.C).bool()
            oh_t = torch.nn.functional.one_hot(t, self.C).bool()
        else:
            p = _binarize(preds, self.threshold)
            t = target.long()
            if self.task == "binary":
                p, t = p.reshape(-1, 1), t.reshape(-1, 1)
            else:
                p, t = p.reshape(-1, self.C), t.reshape(-1, self.C)
            if self.ignore_index is not None:
                keep = (t != self.ignore_index)
                p, t = p * keep, t * keep
            oh_p, oh_t = p.bool(), t.bool()
        self.tp += (oh_p & oh_t).sum(0)
        self.fp += (oh_p & ~oh_t).sum(0)
        self.fn += (~oh_p & oh_t).sum(0)
        self.tn += (~oh_p & ~oh_t).sum(0)

    def _ratio(self, num: Tensor, den: Tensor, weights: Optional[Tensor] = None) -> Tensor:
        num, den = num.double(), den.double()
        if self.average == "micro" or self.C == 1:
            return (num.sum() / den.sum().clamp(min=1e-12)).float()
        per = num / den.clamp(min=1e-12)
        if self.average in ("none", None):
            return per.float()
        if self.average == "weighted":
            w = (self.tp + self.fn).double() if weights is None else weights
            return ((per * w).sum() / w.sum().clamp(min=1e-12)).float()
        return per.mean().float()


def _stat_metric(name, fn, doc):
    def compute(self):
        return fn(self)
    base = type("_" + name, (_Counts,), {"compute": compute, "__doc__": doc})
    out = {}
    for task, prefix in (("binary", "Binary"), ("multiclass", "Multiclass"), ("multilabel", "Multilabel")):
        out[prefix + name] = type(prefix + name, (base,), {"task": task, "__doc__": doc})
    return out


def _fbeta(self):
    b2 = getattr(self, "beta", 1.0) ** 2
    return self._ratio((1 + b2) * self.tp, (1 + b2) * self.tp + b2 * self.fn + self.fp)


_FAMILY = {}
_FAMILY.update(_stat_metric("Accuracy", lambda s: s._ratio(s.tp + s.tn, s.tp + s.tn + s.fp + s.fn)
                            if s.task != "multiclass" else
                            (s._ratio(s.tp, s.tp + s.fn) if s.average != "micro" else
                             (s.tp.sum().double() / (s.tp + s.fn).sum().double().clamp(min=1e-12)).float()),
                            "Fraction of correct decisions (per class recall averaged for macro multiclass)."))
_FAMILY.update(_stat_metric("Precision", lambda s: s._ratio(s.tp, s.tp + s.fp), "tp / (tp + fp)."))
_FAMILY.update(_stat_metric("Recall", lambda s: s._ratio(s.tp, s.tp + s.fn), "tp / (tp + fn)."))
_FAMILY.update(_stat_metric("Specificity", lambda s: s._ratio(s.tn, s.tn + s.fp), "tn / (tn + fp)."))
_FAMILY.update(_stat_metric("NegativePredictiveValue", lambda s: s._ratio(s.tn, s.tn + s.fn), "tn / (tn + fn)."))
_FAMILY.update(_stat_metric("F1Score", _fbeta, "Harmonic mean of precision and recall."))
_FAMILY.update(_stat_metric("JaccardIndex", lambda s: s._ratio(s.tp, s.tp + s.fp + s.fn), "Intersection over union."))
_FAMILY.update(_stat_metric("HammingDistance", lambda s: s._ratio(s.fp + s.fn, s.tp + s.tn + s.fp + s.fn)
                            if s.task != "multiclass" else 1 - s._ratio(s.tp, s.tp + s.fn),
                            "Fraction of wrong labels."))
_FAMILY.update(_stat_metric("StatScores", lambda s: torch.stack((s.tp, s.fp, s.tn, s.fn, s.tp + s.fn), -1).squeeze(0),
                            "``[tp, fp, tn, fn, support]`` (per class)."))
globals().update(_FAMILY)


def _fbeta_class(prefix, task):
    base = _FAMILY[prefix + "F1Score"]

    def __init__(self, beta: float = 1.0, **kw):
        base.__init__(self, **kw)
        self.beta = beta
    return type(prefix + "FBetaScore", (base,), {"__init__": __init__, "task": task,
                                                 "__doc__": "F-beta: recall weighted ``beta`` times as much as precision."})


for _p, _t in (("Binary", "binary"), ("Multiclass", "multiclass"), ("Multilabel", "multilabel")):
    globals()[_p + "FBetaScore"] = _fbeta_class(_p, _t)


def _task_dispatch(name):
    def make(task: str = "multiclass", **kw):
        prefix = {"binary": "Binary", "multiclass": "Multiclass", "multilabel": "Multilabel"}[task]
        return globals()[prefix + name](**kw)
    make.__name__ = name
    make.__doc__ = f"``{name}(task=...)``: the binary / multiclass / multilabel variant."
    return make


Specificity, JaccardIndex, HammingDistance, StatScores, FBetaScore, NegativePredictiveValue = (
    _task_dispatch(n) for n in ("Specificity", "JaccardIndex", "HammingDistance", "StatScores", "FBetaScore",
                                "NegativePredictiveValue"))


class MulticlassConfusionMatrix(Metric):
    def __init__(self, num_classes: int, normalize: Optional[str] = None, **kw) -> None:
        super().__init__()
        self.C, self.normalize = num_classes, normalize
        self.add_state("matrix", torch.zeros(num_classes, num_classes, dtype=torch.long))

    def update(self, preds: Tensor, target: Tensor) -> None:
        self._to(target.device)
        p = preds.argmax(-1) if preds.is_floating_point() and preds.dim() == target.dim() + 1 else preds
        idx = target.reshape(-1).long() * self.C + p.reshape(-1).long()
        self.matrix += torch.bincount(idx, minlength=self.C * self.C).view(self.C, self.C)

    def compute(self) -> Tensor:
        m = self.matrix
        if self.normalize == "true":
            return m.double() / m.sum(1, keepdim=True).clamp(min=1)
        if self.normalize == "pred":
            return m.double() / m.sum(0, keepdim=True).clamp(min=1)
        if self.normalize == "all":
            return m.double() / m.sum().clamp(min=1)
        return m


class BinaryConfusionMatrix(MulticlassConfusionMatrix):
    def __init__(self, threshold: float = 0.5, normalize: Optional[str] = None, **kw) -> None:
        super().__init__(2, normalize)
        self.threshold = threshold

    def update(self, preds: Tensor, target: Tensor) -> None:
        super().update(_binarize(preds, self.threshold), target)


class MultilabelConfusionMatrix(Metric):
    """One 2 x 2 matrix per label: ``[label, true, predicted]``."""

    def __init__(self, num_labels: int, threshold: float = 0.5, **kw) -> None:
        super().__init__()
        self.L, self.threshold = num_labels, threshold
        self.add_state("matrix", torch.zeros(num_labels, 2, 2, dtype=torch.long))

    def update(self, preds: Tensor, target: Tensor) -> None:
        self._to(target.device)
        p, t = _binarize(preds, self.threshold).reshape(-1, self.L), target.reshape(-1, self.L).long()
        for a in (0, 1):
            for b in (0, 1):
                self.matrix[:, a, b] += ((t == a) & (p == b)).sum(0)

    def compute(self) -> Tensor:
        return self.matrix


class MulticlassCohenKappa(MulticlassConfusionMatrix):
    """Agreement beyond chance: ``(p_o - p_e) / (1 - p_e)``."""

    def compute(self) -> Tensor:
        m = self.matrix.double()
        n = m.sum().clamp(min=1)
        po = m.diag().sum() / n
        pe = (m.sum(0) * m.sum(1)).sum() / (n * n)
        return ((po - pe) / (1 - pe).clamp(min=1e-12)).float()


class BinaryCohenKappa(BinaryConfusionMatrix):
    compute = MulticlassCohenKappa.compute


class MulticlassMatthewsCorrCoef(MulticlassConfusionMatrix):
    def compute(self) -> Tensor:
        m = self.matrix.double()
        t, p, c, s = m.sum(1), m.sum(0), m.diag().sum(), m.sum()
        num = c * s - (t * p).sum()
        den = torch.sqrt((s * s - (p * p).sum()) * (s * s - (t * t).sum()))
        return (num / den.clamp(min=1e-12)).float()


class BinaryMatthewsCorrCoef(BinaryConfusionMatrix):
    compute = MulticlassMatthewsCorrCoef.compute


def CohenKappa(task: str = "multiclass", **kw):
    return BinaryCohenKappa(**kw) if task == "binary" else MulticlassCohenKappa(**kw)


def MatthewsCorrCoef(task: str = "multiclass", **kw):
    return BinaryMatthewsCorrCoef(**kw) if task == "binary" else MulticlassMatthewsCorrCoef(**kw)


class _Scores(Metric):
    """Keeps all scores and targets (curve metrics need the ranking of the whole set)."""

    def __init__(self, **kw) -> None:
        super().__init__()
        self.p, self.t = [], []

    def reset(self) -> None:
        self.p, self.t = [], []

    def update(self, preds: Tensor, target: Tensor) -> None:
        self.p.append(preds.detach())
        self.t.append(target.detach())

    def sync(self, group=None) -> None:
        import torch.distributed as dist
        if not (dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1) or not self.p:
            return
        for name in ("p", "t"):
            t = torch.cat(getattr(self, name))
            parts = [None] * dist.get_world_size(group)
            dist.all_gather_object(parts, t.cpu(), group=group)
            setattr(self, name, [torch.cat(parts).to(t.device)])

    def _all(self):
        return torch.cat(self.p), torch.cat(self.t)


def _binary_curve(scores: Tensor, target: Tensor):
    """Cumulative tp / fp at every distinct threshold, scores descending."""
    order = torch.argsort(scores.double(), descending=True)
    s, t = scores.double()[order], target[order].double()
    distinct = torch.nonzero(s[1:] != s[:-1]).reshape(-1)
    idx = torch.cat((distinct, torch.tensor([s.numel() - 1], device=s.device)))
    tps = torch.cumsum(t, 0)[idx]
    fps = (idx + 1).double() - tps
    return fps, tps, s[idx]


class BinaryROC(_Scores):
    """``(fpr, tpr, thresholds)`` starting at (0, 0)."""

    def compute(self):
        p, t = self._all()
        fps, tps, thr = _binary_curve(p.reshape(-1), t.reshape(-1))
        z = torch.zeros(1, dtype=torch.float64, device=fps.device)
        fpr = torch.cat((z, fps)) / fps[-1].clamp(min=1)
        tpr = torch.cat((z, tps)) / tps[-1].clamp(min=1)
        return fpr, tpr, torch.cat((torch.ones(1, dtype=torch.float64, device=thr.device) * float("inf"), thr))


class BinaryPrecisionRecallCurve(_Scores):
    """``(precision, recall, thresholds)`` with recall decreasing, ending at (1, 0)."""

    def compute(self):
        p, t = self._all()
        fps, tps, thr = _binary_curve(p.reshape(-1), t.reshape(-1))
        precision = tps / (tps + fps)
        recall = tps / tps[-1].clamp(min=1)
        one, zero = torch.ones(1, dtype=torch.float64), torch.zeros(1, dtype=torch.float64)
        return (torch.cat((precision.flip(0), one.to(precision.device))), torch.cat((recall.flip(0), zero.to(recall.device))),
                thr.flip(0))


class BinaryAUROC(_Scores):
    def compute(self) -> Tensor:
        from .ranking import binary_auroc
        p, t = self._all()
        return binary_auroc(p, t).float()


class BinaryAveragePrecision(_Scores):
    def compute(self) -> Tensor:
        from .ranking import binary_average_precision
        p, t = self._all()
        return binary_average_precision(p, t).float()


class MulticlassAUROC(_Scores):
    """One-vs-rest AUROC per class, macro-averaged (``average="none"`` keeps the classes)."""

    def __init__(self, num_classes: int, average: Optional[str] = "macro", **kw) -> None:
        super().__init__()
        self.C, self.average = num_classes, average

    def _per_class(self, fn):
        p, t = self._all()
        p = p.reshape(-1, self.C)
        t = t.reshape(-1)
        return torch.stack([fn(p[:, c], (t == c)) for c in range(self.C)])

    def compute(self) -> Tensor:
        from .ranking import binary_auroc
        per = self._per_class(binary_auroc)
        return per.float() if self.average in ("none", None) else per.mean().float()


class MulticlassAveragePrecision(MulticlassAUROC):
    def compute(self) -> Tensor:
        from .ranking import binary_average_precision
        per = self._per_class(binary_average_precision)
        return per.float() if self.average in ("none", None) else per.mean().float()


class MultilabelAUROC(MulticlassAUROC):
    def __init__(self, num_labels: int, average: Optional[str] = "macro", **kw) -> None:
        super().__init__(num_labels, average)

    def _per_class(self, fn):
        p, t = self._all()
        p, t = p.reshape(-1, self.C), t.reshape(-1, self.C)
        return torch.stack([fn(p[:, c], t[:, c]) for c in range(self.C)])


class MultilabelAveragePrecision(MultilabelAUROC):
    compute = MulticlassAveragePrecision.compute


class BinaryCalibrationError(_Scores):
    def __init__(self, n_bins: int = 15, **kw) -> None:
        super().__init__()
        self.n_bins = n_bins

    def compute(self) -> Tensor:
        from .ranking import expected_calibration_error
        p, t = self._all()
        p = p.reshape(-1).double()
        probs = torch.stack((1 - p, p), -1)
        return expected_calibration_error(probs, t.reshape(-1).long(), self.n_bins).float()


class MulticlassCalibrationError(_Scores):
    def __init__(self, num_classes: int, n_bins: int = 15, **kw) -> None:
        super().__init__()
        self.C, self.n_bins = num_classes, n_bins

    def compute(self) -> Tensor:
        from .ranking import expected_calibration_error
        p, t = self._all()
        p = p.reshape(-1, self.C)
        if p.min() < 0 or p.max() > 1:
            p = torch.softmax(p.float(), -1)
        return expected_calibration_error(p, t.reshape(-1), self.n_bins).float()


class BinaryHingeLoss(Metric):
    """Mean of ``max(0, 1 - y f)`` with ``y`` in {-1, +1} (``squared`` squares the margin violations)."""

    def __init__(self, squared: bool = False, **kw) -> None:
        super().__init__()
        self.squared = squared
        self.add_state("total", torch.zeros((), dtype=torch.float64))
        self.add_state("n", torch.zeros((), dtype=torch.float64))

    def update(self, preds: Tensor, target: Tensor) -> None:
        self._to(preds.device)
        y = target.reshape(-1).double() * 2 - 1
        m = (1 - y * preds.reshape(-1).double()).clamp(min=0)
        self.total += (m * m if self.squared else m).sum()
        self.n += m.numel()

    def compute(self) -> Tensor:
        return (self.total / self.n.clamp(min=1)).float()


class MulticlassHingeLoss(BinaryHingeLoss):
    """Crammer-Singer margin: ``max(0, 1 - f_y + max_{j != y} f_j)``."""

    def __init__(self, num_classes: int, squared: bool = False, **kw) -> None:
        super().__init__(squared)
        self.C = num_classes

    def update(self, preds: Tensor, target: Tensor) -> None:
        self._to(preds.device)
        p = preds.reshape(-1, self.C).double()
        t = target.reshape(-1)
        true = p.gather(1, t[:, None])[:, 0]
        other = p.masked_fill(torch.nn.functional.one_hot(t, self.C).bool(), float("-inf")).max(-1).values
        m = (1 - true + other).clamp(min=0)
        self.total += (m * m if self.squared else m).sum()
        self.n += m.numel()


class ExactMatch(Metric):
    """Fraction of samples whose every label (multilabel) or position (multidimensional multiclass) is right."""

    def __init__(self, threshold: float = 0.5, **kw) -> None:
        super().__init__()
        self.threshold = threshold
        self.add_state("hit", torch.zeros((), dtype=torch.float64))
        self.add_state("n", torch.zeros((), dtype=torch.float64))

    def update(self, preds: Tensor, target: Tensor) -> None:
        self._to(target.device)
        p = _binarize(preds, self.threshold) if preds.shape == target.shape else preds.argmax(1)
        ok = (p.reshape(p.shape[0], -1) == target.reshape(target.shape[0], -1)).all(-1)
        self.hit += ok.sum()
        self.n += ok.numel()

    def compute(self) -> Tensor:
        return (self.hit / self.n.clamp(min=1)).float()


__all__ = sorted(n for n in globals() if n[0].isupper() and n not in ("Metric", "Tensor", "Optional"))


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
