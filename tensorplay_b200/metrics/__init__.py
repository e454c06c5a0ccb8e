"""Streaming evaluation metrics with distributed synchronisation.

Each metric keeps its sufficient statistics as tensors on the device of its inputs, ``update``
adds a batch, ``compute`` returns the value and ``sync`` sums the statistics over a process group
first. Covers the core of the reference's ``tensorplay.metrics`` pack (classification,
regression, aggregation, text): tensorplay/metrics/__init__.py.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.distributed as dist
from torch import Tensor

__all__ = ["Metric", "MeanMetric", "SumMetric", "Accuracy", "Precision", "Recall", "F1Score",
           "ConfusionMatrix", "MeanSquaredError", "MeanAbsoluteError", "R2Score", "Perplexity",
           "MetricCollection", "PearsonCorrCoef", "SpearmanCorrCoef", "KendallRankCorrCoef", "AUROC",
           "AveragePrecision", "RetrievalNormalizedDCG", "RetrievalMRR", "CalibrationError", "functional"]


class Metric:
    """Base class: subclasses declare their state with :meth:`add_state`."""

    def __init__(self) -> None:
        self._defaults: Dict[str, Tensor] = {}

    def add_state(self, name: str, default: Tensor) -> None:
        self._defaults[name] = default.clone()
        setattr(self, name, default.clone())

    def reset(self) -> None:
        for k, v in self._defaults.items():
            setattr(self, k, v.clone().to(getattr(self, k).device))

    def _to(self, device) -> None:
        for k in self._defaults:
            setattr(self, k, getattr(self, k).to(device))

    def sync(self, group=None) -> None:
        """Sum every state over ``group`` (no-op outside a process group)."""
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            for k in self._defaults:
                t = getattr(self, k)
                dist.all_reduce(t, group=group)

    def update(self, *args, **kwargs) -> None:  # pragma: no cover - interface
        raise NotImplementedError

    def compute(self) -> Tensor:  # pragma: no cover - interface
        raise NotImplementedError

    def __call__(self, *args, **kwargs) -> Tensor:
        self.update(*args, **kwargs)
        return self.compute()


class SumMetric(Metric):
    def __init__(self) -> None:
        super().__init__()
        self.add_state("total", torch.zeros((), dtype=torch.float64))

    def update(self, value: Tensor) -> None:
        self._to(value.device)
        self.total += value.double().sum()

    def compute(self) -> Tensor:
        return self.total.float()


class MeanMetric(Metric):
    def __init__(self) -> None:
        super().__init__()
        self.add_state("total", torch.zeros((), dtype=torch.float64))
        self.add_state("weight", torch.zeros((), dtype=torch.float64))

    def update(self, value: Tensor, weight: Optional[Tensor] = None) -> None:
        self._to(value.device)
        w = torch.ones_like(value, dtype=torch.float64) if weight is None else weight.double().expand_as(value)
        self.total += (value.double() * w).sum()
        self.weight += w.sum()

    def compute(self) -> Tensor:
        return (self.total / self.weight.clamp(min=1e-12)).float()


def _labels(preds: Tensor, num_classes: int) -> Tensor:
    if preds.dim() >= 2 and preds.shape[-1] == num_classes and preds.is_floating_point():
        return preds.argmax(-1)
    if preds.is_floating_point():
        return (preds > 0.5).long()
    return preds


class ConfusionMatrix(Metric):
    """``matrix[t, p]`` counts samples of true class ``t`` predicted as ``p``."""

    def __init__(self, num_classes: int) -> None:
        super().__init__()
        self.num_classes = num_classes
        self.add_state("matrix", torch.zeros(num_classes, num_classes, dtype=torch.long))

    def update(self, preds: Tensor, target: Tensor) -> None:
        self._to(target.device)
        p = _labels(preds, self.num_classes).reshape(-1)
        t = target.reshape(-1)
        idx = t * self.num_classes + p
        self.matrix += torch.bincount(idx, minlength=self.num_classes ** 2).view(self.num_classes, self.num_classes)

    def compute(self) -> Tensor:
        return self.matrix


class _StatScores(ConfusionMatrix):
    def __init__(self, num_classes: int = 2, average: str = "micro") -> None:
        super().__init__(num_classes)
        if average not in ("micro", "macro", "none"):
            raise ValueError("average must be 'micro', 'macro' or 'none'")
        self.average = average

    def _tp_fp_fn(self):
        m = self.matrix.double()
        tp = m.diag()
        return tp, m.sum(0) - tp, m.sum(1) - tp

    def _reduce(self, num: Tensor, den: Tensor) -> Tensor:
        if self.average == "micro":
            return (num.sum() / den.sum().clamp(min=1e-12)).float()
        per = num / den.clamp(min=1e-12)
        return per.float() if self.average == "none" else per.mean().float()


class Accuracy(_StatScores):
    def compute(self) -> Tensor:
        m = self.matrix.double()
        if self.average == "micro":
            return (m.diag().sum() / m.sum().clamp(min=1e-12)).float()
        return self._reduce(m.diag(), m.sum(1))


class Precision(_StatScores):
    def compute(self) -> Tensor:
        tp, fp, _ = self._tp_fp_fn()
        return self._reduce(tp, tp + fp)


class Recall(_StatScores):
    def compute(self) -> Tensor:
        tp, _, fn = self._tp_fp_fn()
        return self._reduce(tp, tp + fn)


class F1Score(_StatScores):
    def compute(self) -> Tensor:
        tp, fp, fn = self._tp_fp_fn()
        return self._reduce(2 * tp, 2 * tp + fp + fn)


def _native_diff_sum(preds: Tensor, target: Tensor, kind: str):
    """Sum of squared / absolute differences by the host runtime's one-pass reduction for float32 CPU
    inputs, or ``None`` when the inputs do not qualify (other device, dtype or layout)."""
    if (preds.device.type != "cpu" or preds.dtype != torch.float32 or target.dtype != torch.float32
            or preds.shape != target.shape or not preds.is_contiguous() or not target.is_contiguous()):
        return None
    try:
        import ctypes as C

        from .. import _native
        rt = _native.runtime()
        fn = rt.tpb_sum_sq_diff_f32 if kind == "sq" else rt.tpb_sum_abs_diff_f32
        if fn.restype is not C.c_double:
            fn.restype = C.c_double
            fn.argtypes = [C.c_void_p, C.c_void_p, C.c_longlong]
        return fn(preds.data_ptr(), target.data_ptr(), preds.numel())
    except (OSError, AttributeError):
        return None


class MeanSquaredError(Metric):
    def __init__(self, squared: bool = True) -> None:
        super().__init__()
        self.squared = squared
        self.add_state("sse", torch.zeros((), dtype=torch.float64))
        self.add_state("n", torch.zeros((), dtype=torch.float64))

    def update(self, preds: Tensor, target: Tensor) -> None:
        self._to(preds.device)
        # one pass in the input precision; the running sum is kept in double
        v = _native_diff_sum(preds, target, "sq")
        if v is None:
            v = torch.nn.functional.mse_loss(preds.float(), target.float(), reduction="sum").double()
        self.sse += v
        self.n += preds.numel()

    def compute(self) -> Tensor:
        mse = self.sse / self.n.clamp(min=1)
        return (mse if self.squared else mse.sqrt()).float()


class MeanAbsoluteError(Metric):
    def __init__(self) -> None:
        super().__init__()
        self.add_state("sae", torch.zeros((), dtype=torch.float64))
        self.add_state("n", torch.zeros((), dtype=torch.float64))

    def update(self, preds: Tensor, target: Tensor) -> None:
        self._to(preds.device)
        v = _native_diff_sum(preds, target, "abs")
        if v is None:
            v = torch.nn.functional.l1_loss(preds.float(), target.float(), reduction="sum").double()
        self.sae += v
        self.n += preds.numel()

    def compute(self) -> Tensor:
        return (self.sae / self.n.clamp(min=1)).float()


class R2Score(Metric):
    def __init__(self) -> None:
        super().__init__()
        for s in ("sy", "syy", "sres", "n"):
            self.add_state(s, torch.zeros((), dtype=torch.float64))

    def update(self, preds: Tensor, target: Tensor) -> None:
        self._to(preds.device)
        t = target.double()
        self.sy += t.sum()
        self.syy += (t * t).sum()
        self.sres += ((t - preds.double()) ** 2).sum()
        self.n += t.numel()

    def compute(self) -> Tensor:
        tot = self.syy - self.sy * self.sy / self.n.clamp(min=1)
        return (1 - self.sres / tot.clamp(min=1e-12)).float()


class Perplexity(Metric):
    """``exp`` of the mean token negative log-likelihood; ``ignore_index`` tokens are skipped."""

    def __init__(self, ignore_index: Optional[int] = -100) -> None:
        super().__init__()
        self.ignore_index = ignore_index
        self.add_state("nll", torch.zeros((), dtype=torch.float64))
        self.add_state("n", torch.zeros((), dtype=torch.float64))

    def update(self, logits: Tensor, target: Tensor) -> None:
        self._to(logits.device)
        lp = torch.log_softmax(logits.float().reshape(-1, logits.shape[-1]), dim=-1)
        t = target.reshape(-1)
        keep = torch.ones_like(t, dtype=torch.bool) if self.ignore_index is None else t != self.ignore_index
        picked = lp.gather(1, t.clamp(min=0).unsqueeze(1)).squeeze(1)
        self.nll -= (picked * keep).double().sum()
        self.n += keep.sum()

    def compute(self) -> Tensor:
        return torch.exp(self.nll / self.n.clamp(min=1)).float()


class MetricCollection:
    """Dictionary of metrics updated with the same arguments."""

    def __init__(self, metrics: Dict[str, Metric]) -> None:
        self.metrics = dict(metrics)

    def update(self, *args, **kwargs) -> None:
        for m in self.metrics.values():
            m.update(*args, **kwargs)

    def compute(self) -> Dict[str, Tensor]:
        return {k: m.compute() for k, m in self.metrics.items()}

    def sync(self, group=None) -> None:
        for m in self.metrics.values():
            m.sync(group)

    def reset(self) -> None:
        for m in self.metrics.values():
            m.reset()


from .ranking import (AUROC, AveragePrecision, CalibrationError, KendallRankCorrCoef, PearsonCorrCoef,  # noqa: E402
                      RetrievalMRR, RetrievalNormalizedDCG, SpearmanCorrCoef)

from . import classification  # noqa: E402
from .classification import *  # noqa: E402,F401,F403
from . import regression  # noqa: E402
from .regression import *  # noqa: E402,F401,F403
from . import domains  # noqa: E402
from .domains import *  # noqa: E402,F401,F403
from . import more  # noqa: E402
from .more import *  # noqa: E402,F401,F403
from . import generative, panoptic, text_more  # noqa: E402
from .generative import *  # noqa: E402,F401,F403
from .panoptic import *  # noqa: E402,F401,F403
from .text_more import *  # noqa: E402,F401,F403
from . import functional, utilities  # noqa: E402


def _domain_views() -> None:
    """``metrics.text``, ``metrics.image`` ... resolve the same classes as the package itself: the
    classes live in a few files by kind of state, the domain names are views for imports."""
    import sys
    import types
    pkg = sys.modules[__name__]
    for name in ("wrappers", "image", "text", "audio", "retrieval", "nominal", "detection", "multimodal", "aggregation",
                 "collections"):
        if name in pkg.__dict__:
            continue
        mod = types.ModuleType(f"{__name__}.{name}", f"View of {__name__} for the {name} metrics.")
        mod.__getattr__ = lambda attr, _pkg=pkg: getattr(_pkg, attr)
        mod.__path__ = []   # deeper module names (metrics.text.bleu ...) resolve through the view finder
        sys.modules[mod.__name__] = mod
        setattr(pkg, name, mod)


_domain_views()

from .. import _views as _view_finder  # noqa: E402

_view_finder.install(__name__, max_depth=2)
