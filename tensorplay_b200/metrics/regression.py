"""Further regression, divergence and aggregation metrics, and the metric wrappers."""
from __future__ import annotations

import copy
from typing import Dict, List, Optional, Sequence

import torch
from torch import Tensor

from . import Metric


class _SumOver(Metric):
    """Metrics of the form ``finish(sum_i f(pred_i, target_i), n)``."""

    def __init__(self, **kw) -> None:
        super().__init__()
        self.add_state("total", torch.zeros((), dtype=torch.float64))
        self.add_state("n", torch.zeros((), dtype=torch.float64))

    def _term(self, p: Tensor, t: Tensor) -> Tensor:
        raise NotImplementedError

    def _count(self, p: Tensor) -> int:
        return p.numel()

    def update(self, preds: Tensor, target: Tensor) -> None:
        self._to(preds.device)
        self.total += self._term(preds.double(), target.double()).sum()
        self.n += self._count(preds)

    def compute(self) -> Tensor:
        return (self.total / self.n.clamp(min=1)).float()


class LogCoshError(_SumOver):
    def _term(self, p, t):
        d = p - t
        return d + torch.nn.functional.softplus(-2 * d) - 0.6931471805599453


class MeanAbsolutePercentageError(_SumOver):
    def _term(self, p, t):
        return (p - t).abs() / t.abs().clamp(min=1.17e-06)


class SymmetricMeanAbsolutePercentageError(_SumOver):
    def _term(self, p, t):
        return 2 * (p - t).abs() / (p.abs() + t.abs()).clamp(min=1.17e-06)


class MeanSquaredLogError(_SumOver):
    def _term(self, p, t):
        return (torch.log1p(p) - torch.log1p(t)) ** 2


class WeightedMeanAbsolutePercentageError(Metric):
    def __init__(self, **kw) -> None:
        super().__init__()
        self.add_state("err", torch.zeros((), dtype=torch.float64))
        self.add_state("den", torch.zeros((), dtype=torch.float64))

    def update(self, preds, target) -> None:
        self._to(preds.device)
        self.err += (preds.double() - target.double()).abs().sum()
        self.den += target.double().abs().sum()

    def compute(self) -> Tensor:
        return (self.err / self.den.clamp(min=1.17e-06)).float()


class MinkowskiDistance(Metric):
    def __init__(self, p: float = 2.0, **kw) -> None:
        super().__init__()
        self.p = p
        self.add_state("total", torch.zeros((), dtype=torch.float64))

    def update(self, preds, target) -> None:
        self._to(preds.device)
        self.total += (preds.double() - target.double()).abs().pow(self.p).sum()

    def compute(self) -> Tensor:
        return self.total.pow(1.0 / self.p).float()


class CosineSimilarity(_SumOver):
    """Mean cosine similarity of the rows."""

    def _term(self, p, t):
        return torch.nn.functional.cosine_similarity(p.reshape(-1, p.shape[-1]), t.reshape(-1, t.shape[-1]), dim=-1)

    def _count(self, p):
        return p.numel() // p.shape[-1]


class KLDivergence(_SumOver):
    """Mean ``KL(p || q)`` of rows of probabilities (``log_prob=True``: rows of log-probabilities)."""

    def __init__(self, log_prob: bool = False, **kw) -> None:
        super().__init__()
        self.log_prob = log_prob

    def _term(self, p, q):
        if self.log_prob:
            return (p.exp() * (p - q)).sum(-1)
        p, q = p / p.sum(-1, keepdim=True), q / q.sum(-1, keepdim=True)
        return (p * (torch.log(p.clamp(min=1e-300)) - torch.log(q.clamp(min=1e-300)))).sum(-1)

    def _count(self, p):
        return p.numel() // p.shape[-1]


class JensenShannonDivergence(KLDivergence):
    def _term(self, p, q):
        if self.log_prob:
            p, q = p.exp(), q.exp()
        p, q = p / p.sum(-1, keepdim=True), q / q.sum(-1, keepdim=True)
        m = 0.5 * (p + q)
        kl = lambda a, b: (a * (torch.log(a.clamp(min=1e-300)) - torch.log(b.clamp(min=1e-300)))).sum(-1)   # noqa: E731
        return 0.5 * kl(p, m) + 0.5 * kl(q, m)


class _Moments(Metric):
    """Sums needed for variance / covariance statistics of (pred, target) pairs."""

    def __init__(self, **kw) -> None:
        super().__init__()
        for n in ("n", "sp", "st", "spp", "stt", "spt", "sres"):
            self.add_state(n, torch.zeros((), dtype=torch.float64))

    def update(self, preds, target) -> None:
        self._to(preds.device)
        p, t = preds.double().reshape(-1), target.double().reshape(-1)
        self.n += p.numel()
        self.sp += p.sum()
        self.st += t.sum()
        self.spp += (p * p).sum()
        self.stt += (t * t).sum()
        self.spt += (p * t).sum()
        self.sres += ((t - p) ** 2).sum()

    def _var(self, s, ss):
        return ss / self.n - (s / self.n) ** 2


class ExplainedVariance(_Moments):
    def compute(self) -> Tensor:
        d_mean = (self.st - self.sp) / self.n
        var_res = self.sres / self.n - d_mean ** 2
        return (1 - var_res / self._var(self.st, self.stt).clamp(min=1e-300)).float()


class ConcordanceCorrCoef(_Moments):
    def compute(self) -> Tensor:
        mp, mt = self.sp / self.n, self.st / self.n
        cov = self.spt / self.n - mp * mt
        return (2 * cov / (self._var(self.sp, self.spp) + self._var(self.st, self.stt) + (mp - mt) ** 2).clamp(min=1e-300)).float()


class RelativeSquaredError(_Moments):
    def compute(self) -> Tensor:
        return (self.sres / (self.stt - self.st ** 2 / self.n).clamp(min=1e-300)).float()


class NormalizedRootMeanSquaredError(_Moments):
    """RMSE divided by the mean (default), the range is not tracked: ``normalization`` in {"mean", "std"}."""

    def __init__(self, normalization: str = "mean", **kw) -> None:
        super().__init__()
        self.normalization = normalization

    def compute(self) -> Tensor:
        rmse = (self.sres / self.n).sqrt()
        den = (self.st / self.n).abs() if self.normalization == "mean" else self._var(self.st, self.stt).sqrt()
        return (rmse / den.clamp(min=1e-300)).float()


class TweedieDevianceScore(_SumOver):
    def __init__(self, power: float = 0.0, **kw) -> None:
        super().__init__()
        self.power = power

    def _term(self, p, t):
        a = self.power
        if a == 0:
            return (t - p) ** 2
        if a == 1:
            return 2 * (torch.xlogy(t, t / p) + p - t)
        if a == 2:
            return 2 * (torch.log(p / t) + t / p - 1)
        return 2 * (t.clamp(min=0).pow(2 - a) / ((1 - a) * (2 - a)) - t * p.pow(1 - a) / (1 - a) + p.pow(2 - a) / (2 - a))


# ----------------------------------------------------------------------------- aggregation
class MaxMetric(Metric):
    def __init__(self, **kw) -> None:
        super().__init__()
        self.add_state("value", torch.tensor(float("-inf"), dtype=torch.float64))

    def update(self, x) -> None:
        self._to(x.device if isinstance(x, Tensor) else "cpu")
        self.value = torch.maximum(self.value, torch.as_tensor(x, dtype=torch.float64).max())

    def sync(self, group=None) -> None:
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(self.value, op=dist.ReduceOp.MAX, group=group)

    def compute(self) -> Tensor:
        return self.value.float()


class MinMetric(MaxMetric):
    def __init__(self, **kw) -> None:
        Metric.__init__(self)
        self.add_state("value", torch.tensor(float("inf"), dtype=torch.float64))

    def update(self, x) -> None:
        self.value = torch.minimum(self.value, torch.as_tensor(x, dtype=torch.float64).min())

    def sync(self, group=None) -> None:
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(self.value, op=dist.ReduceOp.MIN, group=group)


class CatMetric(Metric):
    def __init__(self, **kw) -> None:
        super().__init__()
        self.values: List[Tensor] = []

    def reset(self) -> None:
        self.values = []

    def update(self, x) -> None:
        self.values.append(torch.as_tensor(x).detach().reshape(-1))

    def compute(self) -> Tensor:
        return torch.cat(self.values) if self.values else torch.zeros(0)


class Running(Metric):
    """The wrapped metric over the last ``window`` updates only."""

    def __init__(self, base: Metric, window: int = 5) -> None:
        super().__init__()
        self.base, self.window = base, window
        self.buffer: List[tuple] = []

    def reset(self) -> None:
        self.buffer = []

    def update(self, *args) -> None:
        self.buffer = (self.buffer + [args])[-self.window:]

    def compute(self):
        m = copy.deepcopy(self.base)
        m.reset()
        for a in self.buffer:
            m.update(*a)
        return m.compute()


class RunningMean(Running):
    def __init__(self, window: int = 5) -> None:
        from . import MeanMetric
        super().__init__(MeanMetric(), window)


class RunningSum(Running):
    def __init__(self, window: int = 5) -> None:
        from . import SumMetric
        super().__init__(SumMetric(), window)


class MinMaxMetric(Metric):
    """Tracks the smallest and the largest value the wrapped metric has computed."""

    def __init__(self, base: Metric) -> None:
        super().__init__()
        self.base = base
        self.lo, self.hi = float("inf"), float("-inf")

    def update(self, *a, **k) -> None:
        self.base.update(*a, **k)

    def compute(self) -> Dict[str, Tensor]:
        v = self.base.compute()
        self.lo, self.hi = min(self.lo, float(v)), max(self.hi, float(v))
        return {"raw": v, "min": torch.tensor(self.lo), "max": torch.tensor(self.hi)}

    def reset(self) -> None:
        self.base.reset()


class MetricTracker:
    """History of a metric over epochs: ``increment()`` starts a fresh copy, ``best_metric()`` picks the best."""

    def __init__(self, metric: Metric, maximize: bool = True) -> None:
        self.proto, self.maximize = metric, maximize
        self.steps: List[Metric] = []

    def increment(self) -> None:
        m = copy.deepcopy(self.proto)
        m.reset()
        self.steps.append(m)

    def update(self, *a, **k) -> None:
        self.steps[-1].update(*a, **k)

    def compute(self):
        return self.steps[-1].compute()

    def compute_all(self) -> Tensor:
        return torch.stack([torch.as_tensor(m.compute()).float() for m in self.steps])

    def best_metric(self, return_step: bool = False):
        allv = self.compute_all()
        idx = int(allv.argmax() if self.maximize else allv.argmin())
        return (float(allv[idx]), idx) if return_step else float(allv[idx])


class ClasswiseWrapper(Metric):
    """Turns a per-class result vector into a dictionary ``{prefix + label: value}``."""

    def __init__(self, metric: Metric, labels: Optional[Sequence[str]] = None, prefix: Optional[str] = None) -> None:
        super().__init__()
        self.metric, self.labels = metric, labels
        self.prefix = prefix if prefix is not None else type(metric).__name__.lower() + "_"

    def update(self, *a, **k) -> None:
        self.metric.update(*a, **k)

    def compute(self) -> Dict[str, Tensor]:
        v = self.metric.compute()
        names = self.labels or [str(i) for i in range(len(v))]
        return {self.prefix + n: x for n, x in zip(names, v)}

    def reset(self) -> None:
        self.metric.reset()

    def sync(self, group=None) -> None:
        self.metric.sync(group)


class MultioutputWrapper(Metric):
    """One copy of the metric per output column (last dimension)."""

    def __init__(self, metric: Metric, num_outputs: int) -> None:
        super().__init__()
        self.metrics = [copy.deepcopy(metric) for _ in range(num_outputs)]

    def update(self, preds, target) -> None:
        for i, m in enumerate(self.metrics):
            m.update(preds[..., i], target[..., i])

    def compute(self) -> Tensor:
        return torch.stack([torch.as_tensor(m.compute()).float() for m in self.metrics])

    def reset(self) -> None:
        for m in self.metrics:
            m.reset()

    def sync(self, group=None) -> None:
        for m in self.metrics:
            m.sync(group)


class BootStrapper(Metric):
    """Bootstrap estimate of a metric's mean and standard deviation: every copy sees a Poisson(1)
    resampling of each batch."""

    def __init__(self, metric: Metric, num_bootstraps: int = 10, generator=None) -> None:
        super().__init__()
        self.metrics = [copy.deepcopy(metric) for _ in range(num_bootstraps)]
        self.generator = generator

    def update(self, *args) -> None:
        n = args[0].shape[0]
        for m in self.metrics:
            idx = torch.multinomial(torch.ones(n), n, replacement=True, generator=self.generator)
            m.update(*[a[idx] for a in args])

    def compute(self) -> Dict[str, Tensor]:
        v = torch.stack([torch.as_tensor(m.compute()).float() for m in self.metrics])
        return {"mean": v.mean(0), "std": v.std(0)}

    def reset(self) -> None:
        for m in self.metrics:
            m.reset()


class CompositionalMetric(Metric):
    """``op(a, b)`` of two metrics (or a metric and a constant), updated together."""

    def __init__(self, op, a, b=None) -> None:
        super().__init__()
        self.op, self.a, self.b = op, a, b

    def update(self, *args, **kw) -> None:
        for m in (self.a, self.b):
            if isinstance(m, Metric):
                m.update(*args, **kw)

    def compute(self):
        va = self.a.compute() if isinstance(self.a, Metric) else self.a
        vb = self.b.compute() if isinstance(self.b, Metric) else self.b
        return self.op(va) if vb is None else self.op(va, vb)

    def reset(self) -> None:
        for m in (self.a, self.b):
            if isinstance(m, Metric):
                m.reset()


__all__ = sorted(n for n in globals() if n[0].isupper() and n not in ("Metric", "Tensor", "Optional", "Dict", "List", "Sequence"))


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
