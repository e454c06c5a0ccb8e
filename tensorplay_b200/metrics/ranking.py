"""Correlation, ranking and retrieval metrics (functional forms and streaming classes): Pearson,
Spearman, Kendall tau-b, AUROC, average precision, NDCG, MRR, top-k accuracy, calibration error.
(The reference's ``tensorplay/metrics`` families ``regression``, ``classification`` and ``retrieval``.)"""
from __future__ import annotations

import torch
from torch import Tensor

from . import Metric


def _rank(x: Tensor) -> Tensor:
    """Average ranks (1-based) with ties sharing the mean of their positions."""
    x = x.reshape(-1).double()
    order = torch.argsort(x)
    ranks = torch.empty_like(x)
    ranks[order] = torch.arange(1, x.numel() + 1, dtype=torch.float64, device=x.device)
    _, inv, counts = torch.unique(x, return_inverse=True, return_counts=True)
    sums = torch.zeros_like(counts, dtype=torch.float64).scatter_add_(0, inv, ranks)
    return (sums / counts)[inv]


def pearson_corrcoef(x: Tensor, y: Tensor) -> Tensor:
    x, y = x.reshape(-1).double(), y.reshape(-1).double()
    xm, ym = x - x.mean(), y - y.mean()
    return (xm * ym).sum() / (xm.norm() * ym.norm()).clamp(min=1e-300)


def spearman_corrcoef(x: Tensor, y: Tensor) -> Tensor:
    return pearson_corrcoef(_rank(x), _rank(y))


def kendall_tau(x: Tensor, y: Tensor, variant: str = "b") -> Tensor:
    """Kendall rank correlation; tau-b corrects for ties. All pairs at once (an ``n x n`` sign
    product on the tensor's device), which is what makes it fast for the sizes metrics see."""
    x, y = x.reshape(-1).double(), y.reshape(-1).double()
    n = x.numel()
    sx = torch.sign(x[:, None] - x[None, :])
    sy = torch.sign(y[:, None] - y[None, :])
    iu = torch.triu_indices(n, n, offset=1, device=x.device)
    px, py = sx[iu[0], iu[1]], sy[iu[0], iu[1]]
    s = (px * py).sum()
    n0 = n * (n - 1) / 2
    if variant == "a":
        return s / n0
    tx, ty = (px == 0).sum(), (py == 0).sum()
    return s / torch.sqrt(((n0 - tx) * (n0 - ty)).clamp(min=1e-300))


def binary_auroc(scores: Tensor, target: Tensor) -> Tensor:
    """Area under the ROC curve = probability that a positive outranks a negative (ties count half)."""
    r = _rank(scores)
    t = target.reshape(-1).bool()
    n_pos, n_neg = t.sum().double(), (~t).sum().double()
    return (r[t].sum() - n_pos * (n_pos + 1) / 2) / (n_pos * n_neg).clamp(min=1)


def binary_average_precision(scores: Tensor, target: Tensor) -> Tensor:
    order = torch.argsort(scores.reshape(-1), descending=True)
    t = target.reshape(-1)[order].double()
    hits = torch.cumsum(t, 0)
    prec = hits / torch.arange(1, t.numel() + 1, dtype=torch.float64, device=t.device)
    return (prec * t).sum() / t.sum().clamp(min=1)


def topk_accuracy(logits: Tensor, target: Tensor, k: int = 5) -> Tensor:
    top = logits.topk(k, dim=-1).indices
    return (top == target.unsqueeze(-1)).any(-1).double().mean()


def dcg(rel: Tensor, k: int = None) -> Tensor:
    rel = rel.double()[..., :k] if k else rel.double()
    disc = 1.0 / torch.log2(torch.arange(2, rel.shape[-1] + 2, dtype=torch.float64, device=rel.device))
    return (rel * disc).sum(-1)


def ndcg(scores: Tensor, relevance: Tensor, k: int = None) -> Tensor:
    """Mean NDCG@k over queries; ``scores`` and ``relevance`` are ``[queries, docs]``."""
    order = torch.argsort(scores, dim=-1, descending=True)
    got = dcg(torch.gather(relevance, -1, order), k)
    ideal = dcg(torch.sort(relevance, dim=-1, descending=True).values, k)
    return (got / ideal.clamp(min=1e-12)).mean()


def mean_reciprocal_rank(scores: Tensor, relevant: Tensor) -> Tensor:
    """``relevant``: boolean ``[queries, docs]``; rank of the first relevant document per query."""
    order = torch.argsort(scores, dim=-1, descending=True)
    rel = torch.gather(relevant.bool(), -1, order)
    first = torch.where(rel.any(-1), rel.double().argmax(-1) + 1, torch.zeros((), dtype=torch.long, device=rel.device))
    return torch.where(first > 0, 1.0 / first.double().clamp(min=1), torch.zeros((), dtype=torch.float64,
                                                                                device=rel.device)).mean()


def expected_calibration_error(probs: Tensor, target: Tensor, bins: int = 15) -> Tensor:
    """Top-label ECE: sum over confidence bins of ``|accuracy - confidence| * share``."""
    conf, pred = probs.max(-1)
    correct = (pred == target).double()
    edges = torch.linspace(0, 1, bins + 1, device=probs.device)
    idx = torch.bucketize(conf.double(), edges.double()[1:-1])
    ece = torch.zeros((), dtype=torch.float64, device=probs.device)
    for b in range(bins):
        m = idx == b
        if m.any():
            ece = ece + m.double().mean() * (correct[m].mean() - conf[m].double().mean()).abs()
    return ece


class _Collecting(Metric):
    """Streaming wrapper for metrics that need all samples: updates are concatenated; ``sync``
    gathers the samples of every rank."""

    fn = None

    def __init__(self, **kw):
        super().__init__()
        self.kw = kw
        self.a, self.b = [], []

    def reset(self) -> None:
        self.a, self.b = [], []

    def update(self, a: Tensor, b: Tensor) -> None:
        self.a.append(a.detach())
        self.b.append(b.detach())

    def sync(self, group=None) -> None:
        """Gather every rank's samples (rank order), so that ``compute`` sees the whole set."""
        import torch.distributed as dist
        if not (dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1) or not self.a:
            return
        for name in ("a", "b"):
            t = torch.cat(getattr(self, name))
            parts = [None] * dist.get_world_size(group)
            dist.all_gather_object(parts, t.cpu(), group=group)
            setattr(self, name, [torch.cat(parts).to(t.device)])

    def compute(self) -> Tensor:
        return type(self).fn(torch.cat(self.a), torch.cat(self.b), **self.kw)


class PearsonCorrCoef(_Collecting):
    fn = staticmethod(pearson_corrcoef)


class SpearmanCorrCoef(_Collecting):
    fn = staticmethod(spearman_corrcoef)


class KendallRankCorrCoef(_Collecting):
    fn = staticmethod(kendall_tau)


class AUROC(_Collecting):
    fn = staticmethod(binary_auroc)


class AveragePrecision(_Collecting):
    fn = staticmethod(binary_average_precision)


class RetrievalNormalizedDCG(_Collecting):
    fn = staticmethod(ndcg)


class RetrievalMRR(_Collecting):
    fn = staticmethod(mean_reciprocal_rank)


class CalibrationError(_Collecting):
    fn = staticmethod(expected_calibration_error)


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
