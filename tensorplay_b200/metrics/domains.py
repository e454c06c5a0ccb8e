"""Text, audio, image and retrieval metrics (the reference's ``metrics`` families ``text``, ``audio``,
``image`` and ``retrieval``)."""
from __future__ import annotations

import math
from collections import Counter
from typing import List, Optional, Sequence, Union

import torch
from torch import Tensor

from . import Metric


# ----------------------------------------------------------------------------- text
def edit_distance(a: Sequence, b: Sequence) -> int:
    """Levenshtein distance between two sequences (tokens or characters)."""
    prev = list(range(len(b) + 1))
    for i, x in enumerate(a, 1):
        cur = [i] + [0] * len(b)
        for j, y in enumerate(b, 1):
            cur[j] = min(prev[j] + 1, cur[j - 1] + 1, prev[j - 1] + (x != y))
        prev = cur
    return prev[-1]


def _as_list(x) -> List[str]:
    return [x] if isinstance(x, str) else list(x)


class _ErrorRate(Metric):
    unit = "word"

    def __init__(self, **kw) -> None:
        super().__init__()
        for n in ("errors", "total", "hits", "pred_total"):
            self.add_state(n, torch.zeros((), dtype=torch.float64))

    def _tok(self, s: str):
        return s.split() if self.unit == "word" else list(s)

    def update(self, preds, target) -> None:
        for p, t in zip(_as_list(preds), _as_list(target)):
            pt, tt = self._tok(p), self._tok(t)
            d = edit_distance(pt, tt)
            self.errors += d
            self.total += len(tt)
            self.pred_total += len(pt)
            # hits of the alignment: positions that are neither substituted, deleted nor inserted
            self.hits += max(len(tt), len(pt)) - d

    def compute(self) -> Tensor:
        return (self.errors / self.total.clamp(min=1)).float()


class WordErrorRate(_ErrorRate):
    unit = "word"


class CharErrorRate(_ErrorRate):
    unit = "char"


class MatchErrorRate(_ErrorRate):
    def compute(self) -> Tensor:
        return (self.errors / (self.errors + self.hits).clamp(min=1)).float()


class WordInfoPreserved(_ErrorRate):
    def compute(self) -> Tensor:
        return ((self.hits / self.total.clamp(min=1)) * (self.hits / self.pred_total.clamp(min=1))).float()


class WordInfoLost(WordInfoPreserved):
    def compute(self) -> Tensor:
        return 1 - super().compute()


class EditDistance(Metric):
    def __init__(self, reduction: str = "mean", **kw) -> None:
        super().__init__()
        self.reduction = reduction
        self.add_state("total", torch.zeros((), dtype=torch.float64))
        self.add_state("n", torch.zeros((), dtype=torch.float64))

    def update(self, preds, target) -> None:
        for p, t in zip(_as_list(preds), _as_list(target)):
            self.total += edit_distance(p, t)
            self.n += 1

    def compute(self) -> Tensor:
        return (self.total if self.reduction == "sum" else self.total / self.n.clamp(min=1)).float()


def _ngrams(tokens: Sequence[str], n: int) -> Counter:
    return Counter(tuple(tokens[i: i + n]) for i in range(len(tokens) - n + 1))


class BLEUScore(Metric):
    """Corpus BLEU with uniform n-gram weights and the brevity penalty (``smooth``: add-one on n > 1)."""

    def __init__(self, n_gram: int = 4, smooth: bool = False, **kw) -> None:
        super().__init__()
        self.n_gram, self.smooth = n_gram, smooth
        self.add_state("match", torch.zeros(n_gram, dtype=torch.float64))
        self.add_state("count", torch.zeros(n_gram, dtype=torch.float64))
        self.add_state("pred_len", torch.zeros((), dtype=torch.float64))
        self.add_state("ref_len", torch.zeros((), dtype=torch.float64))

    def update(self, preds: Sequence[str], target: Sequence[Sequence[str]]) -> None:
        for p, refs in zip(_as_list(preds), target):
            pt = p.split()
            rts = [r.split() for r in _as_list(refs)]
            self.pred_len += len(pt)
            self.ref_len += min((abs(len(r) - len(pt)), len(r)) for r in rts)[1]
            for n in range(1, self.n_gram + 1):
                pc = _ngrams(pt, n)
                best = Counter()
                for r in rts:
                    for g, c in _ngrams(r, n).items():
                        best[g] = max(best[g], c)
                self.match[n - 1] += sum(min(c, best[g]) for g, c in pc.items())
                self.count[n - 1] += max(0, len(pt) - n + 1)

    def compute(self) -> Tensor:
        if self.count.min() == 0 or self.match[0] == 0:
            return torch.zeros(())
        if self.smooth:
            prec = torch.cat((self.match[:1] / self.count[:1], (self.match[1:] + 1) / (self.count[1:] + 1)))
        else:
            prec = self.match / self.count
        if prec.min() == 0:
            return torch.zeros(())
        bp = 1.0 if self.pred_len > self.ref_len else math.exp(1 - float(self.ref_len) / float(self.pred_len))
        return (bp * torch.exp(torch.log(prec).mean())).float()


def _lcs(a: Sequence, b: Sequence) -> int:
    prev = [0] * (len(b) + 1)
    for x in a:
        cur = [0]
        for j, y in enumerate(b, 1):
            cur.append(prev[j - 1] + 1 if x == y else max(prev[j], cur[j - 1]))
        prev = cur
    return prev[-1]


class ROUGEScore(Metric):
    """Mean F-measures of ROUGE-1, ROUGE-2 (n-gram overlap) and ROUGE-L (longest common subsequence)."""

    def __init__(self, **kw) -> None:
        super().__init__()
        self.scores = {"rouge1_fmeasure": [], "rouge2_fmeasure": [], "rougeL_fmeasure": []}

    def reset(self) -> None:
        for v in self.scores.values():
            v.clear()

    @staticmethod
    def _f(match: float, n_pred: int, n_ref: int) -> float:
        if match == 0 or n_pred == 0 or n_ref == 0:
            return 0.0
        p, r = match / n_pred, match / n_ref
        return 2 * p * r / (p + r)

    def update(self, preds, target) -> None:
        for p, t in zip(_as_list(preds), _as_list(target)):
            pt, tt = p.lower().split(), t.lower().split()
            for n in (1, 2):
                pc, tc = _ngrams(pt, n), _ngrams(tt, n)
                m = sum(min(c, tc[g]) for g, c in pc.items())
                self.scores[f"rouge{n}_fmeasure"].append(self._f(m, sum(pc.values()), sum(tc.values())))
            self.scores["rougeL_fmeasure"].append(self._f(_lcs(pt, tt), len(pt), len(tt)))

    def compute(self):
        return {k: torch.tensor(sum(v) / max(1, len(v))) for k, v in self.scores.items()}


# ----------------------------------------------------------------------------- audio
def _snr_db(num: Tensor, den: Tensor) -> Tensor:
    return 10 * torch.log10(num.clamp(min=1e-30) / den.clamp(min=1e-30))


class _MeanOverSignals(Metric):
    def __init__(self, **kw) -> None:
        super().__init__()
        self.add_state("total", torch.zeros((), dtype=torch.float64))
        self.add_state("n", torch.zeros((), dtype=torch.float64))

    def _value(self, p: Tensor, t: Tensor) -> Tensor:
        raise NotImplementedError

    def update(self, preds: Tensor, target: Tensor) -> None:
        self._to(preds.device)
        v = self._value(preds.double().reshape(-1, preds.shape[-1]), target.double().reshape(-1, target.shape[-1]))
        self.total += v.sum()
        self.n += v.numel()

    def compute(self) -> Tensor:
        return (self.total / self.n.clamp(min=1)).float()


class SignalNoiseRatio(_MeanOverSignals):
    def __init__(self, zero_mean: bool = False, **kw) -> None:
        super().__init__()
        self.zero_mean = zero_mean

    def _value(self, p, t):
        if self.zero_mean:
            p, t = p - p.mean(-1, keepdim=True), t - t.mean(-1, keepdim=True)
        return _snr_db((t * t).sum(-1), ((t - p) ** 2).sum(-1))


class ScaleInvariantSignalDistortionRatio(_MeanOverSignals):
    def __init__(self, zero_mean: bool = False, **kw) -> None:
        super().__init__()
        self.zero_mean = zero_mean

    def _value(self, p, t):
        if self.zero_mean:
            p, t = p - p.mean(-1, keepdim=True), t - t.mean(-1, keepdim=True)
        alpha = (p * t).sum(-1, keepdim=True) / (t * t).sum(-1, keepdim=True).clamp(min=1e-30)
        proj = alpha * t
        return _snr_db((proj * proj).sum(-1), ((proj - p) ** 2).sum(-1))


class ScaleInvariantSignalNoiseRatio(ScaleInvariantSignalDistortionRatio):
    def __init__(self, **kw) -> None:
        super().__init__(zero_mean=True)


# ----------------------------------------------------------------------------- image
class PeakSignalNoiseRatio(Metric):
    def __init__(self, data_range: Optional[float] = None, **kw) -> None:
        super().__init__()
        self.data_range = data_range
        self.add_state("sse", torch.zeros((), dtype=torch.float64))
        self.add_state("n", torch.zeros((), dtype=torch.float64))
        self.add_state("lo", torch.tensor(float("inf"), dtype=torch.float64))
        self.add_state("hi", torch.tensor(float("-inf"), dtype=torch.float64))

    def update(self, preds: Tensor, target: Tensor) -> None:
        self._to(preds.device)
        self.sse += ((preds.double() - target.double()) ** 2).sum()
        self.n += preds.numel()
        self.lo = torch.minimum(self.lo, target.double().min())
        self.hi = torch.maximum(self.hi, target.double().max())

    def compute(self) -> Tensor:
        rng = self.data_range if self.data_range is not None else (self.hi - self.lo)
        return (10 * torch.log10(torch.as_tensor(rng, dtype=torch.float64) ** 2 / (self.sse / self.n).clamp(min=1e-30))).float()


def _gaussian_window(size: int, sigma: float, channels: int, device, dtype) -> Tensor:
    x = torch.arange(size, dtype=dtype, device=device) - (size - 1) / 2
    g = torch.exp(-(x ** 2) / (2 * sigma ** 2))
    g = g / g.sum()
    return (g[:, None] * g[None, :]).expand(channels, 1, size, size).contiguous()


def ssim(preds: Tensor, target: Tensor, data_range: float = 1.0, kernel_size: int = 11, sigma: float = 1.5,
         k1: float = 0.01, k2: float = 0.03) -> Tensor:
    """Structural similarity per image (``[B, C, H, W]`` inputs, Gaussian window, valid region)."""
    p, t = preds.double(), target.double()
    c = p.shape[1]
    w = _gaussian_window(kernel_size, sigma, c, p.device, p.dtype)
    conv = lambda x: torch.nn.functional.conv2d(x, w, groups=c)   # noqa: E731
    mp, mt = conv(p), conv(t)
    vp, vt, cov = conv(p * p) - mp * mp, conv(t * t) - mt * mt, conv(p * t) - mp * mt
    c1, c2 = (k1 * data_range) ** 2, (k2 * data_range) ** 2
    s = ((2 * mp * mt + c1) * (2 * cov + c2)) / ((mp * mp + mt * mt + c1) * (vp + vt + c2))
    return s.flatten(1).mean(-1)


class StructuralSimilarityIndexMeasure(_MeanOverSignals):
    def __init__(self, data_range: float = 1.0, kernel_size: int = 11, sigma: float = 1.5, **kw) -> None:
        super().__init__()
        self.kw = dict(data_range=data_range, kernel_size=kernel_size, sigma=sigma)

    def update(self, preds: Tensor, target: Tensor) -> None:
        self._to(preds.device)
        v = ssim(preds, target, **self.kw)
        self.total += v.sum()
        self.n += v.numel()


class TotalVariation(Metric):
    def __init__(self, reduction: str = "sum", **kw) -> None:
        super().__init__()
        self.reduction = reduction
        self.add_state("total", torch.zeros((), dtype=torch.float64))
        self.add_state("n", torch.zeros((), dtype=torch.float64))

    def update(self, img: Tensor) -> None:
        self._to(img.device)
        x = img.double()
        self.total += (x[..., 1:, :] - x[..., :-1, :]).abs().sum() + (x[..., :, 1:] - x[..., :, :-1]).abs().sum()
        self.n += x.shape[0]

    def compute(self) -> Tensor:
        return (self.total if self.reduction == "sum" else self.total / self.n.clamp(min=1)).float()


class UniversalImageQualityIndex(StructuralSimilarityIndexMeasure):
    """SSIM without the stabilising constants."""

    def update(self, preds: Tensor, target: Tensor) -> None:
        self._to(preds.device)
        v = ssim(preds, target, data_range=self.kw["data_range"], kernel_size=self.kw["kernel_size"], sigma=self.kw["sigma"],
                 k1=1e-8, k2=1e-8)
        self.total += v.sum()
        self.n += v.numel()


# ----------------------------------------------------------------------------- retrieval
class _Retrieval(Metric):
    """Scores, relevance and query ids are collected; the value is the mean over queries."""

    def __init__(self, top_k: Optional[int] = None, **kw) -> None:
        super().__init__()
        self.top_k = top_k
        self.p, self.t, self.q = [], [], []

    def reset(self) -> None:
        self.p, self.t, self.q = [], [], []

    def update(self, preds: Tensor, target: Tensor, indexes: Tensor) -> None:
        self.p.append(preds.detach().reshape(-1))
        self.t.append(target.detach().reshape(-1))
        self.q.append(indexes.detach().reshape(-1))

    def _query(self, rel_sorted: Tensor, n_rel: float) -> float:
        raise NotImplementedError

    def compute(self) -> Tensor:
        p, t, q = torch.cat(self.p), torch.cat(self.t), torch.cat(self.q)
        vals = []
        for qi in q.unique().tolist():
            m = q == qi
            order = torch.argsort(p[m], descending=True)
            rel = t[m][order].double()
            if rel.sum() == 0 and not getattr(self, "empty_ok", False):
                vals.append(0.0)
                continue
            vals.append(float(self._query(rel, float(rel.sum()))))
        return torch.tensor(sum(vals) / max(1, len(vals)))


class RetrievalMAP(_Retrieval):
    def _query(self, rel, n_rel):
        rel = rel[: self.top_k] if self.top_k else rel
        prec = torch.cumsum(rel, 0) / torch.arange(1, rel.numel() + 1, dtype=torch.float64)
        return (prec * rel).sum() / max(1.0, float(rel.sum()))


class RetrievalPrecision(_Retrieval):
    def _query(self, rel, n_rel):
        k = self.top_k or rel.numel()
        return rel[:k].sum() / k


class RetrievalRecall(_Retrieval):
    def _query(self, rel, n_rel):
        k = self.top_k or rel.numel()
        return rel[:k].sum() / n_rel


class RetrievalHitRate(_Retrieval):
    def _query(self, rel, n_rel):
        k = self.top_k or rel.numel()
        return (rel[:k].sum() > 0).double()


class RetrievalRPrecision(_Retrieval):
    def _query(self, rel, n_rel):
        r = int(n_rel)
        return rel[:r].sum() / r


class RetrievalFallOut(_Retrieval):
    """Fraction of the non-relevant documents that appear in the top k (lower is better)."""

    empty_ok = True

    def _query(self, rel, n_rel):
        k = self.top_k or rel.numel()
        neg = rel.numel() - n_rel
        return (1 - rel[:k]).sum() / max(1.0, neg)


class RetrievalAUROC(_Retrieval):
    def _query(self, rel, n_rel):
        from .ranking import binary_auroc
        scores = torch.arange(rel.numel(), 0, -1, dtype=torch.float64)     # rank order as score
        return binary_auroc(scores, rel)


__all__ = sorted(n for n in globals() if n[0].isupper() and n not in ("Metric", "Tensor", "Optional", "Counter", "List",
                                                                      "Sequence", "Union")) + ["edit_distance", "ssim"]


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
