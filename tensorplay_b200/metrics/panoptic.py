"""Panoptic quality (Kirillov et al. 2019) and its modified form for stuff classes
(Porzi et al. 2019). Reference: tensorplay/metrics/detection/panoptic_qualities.py."""
from __future__ import annotations

from typing import Collection, Dict, Tuple

import torch
from torch import Tensor

from . import Metric


class PanopticQuality(Metric):
    """Inputs ``[B, *spatial, 2]`` hold ``(category_id, instance_id)`` per point. A predicted and a
    target segment of one category match when their IoU exceeds 0.5 (target points of unknown
    category do not count against a prediction); per category
    ``PQ = sum IoU(matched) / (TP + FP / 2 + FN / 2)``; the value is the mean over the categories seen.
    Classes are ordered things first, then stuffs, each sorted."""

    modified = False

    def __init__(self, things: Collection[int], stuffs: Collection[int], allow_unknown_preds_category: bool = False,
                 return_sq_and_rq: bool = False, return_per_class: bool = False, **kw) -> None:
        super().__init__()
        things, stuffs = set(things), set(stuffs)
        if things & stuffs:
            raise ValueError(f"things and stuffs share the categories {sorted(things & stuffs)}")
        if not all(isinstance(c, int) for c in things | stuffs):
            raise TypeError("category ids must be integers")
        self.things, self.stuffs = things, stuffs
        self.allow_unknown = allow_unknown_preds_category
        self.return_sq_and_rq, self.return_per_class = return_sq_and_rq, return_per_class
        self.order = sorted(things) + sorted(stuffs)
        self.slot = {c: i for i, c in enumerate(self.order)}
        n = len(self.order)
        for name in ("iou_sum", "tp", "fp", "fn"):
            self.add_state(name, torch.zeros(n, dtype=torch.float64))

    def _segments(self, img: Tensor) -> Tuple[Dict[Tuple[int, int], Tensor], Tensor]:
        """Masks per (category, instance) over the flattened points (stuff: one segment per category)
        and the mask of points of unknown category."""
        flat = img.reshape(-1, 2)
        cat, inst = flat[:, 0], flat[:, 1]
        known = torch.zeros_like(cat, dtype=torch.bool)
        segs: Dict[Tuple[int, int], Tensor] = {}
        for c in cat.unique().tolist():
            m = cat == c
            if c in self.stuffs:
                segs[(c, 0)] = m
            elif c in self.things:
                for i in inst[m].unique().tolist():
                    segs[(c, i)] = m & (inst == i)
            else:
                continue
            known |= m
        return segs, ~known

    def update(self, preds: Tensor, target: Tensor) -> None:
        if preds.shape != target.shape or preds.shape[-1] != 2 or preds.dim() < 3:
            raise ValueError("preds and target must both have the shape [B, *spatial, 2]")
        for p_img, t_img in zip(preds.cpu(), target.cpu()):
            p_segs, p_void = self._segments(p_img)
            if bool(p_void.any()) and not self.allow_unknown:
                raise ValueError("preds contain a category that is neither a thing nor a stuff")
            t_segs, t_void = self._segments(t_img)
            matched_p, matched_t = set(), set()
            for tk, tm in t_segs.items():
                for pk, pm in p_segs.items():
                    if pk[0] != tk[0]:
                        continue
                    inter = int((tm & pm).sum())
                    if inter == 0:
                        continue
                    union = int(tm.sum()) + int(pm.sum()) - inter - int((pm & t_void).sum())
                    iou = inter / union
                    s = self.slot[tk[0]]
                    if self.modified and tk[0] in self.stuffs:
                        self.iou_sum[s] += iou
                        matched_p.add(pk)
                    elif iou > 0.5:
                        self.iou_sum[s] += iou
                        self.tp[s] += 1
                        matched_p.add(pk)
                        matched_t.add(tk)
            for tk, tm in t_segs.items():
                s = self.slot[tk[0]]
                if self.modified and tk[0] in self.stuffs:
                    self.tp[s] += 1                       # every target stuff segment counts once
                elif tk not in matched_t and int((tm & p_void).sum()) <= 0.5 * int(tm.sum()):
                    self.fn[s] += 1
            for pk, pm in p_segs.items():
                if pk in matched_p or (self.modified and pk[0] in self.stuffs):
                    continue
                if int((pm & t_void).sum()) <= 0.5 * int(pm.sum()):
                    self.fp[self.slot[pk[0]]] += 1

    def compute(self) -> Tensor:
        den = self.tp + 0.5 * self.fp + 0.5 * self.fn
        seen = den > 0
        pq = torch.where(seen, self.iou_sum / den.clamp(min=1e-12), torch.zeros_like(den))
        sq = torch.where(self.tp > 0, self.iou_sum / self.tp.clamp(min=1e-12), torch.zeros_like(den))
        rq = torch.where(seen, self.tp / den.clamp(min=1e-12), torch.zeros_like(den))
        if self.return_per_class:
            return torch.stack((pq, sq, rq)) if self.return_sq_and_rq else pq.reshape(1, -1)
        mean = lambda v: v[seen].mean() if bool(seen.any()) else torch.zeros((), dtype=torch.float64)   # noqa: E731
        return torch.stack((mean(pq), mean(sq), mean(rq))) if self.return_sq_and_rq else mean(pq)


class ModifiedPanopticQuality(PanopticQuality):
    """For stuff categories the 0.5 threshold is dropped: the value of a stuff category is the mean
    IoU over the images in which the target contains it."""

    modified = True


__all__ = ["PanopticQuality", "ModifiedPanopticQuality"]


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
