"""Perturbation-based and surrogate-model attribution (the reference's ``lumen/_core``:
feature_ablation.py, occlusion.py, feature_permutation.py, shapley_value.py, lime.py,
kernel_shap.py)."""
from __future__ import annotations

import itertools
import math
from typing import Optional, Sequence

import torch
from torch import Tensor

from ._common import Attribution, as_tuple, like_input, make_baselines, run_forward


def _feature_ids(x: Tensor, feature_mask: Optional[Tensor]) -> Tensor:
    """Integer id per input element (shared by the batch); default: every element its own feature."""
    if feature_mask is None:
        return torch.arange(x[0].numel(), device=x.device).reshape(x.shape[1:])
    m = feature_mask
    return m[0] if m.dim() == x.dim() else m


class FeatureAblation(Attribution):
    """Output change when a feature (group of elements) is replaced by its baseline."""

    def attribute(self, inputs, baselines=None, target=None, feature_mask=None, additional_forward_args=None,
                  perturbations_per_eval: int = 1):
        x = as_tuple(inputs)[0]
        base = make_baselines((x,), baselines)[0]
        ids = _feature_ids(x, feature_mask)
        with torch.no_grad():
            ref = run_forward(self.forward_func, (x,), target, additional_forward_args)
            attr = torch.zeros_like(x)
            feats = ids.unique().tolist()
            for s in range(0, len(feats), perturbations_per_eval):
                group = feats[s: s + perturbations_per_eval]
                xs = []
                for f in group:
                    sel = (ids == f).expand_as(x)
                    xs.append(torch.where(sel, base, x))
                out = run_forward(self.forward_func, (torch.cat(xs),), target, additional_forward_args)
                for j, f in enumerate(group):
                    d = ref - out[j * x.shape[0]: (j + 1) * x.shape[0]]
                    sel = (ids == f).expand_as(x)
                    attr = torch.where(sel, d.view(-1, *([1] * (x.dim() - 1))).to(x.dtype).expand_as(x), attr)
        return like_input((attr,), inputs)


class Occlusion(Attribution):
    """Sliding-window ablation; every element receives the mean change of the windows covering it."""

    def attribute(self, inputs, sliding_window_shapes: Sequence[int], strides=None, baselines=None, target=None,
                  additional_forward_args=None):
        x = as_tuple(inputs)[0]
        base = make_baselines((x,), baselines)[0]
        win = tuple(sliding_window_shapes)
        strides = win if strides is None else ((strides,) * len(win) if isinstance(strides, int) else tuple(strides))
        dims = x.shape[1:]
        assert len(win) == len(dims)
        with torch.no_grad():
            ref = run_forward(self.forward_func, (x,), target, additional_forward_args)
            total, count = torch.zeros_like(x), torch.zeros_like(x)
            ranges = [range(0, max(1, d - w + 1 + (s - 1)), s) for d, w, s in zip(dims, win, strides)]
            for origin in itertools.product(*ranges):
                sl = (slice(None),) + tuple(slice(o, min(o + w, d)) for o, w, d in zip(origin, win, dims))
                xp = x.clone()
                xp[sl] = base[sl]
                d = (ref - run_forward(self.forward_func, (xp,), target, additional_forward_args))
                total[sl] += d.view(-1, *([1] * (x.dim() - 1))).to(x.dtype)
                count[sl] += 1
        return like_input((total / count.clamp(min=1),), inputs)


class FeaturePermutation(Attribution):
    """Output change when a feature's values are shuffled across the batch."""

    def attribute(self, inputs, target=None, feature_mask=None, additional_forward_args=None, generator=None):
        x = as_tuple(inputs)[0]
        ids = _feature_ids(x, feature_mask)
        with torch.no_grad():
            ref = run_forward(self.forward_func, (x,), target, additional_forward_args)
            attr = torch.zeros_like(x)
            for f in ids.unique().tolist():
                perm = torch.randperm(x.shape[0], generator=generator).to(x.device)
                sel = (ids == f).expand_as(x)
                out = run_forward(self.forward_func, (torch.where(sel, x[perm], x),), target, additional_forward_args)
                attr = torch.where(sel, (ref - out).view(-1, *([1] * (x.dim() - 1))).to(x.dtype).expand_as(x), attr)
        return like_input((attr,), inputs)


class ShapleyValueSampling(Attribution):
    """Monte-Carlo Shapley values: marginal contributions along random feature orders."""

    def attribute(self, inputs, baselines=None, target=None, feature_mask=None, n_samples: int = 25,
                  additional_forward_args=None, generator=None):
        x = as_tuple(inputs)[0]
        base = make_baselines((x,), baselines)[0]
        ids = _feature_ids(x, feature_mask)
        feats = ids.unique().tolist()
        orders = self._orders(feats, n_samples, generator)
        attr = torch.zeros_like(x)
        with torch.no_grad():
            for order in orders:
                cur = base.clone()
                prev = run_forward(self.forward_func, (cur,), target, additional_forward_args)
                for f in order:
                    sel = (ids == f).expand_as(x)
                    cur = torch.where(sel, x, cur)
                    out = run_forward(self.forward_func, (cur,), target, additional_forward_args)
                    attr += torch.where(sel, (out - prev).view(-1, *([1] * (x.dim() - 1))).to(x.dtype).expand_as(x),
                                        torch.zeros_like(x))
                    prev = out
        return like_input((attr / len(orders),), inputs)

    def _orders(self, feats, n_samples, generator):
        return [[feats[i] for i in torch.randperm(len(feats), generator=generator).tolist()] for _ in range(n_samples)]


class ShapleyValues(ShapleyValueSampling):
    """Exact Shapley values: every permutation (use for a handful of features)."""

    def _orders(self, feats, n_samples, generator):
        if len(feats) > 8:
            raise ValueError("exact Shapley values enumerate n! orders: use ShapleyValueSampling")
        return [list(p) for p in itertools.permutations(feats)]


class Lime(Attribution):
    """Weighted linear surrogate on binary feature-presence vectors around one input."""

    def _kernel(self, z: Tensor, n_feat: int) -> Tensor:
        dist = 1.0 - z.float().mean(1)                      # fraction of features removed
        return torch.exp(-(dist ** 2) / 0.25 ** 2)

    def _sample(self, n_samples: int, n_feat: int, generator) -> Tensor:
        return (torch.rand(n_samples, n_feat, generator=generator) < 0.5).float()

    def attribute(self, inputs, baselines=None, target=None, feature_mask=None, n_samples: int = 64,
                  additional_forward_args=None, generator=None, return_input_shape: bool = True):
        x = as_tuple(inputs)[0]
        assert x.shape[0] == 1, "surrogate methods explain one example per call"
        base = make_baselines((x,), baselines)[0]
        ids = _feature_ids(x, feature_mask)
        feats = ids.unique().tolist()
        z = self._sample(n_samples, len(feats), generator)
        z[0] = 1.0
        if n_samples > 1:
            z[1] = 0.0
        xs = []
        for row in z:
            keep = torch.zeros_like(ids, dtype=torch.bool)
            for j, f in enumerate(feats):
                if row[j] > 0:
                    keep |= ids == f
            xs.append(torch.where(keep.expand_as(x), x, base))
        with torch.no_grad():
            y = torch.cat([run_forward(self.forward_func, (xx,), target, additional_forward_args) for xx in xs]).double()
        w = self._kernel(z, len(feats)).double().to(y.device)
        a = torch.cat((z.double().to(y.device), torch.ones(len(z), 1, dtype=torch.float64, device=y.device)), 1)
        sw = w.sqrt()[:, None]
        coef = torch.linalg.lstsq(a * sw, (y[:, None] * sw)).solution[:-1, 0]
        if not return_input_shape:
            return coef.to(x.dtype)[None]
        attr = torch.zeros_like(x)
        for j, f in enumerate(feats):
            attr = torch.where((ids == f).expand_as(x), coef[j].to(x.dtype), attr)
        return like_input((attr,), inputs)


class KernelShap(Lime):
    """The surrogate with the Shapley kernel: its coefficients estimate Shapley values."""

    def _sample(self, n_samples, n_feat, generator):
        # subset sizes follow the Shapley kernel's mass, members uniform: the regression is then unweighted
        sizes = torch.arange(1, n_feat)
        if n_feat < 2:
            return torch.ones(n_samples, n_feat)
        p = (n_feat - 1) / (sizes * (n_feat - sizes)).float()
        k = sizes[torch.multinomial(p / p.sum(), n_samples, replacement=True, generator=generator)]
        z = torch.zeros(n_samples, n_feat)
        for r in range(n_samples):
            z[r, torch.randperm(n_feat, generator=generator)[: int(k[r])]] = 1.0
        return z

    def _kernel(self, z, n_feat):
        w = torch.ones(len(z))
        w[:2] = 1e6      # the full and the empty coalition pin f(x) and f(baseline)
        return w


# the reference has a package at this path: deeper module names resolve to views of the pack
__path__: list = []
