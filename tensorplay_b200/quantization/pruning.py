"""Weight pruning (the reference's ``tensorplay/ao/pruning``): magnitude masks per tensor or
globally, N:M semi-structured masks (2:4 is what the sparse tensor cores take), a sparsifier that
keeps masks applied through training, and a cubic sparsity schedule."""
from __future__ import annotations

from typing import Dict, Iterable, Optional

import torch
from torch import Tensor, nn


def magnitude_mask(w: Tensor, sparsity: float) -> Tensor:
    """Boolean keep-mask dropping the ``sparsity`` fraction of smallest magnitudes of ``w``."""
    k = int(round(sparsity * w.numel()))
    if k <= 0:
        return torch.ones_like(w, dtype=torch.bool)
    if k >= w.numel():
        return torch.zeros_like(w, dtype=torch.bool)
    thr = w.abs().flatten().kthvalue(k).values
    return w.abs() > thr


def global_magnitude_masks(params: Dict[str, Tensor], sparsity: float) -> Dict[str, Tensor]:
    """One threshold over all tensors: layers with small weights lose more."""
    allw = torch.cat([p.abs().flatten().float() for p in params.values()])
    k = int(round(sparsity * allw.numel()))
    if k <= 0:
        return {n: torch.ones_like(p, dtype=torch.bool) for n, p in params.items()}
    thr = allw.kthvalue(k).values
    return {n: p.abs().float() > thr for n, p in params.items()}


def n_m_mask(w: Tensor, n: int = 2, m: int = 4) -> Tensor:
    """Keep the ``n`` largest magnitudes in every group of ``m`` consecutive input weights."""
    if w.shape[-1] % m:
        raise ValueError(f"the last dimension must be a multiple of {m}")
    g = w.abs().reshape(-1, m)
    idx = g.topk(n, dim=-1).indices
    mask = torch.zeros_like(g, dtype=torch.bool).scatter_(1, idx, True)
    return mask.reshape(w.shape)


class WeightSparsifier:
    """Keeps masks on the weights of selected layers: ``step()`` recomputes them at the current
    target sparsity, a forward pre-hook re-applies them so that optimizer updates cannot revive
    pruned weights, ``squash()`` makes the zeros permanent and removes the hooks."""

    def __init__(self, model: nn.Module, sparsity: float = 0.5, pattern: Optional[tuple] = None, filter_fn=None):
        self.sparsity, self.pattern = sparsity, pattern
        self.layers = {n: m for n, m in model.named_modules()
                       if isinstance(m, nn.Linear) and (filter_fn is None or filter_fn(m, n))}
        self.masks: Dict[str, Tensor] = {}
        self.hooks = [m.register_forward_pre_hook(lambda mod, inp, n=n: self._apply(n)) for n, m in self.layers.items()]

    def _apply(self, name: str) -> None:
        if name in self.masks:
            with torch.no_grad():
                self.layers[name].weight.mul_(self.masks[name].to(self.layers[name].weight.dtype))

    def step(self, sparsity: Optional[float] = None) -> None:
        if sparsity is not None:
            self.sparsity = sparsity
        for n, m in self.layers.items():
            w = m.weight.data
            self.masks[n] = n_m_mask(w, *self.pattern) if self.pattern else magnitude_mask(w, self.sparsity)
            self._apply(n)

    def density(self) -> float:
        kept = sum(int(m.sum()) for m in self.masks.values())
        total = sum(m.numel() for m in self.masks.values())
        return kept / max(1, total)

    def squash(self) -> None:
        for n in self.layers:
            self._apply(n)
        for h in self.hooks:
            h.remove()
        self.hooks = []


def cubic_sparsity(step: int, total_steps: int, final: float, initial: float = 0.0, begin: int = 0) -> float:
    """Gradual pruning schedule ``s_t = s_f + (s_i - s_f) (1 - t / T)^3``."""
    if step <= begin:
        return initial
    t = min(1.0, (step - begin) / max(1, total_steps - begin))
    return final + (initial - final) * (1 - t) ** 3


def sqnr(ref: Tensor, test: Tensor) -> float:
    """Signal-to-quantisation-noise ratio in dB (the numeric-suite comparison of two outputs)."""
    noise = (ref.float() - test.float()).pow(2).mean().clamp(min=1e-30)
    return float(10 * torch.log10(ref.float().pow(2).mean().clamp(min=1e-30) / noise))


def compare_models(ref: nn.Module, test: nn.Module, inputs: Iterable, layer_types=(nn.Linear,)) -> Dict[str, float]:
    """SQNR of every same-named sub-module output between a reference model and its quantised or
    pruned copy (modules present in both by name; the type filter applies to the reference)."""
    names = [n for n, m in ref.named_modules() if isinstance(m, layer_types) and n]
    outs = {"ref": {}, "test": {}}
    hooks = []
    test_mods = dict(test.named_modules())
    for n in names:
        if n not in test_mods:
            continue
        hooks.append(dict(ref.named_modules())[n].register_forward_hook(
            lambda m, i, o, n=n: outs["ref"].setdefault(n, []).append(o.detach())))
        hooks.append(test_mods[n].register_forward_hook(
            lambda m, i, o, n=n: outs["test"].setdefault(n, []).append(o.detach())))
    with torch.no_grad():
        for batch in inputs:
            args = batch if isinstance(batch, (tuple, list)) else (batch,)
            ref(*args)
            test(*args)
    for h in hooks:
        h.remove()
    return {n: sqnr(torch.cat(outs["ref"][n]), torch.cat(outs["test"][n])) for n in outs["ref"] if n in outs["test"]}
