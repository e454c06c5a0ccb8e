"""Layer and neuron attribution (the reference's ``lumen/_core/layer`` and ``neuron``):
activations, gradient x activation, Grad-CAM, layer integrated gradients, conductance."""
from __future__ import annotations

from typing import Callable, Optional

import torch
from torch import Tensor, nn

from ._common import Attribution, as_tuple, make_baselines, select_target
from .gradient import _quadrature


def _extra(additional_forward_args):
    if additional_forward_args is None:
        return ()
    return additional_forward_args if isinstance(additional_forward_args, tuple) else (additional_forward_args,)


class LayerAttribution(Attribution):
    def __init__(self, forward_func: Callable, layer: nn.Module):
        super().__init__(forward_func)
        self.layer = layer

    def _forward_capture(self, inputs, target, additional_forward_args, replace: Optional[Tensor] = None,
                         need_grad: bool = False):
        """Run the model; returns (selected output, the layer's output tensor). ``replace`` swaps
        the layer's output for a given tensor (which may require grad)."""
        box = {}

        def hook(mod, inp, out):
            o = out[0] if isinstance(out, tuple) else out
            if replace is not None:
                o = replace
            elif need_grad:
                o = o.detach().requires_grad_() if not o.requires_grad else o
                if not o.is_leaf:
                    o.retain_grad()
            box["act"] = o
            return (o,) + tuple(out[1:]) if isinstance(out, tuple) else o
        h = self.layer.register_forward_hook(hook)
        try:
            out = select_target(self.forward_func(*as_tuple(inputs), *_extra(additional_forward_args)), target)
        finally:
            h.remove()
        return out, box["act"]


class LayerActivation(LayerAttribution):
    def attribute(self, inputs, additional_forward_args=None):
        with torch.no_grad():
            box = {}
            h = self.layer.register_forward_hook(lambda m, i, o: box.__setitem__("a", o[0] if isinstance(o, tuple) else o))
            try:
                self.forward_func(*as_tuple(inputs), *_extra(additional_forward_args))
            finally:
                h.remove()
        return box["a"]


class LayerGradientXActivation(LayerAttribution):
    def attribute(self, inputs, target=None, additional_forward_args=None, multiply_by_inputs: bool = True):
        with torch.enable_grad():
            out, act = self._forward_capture(inputs, target, additional_forward_args, need_grad=True)
            g = torch.autograd.grad(out.sum(), act)[0]
        return (g * act).detach() if multiply_by_inputs else g.detach()


class LayerGradCam(LayerAttribution):
    """Channel weights = spatial mean of the gradients; map = weighted sum of the activations."""

    def attribute(self, inputs, target=None, additional_forward_args=None, relu_attributions: bool = False):
        with torch.enable_grad():
            out, act = self._forward_capture(inputs, target, additional_forward_args, need_grad=True)
            g = torch.autograd.grad(out.sum(), act)[0]
        w = g.mean(dim=tuple(range(2, g.dim())), keepdim=True) if g.dim() > 2 else g
        cam = (w * act).sum(1, keepdim=True).detach()
        return cam.clamp(min=0) if relu_attributions else cam


class LayerIntegratedGradients(LayerAttribution):
    """Integrated gradients taken along the straight path between the layer's activations at the
    baseline and at the input (e.g. an embedding layer of a token model)."""

    def has_convergence_delta(self) -> bool:
        return True

    def attribute(self, inputs, baselines=None, target=None, additional_forward_args=None, n_steps: int = 50,
                  method: str = "gausslegendre", return_convergence_delta: bool = False):
        ins = as_tuple(inputs)
        base = as_tuple(baselines) if baselines is not None else tuple(torch.zeros_like(i) for i in ins)
        with torch.no_grad():
            f1, a1 = self._forward_capture(ins, target, additional_forward_args)
            f0, a0 = self._forward_capture(base, target, additional_forward_args)
        alphas, weights = _quadrature(n_steps, method)
        total = torch.zeros_like(a1)
        for al, w in zip(alphas, weights):
            with torch.enable_grad():
                point = (a0 + al * (a1 - a0)).detach().requires_grad_()
                out, _ = self._forward_capture(ins, target, additional_forward_args, replace=point)
                total += w * torch.autograd.grad(out.sum(), point)[0]
        attr = total * (a1 - a0)
        if return_convergence_delta:
            return attr, attr.reshape(attr.shape[0], -1).sum(1) - (f1 - f0)
        return attr


class LayerConductance(LayerAttribution):
    """Flow of the input's integrated gradients through each unit of the layer:
    ``sum_steps dF/dh(x_a) * (h(x_{a+1}) - h(x_a))`` along the input path."""

    def attribute(self, inputs, baselines=None, target=None, additional_forward_args=None, n_steps: int = 50):
        ins = as_tuple(inputs)
        base = make_baselines(ins, baselines)
        total, prev = None, None
        for s in range(n_steps + 1):
            al = s / n_steps
            pts = tuple(b + al * (i - b) for i, b in zip(ins, base))
            with torch.enable_grad():
                out, act = self._forward_capture(pts, target, additional_forward_args, need_grad=True)
                g = torch.autograd.grad(out.sum(), act)[0]
            a = act.detach()
            if prev is not None:
                step = 0.5 * (g + prev[1]) * (a - prev[0])
                total = step if total is None else total + step
            prev = (a, g)
        return total


class NeuronConductance(LayerConductance):
    def attribute(self, inputs, neuron_selector, **kwargs):
        sel = neuron_selector if isinstance(neuron_selector, tuple) else (neuron_selector,)
        return super().attribute(inputs, **kwargs)[(slice(None),) + sel]


class InternalInfluence(LayerAttribution):
    """Integral of the layer gradient along the input path (no multiplication by activations)."""

    def attribute(self, inputs, baselines=None, target=None, additional_forward_args=None, n_steps: int = 50):
        ins = as_tuple(inputs)
        base = make_baselines(ins, baselines)
        alphas, weights = _quadrature(n_steps, "gausslegendre")
        total = None
        for al, w in zip(alphas, weights):
            pts = tuple(b + al * (i - b) for i, b in zip(ins, base))
            with torch.enable_grad():
                out, act = self._forward_capture(pts, target, additional_forward_args, need_grad=True)
                g = torch.autograd.grad(out.sum(), act)[0] * w
            total = g if total is None else total + g
        return total


# the reference has a package at this path: deeper module names resolve to views of the pack
__path__: list = []
