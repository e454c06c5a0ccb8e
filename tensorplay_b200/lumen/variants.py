"""Combined, layer-level and neuron-level variants of the attribution algorithms, layer-wise relevance
propagation, and summary statistics (the reference's ``lumen/_core/layer``, ``neuron``, ``lrp.py``,
``_utils/stat.py`` / ``summarizer.py``)."""
from __future__ import annotations

from typing import Callable, Dict, Optional, Sequence

import torch
from torch import Tensor, nn

from ._common import Attribution, as_tuple, gradients, like_input, make_baselines, select_target
from .gradient import DeepLift, GradientShap, GuidedBackprop, IntegratedGradients, Deconvolution
from .layer import LayerAttribution, LayerGradCam, _extra
from .perturbation import FeatureAblation, FeaturePermutation


class GradientAttribution(Attribution):
    """Marker base of the gradient-based algorithms."""


class PerturbationAttribution(Attribution):
    """Marker base of the perturbation-based algorithms."""


class NeuronAttribution(LayerAttribution):
    """Marker base of the neuron-level algorithms (a layer plus a neuron selector)."""


class DeepLiftShap(Attribution):
    """DeepLift averaged over a distribution of baselines (rows of ``baselines``)."""

    def __init__(self, model: nn.Module):
        super().__init__(model)
        self.dl = DeepLift(model)

    def attribute(self, inputs, baselines, target=None, additional_forward_args=None):
        base = as_tuple(baselines)
        total = None
        for i in range(base[0].shape[0]):
            b = tuple(x[i: i + 1] for x in base)
            a = as_tuple(self.dl.attribute(inputs, b if isinstance(inputs, tuple) else b[0], target, additional_forward_args))
            total = a if total is None else tuple(t + x for t, x in zip(total, a))
        return like_input(tuple(t / base[0].shape[0] for t in total), inputs)


class GuidedGradCam(Attribution):
    """Guided backpropagation at the input, weighted by the up-sampled Grad-CAM map of a layer."""

    def __init__(self, model: nn.Module, layer: nn.Module):
        super().__init__(model)
        self.cam, self.gb = LayerGradCam(model, layer), GuidedBackprop(model)

    def attribute(self, inputs, target=None, additional_forward_args=None, interpolate_mode: str = "nearest"):
        cam = self.cam.attribute(inputs, target, additional_forward_args, relu_attributions=True)
        g = self.gb.attribute(inputs, target, additional_forward_args)
        up = torch.nn.functional.interpolate(cam, size=g.shape[2:], mode=interpolate_mode)
        return g * up


class LRP(Attribution):
    """Layer-wise relevance propagation with the epsilon rule for ``nn.Sequential``-like stacks of
    linear / convolution layers and element-wise activations: relevance of a layer's output is
    redistributed to its inputs in proportion to their contributions ``x_i w_ij``."""

    def __init__(self, model: nn.Module, eps: float = 1e-9):
        super().__init__(model)
        self.model, self.eps = model, eps

    def attribute(self, inputs: Tensor, target=None, return_convergence_delta: bool = False):
        layers = [m for m in self.model.modules() if not list(m.children())]
        acts = [inputs.detach()]
        with torch.no_grad():
            for m in layers:
                acts.append(m(acts[-1]))
        out = acts[-1]
        rel = torch.zeros_like(out)
        sel = select_target(out, target)
        if target is None:
            rel = out.clone()
        else:
            idx = torch.as_tensor(target, device=out.device).expand(out.shape[0]) if not isinstance(target, Tensor) else target
            rel.scatter_(1, idx.view(-1, 1).long(), sel.view(-1, 1))
        for m, a in zip(reversed(layers), reversed(acts[:-1])):
            if isinstance(m, (nn.Linear, nn.Conv2d)):
                with torch.enable_grad():
                    x = a.clone().requires_grad_()
                    z = m(x)
                    stab = z + self.eps * torch.where(z >= 0, torch.ones_like(z), -torch.ones_like(z))
                    (c,) = torch.autograd.grad(z, x, grad_outputs=(rel / stab).detach())
                rel = (a * c).detach()
            elif isinstance(m, (nn.Flatten,)):
                rel = rel.reshape(a.shape)
            # element-wise activations, dropout, pooling-free stacks: relevance passes through
        if return_convergence_delta:
            return rel, rel.reshape(rel.shape[0], -1).sum(1) - sel
        return rel


class _LayerOutputAs(LayerAttribution):
    """Runs an input-attribution algorithm with the layer's output playing the role of the input."""

    algo = None

    def __init__(self, forward_func: Callable, layer: nn.Module, **algo_kw):
        super().__init__(forward_func, layer)
        self.algo_kw = algo_kw

    def _tail(self, inputs, additional_forward_args):
        """Function of the layer output: the rest of the network with the layer's output replaced."""
        def f(h):
            out, _ = self._forward_capture(inputs, None, additional_forward_args, replace=h)
            return out
        return f

    def _layer_value(self, inputs, additional_forward_args):
        with torch.no_grad():
            _, act = self._forward_capture(inputs, None, additional_forward_args)
        return act

    def _forward_capture(self, inputs, target, additional_forward_args, replace=None, need_grad=False):
        box = {}

        def hook(mod, inp, out):
            o = out[0] if isinstance(out, tuple) else out
            if replace is not None:
                o = replace
            box["act"] = o
            return (o,) + tuple(out[1:]) if isinstance(out, tuple) else o
        h = self.layer.register_forward_hook(hook)
        try:
            out = self.forward_func(*as_tuple(inputs), *_extra(additional_forward_args))
        finally:
            h.remove()
        return out, box["act"]


class LayerFeatureAblation(_LayerOutputAs):
    def attribute(self, inputs, layer_baselines=None, target=None, additional_forward_args=None, layer_mask=None):
        act = self._layer_value(inputs, additional_forward_args)
        return FeatureAblation(self._tail(inputs, additional_forward_args)).attribute(
            act, baselines=layer_baselines, target=target, feature_mask=layer_mask)


class LayerFeaturePermutation(_LayerOutputAs):
    def attribute(self, inputs, target=None, additional_forward_args=None, layer_mask=None, generator=None):
        act = self._layer_value(inputs, additional_forward_args)
        return FeaturePermutation(self._tail(inputs, additional_forward_args)).attribute(
            act, target=target, feature_mask=layer_mask, generator=generator)


class LayerGradientShap(_LayerOutputAs):
    def attribute(self, inputs, baselines, target=None, additional_forward_args=None, n_samples: int = 5, generator=None):
        act = self._layer_value(inputs, additional_forward_args)
        base_act = self._layer_value(baselines, additional_forward_args)
        # the tail ignores `inputs` once the layer output is replaced, so any batch-compatible input works
        return GradientShap(self._tail(inputs, additional_forward_args)).attribute(
            act, base_act, target=target, n_samples=n_samples, generator=generator)


class LayerDeepLift(_LayerOutputAs):
    """Rescale-rule multipliers for the part of the network after the layer."""

    def __init__(self, model: nn.Module, layer: nn.Module):
        super().__init__(model, layer)
        self.model = model

    def attribute(self, inputs, baselines=None, target=None, additional_forward_args=None):
        act = self._layer_value(inputs, additional_forward_args)
        base_in = make_baselines(as_tuple(inputs), baselines)
        base_act = self._layer_value(base_in if isinstance(inputs, tuple) else base_in[0], additional_forward_args)
        tail = self._tail(inputs, additional_forward_args)
        ig = IntegratedGradients(tail)        # path integral = exact multipliers for the tail
        return ig.attribute(act, baselines=base_act, target=target, n_steps=64)


class LayerLRP(LRP):
    """Relevance at the output of ``layer`` (propagation stops there)."""

    def __init__(self, model: nn.Module, layer: nn.Module, eps: float = 1e-9):
        super().__init__(model, eps)
        self.layer = layer

    def attribute(self, inputs: Tensor, target=None):
        layers = [m for m in self.model.modules() if not list(m.children())]
        stop = layers.index(self.layer)
        head = nn.Sequential(*layers[: stop + 1])
        tail = nn.Sequential(*layers[stop + 1:])
        with torch.no_grad():
            h = head(inputs)
        return LRP(tail, self.eps).attribute(h, target)


class _NeuronOf(NeuronAttribution):
    """Input attribution of one neuron of ``layer``: the forward function becomes ``layer(x)[neuron]``."""

    algo_cls = None

    def _neuron_func(self, neuron_selector):
        sel = neuron_selector if isinstance(neuron_selector, tuple) else (neuron_selector,)

        def f(*args):
            box = {}
            h = self.layer.register_forward_hook(lambda m, i, o: box.__setitem__("a", o[0] if isinstance(o, tuple) else o))
            try:
                self.forward_func(*args)
            finally:
                h.remove()
            return box["a"][(slice(None),) + sel]
        return f

    def attribute(self, inputs, neuron_selector, **kw):
        algo = type(self).algo_cls
        target_model = self.forward_func if isinstance(self.forward_func, nn.Module) else None
        inst = algo(self._neuron_func(neuron_selector))
        if target_model is not None and hasattr(inst, "model"):
            inst.model = target_model
        return inst.attribute(inputs, **kw)


def _neuron_variant(name, algo, doc):
    return type(name, (_NeuronOf,), {"algo_cls": algo, "__doc__": doc})


class _PlainGradient(Attribution):
    def attribute(self, inputs, additional_forward_args=None):
        g, _ = gradients(self.forward_func, as_tuple(inputs), None, additional_forward_args)
        return like_input(g, inputs)


NeuronGradient = _neuron_variant("NeuronGradient", _PlainGradient, "Gradient of the neuron with respect to the input.")
NeuronIntegratedGradients = _neuron_variant("NeuronIntegratedGradients", IntegratedGradients,
                                            "Integrated gradients of the neuron's activation.")
NeuronFeatureAblation = _neuron_variant("NeuronFeatureAblation", FeatureAblation, "Ablation effect on the neuron.")
NeuronGradientShap = _neuron_variant("NeuronGradientShap", GradientShap, "Expected gradients of the neuron.")


class _NeuronHooked(_NeuronOf):
    """Variants whose algorithm installs hooks on the model (guided backprop, deconvolution, DeepLift)."""

    def attribute(self, inputs, neuron_selector, **kw):
        inst = type(self).algo_cls(self.forward_func)
        inst.forward_func = self._neuron_func(neuron_selector)
        return inst.attribute(inputs, **kw)


NeuronGuidedBackprop = type("NeuronGuidedBackprop", (_NeuronHooked,), {"algo_cls": GuidedBackprop})
NeuronDeconvolution = type("NeuronDeconvolution", (_NeuronHooked,), {"algo_cls": Deconvolution})
NeuronDeepLift = type("NeuronDeepLift", (_NeuronHooked,), {"algo_cls": DeepLift})


# ----------------------------------------------------------------------------- statistics
class Summarizer:
    """Streaming statistics of attribution tensors: ``update`` with batches, ``summary`` returns
    mean / variance / std / min / max / sum / count per element."""

    def __init__(self, stats: Optional[Sequence[str]] = None):
        self.stats = list(stats) if stats else ["mean", "var", "std_dev", "min", "max", "sum", "count"]
        self.n, self.mean_, self.m2, self.lo, self.hi = 0, None, None, None, None

    def update(self, x: Tensor) -> None:
        x = x.detach().double()
        for row in x.reshape(-1, *x.shape[1:]) if x.dim() > 1 else x.reshape(-1, 1):
            self.n += 1
            if self.mean_ is None:
                self.mean_, self.m2 = row.clone(), torch.zeros_like(row)
                self.lo, self.hi = row.clone(), row.clone()
                continue
            d = row - self.mean_
            self.mean_ += d / self.n
            self.m2 += d * (row - self.mean_)          # Welford
            self.lo, self.hi = torch.minimum(self.lo, row), torch.maximum(self.hi, row)

    @property
    def summary(self) -> Dict[str, Tensor]:
        var = self.m2 / max(1, self.n)
        allv = {"mean": self.mean_, "var": var, "std_dev": var.sqrt(), "min": self.lo, "max": self.hi,
                "sum": self.mean_ * self.n, "count": torch.tensor(self.n)}
        return {k: allv[k] for k in self.stats}


def CommonStats():
    return ["mean", "var", "std_dev", "min", "max"]


class ClassSummarizer:
    """One :class:`Summarizer` per class label."""

    def __init__(self, stats: Optional[Sequence[str]] = None):
        self.stats, self.per = stats, {}

    def update(self, x: Tensor, labels: Tensor) -> None:
        for lab in labels.unique().tolist():
            self.per.setdefault(lab, Summarizer(self.stats)).update(x[labels == lab])

    @property
    def class_summaries(self):
        return {k: v.summary for k, v in self.per.items()}


# the reference has a package at this path: deeper module names resolve to views of the pack
__path__: list = []
