"""Generic LIME, DeepLiftShap at layers and neurons, attribution over a whole data loader, and the
graph-mode helpers (trace once, rewrite the ReLU gradients in the traced graph).
Reference: tensorplay/lumen/_core/lime.py (LimeBase), _core/dataloader_attr.py,
_utils/graph.py, _core/graph_guided_backprop.py."""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple, Union

import torch
from torch import Tensor, nn

from ._common import Attribution, as_tuple, gradients, like_input, run_forward
from .variants import DeepLiftShap, LayerDeepLift, _NeuronHooked


class LimeBase(Attribution):
    """LIME with every part supplied by the caller: ``perturb_func(inputs, **kw)`` draws a sample
    (in the interpretable space when ``perturb_interpretable_space``, else in input space),
    ``from_interp_rep_transform`` / ``to_interp_rep_transform`` convert between the two,
    ``similarity_func(inputs, perturbed_input, interpretable_sample, **kw)`` weights it, and
    ``interpretable_model`` is fit on (samples, outputs, weights): an object with
    ``fit(x, y, sample_weight)`` and ``representation()`` (or ``coef_``), or a callable
    ``(x, y, w) -> coefficients``. Returns the surrogate's coefficients."""

    def __init__(self, forward_func: Callable, interpretable_model, similarity_func: Callable, perturb_func: Callable,
                 perturb_interpretable_space: bool, from_interp_rep_transform: Optional[Callable],
                 to_interp_rep_transform: Optional[Callable]) -> None:
        super().__init__(forward_func)
        self.interpretable_model, self.similarity_func, self.perturb_func = interpretable_model, similarity_func, perturb_func
        self.perturb_interpretable_space = perturb_interpretable_space
        self.from_interp, self.to_interp = from_interp_rep_transform, to_interp_rep_transform
        if perturb_interpretable_space and from_interp_rep_transform is None:
            raise AssertionError("from_interp_rep_transform is needed when perturbing the interpretable space")
        if not perturb_interpretable_space and to_interp_rep_transform is None:
            raise AssertionError("to_interp_rep_transform is needed when perturbing the input space")

    def attribute(self, inputs, target=None, additional_forward_args=None, n_samples: int = 50, **kwargs) -> Tensor:
        xs, ys, ws = [], [], []
        gen = self.perturb_func(inputs, **kwargs)
        is_iter = hasattr(gen, "__next__")
        with torch.no_grad():
            for _ in range(n_samples):
                sample = next(gen) if is_iter else (gen if _ == 0 else self.perturb_func(inputs, **kwargs))
                if self.perturb_interpretable_space:
                    interp, model_in = sample, self.from_interp(sample, inputs, **kwargs)
                else:
                    model_in, interp = sample, self.to_interp(sample, inputs, **kwargs)
                y = run_forward(self.forward_func, as_tuple(model_in), target, additional_forward_args)
                xs.append(torch.as_tensor(interp).reshape(1, -1).double())
                ys.append(y.reshape(-1)[:1].double().cpu())
                ws.append(torch.as_tensor(self.similarity_func(inputs, model_in, interp, **kwargs)).reshape(-1)[:1].double())
        x, y, w = torch.cat(xs), torch.cat(ys), torch.cat(ws)
        model = self.interpretable_model
        if hasattr(model, "fit"):
            model.fit(x.numpy() if not isinstance(model, nn.Module) else x, y.numpy() if not isinstance(model, nn.Module) else y,
                      sample_weight=w.numpy() if not isinstance(model, nn.Module) else w)
            rep = model.representation() if hasattr(model, "representation") else model.coef_
            return torch.as_tensor(rep).reshape(1, -1).float()
        return torch.as_tensor(model(x, y, w)).reshape(1, -1).float()


class LayerDeepLiftShap(LayerDeepLift):
    """Layer DeepLift averaged over a distribution of baselines (one row of ``baselines`` each)."""

    def attribute(self, inputs, baselines, target=None, additional_forward_args=None):
        base = as_tuple(baselines)[0]
        total = None
        for b in base:
            ref = b[None].expand_as(as_tuple(inputs)[0])
            a = super().attribute(inputs, baselines=ref, target=target, additional_forward_args=additional_forward_args)
            total = a if total is None else total + a
        return total / base.shape[0]


class NeuronDeepLiftShap(_NeuronHooked):
    """DeepLiftShap of one neuron of a layer with respect to the input."""

    def attribute(self, inputs, neuron_selector, **kw):
        inst = DeepLiftShap(self.forward_func)
        inst.dl.forward_func = self._neuron_func(neuron_selector)
        return inst.attribute(inputs, **kw)


class DataLoaderAttribution(Attribution):
    """Feature ablation where one evaluation is a pass over a whole data loader: ``reduce(accum,
    batch_output, batch_inputs)`` folds the batches, ``to_metric(accum)`` turns the result into the
    tensor that is explained (a loss, an accuracy). Feature ``k`` of ``feature_mask`` (one id tensor
    per attributed input, broadcastable to a batch) is replaced by the baseline in every batch; its
    attribution is ``metric(original) - metric(ablated)``. ``input_roles``: 0 = attributed input,
    1 = forwarded unchanged, 2 = not given to the model (labels for ``reduce``)."""

    def __init__(self, attr_method) -> None:
        from .perturbation import FeatureAblation
        if not isinstance(attr_method, FeatureAblation):
            raise AssertionError("DataLoaderAttribution supports FeatureAblation as its attribution method")
        super().__init__(attr_method.forward_func)

    def attribute(self, dataloader, input_roles: Optional[Sequence[int]] = None, baselines=None, feature_mask=None,
                  reduce: Optional[Callable] = None, to_metric: Optional[Callable] = None, return_input_shape: bool = True):
        first = next(iter(dataloader))
        first = first if isinstance(first, (tuple, list)) else (first,)
        roles = list(input_roles) if input_roles is not None else [0] * len(first)
        attributed = [i for i, r in enumerate(roles) if r == 0]
        masks = list(as_tuple(feature_mask)) if feature_mask is not None else None
        if masks is None:
            masks, nxt = [], 0
            for i in attributed:
                n = first[i][0].numel()
                masks.append(torch.arange(nxt, nxt + n).reshape(1, *first[i].shape[1:]))
                nxt += n
        bases = list(as_tuple(baselines)) if baselines is not None else [0] * len(attributed)
        reduce = reduce or (lambda acc, out, inp: out if acc is None else torch.cat((acc, out)))
        to_metric = to_metric or (lambda acc: acc)
        feats = sorted(set(int(v) for m in masks for v in m.unique().tolist()))

        def run(ablate: Optional[int]):
            acc = None
            with torch.no_grad():
                for batch in dataloader:
                    batch = list(batch if isinstance(batch, (tuple, list)) else (batch,))
                    if ablate is not None:
                        for j, i in enumerate(attributed):
                            sel = (masks[j] == ablate).expand_as(batch[i])
                            b = bases[j] if isinstance(bases[j], Tensor) else torch.full_like(batch[i], bases[j])
                            batch[i] = torch.where(sel, b.expand_as(batch[i]).to(batch[i].dtype), batch[i])
                    out = self.forward_func(*[x for x, r in zip(batch, roles) if r != 2])
                    acc = reduce(acc, out, batch)
            return torch.as_tensor(to_metric(acc)).double()

        ref = run(None)
        deltas = {f: ref - run(f) for f in feats}
        if not return_input_shape:
            return torch.stack([deltas[f] for f in feats], -1).float()
        out = []
        for j, i in enumerate(attributed):
            shape = first[i].shape[1:]
            a = torch.zeros(*ref.shape, *shape, dtype=torch.float64)
            m = masks[j].expand(1, *shape)[0]
            for f in feats:
                a = torch.where(m == f, deltas[f].reshape(*ref.shape, *([1] * len(shape))), a)
            out.append(a.float())
        return tuple(out) if len(out) > 1 else out[0]


# ----------------------------------------------------------------------------- graph mode
def trace(forward_func: Callable) -> Callable:
    """``forward_func`` captured once as a ``torch.fx.GraphModule`` (returned as it is when it cannot be
    traced symbolically: data-dependent control flow, opaque Python)."""
    import torch.fx as fx
    if isinstance(forward_func, fx.GraphModule):
        return forward_func
    try:
        return fx.symbolic_trace(forward_func)
    except Exception:
        return forward_func


def node_names(model: Callable) -> List[str]:
    import torch.fx as fx
    gm = trace(model)
    if not isinstance(gm, fx.GraphModule):
        raise ValueError("the model cannot be traced, so it has no graph nodes to name")
    return [n.name for n in gm.graph.nodes]


def graph_gradient_func(forward_fn: Callable, inputs, target_ind=None, additional_forward_args=None) -> Tuple[Tensor, ...]:
    """Gradients of the (target-selected) output with respect to ``inputs`` through the traced graph."""
    g, _ = gradients(trace(forward_fn), as_tuple(inputs), target_ind, additional_forward_args)
    return g


class _GuidedRelu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        ctx.save_for_backward(x)
        return x.clamp(min=0)

    @staticmethod
    def backward(ctx, g):
        (x,) = ctx.saved_tensors
        return g.clamp(min=0) * (x > 0)


class _DeconvRelu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return x.clamp(min=0)

    @staticmethod
    def backward(ctx, g):
        return g.clamp(min=0)


def _guided_relu(x: Tensor) -> Tensor:
    return _GuidedRelu.apply(x)


def _deconv_relu(x: Tensor) -> Tensor:
    return _DeconvRelu.apply(x)


class _GraphModifiedRelu(Attribution):
    """Traces the model and replaces every ReLU node of the graph by a function with the modified
    backward rule, instead of installing backward hooks on modules: functional ``relu`` calls are
    covered too, and the rewritten graph is built once and reused."""

    relu_fn = None

    def __init__(self, model: nn.Module) -> None:
        import torch.fx as fx
        super().__init__(model)
        gm = fx.symbolic_trace(model)
        mods = dict(gm.named_modules())
        fn = type(self).relu_fn
        for node in list(gm.graph.nodes):
            is_relu = (node.op == "call_module" and isinstance(mods.get(node.target), nn.ReLU)) or \
                      (node.op == "call_function" and node.target in (torch.relu, torch.nn.functional.relu)) or \
                      (node.op == "call_method" and node.target == "relu")
            if is_relu:
                with gm.graph.inserting_after(node):
                    new = gm.graph.call_function(fn, (node.args[0],))
                node.replace_all_uses_with(new)
                gm.graph.erase_node(node)
        gm.recompile()
        self.graph_module = gm

    def attribute(self, inputs, target=None, additional_forward_args=None):
        g, _ = gradients(self.graph_module, as_tuple(inputs), target, additional_forward_args)
        return like_input(g, inputs)


class GraphGuidedBackprop(_GraphModifiedRelu):
    relu_fn = staticmethod(_guided_relu)


class GraphDeconvolution(_GraphModifiedRelu):
    relu_fn = staticmethod(_deconv_relu)


__all__ = ["LimeBase", "LayerDeepLiftShap", "NeuronDeepLiftShap", "DataLoaderAttribution", "trace", "node_names",
           "graph_gradient_func", "GraphGuidedBackprop", "GraphDeconvolution"]


# the reference has a package at this path: deeper module names resolve to views of the pack
__path__: list = []
