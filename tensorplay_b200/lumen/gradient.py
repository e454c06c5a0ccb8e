"""Gradient-based input attribution (the reference's ``lumen/_core``: saliency.py,
input_x_gradient.py, integrated_gradients.py, gradient_shap.py, noise_tunnel.py,
guided_backprop_deconvnet.py, deep_lift.py)."""
from __future__ import annotations

from typing import Callable, Optional

import numpy as np
import torch
from torch import Tensor, nn

from ._common import Attribution, as_tuple, gradients, like_input, make_baselines, run_forward


class Saliency(Attribution):
    def attribute(self, inputs, target=None, abs: bool = True, additional_forward_args=None):
        g, _ = gradients(self.forward_func, as_tuple(inputs), target, additional_forward_args)
        return like_input(tuple(x.abs() if abs else x for x in g), inputs)


class InputXGradient(Attribution):
    def attribute(self, inputs, target=None, additional_forward_args=None):
        ins = as_tuple(inputs)
        g, _ = gradients(self.forward_func, ins, target, additional_forward_args)
        return like_input(tuple(i * x for i, x in zip(ins, g)), inputs)


def _quadrature(n_steps: int, method: str):
    """Nodes and weights on [0, 1] (Gauss-Legendre by default, Riemann variants otherwise)."""
    if method == "gausslegendre":
        x, w = np.polynomial.legendre.leggauss(n_steps)
        return (0.5 * (x + 1)).tolist(), (0.5 * w).tolist()
    if method == "riemann_trapezoid":
        xs = np.linspace(0, 1, n_steps)
        w = np.full(n_steps, 1.0 / (n_steps - 1))
        w[0] = w[-1] = 0.5 / (n_steps - 1)
        return xs.tolist(), w.tolist()
    if method == "riemann_middle":
        return ((np.arange(n_steps) + 0.5) / n_steps).tolist(), [1.0 / n_steps] * n_steps
    if method == "riemann_left":
        return (np.arange(n_steps) / n_steps).tolist(), [1.0 / n_steps] * n_steps
    if method == "riemann_right":
        return ((np.arange(n_steps) + 1) / n_steps).tolist(), [1.0 / n_steps] * n_steps
    raise ValueError(method)


class IntegratedGradients(Attribution):
    """``(x - x') * integral_0^1 grad f(x' + a (x - x')) da``; the completeness axiom gives the
    convergence delta ``sum(attr) - (f(x) - f(x'))``."""

    def has_convergence_delta(self) -> bool:
        return True

    def attribute(self, inputs, baselines=None, target=None, additional_forward_args=None, n_steps: int = 50,
                  method: str = "gausslegendre", internal_batch_size: Optional[int] = None,
                  return_convergence_delta: bool = False):
        ins = as_tuple(inputs)
        base = make_baselines(ins, baselines)
        alphas, weights = _quadrature(n_steps, method)
        total = [torch.zeros_like(i) for i in ins]
        chunk = internal_batch_size or n_steps
        for s in range(0, n_steps, chunk):
            a = alphas[s: s + chunk]
            # all steps of the chunk in one batched forward / backward
            scaled = tuple(torch.cat([b + al * (i - b) for al in a]) for i, b in zip(ins, base))
            extra = additional_forward_args
            tgt = target
            g, _ = gradients(self.forward_func, scaled, tgt, extra)
            for k, gk in enumerate(g):
                parts = gk.chunk(len(a))
                for w, p in zip(weights[s: s + chunk], parts):
                    total[k] += w * p
        attr = tuple(t * (i - b) for t, i, b in zip(total, ins, base))
        if not return_convergence_delta:
            return like_input(attr, inputs)
        with torch.no_grad():
            f1 = run_forward(self.forward_func, ins, target, additional_forward_args)
            f0 = run_forward(self.forward_func, base, target, additional_forward_args)
        delta = sum(a.reshape(a.shape[0], -1).sum(1) for a in attr) - (f1 - f0)
        return like_input(attr, inputs), delta


class GradientShap(Attribution):
    """Expected gradients: random baselines from a distribution, random point on each path."""

    def attribute(self, inputs, baselines, target=None, n_samples: int = 5, stdevs: float = 0.0,
                  additional_forward_args=None, generator=None):
        ins = as_tuple(inputs)
        bdist = as_tuple(baselines)
        total = [torch.zeros_like(i) for i in ins]
        for _ in range(n_samples):
            idx = torch.randint(0, bdist[0].shape[0], (ins[0].shape[0],), generator=generator)
            base = tuple(b[idx.to(b.device)] for b in bdist)
            alpha = torch.rand(ins[0].shape[0], generator=generator).to(ins[0].device)
            pts = []
            for i, b in zip(ins, base):
                noisy = i + stdevs * torch.randn(i.shape, generator=generator).to(i.device) if stdevs else i
                a = alpha.view(-1, *([1] * (i.dim() - 1))).to(i.dtype)
                pts.append(b + a * (noisy - b))
            g, _ = gradients(self.forward_func, tuple(pts), target, additional_forward_args)
            for k in range(len(ins)):
                total[k] += g[k] * (ins[k] - base[k]) / n_samples
        return like_input(tuple(total), inputs)


class NoiseTunnel:
    """SmoothGrad / SmoothGrad-squared / VarGrad around any attribution method."""

    def __init__(self, attribution_method: Attribution):
        self.method = attribution_method

    def attribute(self, inputs, nt_type: str = "smoothgrad", nt_samples: int = 5, stdevs: float = 1.0,
                  generator=None, **kwargs):
        ins = as_tuple(inputs)
        acc = [torch.zeros_like(i) for i in ins]
        acc2 = [torch.zeros_like(i) for i in ins]
        for _ in range(nt_samples):
            noisy = tuple(i + stdevs * torch.randn(i.shape, generator=generator).to(i.device) for i in ins)
            a = as_tuple(self.method.attribute(noisy if isinstance(inputs, tuple) else noisy[0], **kwargs))
            for k in range(len(ins)):
                acc[k] += a[k]
                acc2[k] += a[k] * a[k]
        mean = [a / nt_samples for a in acc]
        if nt_type == "smoothgrad":
            out = mean
        elif nt_type == "smoothgrad_sq":
            out = [a / nt_samples for a in acc2]
        elif nt_type == "vargrad":
            out = [a2 / nt_samples - m * m for a2, m in zip(acc2, mean)]
        else:
            raise ValueError(nt_type)
        return like_input(tuple(out), inputs)


class _ReluOverride(Attribution):
    """Gradient with a modified ReLU backward rule, installed by hooks for the call's duration."""

    def __init__(self, model: nn.Module):
        super().__init__(model)
        self.model = model

    def _rule(self, grad_in: Tensor, grad_out: Tensor) -> Tensor:
        raise NotImplementedError

    def attribute(self, inputs, target=None, additional_forward_args=None):
        handles = []

        def hook(mod, gi, go):
            return (self._rule(gi[0], go[0]),)
        for m in self.model.modules():
            if isinstance(m, nn.ReLU):
                handles.append(m.register_full_backward_hook(hook))
        try:
            g, _ = gradients(self.forward_func, as_tuple(inputs), target, additional_forward_args)
        finally:
            for h in handles:
                h.remove()
        return like_input(g, inputs)


class GuidedBackprop(_ReluOverride):
    """Only positive gradients pass a ReLU (on top of its usual gate)."""

    def _rule(self, grad_in, grad_out):
        return grad_in.clamp(min=0)


class Deconvolution(_ReluOverride):
    """The ReLU is applied to the gradient itself, ignoring the forward gate."""

    def _rule(self, grad_in, grad_out):
        return grad_out.clamp(min=0)


class DeepLift(Attribution):
    """Rescale rule: every ReLU passes ``delta_out / delta_in`` (input against baseline) instead
    of its gradient, which makes the attributions sum to ``f(x) - f(x')`` exactly for piecewise
    linear networks."""

    def __init__(self, model: nn.Module, eps: float = 1e-10):
        super().__init__(model)
        self.model, self.eps = model, eps

    def has_convergence_delta(self) -> bool:
        return True

    def attribute(self, inputs, baselines=None, target=None, additional_forward_args=None,
                  return_convergence_delta: bool = False):
        ins = as_tuple(inputs)
        base = make_baselines(ins, baselines)
        n = ins[0].shape[0]
        handles, saved = [], {}

        def fwd(mod, inp, out):
            saved[mod] = (inp[0].detach(), out.detach())

        def bwd(mod, gi, go):
            x, y = saved[mod]
            dx, dy = x[:n] - x[n:], y[:n] - y[n:]
            mult = torch.where(dx.abs() > self.eps, dy / torch.where(dx.abs() > self.eps, dx, torch.ones_like(dx)),
                               gi[0][:n] / torch.where(go[0][:n] != 0, go[0][:n], torch.ones_like(go[0][:n])))
            new = gi[0].clone()
            new[:n] = go[0][:n] * mult
            return (new,)
        for m in self.model.modules():
            if isinstance(m, (nn.ReLU, nn.Sigmoid, nn.Tanh, nn.GELU, nn.SiLU)):
                handles.append(m.register_forward_hook(fwd))
                handles.append(m.register_full_backward_hook(bwd))
        try:
            both = tuple(torch.cat((i, b)) for i, b in zip(ins, base))
            with torch.enable_grad():
                xs = tuple(b.detach().requires_grad_() for b in both)
                extra = () if additional_forward_args is None else (
                    additional_forward_args if isinstance(additional_forward_args, tuple) else (additional_forward_args,))
                from ._common import select_target
                out = select_target(self.forward_func(*xs, *extra), target)
                grads = torch.autograd.grad(out[:n].sum(), xs)
        finally:
            for h in handles:
                h.remove()
        attr = tuple(g[:n] * (i - b) for g, i, b in zip(grads, ins, base))
        if not return_convergence_delta:
            return like_input(attr, inputs)
        delta = sum(a.reshape(n, -1).sum(1) for a in attr) - (out[:n] - out[n:]).detach()
        return like_input(attr, inputs), delta


# the reference has a package at this path: deeper module names resolve to views of the pack
__path__: list = []
