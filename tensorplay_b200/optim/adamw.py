"""AdamW / Adam with a fused multi-tensor CUDA step.

State per parameter: ``exp_avg``, ``exp_avg_sq`` (fp32) and, for bf16 parameters, an fp32
``master`` copy - the kernel updates all three and writes the bf16 parameter in one pass.
Hyper-parameters and state-dict keys follow torch's (and the reference's, tensorplay/optim/adam.py:27-520,
adamw.py:9-62: ``_multi_tensor_adam`` -> ``_fused_adamw_``).
"""
from __future__ import annotations

from typing import List, Optional

import torch
from torch.optim import Optimizer

from .. import ops


class AdamW(Optimizer):
    _decoupled = True

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 1e-2, amsgrad: bool = False, *, maximize: bool = False,
                 foreach: Optional[bool] = None, capturable: bool = False,
                 differentiable: bool = False, fused: Optional[bool] = None):
        if lr < 0 or eps < 0 or not 0 <= betas[0] < 1 or not 0 <= betas[1] < 1 or weight_decay < 0:
            raise ValueError("invalid AdamW hyper-parameter")
        if amsgrad:
            raise NotImplementedError("amsgrad is not supported by the fused kernel; use torch.optim.AdamW")
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, maximize=maximize)
        super().__init__(params, defaults)
        self._found_inf: Optional[torch.Tensor] = None
        self._grad_scale: Optional[torch.Tensor] = None

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        # torch.amp.GradScaler hands these over as attributes when the optimizer accepts them
        found_inf = getattr(self, "found_inf", None)
        grad_scale_t = getattr(self, "grad_scale", None)
        for group in self.param_groups:
            buckets = {}
            for p in group["params"]:
                if p.grad is None:
                    continue
                if p.grad.is_sparse:
                    raise RuntimeError("AdamW does not support sparse gradients")
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                    st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
                    if p.dtype != torch.float32:
                        st["master"] = p.detach().float().clone()
                st["step"] += 1
                key = (p.device, p.dtype, p.grad.dtype, st["step"])
                buckets.setdefault(key, []).append(p)
            b1, b2 = group["betas"]
            wd = group["weight_decay"] if self._decoupled else 0.0
            for (dev, pdt, gdt, step), ps in buckets.items():
                masters, models = [], []
                for p in ps:
                    st = self.state[p]
                    if "master" in st:
                        masters.append(st["master"].view(-1))
                        models.append(p.data.view(-1) if p.is_contiguous() else None)
                    else:
                        masters.append(p.data.view(-1))
                        models.append(None)
                grads = [p.grad.contiguous().view(-1) for p in ps]
                if not self._decoupled and group["weight_decay"] != 0:
                    grads = [g.float().add(m, alpha=group["weight_decay"]) for g, m in zip(grads, masters)]
                m1 = [self.state[p]["exp_avg"].view(-1) for p in ps]
                m2 = [self.state[p]["exp_avg_sq"].view(-1) for p in ps]
                gscale = 1.0
                if grad_scale_t is not None:
                    gscale = 1.0 / float(grad_scale_t)
                fused_ok = dev.type == "cuda" and all(g.dtype in (torch.bfloat16, torch.float32) for g in grads) \
                    and pdt in (torch.bfloat16, torch.float32) and len({g.dtype for g in grads}) == 1
                has_models = any(m is not None for m in models)
                if fused_ok and (not has_models or all(m is not None for m in models)):
                    ops.adamw_multi_(masters, m1, m2, grads, models if has_models else None,
                                     lr=group["lr"], beta1=b1, beta2=b2, eps=group["eps"],
                                     weight_decay=wd, step=step, grad_scale=gscale,
                                     maximize=group["maximize"], found_inf=found_inf)
                else:
                    for i, p in enumerate(ps):
                        ops.optim.adamw_flat_(masters[i], m1[i], m2[i], grads[i], None, lr=group["lr"],
                                              beta1=b1, beta2=b2, eps=group["eps"], weight_decay=wd,
                                              step=step, grad_scale=gscale, maximize=group["maximize"],
                                              found_inf=found_inf)
                        if "master" in self.state[p]:
                            p.data.copy_(self.state[p]["master"].view_as(p))
        return loss


class Adam(AdamW):
    """Adam with L2 regularisation folded into the gradient (``weight_decay`` is not decoupled)."""
    _decoupled = False

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.0, **kw):
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, **kw)
