"""SGD, Adagrad, RMSprop and Adafactor with fused CUDA steps.

Constructor arguments, state-dict keys and update rules are torch's (and the reference's,
tensorplay/optim/sgd.py, adagrad.py, rmsprop.py over p10/include/OptimizerMTA.cuh:438 / :847 /
:988). On CUDA every parameter group is updated by a handful of launches of
``tpb_optim_multi`` (fp32 state; bf16 parameters keep an fp32 ``master`` copy and are written in the
same pass); on CPU, for sparse gradients and for dtypes the kernel does not take, the step falls
back to torch's implementation of the same class.
"""
from __future__ import annotations

from typing import Dict, List

import torch
from torch.optim import SGD as _SGD
from torch.optim import Adafactor as _Adafactor
from torch.optim import Adagrad as _Adagrad
from torch.optim import RMSprop as _RMSprop

from ..ops import optim as K


def _fusable(p: torch.Tensor) -> bool:
    return (p.is_cuda and p.grad is not None and not p.grad.is_sparse and p.is_contiguous()
            and p.dtype in (torch.float32, torch.bfloat16) and p.grad.dtype in (torch.float32, torch.bfloat16))


class _FusedMixin:
    def _weights(self, ps: List[torch.Tensor]):
        """fp32 weights the kernel updates, and the bf16 parameters it also writes (or None)."""
        masters, models = [], []
        for p in ps:
            st = self.state[p]
            if p.dtype == torch.float32:
                masters.append(p.data.view(-1))
                models.append(None)
            else:
                if "master" not in st:
                    st["master"] = p.detach().float().clone()
                masters.append(st["master"].view(-1))
                models.append(p.data.view(-1))
        return masters, models

    def _by_grad_dtype(self, ps: List[torch.Tensor]) -> Dict:
        out: Dict = {}
        for p in ps:
            out.setdefault((p.dtype, p.grad.dtype), []).append(p)
        return out

    def _run(self, ps, algo, flags, states, **hyper) -> None:
        masters, models = self._weights(ps)
        has_model = models[0] is not None
        grads = [p.grad.contiguous().view(-1) for p in ps]
        found_inf = getattr(self, "found_inf", None)
        gs = getattr(self, "grad_scale", None)
        K.optim_multi_(algo, flags, masters, *states, grads, models if has_model else None,
                       grad_scale=1.0 / float(gs) if gs is not None else 1.0, found_inf=found_inf, **hyper)


class SGD(_FusedMixin, _SGD):
    @torch.no_grad()
    def step(self, closure=None):
        if not all(_fusable(p) for g in self.param_groups for p in g["params"] if p.grad is not None) or \
                any(g.get("differentiable") for g in self.param_groups):
            return super().step(closure)
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            mom = group["momentum"]
            with_grad = [p for p in group["params"] if p.grad is not None]
            first = [p for p in with_grad if mom != 0 and "momentum_buffer" not in self.state[p]]
            for subset, is_first in ((first, True), ([p for p in with_grad if p not in set(first)], False)):
                for (_, _), ps in self._by_grad_dtype(subset).items():
                    flags = (K.FLAG_NESTEROV if group["nesterov"] else 0) | (K.FLAG_MAXIMIZE if group["maximize"] else 0)
                    bufs = None
                    if mom != 0:
                        flags |= K.FLAG_MOMENTUM | (K.FLAG_FIRST_STEP if is_first else 0)
                        for p in ps:
                            if "momentum_buffer" not in self.state[p] or self.state[p]["momentum_buffer"] is None:
                                self.state[p]["momentum_buffer"] = torch.zeros_like(p, dtype=torch.float32)
                        bufs = [self.state[p]["momentum_buffer"].view(-1) for p in ps]
                    self._run(ps, K.OPT_SGD, flags, (bufs, None, None), lr=float(group["lr"]),
                              weight_decay=group["weight_decay"], a=mom, b=group["dampening"])
        return loss


class Adagrad(_FusedMixin, _Adagrad):
    @torch.no_grad()
    def step(self, closure=None):
        if not all(_fusable(p) for g in self.param_groups for p in g["params"] if p.grad is not None):
            return super().step(closure)
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            by_step: Dict = {}
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                st["step"] += 1
                if st["sum"].dtype != torch.float32:
                    st["sum"] = st["sum"].float()
                by_step.setdefault((int(st["step"]), p.dtype, p.grad.dtype), []).append(p)
            for (step, _, _), ps in by_step.items():
                clr = float(group["lr"]) / (1 + (step - 1) * group["lr_decay"])
                sums = [self.state[p]["sum"].view(-1) for p in ps]
                self._run(ps, K.OPT_ADAGRAD, K.FLAG_MAXIMIZE if group["maximize"] else 0, (sums, None, None),
                          lr=clr, weight_decay=group["weight_decay"], eps=group["eps"])
        return loss


class RMSprop(_FusedMixin, _RMSprop):
    @torch.no_grad()
    def step(self, closure=None):
        if not all(_fusable(p) for g in self.param_groups for p in g["params"] if p.grad is not None):
            return super().step(closure)
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            with_grad = [p for p in group["params"] if p.grad is not None]
            for p in with_grad:
                st = self.state[p]
                if not st:
                    st["step"] = torch.tensor(0.0)
                    st["square_avg"] = torch.zeros_like(p, dtype=torch.float32)
                    if group["momentum"] > 0:
                        st["momentum_buffer"] = torch.zeros_like(p, dtype=torch.float32)
                    if group["centered"]:
                        st["grad_avg"] = torch.zeros_like(p, dtype=torch.float32)
                st["step"] += 1
            for (_, _), ps in self._by_grad_dtype(with_grad).items():
                flags = (K.FLAG_MAXIMIZE if group["maximize"] else 0) | (K.FLAG_CENTERED if group["centered"] else 0) | \
                        (K.FLAG_MOMENTUM if group["momentum"] > 0 else 0)
                sq = [self.state[p]["square_avg"].view(-1) for p in ps]
                mb = [self.state[p]["momentum_buffer"].view(-1) for p in ps] if group["momentum"] > 0 else None
                ga = [self.state[p]["grad_avg"].view(-1) for p in ps] if group["centered"] else None
                self._run(ps, K.OPT_RMSPROP, flags, (sq, mb, ga), lr=float(group["lr"]),
                          weight_decay=group["weight_decay"], a=group["alpha"], b=group["momentum"], eps=group["eps"])
        return loss


class Adafactor(_Adafactor):
    """torch's Adafactor (same arguments, state keys and rule; the reference's fused kernels are
    p10/include/OptimizerMTA.cuh:1522-1753) with the step of every vector and matrix parameter on CUDA
    done by ``tpb_adafactor_step``: two launches for a vector, four for a matrix, every norm and mean
    of the rule kept on the device. State is fp32 (bf16 parameters keep an fp32 ``master``). Tensors of
    three or more dimensions, CPU tensors and other dtypes take torch's step of the same class."""

    @torch.no_grad()
    def step(self, closure=None):
        fusable = [p for g in self.param_groups for p in g["params"] if p.grad is not None]
        if not fusable or not all(_fusable(p) and p.dim() in (1, 2) for p in fusable) or \
                any(isinstance(g["lr"], torch.Tensor) for g in self.param_groups):
            return super().step(closure)
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        found_inf = getattr(self, "found_inf", None)
        gs = getattr(self, "grad_scale", None)
        grad_scale = 1.0 / float(gs) if gs is not None else 1.0
        for group in self.param_groups:
            eps1, eps2 = group["eps"]
            lr = float(group["lr"])
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if len(st) == 0:
                    st["step"] = torch.tensor(0.0)
                    if p.dim() > 1:
                        st["row_var"] = torch.zeros(p.shape[0], 1, dtype=torch.float32, device=p.device)
                        st["col_var"] = torch.zeros(1, p.shape[1], dtype=torch.float32, device=p.device)
                    else:
                        st["variance"] = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
                for key in ("row_var", "col_var", "variance"):
                    if key in st and st[key].dtype != torch.float32:
                        st[key] = st[key].float()
                st["step"] += 1
                step = float(st["step"])
                if p.dtype == torch.float32:
                    master, model = p.data, None
                else:
                    if "master" not in st:
                        st["master"] = p.detach().float().clone()
                    master, model = st["master"], p.data
                e1 = eps1 if eps1 is not None else torch.finfo(p.dtype).eps
                grad = p.grad.contiguous()
                K.adafactor_step_(master, grad, model, st.get("row_var"), st.get("col_var"), st.get("variance"), st,
                                  lr=lr, weight_decay=group["weight_decay"], eps1=e1, eps2=eps2, d=group["d"],
                                  omb2=step ** group["beta2_decay"], rho=min(lr, 1.0 / (step ** 0.5)),
                                  grad_scale=-grad_scale if group["maximize"] else grad_scale, found_inf=found_inf)
        return loss
