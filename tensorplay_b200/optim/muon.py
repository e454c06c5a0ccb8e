"""Muon: momentum + Newton-Schulz orthogonalisation of 2-D updates (matrix parameters only).

The quintic Newton-Schulz iteration runs in bf16 on the tcgen05 GEMM when the matrices live
on a CUDA device; other parameters should be given to AdamW.
"""
from __future__ import annotations

import torch
from torch.optim import Optimizer

from .. import ops


def _mm_nt(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``a @ b.T`` for 2-D tensors."""
    if a.is_cuda and a.dtype == torch.bfloat16 and a.shape[1] % 8 == 0:
        return ops.gemm(a.contiguous(), b.contiguous())
    return a @ b.t()


def newton_schulz(g: torch.Tensor, steps: int = 5, eps: float = 1e-7) -> torch.Tensor:
    """Approximate the orthogonal polar factor of ``g`` (2-D)."""
    a, b, c = 3.4445, -4.7750, 2.0315
    x = g.to(torch.bfloat16) if g.is_cuda else g.float()
    transposed = x.shape[0] > x.shape[1]
    if transposed:
        x = x.t().contiguous()
    x = x / (x.float().norm() + eps).to(x.dtype)
    for _ in range(steps):
        A = _mm_nt(x, x)                      # X X^T
        B = b * A + c * _mm_nt(A, A)          # A is symmetric: A A^T = A^2
        x = a * x + _mm_nt(B, x.t().contiguous())  # B X
    if transposed:
        x = x.t()
    return x.to(g.dtype)


class Muon(Optimizer):
    def __init__(self, params, lr: float = 0.02, momentum: float = 0.95, nesterov: bool = True,
                 ns_steps: int = 5, weight_decay: float = 0.0):
        defaults = dict(lr=lr, momentum=momentum, nesterov=nesterov, ns_steps=ns_steps,
                        weight_decay=weight_decay)
        super().__init__(params, defaults)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                if p.dim() != 2:
                    raise ValueError("Muon handles 2-D parameters only; give the rest to AdamW")
                g = p.grad
                st = self.state[p]
                if "momentum_buffer" not in st:
                    st["momentum_buffer"] = torch.zeros_like(g, dtype=torch.float32)
                buf = st["momentum_buffer"]
                buf.mul_(group["momentum"]).add_(g.float())
                upd = g.float().add(buf, alpha=group["momentum"]) if group["nesterov"] else buf
                o = newton_schulz(upd, group["ns_steps"]).float()
                scale = max(1.0, p.shape[0] / p.shape[1]) ** 0.5
                if group["weight_decay"]:
                    p.mul_(1 - group["lr"] * group["weight_decay"])
                p.add_(o.to(p.dtype), alpha=-group["lr"] * scale)
        return loss
