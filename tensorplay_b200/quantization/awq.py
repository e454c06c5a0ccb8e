"""Activation-aware weight quantisation for the W4A16 / W8A16 layers (the reference's
``tensorplay/ao/quantization/awq.py``): input channels that carry large activations are scaled up
before rounding (and the activations down by the same factor), with the exponent of the scaling
chosen per layer to minimise the layer's output error on calibration data."""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional

import torch
from torch import Tensor, nn

from . import WeightOnlyLinear


def _fake_quant(w: Tensor, bits: int, group: int) -> Tensor:
    from ..ops import dequantize_weight, quantize_weight_int4, quantize_weight_int8
    if bits == 4:
        q, s, z = quantize_weight_int4(w, group)
        return dequantize_weight(q, s, z, 4, group).float()
    q, s = quantize_weight_int8(w, group)
    return dequantize_weight(q, s, None, 8, group).float()


def search_scales(weight: Tensor, x: Tensor, bits: int = 4, group_size: int = 128, grid: int = 20):
    """Per-input-channel scales ``s = mean|x|^alpha`` (normalised), ``alpha`` on a grid in [0, 1],
    minimising ``|| Q(W diag(s)) diag(1/s) x - W x ||``. Returns ``(scales, best_alpha, errors)``."""
    w = weight.float()
    xf = x.reshape(-1, x.shape[-1]).float()
    act = xf.abs().mean(0).clamp(min=1e-5)
    ref = xf @ w.t()
    best, best_err, best_alpha, errs = None, float("inf"), 0.0, []
    for i in range(grid + 1):
        alpha = i / grid
        s = act.pow(alpha)
        s = s / (s.max() * s.min()).sqrt()
        out = (xf / s) @ _fake_quant(w * s, bits, group_size).t()
        err = (out - ref).pow(2).mean().item()
        errs.append(err)
        if err < best_err:
            best, best_err, best_alpha = s, err, alpha
    return best, best_alpha, errs


class AWQLinear(nn.Module):
    """Weight-only quantised linear whose input is divided by the searched channel scales. (When
    the producer of the input is a norm or another linear layer, ``fold_into`` moves the division
    into that layer's weights and this wrapper becomes a plain :class:`WeightOnlyLinear`.)"""

    def __init__(self, linear: nn.Linear, scales: Tensor, bits: int = 4, group_size: int = 128):
        super().__init__()
        scaled = nn.Linear(linear.in_features, linear.out_features, bias=linear.bias is not None,
                           device=linear.weight.device, dtype=linear.weight.dtype)
        with torch.no_grad():
            scaled.weight.copy_(linear.weight.float() * scales.to(linear.weight.device))
            if linear.bias is not None:
                scaled.bias.copy_(linear.bias)
        self.inner = WeightOnlyLinear(scaled, bits, group_size)
        self.register_buffer("inv_scales", (1.0 / scales).to(linear.weight.dtype))
        self.folded = False

    def fold_into(self, producer: nn.Module) -> None:
        """Multiply the producer's output channels (a norm's weight, or a linear layer's rows and
        bias) by ``1 / s`` so that no run-time division remains."""
        with torch.no_grad():
            inv = self.inv_scales.to(producer.weight.dtype)
            if producer.weight.dim() == 1:
                producer.weight.mul_(inv)
                if getattr(producer, "bias", None) is not None:
                    producer.bias.mul_(inv)
            else:
                producer.weight.mul_(inv[:, None])
                if producer.bias is not None:
                    producer.bias.mul_(inv)
        self.folded = True

    def forward(self, x: Tensor) -> Tensor:
        return self.inner(x if self.folded else x * self.inv_scales.to(x.dtype))


def awq_quantize_(model: nn.Module, calibration: Iterable, bits: int = 4, group_size: int = 128, grid: int = 20,
                  filter_fn=None) -> Dict[str, float]:
    """Quantise every ``nn.Linear`` of ``model`` in place with searched scales. ``calibration`` yields
    model inputs (tensors or tuples); the inputs of each linear layer are captured with hooks in one
    pass. Returns the chosen exponent per layer name."""
    targets = {n: m for n, m in model.named_modules()
               if isinstance(m, nn.Linear) and (filter_fn is None or filter_fn(m, n))}
    seen: Dict[str, List[Tensor]] = {n: [] for n in targets}
    hooks = [m.register_forward_hook(lambda mod, inp, out, n=n: seen[n].append(inp[0].detach().reshape(-1, inp[0].shape[-1])))
             for n, m in targets.items()]
    with torch.no_grad():
        for batch in calibration:
            model(*batch) if isinstance(batch, (tuple, list)) else model(batch)
    for h in hooks:
        h.remove()
    chosen = {}
    for name, lin in targets.items():
        if not seen[name] or lin.in_features % group_size:
            continue
        x = torch.cat(seen[name])[:4096]
        scales, alpha, _ = search_scales(lin.weight.data, x, bits, group_size, grid)
        parent = model
        *path, leaf = name.split(".")
        for p in path:
            parent = getattr(parent, p)
        setattr(parent, leaf, AWQLinear(lin, scales, bits, group_size))
        chosen[name] = alpha
    return chosen
