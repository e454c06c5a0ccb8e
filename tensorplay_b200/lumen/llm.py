"""Interpretability tools for decoder language models (the reference's ``lumen/llm``:
logit_lens.py, patching.py, attention.py; ``_core/llm_attr.py``)."""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence

import torch
from torch import Tensor, nn


def _block_outputs(model: nn.Module, layers: Sequence[nn.Module], run: Callable[[], Tensor]):
    acts: List[Tensor] = []
    hs = [l.register_forward_hook(lambda m, i, o: acts.append((o[0] if isinstance(o, tuple) else o).detach()))
          for l in layers]
    try:
        out = run()
    finally:
        for h in hs:
            h.remove()
    return out, acts


def logit_lens(model: nn.Module, tokens: Tensor, layers: Optional[Sequence[nn.Module]] = None,
               head: Optional[Callable[[Tensor], Tensor]] = None) -> Tensor:
    """Logits decoded from the residual stream after every block: ``[layers, B, T, V]``. ``head``
    maps hidden states to logits (default: the model's ``head`` method: final norm + LM head)."""
    layers = list(model.layers) if layers is None else list(layers)
    head = head or model.head
    with torch.no_grad():
        _, acts = _block_outputs(model, layers, lambda: model(tokens))
        return torch.stack([head(a) for a in acts])


def activation_patching(model: nn.Module, clean_tokens: Tensor, corrupt_tokens: Tensor,
                        metric: Callable[[Tensor], Tensor], layers: Optional[Sequence[nn.Module]] = None,
                        positions: Optional[Sequence[int]] = None) -> Tensor:
    """Causal tracing: run the corrupted prompt with one (layer, position) of the residual stream
    restored from the clean run; returns ``metric(logits)`` for every choice, ``[layers, positions]``."""
    layers = list(model.layers) if layers is None else list(layers)
    with torch.no_grad():
        _, clean = _block_outputs(model, layers, lambda: model(clean_tokens))
        T = clean_tokens.shape[1]
        positions = list(range(T)) if positions is None else list(positions)
        out = torch.zeros(len(layers), len(positions))
        for li, layer in enumerate(layers):
            for pi, pos in enumerate(positions):
                def hook(m, i, o, li=li, pos=pos):
                    t = (o[0] if isinstance(o, tuple) else o).clone()
                    t[:, pos] = clean[li][:, pos]
                    return (t,) + tuple(o[1:]) if isinstance(o, tuple) else t
                h = layer.register_forward_hook(hook)
                try:
                    out[li, pi] = float(metric(model(corrupt_tokens)))
                finally:
                    h.remove()
    return out


def attention_rollout(attentions: Sequence[Tensor], residual: bool = True) -> Tensor:
    """Product over layers of the head-averaged attention maps (with the identity mixed in for the
    residual connection): ``[B, T, T]`` token-to-token influence."""
    roll = None
    for a in attentions:
        m = a.mean(1)
        if residual:
            eye = torch.eye(m.shape[-1], dtype=m.dtype, device=m.device)
            m = 0.5 * m + 0.5 * eye
        m = m / m.sum(-1, keepdim=True)
        roll = m if roll is None else m @ roll
    return roll


class LLMGradientAttribution:
    """Token attribution of a continuation's log-probability by gradient x embedding."""

    def __init__(self, model: nn.Module, embed: Callable[[Tensor], Tensor], forward_embeds: Callable[[Tensor], Tensor]):
        self.model, self.embed, self.forward_embeds = model, embed, forward_embeds

    def attribute(self, prompt: Tensor, continuation: Tensor) -> Dict[str, Tensor]:
        toks = torch.cat((prompt, continuation), 1)
        with torch.enable_grad():
            e = self.embed(toks).detach().requires_grad_()
            logits = self.forward_embeds(e)
            lp = torch.log_softmax(logits.float(), -1)
            P = prompt.shape[1]
            sel = lp[:, P - 1: -1].gather(-1, continuation[..., None])[..., 0]   # log p of each continuation token
            total = sel.sum()
            g = torch.autograd.grad(total, e)[0]
        scores = (g * e).sum(-1).detach()
        return {"token_attr": scores, "log_prob": sel.detach(), "seq_attr": scores[:, :P]}


# the reference has a package at this path: deeper module names resolve to views of the pack
__path__: list = []
