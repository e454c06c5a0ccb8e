"""Autoregressive decoding: ``generate`` with greedy / temperature / top-k / top-p sampling.

API after tensorplay/nn/generation.py:73-164.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from .cache import DynamicCache


def top_k_top_p_filtering(logits: Tensor, top_k: int = 0, top_p: float = 1.0) -> Tensor:
    """Set logits outside the top-k / nucleus support to ``-inf`` (returns a new tensor)."""
    logits = logits.clone()
    V = logits.shape[-1]
    if 0 < top_k < V:
        kth = torch.topk(logits, top_k, dim=-1).values[..., -1:]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    if top_p < 1.0:
        sorted_logits, idx = torch.sort(logits, descending=True, dim=-1)
        probs = torch.softmax(sorted_logits, dim=-1)
        cum = probs.cumsum(dim=-1)
        remove = (cum - probs) > top_p  # keep the first token that crosses the threshold
        sorted_logits = sorted_logits.masked_fill(remove, float("-inf"))
        logits = torch.full_like(logits, float("-inf")).scatter(-1, idx, sorted_logits)
    return logits


def _apply_repetition_penalty(logits: Tensor, sequences: Tensor, penalty: float) -> Tensor:
    picked = logits.gather(-1, sequences)
    picked = torch.where(picked > 0, picked / penalty, picked * penalty)
    return logits.scatter(-1, sequences, picked)


def sample(logits: Tensor, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0) -> Tensor:
    """One token id per row from the filtered, tempered distribution."""
    if logits.is_cuda and logits.dim() == 2:
        # one kernel: sort-free top-k / nucleus support + inverse-CDF draw
        from .. import ops
        return ops.sample(logits, temperature, top_k, top_p)
    scaled = logits.float() / max(temperature, 1e-6)
    filtered = top_k_top_p_filtering(scaled, top_k, top_p)
    return torch.multinomial(torch.softmax(filtered, dim=-1), num_samples=1).squeeze(-1)


@torch.no_grad()
def generate(model, input_ids: Tensor, max_new_tokens: int = 20, do_sample: bool = False,
             temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0,
             repetition_penalty: float = 1.0, eos_token_id: Optional[int] = None,
             pad_token_id: Optional[int] = None, use_cache: bool = True,
             past_key_values=None) -> Tensor:
    """Returns ``[batch, prompt_len + n_generated]`` (prompt followed by generated / pad tokens)."""
    if input_ids.dim() != 2:
        raise ValueError(f"generate: expected a [batch, prompt_len] tensor of token ids, got {input_ids.dim()} dimensions")
    B, T0 = input_ids.shape
    device = input_ids.device
    if max_new_tokens < 1:
        return input_ids
    # finished sequences are filled with the padding id; without one, the end-of-sequence id (or 0) stands in
    fill = pad_token_id
    if fill is None:
        fill = 0 if eos_token_id is None else eos_token_id
    pad_token_id = fill
    cache = past_key_values
    if use_cache and cache is None:
        # models that need a particular cache kind (static, paged, linear-state) build it themselves
        factory = getattr(model, "create_empty_cache", None)
        cache = DynamicCache() if factory is None else factory()
    past_key_values = cache
    out = torch.full((B, T0 + max_new_tokens), pad_token_id, dtype=input_ids.dtype, device=device)
    out[:, :T0] = input_ids
    finished = torch.zeros(B, dtype=torch.bool, device=device)
    cur = T0
    next_input = input_ids
    for _ in range(max_new_tokens):
        start = cur - next_input.shape[1]
        position_ids = torch.arange(start, cur, device=device).unsqueeze(0).expand(B, -1)
        logits = model(next_input, position_ids=position_ids,
                       past_key_values=past_key_values if use_cache else None)[:, -1, :]
        if not do_sample or temperature <= 1e-5:
            token = logits.argmax(dim=-1)
        else:
            lg = logits.float()
            if repetition_penalty != 1.0:
                lg = _apply_repetition_penalty(lg, out[:, :cur], repetition_penalty)
            token = sample(lg, temperature, top_k, top_p)
        token = torch.where(finished, torch.full_like(token, pad_token_id), token)
        out[:, cur] = token
        cur += 1
        if eos_token_id is not None:
            finished = finished | (token == eos_token_id)
            if bool(finished.all()):
                break
        next_input = token.unsqueeze(1) if use_cache else out[:, :cur]
    return out[:, :cur]
