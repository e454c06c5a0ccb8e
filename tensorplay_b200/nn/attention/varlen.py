"""Variable-length attention over packed sequences.

``query [total_q, Hq, D]``, ``key / value [total_k, Hkv, D]`` hold the tokens of all sequences back
to back; ``cu_seq_q / cu_seq_k`` (int32, ``[n + 1]``) are the cumulative lengths. Self-attention over
the packed tokens (``cu_seq_q == cu_seq_k``; causal, optionally with a left window) is ONE launch of
the tcgen05 flash kernels over the whole packed row: every token carries the bounds of its sequence,
query tiles skip the KV blocks of other sequences and mask inside the blocks on a boundary. Cross
attention between packed sets of different lengths takes one launch per sequence on strided views
(no padding, no copy); a right-bounded non-causal window and head dims other than 64 / 128 run the
fp32 formula per sequence. Differentiable. (tensorplay/nn/attention/varlen.py:287 ``varlen_attn``; the reference's
kernels take ``cu_seqlens`` inside one launch, p10/src/backend/cuda/transformers/AttentionKernels.cu:1782-1969.)
"""
from __future__ import annotations

import math
from typing import NamedTuple, Optional, Sequence

import torch


class AuxRequest(NamedTuple):
    lse: bool = False


def _window_math(q, k, v, causal, scale, window):
    """fp32 attention of one sequence ``[T, H, D]`` with a (left, right) window; -1 = unbounded."""
    Tq, Hq, D = q.shape
    Tk, Hkv = k.shape[0], k.shape[1]
    g = Hq // Hkv
    kf = k.float().repeat_interleave(g, dim=1)
    vf = v.float().repeat_interleave(g, dim=1)
    s = torch.einsum("qhd,khd->hqk", q.float(), kf) * scale
    i = torch.arange(Tq, device=q.device).view(-1, 1) + (Tk - Tq)
    j = torch.arange(Tk, device=q.device).view(1, -1)
    ok = torch.ones(Tq, Tk, dtype=torch.bool, device=q.device)
    left, right = window
    if causal:
        right = 0 if right < 0 else min(right, 0)
    if left >= 0:
        ok &= j >= i - left
    if right >= 0:
        ok &= j <= i + right
    s = s.masked_fill(~ok, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.softmax(s, dim=-1).nan_to_num(0.0)
    return torch.einsum("hqk,khd->qhd", p, vf).to(q.dtype), lse


def varlen_attn(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, cu_seq_q: torch.Tensor,
                cu_seq_k: torch.Tensor, max_q: int, max_k: int, is_causal: bool = False,
                return_aux: Optional[AuxRequest] = None, scale: Optional[float] = None,
                window_size: Optional[Sequence[int]] = None):
    if query.dim() != 3 or key.dim() != 3 or value.dim() != 3:
        raise ValueError("varlen_attn expects packed [total_tokens, heads, head_dim] tensors")
    window = (-1, -1) if window_size is None else tuple(window_size)
    if len(window) != 2:
        raise ValueError(f"window_size must have length 2, got {len(window)}")
    if scale is not None and not scale > 0:
        raise ValueError("scale must be positive")
    D = query.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    bq, bk = cu_seq_q.tolist(), cu_seq_k.tolist()
    if len(bq) != len(bk) or bq[-1] != query.shape[0] or bk[-1] != key.shape[0]:
        raise ValueError("cumulative sequence lengths do not match the packed tensors")
    want_lse = bool(return_aux and return_aux.lse)
    use_kernel = (window == (-1, -1) and not want_lse and query.is_cuda and query.dtype == torch.bfloat16
                  and D in (64, 128))
    from . import _flash
    left, right = window
    one_launch = (query.is_cuda and query.dtype == torch.bfloat16 and D in (64, 128) and not want_lse and bq == bk
                  and key.shape[0] == query.shape[0] and max(a1 - a0 for a0, a1 in zip(bq[:-1], bq[1:])) <= max_q
                  and (right < 0 or (is_causal and right >= 0)) and (is_causal or left < 0))
    if one_launch:
        from ...ops.attention import flash_attention, segment_bounds
        seg_start, seg_end = segment_bounds(cu_seq_q.to(query.device), query.shape[0])
        return flash_attention(query.unsqueeze(0), key.unsqueeze(0), value.unsqueeze(0), causal=is_causal,
                               scale=scale, window=(left + 1) if left >= 0 else 0,
                               seg_start=seg_start.view(1, -1), seg_end=seg_end.view(1, -1)).squeeze(0)
    outs, lses = [], []
    for a0, a1, b0, b1 in zip(bq[:-1], bq[1:], bk[:-1], bk[1:]):
        if a1 - a0 > max_q or b1 - b0 > max_k:
            raise ValueError("a sequence is longer than max_q / max_k")
        q, k, v = query[a0:a1], key[b0:b1], value[b0:b1]
        if a1 == a0:
            continue
        if use_kernel and b1 > b0:
            outs.append(_flash(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), is_causal, scale).squeeze(0))
        else:
            o, lse = _window_math(q, k, v, is_causal, scale, window)
            outs.append(o)
            lses.append(lse)
    out = torch.cat(outs, dim=0) if outs else query.new_zeros(query.shape)
    if want_lse:
        return out, torch.cat(lses, dim=1) if lses else query.new_zeros(query.shape[1], 0, dtype=torch.float32)
    return out
