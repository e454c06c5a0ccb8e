"""Token-level ops around the transformer body: embedding (gather / scatter-add backward),
KV-cache append (contiguous and paged) and top-k / top-p sampling.

CUDA tensors run ``csrc/kernels/decode_ops.cu``; CPU tensors run the PyTorch expressions below.
Capability reference: p10/src/backend/cuda/EmbeddingKernels.cu, SamplingKernels.cu:350,
tensorplay/nn/cache.py:51-457, tensorplay/nn/generation.py:73-164.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from .. import _native
from ._common import lib, ptr, stream_ptr, use_native


class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight):
        ctx.save_for_backward(ids)
        ctx.wshape, ctx.wdtype = weight.shape, weight.dtype
        # an engine may own the gradient storage; its view is bound only by the time backward runs
        ctx.weight_ref = weight if hasattr(weight, "_tpb_grad_view") else None
        return embedding_forward(ids, weight)

    @staticmethod
    def backward(ctx, dy):
        (ids,) = ctx.saved_tensors
        w = ctx.weight_ref
        dst = None if w is None else w._tpb_grad_view
        if dst is not None:
            # engine-owned flat gradient: accumulate in place, nothing flows through autograd
            if not getattr(w, "_tpb_grad_written", False):
                dst.zero_()
                w._tpb_grad_written = True
            embedding_backward_(dst, ids, dy)
            return None, None
        dw = torch.zeros(ctx.wshape, dtype=ctx.wdtype, device=dy.device)
        embedding_backward_(dw, ids, dy)
        return None, dw


def embedding_forward(ids: Tensor, weight: Tensor) -> Tensor:
    H = weight.shape[1]
    if use_native(ids, weight) and weight.dtype == torch.bfloat16 and H % 8 == 0 and weight.is_contiguous():
        flat = ids.reshape(-1).to(torch.int64).contiguous()
        out = torch.empty(flat.numel(), H, dtype=weight.dtype, device=weight.device)
        _native.check(lib().tpb_embedding_fwd(ptr(flat), ptr(weight), ptr(out), flat.numel(), H,
                                              weight.shape[0], stream_ptr()), "tpb_embedding_fwd")
        return out.view(*ids.shape, H)
    return weight.index_select(0, ids.reshape(-1)).view(*ids.shape, H)


def embedding_backward_(dw: Tensor, ids: Tensor, dy: Tensor) -> Tensor:
    """``dw[ids[i]] += dy[i]`` in place (``dw`` bf16 or fp32)."""
    H = dw.shape[1]
    dy2 = dy.reshape(-1, H)
    if (use_native(dw, ids, dy2) and dy2.dtype == torch.bfloat16 and H % 2 == 0 and dw.is_contiguous()
            and dw.dtype in (torch.bfloat16, torch.float32)):
        flat = ids.reshape(-1).to(torch.int64).contiguous()
        _native.check(lib().tpb_embedding_bwd(ptr(flat), ptr(dy2.contiguous()), ptr(dw), flat.numel(), H,
                                              dw.shape[0], int(dw.dtype == torch.float32), stream_ptr()),
                      "tpb_embedding_bwd")
        return dw
    return dw.index_add_(0, ids.reshape(-1), dy2.to(dw.dtype))


def embedding(ids: Tensor, weight: Tensor) -> Tensor:
    """Differentiable row gather."""
    if weight.requires_grad and torch.is_grad_enabled():
        return _EmbeddingFn.apply(ids, weight)
    return embedding_forward(ids, weight)


def kv_append(cache: Tensor, new: Tensor, pos, block_table: Optional[Tensor] = None,
              block_size: int = 0) -> Tensor:
    """Write ``new`` [B, H, T, D] into a cache at token position ``pos`` (int, or int32 tensor [B]).

    Contiguous cache: ``cache`` is [B, H, S, D]. Paged cache: ``cache`` is the page pool
    [num_blocks, H, block_size, D] and ``block_table`` int32 [B, max_blocks] maps logical to
    physical pages.
    """
    B, H, T, D = new.shape
    pos_t = pos if isinstance(pos, Tensor) else None
    if use_native(cache, new) and new.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16 and D % 8 == 0 \
            and new.stride(3) == 1 and cache.stride(3) == 1 \
            and all(s % 8 == 0 for s in new.stride()[:3] + cache.stride()[:3]):
        bt = None if block_table is None else block_table.to(torch.int32).contiguous()
        pt = None if pos_t is None else pos_t.to(torch.int32).contiguous()
        _native.check(lib().tpb_kv_append(
            ptr(new), ptr(cache), ptr(pt), ptr(bt), 0 if pos_t is not None else int(pos), B, T, H, D,
            block_size, 0 if bt is None else bt.shape[1], new.stride(0), new.stride(2), new.stride(1),
            cache.stride(0), cache.stride(2), cache.stride(1), stream_ptr()), "tpb_kv_append")
        return cache
    for b in range(B):
        p0 = int(pos_t[b]) if pos_t is not None else int(pos)
        for t in range(T):
            at = p0 + t
            if block_table is None:
                cache[b, :, at] = new[b, :, t]
            else:
                cache[int(block_table[b, at // block_size]), :, at % block_size] = new[b, :, t]
    return cache


def decode_qkv_prep(qkv: Tensor, cos: Tensor, sin: Tensor, pos: Tensor, num_heads: int, num_kv_heads: int,
                    k_cache: Tensor, v_cache: Tensor) -> Tensor:
    """One decode step's QKV projection ``[B, Hq + 2 Hkv, D]`` -> rotated queries ``[B, Hq, D]``; the rotated keys
    and the values are written into the caches ``[B, S, Hkv, D]`` at row ``pos[b]`` (int32 ``[B]``, also the
    rotary position). One launch for the rotation and both appends (NeoX half-split rotation)."""
    B, heads, D = qkv.shape
    Hq, Hkv = num_heads, num_kv_heads
    assert heads == Hq + 2 * Hkv and k_cache.shape == v_cache.shape and k_cache.stride() == v_cache.stride()
    if use_native(qkv, k_cache) and qkv.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and D % 16 == 0 \
            and qkv.stride(2) == 1 and qkv.stride(1) == D and k_cache.stride(3) == 1 and pos.dtype == torch.int32:
        q = torch.empty((B, Hq, D), dtype=qkv.dtype, device=qkv.device)
        _native.check(lib().tpb_decode_qkv_prep(
            ptr(qkv), ptr(q), ptr(k_cache), ptr(v_cache), ptr(cos), ptr(sin), ptr(pos), B, Hq, Hkv, D,
            k_cache.shape[1], cos.shape[0], qkv.stride(0), k_cache.stride(0), k_cache.stride(1), k_cache.stride(2),
            stream_ptr()), "tpb_decode_qkv_prep")
        return q
    from .rope import _rope_ref
    pos64 = pos.to(torch.int64)
    qk = _rope_ref(qkv[:, None, : Hq + Hkv], cos, sin, pos64.view(B, 1), False, 1.0)[:, 0]
    idx = torch.arange(B, device=qkv.device)
    k_cache[idx, pos64] = qk[:, Hq:].to(k_cache.dtype)
    v_cache[idx, pos64] = qkv[:, Hq + Hkv:].to(v_cache.dtype)
    return qk[:, :Hq].contiguous()


def sample_reference(logits: Tensor, uniform: Tensor, temperature: float = 1.0, top_k: int = 0,
                     top_p: float = 1.0) -> Tensor:
    """Oracle of ``sample``: same support rule and the same inverse CDF in index order."""
    x = logits.float() / temperature
    V = x.shape[-1]
    keep = torch.ones_like(x, dtype=torch.bool)
    if 0 < top_k < V:
        kth = torch.topk(x, top_k, dim=-1).values[..., -1:]
        keep &= x >= kth
    w = torch.where(keep, torch.exp(x - x.amax(dim=-1, keepdim=True)), torch.zeros_like(x))
    if top_p < 1.0:
        z = w.sum(-1, keepdim=True)
        sw, idx = torch.sort(torch.where(keep, x, torch.full_like(x, float("-inf"))), descending=True, dim=-1)
        sp = torch.gather(w, -1, idx)
        # mass of strictly larger logits (ties share the mass above the tie group)
        csum = sp.cumsum(-1) - sp
        first_of_tie = torch.ones_like(sw, dtype=torch.bool)
        first_of_tie[..., 1:] = sw[..., 1:] != sw[..., :-1]
        above = torch.where(first_of_tie, csum, torch.zeros_like(csum)).cummax(-1).values
        keep_sorted = above <= top_p * z
        keep = torch.zeros_like(keep).scatter(-1, idx, keep_sorted) & keep
        w = torch.where(keep, w, torch.zeros_like(w))
    cdf = w.cumsum(-1)
    target = uniform.reshape(-1, 1).float() * cdf[..., -1:]
    return (cdf <= target).sum(-1).clamp_(max=V - 1)


def sample(logits: Tensor, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0,
           uniform: Optional[Tensor] = None, generator=None) -> Tensor:
    """One token id per row of ``logits`` [rows, V] from the tempered top-k / top-p distribution."""
    rows, V = logits.shape
    if uniform is None:
        uniform = torch.rand(rows, device=logits.device, generator=generator)
    if use_native(logits) and logits.dtype in (torch.float32, torch.bfloat16) and logits.stride(1) == 1:
        out = torch.empty(rows, dtype=torch.int64, device=logits.device)
        u = uniform.float().contiguous()
        _native.check(lib().tpb_sample(ptr(logits), ptr(u), ptr(out), None, rows, V, logits.stride(0),
                                       int(logits.dtype == torch.float32), float(max(temperature, 1e-6)),
                                       int(top_k), float(top_p), stream_ptr()), "tpb_sample")
        return out
    return sample_reference(logits, uniform, max(temperature, 1e-6), top_k, top_p)
