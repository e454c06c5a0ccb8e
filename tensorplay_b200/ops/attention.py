"""Flash attention (GQA-native, causal / full) on the tcgen05 kernels.

Layout is token-major ``[B, T, H, D]`` with arbitrary token / head / batch strides, so q, k
and v may be slices of one fused QKV projection buffer.

Reference counterparts: FlashAttention-2 sm80 forward/backward leaves
(p10/src/backend/cuda/transformers/AttentionKernels.cu:1782-1969, :2286-2543) behind
``scaled_dot_product_attention`` (tensorplay/nn/functional.py:3589-3615); the reference expands
K/V to the query head count for GQA training (:3571-3586) while these kernels take grouped
heads natively and reduce dK/dV over the group inside the kernel.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import _native
from . import _ckpt
from ._common import lib, status_word, stream_ptr, use_native


def _strides_ok(t: torch.Tensor) -> bool:
    return t.stride(3) == 1 and all(s % 8 == 0 for s in t.stride()[:3]) and t.data_ptr() % 16 == 0


def segment_bounds(cu_seqlens: torch.Tensor, total: int):
    """Per-token ``(seg_start, seg_end)`` int32 arrays of ``total`` packed tokens whose sequence boundaries are
    ``cu_seqlens`` (``[n + 1]``, first 0, last ``total``): token ``i`` of sequence ``s`` gets
    ``(cu_seqlens[s], cu_seqlens[s + 1])``."""
    cu = cu_seqlens.to(torch.int64)
    pos = torch.arange(total, device=cu.device)
    seq = torch.searchsorted(cu[1:].contiguous(), pos, right=True).clamp_(max=cu.numel() - 2)
    return cu[seq].to(torch.int32).contiguous(), cu[seq + 1].to(torch.int32).contiguous()


def attention_reference(q, k, v, causal: bool = True, scale: Optional[float] = None, window: int = 0,
                        seg_start: Optional[torch.Tensor] = None, seg_end: Optional[torch.Tensor] = None):
    """Plain fp32 attention in ``[B, T, H, D]`` layout (the correctness oracle). ``window`` / ``seg_start`` /
    ``seg_end`` as in :func:`flash_attention`; a query without any admissible key gives zeros."""
    B, Tq, Hq, D = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    g = Hq // Hkv
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    i = torch.arange(Tq, device=q.device).view(-1, 1)
    j = torch.arange(Tk, device=q.device).view(1, -1)
    if causal:
        s = s.masked_fill(j > i + (Tk - Tq), float("-inf"))
    if window and window > 0:
        s = s.masked_fill(j < i + (Tk - Tq) - window + 1, float("-inf"))
    if seg_start is not None:
        s = s.masked_fill((j.view(1, 1, 1, Tk) < seg_start.view(B, 1, Tq, 1)), float("-inf"))
    if seg_end is not None:
        s = s.masked_fill((j.view(1, 1, 1, Tk) >= seg_end.view(B, 1, Tq, 1)), float("-inf"))
    empty = torch.isinf(s).all(dim=-1, keepdim=True)
    p = torch.softmax(s.masked_fill(empty, 0.0), dim=-1).masked_fill(empty, 0.0)
    o = torch.matmul(p, vf)
    return o.permute(0, 2, 1, 3).to(q.dtype)


def flash_fwd(q, k, v, causal: bool, scale: float, kv_len: Optional[torch.Tensor] = None, n_splits: int = 1,
              window: int = 0, seg_start: Optional[torch.Tensor] = None, seg_end: Optional[torch.Tensor] = None,
              out: Optional[torch.Tensor] = None):
    """Forward kernel. ``kv_len`` (int32 device scalar) limits the keys to the first ``kv_len`` of
    ``k``/``v`` without a host-side shape change, so that a decode step over a preallocated cache
    can be captured in a CUDA graph. ``n_splits > 1`` (non-causal, i.e. decode) spreads the keys of
    every (batch, head) over that many CTAs and merges the partial outputs by their LSE. ``out``: a
    ``[B, Tq, Hq, D]`` view (any batch / token / head strides, contiguous ``D``) that receives the output, e.g.
    one laid out for the projection that follows."""
    B, Tq, Hq, D = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    if out is not None:
        if out.shape != (B, Tq, Hq, D) or out.stride(3) != 1 or out.dtype != q.dtype or \
                any(s % 8 for s in out.stride()[:3]) or out.data_ptr() % 16:
            raise ValueError("flash_fwd: out must be [B, Tq, Hq, D] with contiguous D and 16-byte aligned rows")
        o = out
    else:
        o = torch.empty((B, Tq, Hq, D), dtype=q.dtype, device=q.device)
    # rows padded to the backward kernels' 64-query vector loads
    lse_stride = (Tq + 127) // 128 * 128
    lse = torch.empty((B, Hq, lse_stride), dtype=torch.float32, device=q.device)
    n_splits = max(1, min(int(n_splits), (Tk + 127) // 128)) if not causal else 1
    if n_splits > 1:
        part = torch.empty((n_splits, B, Tq, Hq, D), dtype=q.dtype, device=q.device)
        lse_part = torch.empty((n_splits, B, Hq, lse_stride), dtype=torch.float32, device=q.device)
        dst, dst_lse = part[0], lse_part
        o_split, lse_split = part.stride(0), lse_part.stride(0)
    else:
        dst, dst_lse, o_split, lse_split = o, lse, 0, 0
    code = lib().tpb_flash_fwd_ex(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), dst.data_ptr(), dst_lse.data_ptr(), B, Tq, Tk, Hq, Hkv,
        D, q.stride(1), q.stride(2), q.stride(0), k.stride(1), k.stride(2), k.stride(0),
        v.stride(1), v.stride(2), v.stride(0), dst.stride(1), dst.stride(2), dst.stride(0), lse_stride,
        int(causal), float(scale), status_word(q.device).data_ptr(), stream_ptr(),
        None if kv_len is None else kv_len.data_ptr(), n_splits, o_split, lse_split, int(window or 0),
        None if seg_start is None else seg_start.data_ptr(), None if seg_end is None else seg_end.data_ptr())
    _native.check(code, "tpb_flash_fwd")
    if _native.flop_sinks:   # QK^T and PV over the unmasked part (a causal square is half full)
        _native.add_flops("tpb.flash_attention_forward", 4 * B * Hq * Tq * Tk * D // (2 if causal and Tq == Tk else 1))
    if n_splits > 1:
        code = lib().tpb_attn_split_merge(part.data_ptr(), lse_part.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                          n_splits, B, Tq, Hq, D, o_split, lse_split, lse_stride, o.stride(1),
                                          o.stride(2), o.stride(0), stream_ptr())
        _native.check(code, "tpb_attn_split_merge")
    return o, lse


def flash_bwd(do, q, k, v, o, lse, causal: bool, scale: float, dq=None, dk=None, dv=None, window: int = 0,
              seg_start: Optional[torch.Tensor] = None, seg_end: Optional[torch.Tensor] = None):
    """Backward of ``flash_fwd``. ``dq``/``dk``/``dv`` may be preallocated (strided) views, e.g.
    slices of one fused dQKV buffer; ``dk`` and ``dv`` must share their strides."""
    B, Tq, Hq, D = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    if dq is None:
        dq = torch.empty((B, Tq, Hq, D), dtype=q.dtype, device=q.device)
    if dk is None:
        dk = torch.empty((B, Tk, Hkv, D), dtype=q.dtype, device=q.device)
    if dv is None:
        dv = torch.empty((B, Tk, Hkv, D), dtype=q.dtype, device=q.device)
    assert dk.stride() == dv.stride()
    delta = torch.empty_like(lse)
    if not _strides_ok(do):
        do = do.contiguous()
    code = lib().tpb_flash_bwd_ex(
        do.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
        delta.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), B, Tq, Tk, Hq, Hkv, D,
        q.stride(1), q.stride(2), q.stride(0), k.stride(1), k.stride(2), k.stride(0),
        v.stride(1), v.stride(2), v.stride(0), o.stride(1), o.stride(2), o.stride(0),
        do.stride(1), do.stride(2), do.stride(0), dq.stride(1), dq.stride(2), dq.stride(0),
        dk.stride(1), dk.stride(2), dk.stride(0), lse.shape[2], int(causal), float(scale),
        status_word(q.device).data_ptr(), stream_ptr(), int(window or 0),
        None if seg_start is None else seg_start.data_ptr(), None if seg_end is None else seg_end.data_ptr())
    _native.check(code, "tpb_flash_bwd")
    if _native.flop_sinks:   # five products: S and dP again, dV, dK, dQ
        _native.add_flops("tpb.flash_attention_backward", 10 * B * Hq * Tq * Tk * D // (2 if causal and Tq == Tk else 1))
    return dq, dk, dv


class _FlashAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale, window=0, seg_start=None, seg_end=None):
        o, lse = flash_fwd(q, k, v, causal, scale, window=window, seg_start=seg_start, seg_end=seg_end)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.causal, ctx.scale, ctx.window, ctx.seg = causal, scale, window, (seg_start, seg_end)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = flash_bwd(do, q, k, v, o, lse, ctx.causal, ctx.scale, window=ctx.window,
                               seg_start=ctx.seg[0], seg_end=ctx.seg[1])
        return dq, dk, dv, None, None, None, None, None


def flash_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True,
                    scale: Optional[float] = None, window: int = 0, seg_start: Optional[torch.Tensor] = None,
                    seg_end: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``softmax(q k^T * scale [+ mask]) v`` for ``q [B, Tq, Hq, D]``, ``k/v [B, Tk, Hkv, D]``.

    ``Hq`` must be a multiple of ``Hkv`` (grouped-query attention). With ``causal`` the last
    query is aligned with the last key. ``window > 0`` is local attention: a query sees its last
    ``window`` keys (its own position included). ``seg_start`` / ``seg_end`` (int32 ``[B, Tq]``,
    non-decreasing along the sequence, see :func:`segment_bounds`) restrict query ``i`` to the keys
    ``[seg_start[i], seg_end[i])``: several sequences packed into one row attend only within
    themselves (``Tq == Tk``). The kernels skip the KV blocks that lie outside the bounds of a
    whole query tile and mask inside the blocks on their edges
    (p10/src/backend/cuda/transformers/AttentionKernels.cu:1907-1918 has the window of the reference).
    """
    D = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if (seg_start is not None or seg_end is not None) and q.shape[1] != k.shape[1]:
        raise ValueError("flash_attention: segment bounds need Tq == Tk (packed self-attention)")
    if seg_start is not None:
        seg_start = seg_start.to(torch.int32).contiguous()
    if seg_end is not None:
        seg_end = seg_end.to(torch.int32).contiguous()
    native = (q.is_cuda and q.dtype == torch.bfloat16 and D in (64, 128) and use_native(q, k, v))
    if not native:
        if (q.is_cuda and q.dtype in (torch.bfloat16, torch.float16) and not window and seg_start is None and seg_end is None
                and (not causal or q.shape[1] == k.shape[1]) and q.shape[2] % k.shape[2] == 0):
            # head dims without a kernel here (32, 96, 256 ...): PyTorch's library attention instead of the fp32
            # formula, which materialises the whole score matrix
            o = torch.nn.functional.scaled_dot_product_attention(
                q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=causal, scale=scale,
                enable_gqa=q.shape[2] != k.shape[2])
            return o.transpose(1, 2)
        return attention_reference(q, k, v, causal, scale, window, seg_start, seg_end)
    if not _strides_ok(q):
        q = q.contiguous()
    if not _strides_ok(k):
        k = k.contiguous()
    if not _strides_ok(v):
        v = v.contiguous()
    return _FlashAttnFn.apply(q, k, v, causal, scale, int(window or 0), seg_start, seg_end)


class _QKVAttnFn(torch.autograd.Function):
    """RoPE + flash attention on a packed QKV projection ``[B, T, (Hq + 2 Hkv) * D]``.

    Forward rotates q and k out of the packed buffer into a fresh ``[B, T, Hq + Hkv, D]`` one with one launch
    (no copy before the rotation) and
    attends with v read in place from the packed buffer. Backward has the flash kernels
    write dq, dk and dv straight into the slices of one packed gradient buffer and un-rotates
    its q/k part in place, so that no concatenation or copy is needed around the projection.
    """

    @staticmethod
    def forward(ctx, qkv, cos, sin, pos, Hq, Hkv, D, causal, scale, interleaved):
        from .rope import _rope_native_out
        B, T, _ = qkv.shape
        tot = Hq + 2 * Hkv
        packed = qkv.view(B, T, tot, D)
        qk = torch.empty((B, T, Hq + Hkv, D), device=qkv.device, dtype=qkv.dtype)
        _rope_native_out(packed[:, :, : Hq + Hkv], qk, cos, sin, pos, interleaved, False)
        q, k, v = qk[:, :, :Hq], qk[:, :, Hq:], packed[:, :, Hq + Hkv:]
        kept = _ckpt.take()  # selective checkpointing: output and LSE of the first forward pass
        if kept is not None:
            o, lse = kept
        else:
            o, lse = flash_fwd(q, k, v, causal, scale)
            _ckpt.stash(o, lse)
        ctx.save_for_backward(qk, qkv, o, lse, cos, sin, pos if pos is not None else torch.empty(0))
        ctx.cfg = (Hq, Hkv, D, causal, scale, interleaved, pos is not None)
        return o.view(B, T, Hq * D)

    @staticmethod
    def backward(ctx, do):
        from .rope import _rope_native_
        qk, qkv, o, lse, cos, sin, pos = ctx.saved_tensors
        Hq, Hkv, D, causal, scale, interleaved, has_pos = ctx.cfg
        B, T, _ = qkv.shape
        tot = Hq + 2 * Hkv
        packed = qkv.view(B, T, tot, D)
        dqkv = torch.empty_like(qkv)
        dp = dqkv.view(B, T, tot, D)
        do4 = do.reshape(B, T, Hq, D)
        if not _strides_ok(do4):
            do4 = do4.contiguous()
        flash_bwd(do4, qk[:, :, :Hq], qk[:, :, Hq:], packed[:, :, Hq + Hkv:], o, lse, causal, scale,
                  dq=dp[:, :, :Hq], dk=dp[:, :, Hq:Hq + Hkv], dv=dp[:, :, Hq + Hkv:])
        _rope_native_(dp[:, :, : Hq + Hkv], cos, sin, pos if has_pos else None, interleaved, True)
        return dqkv, None, None, None, None, None, None, None, None, None


def qkv_attention(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                  position_ids: Optional[torch.Tensor], num_heads: int, num_kv_heads: int,
                  head_dim: int, causal: bool = True, scale: Optional[float] = None,
                  interleaved: bool = False) -> torch.Tensor:
    """Attention over a packed QKV projection; returns ``[B, T, num_heads * head_dim]``."""
    scale = scale if scale is not None else 1.0 / math.sqrt(head_dim)
    B, T, _ = qkv.shape
    native = (qkv.is_cuda and qkv.dtype == torch.bfloat16 and head_dim in (64, 128)
              and use_native(qkv))
    pos = None if position_ids is None else position_ids.reshape(-1).to(torch.int64).contiguous()
    if native:
        if not qkv.is_contiguous():
            qkv = qkv.contiguous()
        return _QKVAttnFn.apply(qkv, cos, sin, pos, num_heads, num_kv_heads, head_dim, causal, scale,
                                interleaved)
    from .rope import _rope_ref
    packed = qkv.view(B, T, num_heads + 2 * num_kv_heads, head_dim)
    qk = _rope_ref(packed[:, :, : num_heads + num_kv_heads], cos, sin, position_ids, interleaved, 1.0)
    o = attention_reference(qk[:, :, :num_heads], qk[:, :, num_heads:],
                            packed[:, :, num_heads + num_kv_heads:], causal, scale)
    return o.reshape(B, T, num_heads * head_dim)
