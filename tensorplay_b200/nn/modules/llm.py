"""The LLM building blocks of the reference's ``nn`` package, computed by the sm_100a ops.

Public names and constructor arguments follow tensorplay/nn/modules/rotary.py:79-199
(``apply_rotary_emb``, ``RotaryEmbedding``), causal_attention.py:30-187
(``GroupedQueryAttention``) and modern_block.py:29-103 (``SwiGLUMLP``, ``TransformerBlock``);
parameter names match so that checkpoints interchange.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import Tensor
from torch.nn import Module, Parameter

from ... import ops as _ops
from ...ops.attention import flash_attention
from .. import functional as F


class Linear(torch.nn.Linear):
    """``torch.nn.Linear`` whose bf16 CUDA products run on the tcgen05 GEMM."""

    def forward(self, input: Tensor) -> Tensor:
        return F.linear(input, self.weight, self.bias)


class RMSNorm(Module):
    def __init__(self, normalized_shape, eps: Optional[float] = None, elementwise_affine: bool = True,
                 device=None, dtype=None) -> None:
        super().__init__()
        if isinstance(normalized_shape, int):
            normalized_shape = (normalized_shape,)
        self.normalized_shape = tuple(normalized_shape)
        self.eps = eps
        self.elementwise_affine = elementwise_affine
        if elementwise_affine:
            self.weight = Parameter(torch.ones(self.normalized_shape, device=device, dtype=dtype))
        else:
            self.register_parameter("weight", None)

    def forward(self, x: Tensor, residual: Optional[Tensor] = None):
        eps = self.eps if self.eps is not None else torch.finfo(x.dtype).eps
        if self.weight is not None and len(self.normalized_shape) == 1:
            w = self.weight
            if w.dtype != x.dtype:
                w = w.to(x.dtype)
            return _ops.rms_norm(x, w, eps, residual)
        if residual is not None:
            x = x + residual
            return torch.nn.functional.rms_norm(x, self.normalized_shape, self.weight, eps), x
        return torch.nn.functional.rms_norm(x, self.normalized_shape, self.weight, eps)

    def extra_repr(self) -> str:
        return f"{self.normalized_shape}, eps={self.eps}, elementwise_affine={self.elementwise_affine}"


class LayerNorm(torch.nn.LayerNorm):
    def forward(self, input: Tensor) -> Tensor:
        return F.layer_norm(input, self.normalized_shape, self.weight, self.bias, self.eps)


def _rotate_ref(x: Tensor, cos: Tensor, sin: Tensor, interleaved: bool) -> Tensor:
    # x: [B, H, T, D]; cos/sin: [B, T, R/2]
    r = cos.shape[-1] * 2
    xr, xp = x[..., :r].float(), x[..., r:]
    c = cos.float().unsqueeze(1)
    s = sin.float().unsqueeze(1)
    if interleaved:
        a, b = xr[..., 0::2], xr[..., 1::2]
        out = torch.stack((a * c - b * s, b * c + a * s), dim=-1).flatten(-2)
    else:
        a, b = xr[..., : r // 2], xr[..., r // 2:]
        out = torch.cat((a * c - b * s, b * c + a * s), dim=-1)
    out = out.to(x.dtype)
    return out if xp.shape[-1] == 0 else torch.cat((out, xp), dim=-1)


def apply_rotary_emb(q: Tensor, k: Tensor, cos: Tensor, sin: Tensor,
                     interleaved: bool = False) -> Tuple[Tensor, Tensor]:
    """Rotate the trailing ``2 * cos.shape[-1]`` dims of ``q`` and ``k`` (``[B, H, T, D]``) with
    gathered ``[B, T, R/2]`` tables."""
    return _rotate_ref(q, cos, sin, interleaved), _rotate_ref(k, cos, sin, interleaved)


class RotaryEmbedding(Module):
    """cos/sin tables for given positions. ``tables(max_pos)`` exposes the raw fp32
    ``[max_pos, dim/2]`` tables that the fused kernel indexes by position itself."""

    def __init__(self, dim: int, base: float = 10000.0, interleaved: bool = False, device=None) -> None:
        super().__init__()
        if dim % 2:
            raise ValueError(f"rotary dim must be even, got {dim}")
        self.dim = dim
        self.base = float(base)
        self.interleaved = interleaved
        inv_freq = 1.0 / (self.base ** (torch.arange(0, dim, 2, device=device, dtype=torch.float32) / dim))
        self.register_buffer("inv_freq", inv_freq, persistent=False)
        self._n = 0
        self._cos: Optional[Tensor] = None
        self._sin: Optional[Tensor] = None

    def tables(self, max_position: int, device) -> Tuple[Tensor, Tensor]:
        if self._cos is None or self._n < max_position or self._cos.device != torch.device(device):
            n = max(max_position, 2 * self._n, 16)
            cos, sin = _ops.rope_tables(n, self.dim, self.base, device=device)
            self._cos, self._sin, self._n = cos, sin, n
        return self._cos, self._sin

    def forward(self, x: Tensor, position_ids: Tensor, max_position: Optional[int] = None):
        if max_position is None:
            max_position = int(position_ids.max().item()) + 1
        cos, sin = self.tables(int(max_position), x.device)
        return cos[position_ids].to(x.dtype), sin[position_ids].to(x.dtype)

    def extra_repr(self) -> str:
        return f"dim={self.dim}, base={self.base}, interleaved={self.interleaved}"


class GroupedQueryAttention(Module):
    """Causal self-attention with grouped KV heads, optional QK-RMSNorm, RoPE and a KV cache."""

    def __init__(self, embed_dim: int, num_heads: int, num_kv_heads: Optional[int] = None,
                 head_dim: Optional[int] = None, dropout: float = 0.0, bias: bool = False,
                 qk_norm: bool = False, rms_norm_eps: float = 1e-6, rope_base: float = 10000.0,
                 rope_interleaved: bool = False, layer_idx: int = 0, device=None, dtype=None) -> None:
        kw = {"device": device, "dtype": dtype}
        super().__init__()
        if embed_dim % num_heads:
            raise ValueError(f"embed_dim ({embed_dim}) must be divisible by num_heads ({num_heads})")
        num_kv_heads = num_heads if num_kv_heads is None else num_kv_heads
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads ({num_heads}) must be divisible by num_kv_heads ({num_kv_heads})")
        head_dim = embed_dim // num_heads if head_dim is None else head_dim
        self.embed_dim, self.num_heads, self.num_kv_heads = embed_dim, num_heads, num_kv_heads
        self.head_dim, self.dropout, self.layer_idx = head_dim, dropout, layer_idx
        self.scaling = head_dim ** -0.5
        self.q_proj = Linear(embed_dim, num_heads * head_dim, bias=bias, **kw)
        self.k_proj = Linear(embed_dim, num_kv_heads * head_dim, bias=bias, **kw)
        self.v_proj = Linear(embed_dim, num_kv_heads * head_dim, bias=bias, **kw)
        self.o_proj = Linear(num_heads * head_dim, embed_dim, bias=bias, **kw)
        self.qk_norm = qk_norm
        self.q_norm = RMSNorm(head_dim, eps=rms_norm_eps, **kw) if qk_norm else None
        self.k_norm = RMSNorm(head_dim, eps=rms_norm_eps, **kw) if qk_norm else None
        self.rope = RotaryEmbedding(head_dim, base=rope_base, interleaved=rope_interleaved, device=device)

    def forward(self, hidden_states: Tensor, position_ids: Optional[Tensor] = None,
                past_key_values=None) -> Tensor:
        B, T, _ = hidden_states.shape
        offset = past_key_values.get_seq_length(self.layer_idx) if past_key_values is not None else 0
        if position_ids is None:
            max_pos = offset + T
            pos = None if offset == 0 else torch.arange(offset, offset + T, device=hidden_states.device).expand(B, T)
        else:
            pos = position_ids
            max_pos = None
        q = self.q_proj(hidden_states).view(B, T, self.num_heads, self.head_dim)
        k = self.k_proj(hidden_states).view(B, T, self.num_kv_heads, self.head_dim)
        v = self.v_proj(hidden_states).view(B, T, self.num_kv_heads, self.head_dim)
        if self.qk_norm:
            q = self.q_norm(q)
            k = self.k_norm(k)
        if max_pos is None:
            max_pos = int(pos.max().item()) + 1
        cos, sin = self.rope.tables(max_pos, hidden_states.device)
        q = _ops.apply_rope(q, cos, sin, pos, self.rope.interleaved)
        k = _ops.apply_rope(k, cos, sin, pos, self.rope.interleaved)
        if past_key_values is not None:
            # caches keep the reference's [B, H, T, D] layout
            kc, vc = past_key_values.update(k.transpose(1, 2), v.transpose(1, 2), self.layer_idx)
            k, v = kc.transpose(1, 2), vc.transpose(1, 2)
        if self.training and self.dropout > 0.0:
            o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                               dropout_p=self.dropout, is_causal=q.shape[1] == k.shape[1],
                                               scale=self.scaling, enable_gqa=True).transpose(1, 2)
        else:
            # bottom-right aligned causal mask: equals the reference's rule (causal when the
            # query covers the prefix, unmasked for a single decode token) and also covers
            # chunked prefill
            o = flash_attention(q, k, v, causal=True, scale=self.scaling)
        return self.o_proj(o.reshape(B, T, self.num_heads * self.head_dim))

    def extra_repr(self) -> str:
        return (f"embed_dim={self.embed_dim}, num_heads={self.num_heads}, num_kv_heads={self.num_kv_heads}, "
                f"head_dim={self.head_dim}, qk_norm={self.qk_norm}, layer_idx={self.layer_idx}")


class SwiGLUMLP(Module):
    """``down(silu(gate(x)) * up(x))``."""

    def __init__(self, hidden_size: int, intermediate_size: Optional[int] = None, bias: bool = False,
                 device=None, dtype=None) -> None:
        kw = {"device": device, "dtype": dtype}
        super().__init__()
        if intermediate_size is None:
            intermediate_size = 4 * hidden_size * 2 // 3
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.gate_proj = Linear(hidden_size, intermediate_size, bias=bias, **kw)
        self.up_proj = Linear(hidden_size, intermediate_size, bias=bias, **kw)
        self.down_proj = Linear(intermediate_size, hidden_size, bias=bias, **kw)

    def forward(self, x: Tensor) -> Tensor:
        return self.down_proj(_ops.swiglu(self.gate_proj(x), self.up_proj(x)))


class TransformerBlock(Module):
    """Pre-norm residual block around an injected mixer."""

    def __init__(self, hidden_size: int, mixer: Module, mlp_intermediate_size: Optional[int] = None,
                 rms_norm_eps: float = 1e-6, device=None, dtype=None) -> None:
        kw = {"device": device, "dtype": dtype}
        super().__init__()
        self.hidden_size = hidden_size
        self.mixer = mixer
        self.mlp = SwiGLUMLP(hidden_size, intermediate_size=mlp_intermediate_size, **kw)
        self.input_norm = RMSNorm(hidden_size, eps=rms_norm_eps, **kw)
        self.post_norm = RMSNorm(hidden_size, eps=rms_norm_eps, **kw)

    def forward(self, hidden_states: Tensor, position_ids: Optional[Tensor] = None,
                past_key_values=None) -> Tensor:
        a = self.mixer(self.input_norm(hidden_states), position_ids=position_ids,
                       past_key_values=past_key_values)
        # the residual add is fused into the second norm's pass over the stream
        h, hidden_states = self.post_norm(a, residual=hidden_states)
        return hidden_states + self.mlp(h)
