"""Sequence mixers beyond grouped-query attention: multi-head latent attention (compressed KV
cache) and the gated delta rule (linear-time recurrent mixer).

API after tensorplay/nn/modules/latent_attention.py:30-224 (``MultiheadLatentAttention``) and
tensorplay/nn/modules/gated_delta.py (``GatedDeltaNet``); the math follows the published
formulations (DeepSeek-V2 MLA; gated DeltaNet), written for this package's ops: attention runs on
the flash kernels whenever the head width allows, everything else is plain tensor algebra.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F
from torch import Tensor
from torch.nn import Module

from ... import ops as _ops
from .llm import Linear, RMSNorm, RotaryEmbedding


class MultiheadLatentAttention(Module):
    """Causal attention whose cache holds one compressed latent (``kv_lora_rank`` wide) plus one
    rotary key (``qk_rope_head_dim`` wide) per token instead of per-head keys and values.

    Queries and keys have a content part (``qk_nope_head_dim``, no position) and a rotary part
    (``qk_rope_head_dim``; the rotary key is shared by all heads). Keys and values are
    up-projected from the cached latent on every call.
    """

    def __init__(self, embed_dim: int, num_heads: int, kv_lora_rank: int, qk_nope_head_dim: int,
                 qk_rope_head_dim: int, v_head_dim: Optional[int] = None, q_lora_rank: Optional[int] = None,
                 dropout: float = 0.0, bias: bool = False, rope_base: float = 10000.0,
                 rope_interleaved: bool = False, layer_idx: int = 0, device=None, dtype=None) -> None:
        kw = {"device": device, "dtype": dtype}
        super().__init__()
        if embed_dim % num_heads:
            raise ValueError(f"embed_dim ({embed_dim}) must be divisible by num_heads ({num_heads})")
        if qk_rope_head_dim % 2:
            raise ValueError(f"qk_rope_head_dim must be even for rotary embedding, got {qk_rope_head_dim}")
        v_head_dim = qk_nope_head_dim if v_head_dim is None else v_head_dim
        self.embed_dim, self.num_heads, self.kv_lora_rank = embed_dim, num_heads, kv_lora_rank
        self.qk_nope_head_dim, self.qk_rope_head_dim = qk_nope_head_dim, qk_rope_head_dim
        self.qk_head_dim = qk_nope_head_dim + qk_rope_head_dim
        self.v_head_dim, self.q_lora_rank = v_head_dim, q_lora_rank
        self.dropout, self.layer_idx = dropout, layer_idx
        self.scaling = self.qk_head_dim ** -0.5
        if q_lora_rank is None:
            self.q_proj = Linear(embed_dim, num_heads * self.qk_head_dim, bias=bias, **kw)
            self.q_a_proj = self.q_a_layernorm = self.q_b_proj = None
        else:
            self.q_proj = None
            self.q_a_proj = Linear(embed_dim, q_lora_rank, bias=bias, **kw)
            self.q_a_layernorm = RMSNorm(q_lora_rank, **kw)
            self.q_b_proj = Linear(q_lora_rank, num_heads * self.qk_head_dim, bias=False, **kw)
        self.kv_a_proj_with_mqa = Linear(embed_dim, kv_lora_rank + qk_rope_head_dim, bias=bias, **kw)
        self.kv_a_layernorm = RMSNorm(kv_lora_rank, **kw)
        self.kv_b_proj = Linear(kv_lora_rank, num_heads * (qk_nope_head_dim + v_head_dim), bias=False, **kw)
        self.o_proj = Linear(num_heads * v_head_dim, embed_dim, bias=bias, **kw)
        self.rope = RotaryEmbedding(qk_rope_head_dim, base=rope_base, interleaved=rope_interleaved, device=device)

    def forward(self, hidden_states: Tensor, position_ids: Optional[Tensor] = None, past_key_values=None) -> Tensor:
        B, T, _ = hidden_states.shape
        H, dn, dr, dv = self.num_heads, self.qk_nope_head_dim, self.qk_rope_head_dim, self.v_head_dim
        offset = past_key_values.get_seq_length(self.layer_idx) if past_key_values is not None else 0
        pos = position_ids
        if pos is None:
            pos = torch.arange(offset, offset + T, device=hidden_states.device).expand(B, T)
        if self.q_proj is not None:
            q = self.q_proj(hidden_states)
        else:
            q = self.q_b_proj(self.q_a_layernorm(self.q_a_proj(hidden_states)))
        q = q.view(B, T, H, dn + dr)
        q_nope, q_rot = q[..., :dn], q[..., dn:]
        ckv = self.kv_a_proj_with_mqa(hidden_states)
        latent, k_rot = self.kv_a_layernorm(ckv[..., : self.kv_lora_rank]), ckv[..., self.kv_lora_rank:]
        cos, sin = self.rope.tables(int(pos.max().item()) + 1, hidden_states.device)
        q_rot = _ops.apply_rope(q_rot.contiguous(), cos, sin, pos, self.rope.interleaved)
        k_rot = _ops.apply_rope(k_rot.reshape(B, T, 1, dr).contiguous(), cos, sin, pos, self.rope.interleaved)
        if past_key_values is not None:
            # the cache keeps [B, 1, S, width] entries: latent as "key", rotary key as "value"
            lat_c, rot_c = past_key_values.update(latent.unsqueeze(1), k_rot.transpose(1, 2), self.layer_idx)
            latent, k_rot = lat_c.squeeze(1), rot_c.transpose(1, 2)
        S = latent.shape[1]
        kv = self.kv_b_proj(latent).view(B, S, H, dn + dv)
        k = torch.cat((kv[..., :dn], k_rot.expand(B, S, H, dr)), dim=-1)
        v = kv[..., dn:]
        qf = torch.cat((q_nope, q_rot), dim=-1)
        drop = self.dropout if self.training else 0.0
        if drop == 0.0 and k.shape[-1] == v.shape[-1] and k.shape[-1] in (64, 128):
            o = _ops.flash_attention(qf, k, v, causal=True, scale=self.scaling)
        else:
            # widths the flash kernels do not cover (q/k wider than v): SDPA with a bottom-right mask
            i = torch.arange(T, device=qf.device).view(-1, 1) + (S - T)
            mask = torch.arange(S, device=qf.device).view(1, -1) <= i
            o = F.scaled_dot_product_attention(qf.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                               attn_mask=mask, dropout_p=drop, scale=self.scaling).transpose(1, 2)
        return self.o_proj(o.reshape(B, T, H * dv))

    def extra_repr(self) -> str:
        return (f"embed_dim={self.embed_dim}, num_heads={self.num_heads}, kv_lora_rank={self.kv_lora_rank}, "
                f"qk_nope_head_dim={self.qk_nope_head_dim}, qk_rope_head_dim={self.qk_rope_head_dim}, "
                f"v_head_dim={self.v_head_dim}, q_lora_rank={self.q_lora_rank}")


def gated_delta_rule(q: Tensor, k: Tensor, v: Tensor, g: Tensor, beta: Tensor,
                     state: Optional[Tensor] = None) -> Tuple[Tensor, Tensor]:
    """Gated delta rule, one step per token.

    ``q, k``: [B, T, H, Dk] (keys L2-normalised by the caller), ``v``: [B, T, H, Dv], ``beta``:
    [B, T, H] write strength in (0, 1), ``g``: log-decay (<= 0), either one value per head
    ([B, T, H]) or one per key channel ([B, T, H, Dk]: the fine-grained variant); ``state``:
    [B, H, Dk, Dv]. Per token: ``S <- diag(exp(g)) S``; ``S <- S + beta * k (v - S^T k)^T``;
    ``o = S^T q``. Returns (o [B, T, H, Dv], final state).
    """
    B, T, H, Dk = k.shape
    Dv = v.shape[-1]
    S = torch.zeros(B, H, Dk, Dv, dtype=torch.float32, device=k.device) if state is None else state.float()
    qf, kf, vf = q.float(), k.float(), v.float()
    per_channel = g.dim() == 4
    out = []
    for t in range(T):
        decay = torch.exp(g[:, t].float())
        S = S * (decay[..., None] if per_channel else decay[..., None, None])
        kt, vt = kf[:, t], vf[:, t]
        pred = torch.einsum("bhkv,bhk->bhv", S, kt)
        S = S + torch.einsum("bhk,bhv->bhkv", kt, (vt - pred) * beta[:, t].float()[..., None])
        out.append(torch.einsum("bhkv,bhk->bhv", S, qf[:, t]))
    return torch.stack(out, dim=1).to(v.dtype), S


def chunk_gated_delta_rule(q: Tensor, k: Tensor, v: Tensor, g: Tensor, beta: Tensor, state: Optional[Tensor] = None,
                           chunk: int = 64) -> Tuple[Tensor, Tensor]:
    """Same result as :func:`gated_delta_rule` (head-scalar decay) with matrix algebra per chunk of
    ``chunk`` tokens: inside a chunk the delta-rule writes form a unit lower-triangular system
    ``(I + tril(beta * decay * K K^T, -1)) U = beta * (V - decay_in * K S)`` solved in closed form,
    so the sequential depth is T / chunk instead of T (the GEMM-shaped form used for training)."""
    B, T, H, Dk = k.shape
    Dv = v.shape[-1]
    S = torch.zeros(B, H, Dk, Dv, dtype=torch.float32, device=k.device) if state is None else state.float()
    qf, kf, vf = (t.float().transpose(1, 2) for t in (q, k, v))      # [B, H, T, D]
    gf, bf = g.float().transpose(1, 2), beta.float().transpose(1, 2)  # [B, H, T]
    outs = []
    for c0 in range(0, T, chunk):
        c1 = min(c0 + chunk, T)
        n = c1 - c0
        qc, kc, vc, bc = qf[:, :, c0:c1], kf[:, :, c0:c1], vf[:, :, c0:c1], bf[:, :, c0:c1]
        gc = torch.cumsum(gf[:, :, c0:c1], dim=-1)                    # log-decay from chunk start to token i (incl.)
        # decay between tokens: D[i, j] = exp(gc[i] - gc[j]) for j <= i
        diff = gc.unsqueeze(-1) - gc.unsqueeze(-2)
        tri = torch.tril(torch.ones(n, n, dtype=torch.bool, device=k.device))
        Dm = torch.where(tri, torch.exp(diff.masked_fill(~tri, 0.0)), torch.zeros_like(diff))
        kk = torch.einsum("bhik,bhjk->bhij", kc, kc) * Dm
        A = torch.tril(kk * bc.unsqueeze(-1), diagonal=-1)            # strictly lower part: earlier writes seen by token i
        rhs = bc.unsqueeze(-1) * (vc - torch.exp(gc).unsqueeze(-1) * torch.einsum("bhik,bhkv->bhiv", kc, S))
        eye = torch.eye(n, device=k.device).expand(B, H, n, n)
        U = torch.linalg.solve_triangular(eye + A, rhs, upper=False)  # the per-token write vectors
        qk = torch.einsum("bhik,bhjk->bhij", qc, kc) * Dm
        o = torch.exp(gc).unsqueeze(-1) * torch.einsum("bhik,bhkv->bhiv", qc, S) + torch.einsum("bhij,bhjv->bhiv", qk, U)
        outs.append(o)
        tail = torch.exp(gc[..., -1:] - gc)                           # decay from token j to the chunk end
        S = torch.exp(gc[..., -1])[..., None, None] * S + torch.einsum("bhjk,bhjv->bhkv", kc * tail.unsqueeze(-1), U)
    return torch.cat(outs, dim=2).transpose(1, 2).to(v.dtype), S


class GatedDeltaNet(Module):
    """Linear-time token mixer: short causal depthwise convolutions on q / k / v, a decaying
    matrix-valued state updated by the delta rule with a learned write strength, and a gated,
    normalised read-out. ``past_key_values`` is a ``LinearStateCache`` (conv window + state)."""

    def __init__(self, embed_dim: int, num_heads: int, head_dim: Optional[int] = None, expand_v: float = 2.0,
                 conv_size: int = 4, layer_idx: int = 0, norm_eps: float = 1e-6, device=None, dtype=None) -> None:
        kw = {"device": device, "dtype": dtype}
        super().__init__()
        head_dim = embed_dim // num_heads if head_dim is None else head_dim
        self.embed_dim, self.num_heads, self.head_k_dim = embed_dim, num_heads, head_dim
        self.head_v_dim = int(head_dim * expand_v)
        self.conv_size, self.layer_idx = conv_size, layer_idx
        kd, vd = num_heads * self.head_k_dim, num_heads * self.head_v_dim
        self.q_proj = Linear(embed_dim, kd, bias=False, **kw)
        self.k_proj = Linear(embed_dim, kd, bias=False, **kw)
        self.v_proj = Linear(embed_dim, vd, bias=False, **kw)
        self.a_proj = Linear(embed_dim, num_heads, bias=False, **kw)   # decay input
        self.b_proj = Linear(embed_dim, num_heads, bias=False, **kw)   # write strength
        self.g_proj = Linear(embed_dim, vd, bias=False, **kw)          # output gate
        self.o_proj = Linear(vd, embed_dim, bias=False, **kw)
        self.conv_weight = torch.nn.Parameter(torch.empty(2 * kd + vd, conv_size, **kw))
        torch.nn.init.normal_(self.conv_weight, std=conv_size ** -0.5)
        self.A_log = torch.nn.Parameter(torch.log(torch.empty(num_heads, **kw).uniform_(1.0, 16.0)))
        self.dt_bias = torch.nn.Parameter(torch.zeros(num_heads, **kw))
        self.o_norm = RMSNorm(self.head_v_dim, eps=norm_eps, **kw)

    def _conv(self, x: Tensor, cache) -> Tensor:
        """Causal depthwise convolution over time of ``x [B, T, C]`` followed by SiLU."""
        xt = x.transpose(1, 2)  # [B, C, T]
        if cache is not None:
            full = cache.update_conv_state(self.layer_idx, xt, self.conv_size)
            pad = self.conv_size - 1 - (full.shape[-1] - xt.shape[-1])
        else:
            full, pad = xt, self.conv_size - 1
        full = F.pad(full, (max(pad, 0), 0))
        y = F.conv1d(full, self.conv_weight.unsqueeze(1).to(full.dtype), groups=full.shape[1])
        return F.silu(y[..., -xt.shape[-1]:]).transpose(1, 2)

    def forward(self, hidden_states: Tensor, position_ids: Optional[Tensor] = None, past_key_values=None) -> Tensor:
        B, T, _ = hidden_states.shape
        H, dk, dv = self.num_heads, self.head_k_dim, self.head_v_dim
        qkv = torch.cat((self.q_proj(hidden_states), self.k_proj(hidden_states), self.v_proj(hidden_states)), dim=-1)
        qkv = self._conv(qkv, past_key_values)
        q, k, v = qkv.split((H * dk, H * dk, H * dv), dim=-1)
        q = F.normalize(q.view(B, T, H, dk).float(), dim=-1) * dk ** -0.5
        k = F.normalize(k.view(B, T, H, dk).float(), dim=-1)
        v = v.reshape(B, T, H, dv)
        beta = torch.sigmoid(self.b_proj(hidden_states).float())
        g = -torch.exp(self.A_log.float()) * F.softplus(self.a_proj(hidden_states).float() + self.dt_bias.float())
        state = past_key_values.recurrent_states.get(self.layer_idx) if past_key_values is not None else None
        rule = chunk_gated_delta_rule if T > 16 else gated_delta_rule
        o, state = rule(q, k, v, g, beta, state)
        if past_key_values is not None:
            past_key_values.update_recurrent_state(self.layer_idx, state)
        o = self.o_norm(o) * F.silu(self.g_proj(hidden_states).view(B, T, H, dv))
        return self.o_proj(o.reshape(B, T, H * dv).to(hidden_states.dtype))


def _l2norm(x: Tensor) -> Tensor:
    return F.normalize(x.float(), dim=-1)


def recurrent_gated_delta_rule(query: Tensor, key: Tensor, value: Tensor, g: Tensor, beta: Tensor,
                               initial_state: Optional[Tensor] = None, output_final_state: bool = False,
                               use_qk_l2norm_in_kernel: bool = False) -> Tuple[Tensor, Optional[Tensor]]:
    """The reference's spelling of the token-by-token gated delta rule (nn/modules/gated_delta.py:171): queries are
    scaled by ``key_dim ** -0.5``, ``q`` / ``k`` optionally L2-normalised here, and the final state is returned only
    on request. ``g``: ``[B, T, H]``."""
    if use_qk_l2norm_in_kernel:
        query, key = _l2norm(query), _l2norm(key)
    out, state = gated_delta_rule(query.float() * key.shape[-1] ** -0.5, key, value, g, beta, initial_state)
    return out.to(value.dtype), (state if output_final_state else None)


def recurrent_kimi_delta_rule(query: Tensor, key: Tensor, value: Tensor, g: Tensor, beta: Tensor,
                              initial_state: Optional[Tensor] = None, output_final_state: bool = False,
                              use_qk_l2norm_in_kernel: bool = False) -> Tuple[Tensor, Optional[Tensor]]:
    """Token-by-token delta rule with one decay per key channel, ``g``: ``[B, T, H, Dk]``
    (nn/modules/kimi_delta.py:38)."""
    if g.dim() != 4:
        raise ValueError("recurrent_kimi_delta_rule: g must be [batch, seq, heads, key_dim]")
    if use_qk_l2norm_in_kernel:
        query, key = _l2norm(query), _l2norm(key)
    out, state = gated_delta_rule(query.float() * key.shape[-1] ** -0.5, key, value, g, beta, initial_state)
    return out.to(value.dtype), (state if output_final_state else None)


def chunk_kimi_delta_rule(query: Tensor, key: Tensor, value: Tensor, g: Tensor, beta: Tensor, chunk_size: int = 64,
                          initial_state: Optional[Tensor] = None, output_final_state: bool = False,
                          use_qk_l2norm_in_kernel: bool = False) -> Tuple[Tensor, Optional[Tensor]]:
    """Chunked form of :func:`recurrent_kimi_delta_rule` (nn/modules/kimi_delta.py:92). With a decay per key channel
    the decay between two tokens of a chunk factorises over the channels, ``exp(G_i - G_j) = exp(G_i) * exp(-G_j)``
    (``G``: cumulative log-decay inside the chunk), so the chunk's interaction matrices are plain products of decayed
    keys: ``K+ = K * exp(G)``, ``K- = K * exp(-G)``, ``A = tril(beta * K+ K-^T, -1)``. ``exp(-G)`` grows with the
    chunk length: the chunk matrices are formed in float64."""
    if use_qk_l2norm_in_kernel:
        query, key = _l2norm(query), _l2norm(key)
    B, T, H, Dk = key.shape
    Dv = value.shape[-1]
    f64 = torch.float64
    S = (torch.zeros(B, H, Dk, Dv, dtype=f64, device=key.device) if initial_state is None else initial_state.to(f64))
    qf = (query.to(f64) * Dk ** -0.5).transpose(1, 2)
    kf, vf = key.to(f64).transpose(1, 2), value.to(f64).transpose(1, 2)          # [B, H, T, D]
    gf, bf = g.to(f64).transpose(1, 2), beta.to(f64).transpose(1, 2)              # [B, H, T, Dk], [B, H, T]
    outs = []
    for c0 in range(0, T, chunk_size):
        c1 = min(c0 + chunk_size, T)
        n = c1 - c0
        qc, kc, vc, bc = qf[:, :, c0:c1], kf[:, :, c0:c1], vf[:, :, c0:c1], bf[:, :, c0:c1]
        G = torch.cumsum(gf[:, :, c0:c1], dim=2)                                  # [B, H, n, Dk]
        kp, km, qp = kc * torch.exp(G), kc * torch.exp(-G), qc * torch.exp(G)
        A = torch.tril(torch.einsum("bhik,bhjk->bhij", kp, km) * bc.unsqueeze(-1), diagonal=-1)
        rhs = bc.unsqueeze(-1) * (vc - torch.einsum("bhik,bhkv->bhiv", kp, S))
        eye = torch.eye(n, dtype=f64, device=key.device).expand(B, H, n, n)
        U = torch.linalg.solve_triangular(eye + A, rhs, upper=False)
        qk = torch.tril(torch.einsum("bhik,bhjk->bhij", qp, km))
        outs.append(torch.einsum("bhik,bhkv->bhiv", qp, S) + torch.einsum("bhij,bhjv->bhiv", qk, U))
        tail = torch.exp(G[:, :, -1:] - G)                                        # decay from token j to the chunk end
        S = torch.exp(G[:, :, -1]).unsqueeze(-1) * S + torch.einsum("bhjk,bhjv->bhkv", kc * tail, U)
    out = torch.cat(outs, dim=2).transpose(1, 2).to(value.dtype)
    return out, (S.float() if output_final_state else None)


class GatedRMSNorm(Module):
    """RMSNorm whose output is multiplied by an activated gate: ``norm(x) * weight * act(gate)``, computed in fp32
    (nn/modules/gated_delta.py:214; ``activation``: ``"silu"`` or ``"sigmoid"``)."""

    def __init__(self, dim: int, eps: float = 1e-6, activation: str = "silu", device=None, dtype=None) -> None:
        super().__init__()
        if activation not in ("silu", "sigmoid"):
            raise ValueError(f"unsupported gate activation {activation!r}")
        self.weight = torch.nn.Parameter(torch.ones(dim, device=device, dtype=dtype))
        self.eps, self.activation = eps, activation

    def forward(self, x: Tensor, gate: Tensor) -> Tensor:
        xf = x.float()
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight.float()
        a = F.silu(gate.float()) if self.activation == "silu" else torch.sigmoid(gate.float())
        return (y * a).to(x.dtype)

    def extra_repr(self) -> str:
        return f"{self.weight.numel()}, eps={self.eps}, activation={self.activation}"


class DepthwiseConv2d(torch.nn.Conv2d):
    """``Conv2d`` with one group per input channel (nn/modules/conv.py:292)."""

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, bias=True,
                 padding_mode="zeros", device=None, dtype=None):
        if out_channels % in_channels != 0:
            raise ValueError("out_channels must be divisible by in_channels for DepthwiseConv2d")
        super().__init__(in_channels, out_channels, kernel_size, stride, padding, dilation, groups=in_channels,
                         bias=bias, padding_mode=padding_mode, device=device, dtype=dtype)


class KimiDeltaAttention(GatedDeltaNet):
    """Gated delta rule with the decay resolved per key channel: the forget gate comes from a
    low-rank projection and has shape ``[B, T, H, Dk]``, so that different key coordinates keep
    their associations for different time spans; the write rule is unchanged
    (tensorplay/nn/modules/kimi_delta.py)."""

    def __init__(self, embed_dim: int, num_heads: int, head_dim: Optional[int] = None, expand_v: float = 1.0,
                 conv_size: int = 4, gate_rank: Optional[int] = None, layer_idx: int = 0, norm_eps: float = 1e-6,
                 device=None, dtype=None) -> None:
        super().__init__(embed_dim, num_heads, head_dim, expand_v, conv_size, layer_idx, norm_eps, device, dtype)
        kw = {"device": device, "dtype": dtype}
        rank = gate_rank if gate_rank is not None else self.head_k_dim
        self.f_a_proj = Linear(embed_dim, rank, bias=False, **kw)
        self.f_b_proj = Linear(rank, num_heads * self.head_k_dim, bias=False, **kw)
        self.a_proj = None  # the head-scalar decay input is replaced by the low-rank channel gate
        self.dt_bias = torch.nn.Parameter(torch.zeros(num_heads * self.head_k_dim, **kw))

    def forward(self, hidden_states: Tensor, position_ids: Optional[Tensor] = None, past_key_values=None) -> Tensor:
        B, T, _ = hidden_states.shape
        H, dk, dv = self.num_heads, self.head_k_dim, self.head_v_dim
        qkv = torch.cat((self.q_proj(hidden_states), self.k_proj(hidden_states), self.v_proj(hidden_states)), dim=-1)
        qkv = self._conv(qkv, past_key_values)
        q, k, v = qkv.split((H * dk, H * dk, H * dv), dim=-1)
        q = F.normalize(q.view(B, T, H, dk).float(), dim=-1) * dk ** -0.5
        k = F.normalize(k.view(B, T, H, dk).float(), dim=-1)
        v = v.reshape(B, T, H, dv)
        beta = torch.sigmoid(self.b_proj(hidden_states).float())
        gate_in = self.f_b_proj(self.f_a_proj(hidden_states)).float() + self.dt_bias.float()
        g = (-torch.exp(self.A_log.float()).view(1, 1, H, 1) * F.softplus(gate_in.view(B, T, H, dk)))
        state = past_key_values.recurrent_states.get(self.layer_idx) if past_key_values is not None else None
        o, state = gated_delta_rule(q, k, v, g, beta, state)
        if past_key_values is not None:
            past_key_values.update_recurrent_state(self.layer_idx, state)
        o = self.o_norm(o) * F.silu(self.g_proj(hidden_states).view(B, T, H, dv))
        return self.o_proj(o.reshape(B, T, H * dv).to(hidden_states.dtype))


class CrossAttention(Module):
    """Pre-norm multi-head attention from a decoder stream onto an encoder memory (no mask: every
    decoder position may read the whole memory), added to the stream as a residual."""

    def __init__(self, hidden_size: int, num_heads: int, rms_norm_eps: float = 1e-6, device=None, dtype=None) -> None:
        kw = {"device": device, "dtype": dtype}
        super().__init__()
        if hidden_size % num_heads:
            raise ValueError(f"hidden_size ({hidden_size}) must be divisible by num_heads ({num_heads})")
        self.num_heads, self.head_dim = num_heads, hidden_size // num_heads
        self.norm = RMSNorm(hidden_size, eps=rms_norm_eps, **kw)
        self.q_proj = Linear(hidden_size, hidden_size, bias=False, **kw)
        self.kv_proj = Linear(hidden_size, 2 * hidden_size, bias=False, **kw)
        self.o_proj = Linear(hidden_size, hidden_size, bias=False, **kw)

    def forward(self, x: Tensor, memory: Tensor) -> Tensor:
        B, T, C = x.shape
        S = memory.shape[1]
        q = self.q_proj(self.norm(x)).view(B, T, self.num_heads, self.head_dim)
        kv = self.kv_proj(memory).view(B, S, 2, self.num_heads, self.head_dim)
        o = _ops.flash_attention(q, kv[:, :, 0], kv[:, :, 1], causal=False, scale=self.head_dim ** -0.5)
        return x + self.o_proj(o.reshape(B, T, C))


class CausalEncoderDecoder(Module):
    """Two causal stacks of :class:`TransformerBlock`: the encoder digests the sequence into a
    memory (final norm + projection), the decoder processes the same sequence and reads that
    memory through a :class:`CrossAttention` after each of its blocks. ``mixer_factory(hidden_size,
    layer_idx)`` chooses the token mixer per layer (default: grouped-query attention), so linear
    and latent-attention mixers can be swapped in (tensorplay/nn/modules/causal_encoder_decoder.py:80-163).
    """

    def __init__(self, hidden_size: int, num_heads: int, n_encoder_layers: int = 2, n_decoder_layers: int = 2,
                 mixer_factory=None, num_kv_heads: Optional[int] = None, mlp_intermediate_size: Optional[int] = None,
                 rms_norm_eps: float = 1e-6, device=None, dtype=None) -> None:
        from .llm import GroupedQueryAttention, TransformerBlock
        kw = {"device": device, "dtype": dtype}
        super().__init__()
        if mixer_factory is None:
            def mixer_factory(width, layer_idx):
                return GroupedQueryAttention(width, num_heads, num_kv_heads=num_kv_heads, layer_idx=layer_idx, **kw)
        self.hidden_size = hidden_size

        def stack(n):
            return torch.nn.ModuleList(
                TransformerBlock(hidden_size, mixer_factory(hidden_size, i), mlp_intermediate_size=mlp_intermediate_size,
                                 rms_norm_eps=rms_norm_eps, **kw) for i in range(n))

        self.encoder, self.decoder = stack(n_encoder_layers), stack(n_decoder_layers)
        self.cross_attention = torch.nn.ModuleList(
            CrossAttention(hidden_size, num_heads, rms_norm_eps=rms_norm_eps, **kw) for _ in range(n_decoder_layers))
        self.memory_proj = Linear(hidden_size, hidden_size, bias=False, **kw)
        self.encoder_final_norm = RMSNorm(hidden_size, eps=rms_norm_eps, **kw)

    def forward(self, hidden_states: Tensor) -> Tensor:
        memory = hidden_states
        for block in self.encoder:
            memory = block(memory)
        memory = self.memory_proj(self.encoder_final_norm(memory))
        x = hidden_states
        for block, cross in zip(self.decoder, self.cross_attention):
            x = cross(block(x), memory)
        return x


class CompressedSparseAttention(Module):
    """Long-context mixer with two key/value tiers (tensorplay/nn/modules/compressed_attention.py):

    * a sliding window of the last ``window_size`` tokens, attended at full resolution through one
      shared key/value head with ``k == v``;
    * one compressed entry per ``compress_rate`` source tokens (a softmax-gated reduction of the
      window's key/value vectors), of which every query sees at most ``index_topk``: a small
      indexer scores the entries per query, ``sum_h w[t, h] * relu(q_idx[t, h] . k_idx[s])``, and
      only entries that lie completely in the query's past are eligible.

    Each head also has a learned sink logit that takes part in the softmax without contributing a
    value. This implementation processes whole sequences (training / prefill); it keeps no
    incremental state between calls.
    """

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, q_lora_rank: int, compress_rate: int = 4,
                 window_size: int = 128, rope_head_dim: Optional[int] = None, index_n_heads: int = 4,
                 index_head_dim: int = 32, index_topk: int = 16, rope_base: float = 10000.0,
                 rms_norm_eps: float = 1e-6, layer_idx: int = 0, device=None, dtype=None) -> None:
        kw = {"device": device, "dtype": dtype}
        super().__init__()
        if hidden_size % num_heads:
            raise ValueError(f"hidden_size ({hidden_size}) must be divisible by num_heads ({num_heads})")
        self.hidden_size, self.num_heads, self.head_dim = hidden_size, num_heads, head_dim
        self.sliding_window, self.compress_rate, self.index_topk = window_size, compress_rate, index_topk
        self.index_n_heads, self.index_head_dim, self.layer_idx = index_n_heads, index_head_dim, layer_idx
        self.scaling = head_dim ** -0.5
        self.q_a_proj = Linear(hidden_size, q_lora_rank, bias=False, **kw)
        self.q_a_norm = RMSNorm(q_lora_rank, eps=rms_norm_eps, **kw)
        self.q_b_proj = Linear(q_lora_rank, num_heads * head_dim, bias=False, **kw)
        self.kv_proj = Linear(hidden_size, head_dim, bias=False, **kw)
        self.kv_norm = RMSNorm(head_dim, eps=rms_norm_eps, **kw)
        self.o_proj = Linear(num_heads * head_dim, hidden_size, bias=False, **kw)
        self.sinks = torch.nn.Parameter(torch.zeros(num_heads, **kw))
        self.rope_dim = rope_head_dim if rope_head_dim is not None else head_dim
        self.rope = RotaryEmbedding(self.rope_dim, base=rope_base, device=device)
        # compressor: per-token gate logit; entries are gate-softmax-weighted means of the window's kv
        self.compress_gate = Linear(hidden_size, 1, bias=False, **kw)
        self.compress_norm = RMSNorm(head_dim, eps=rms_norm_eps, **kw)
        # indexer: its own small keys per entry, queries and head weights per token
        self.idx_k_proj = Linear(hidden_size, index_head_dim, bias=False, **kw)
        self.idx_q_proj = Linear(q_lora_rank, index_n_heads * index_head_dim, bias=False, **kw)
        self.idx_w_proj = Linear(hidden_size, index_n_heads, bias=False, **kw)

    def _compress(self, x: Tensor, feats: Tensor) -> Tensor:
        """[B, T, C] features -> [B, T // rate, C] gate-weighted window means (incomplete tail dropped)."""
        B, T, C = feats.shape
        r = self.compress_rate
        n = T // r
        if n == 0:
            return feats.new_zeros(B, 0, C)
        gate = torch.softmax(self.compress_gate(x[:, : n * r]).float().view(B, n, r), dim=-1)
        return (feats[:, : n * r].float().view(B, n, r, C) * gate.unsqueeze(-1)).sum(2).to(feats.dtype)

    def forward(self, hidden_states: Tensor, position_ids: Optional[Tensor] = None, past_key_values=None) -> Tensor:
        if past_key_values is not None:
            raise NotImplementedError("CompressedSparseAttention keeps no incremental state in this build")
        B, T, _ = hidden_states.shape
        H, D, r = self.num_heads, self.head_dim, self.compress_rate
        dev = hidden_states.device
        pos = position_ids if position_ids is not None else torch.arange(T, device=dev).expand(B, T)
        q_lat = self.q_a_norm(self.q_a_proj(hidden_states))
        q = self.q_b_proj(q_lat).view(B, T, H, D)
        kv = self.kv_norm(self.kv_proj(hidden_states)).view(B, T, 1, D)
        cos, sin = self.rope.tables(int(pos.max().item()) + 1, dev)
        rd = self.rope_dim
        q = torch.cat((_ops.apply_rope(q[..., :rd].contiguous(), cos, sin, pos), q[..., rd:]), dim=-1)
        k_win = torch.cat((_ops.apply_rope(kv[..., :rd].contiguous(), cos, sin, pos), kv[..., rd:]), dim=-1)
        # ---- tier 1: sliding window (shared head, k == v up to the rotation of k)
        i = torch.arange(T, device=dev).view(T, 1)
        j = torch.arange(T, device=dev).view(1, T)
        win_ok = (j <= i) & (j > i - self.sliding_window)
        s_win = torch.einsum("bthd,bsd->bhts", q.float(), k_win[:, :, 0].float()) * self.scaling
        s_win = s_win.masked_fill(~win_ok, float("-inf"))
        # ---- tier 2: compressed entries selected by the indexer
        ent = self.compress_norm(self._compress(hidden_states, kv[:, :, 0]))        # [B, n, D]
        n = ent.shape[1]
        if n > 0:
            ent_end = (torch.arange(n, device=dev) + 1) * r - 1                     # last source position of an entry
            eligible = ent_end.view(1, 1, n) <= pos.unsqueeze(-1)                   # completely in the query's past
            k_idx = self._compress(hidden_states, self.idx_k_proj(hidden_states))   # [B, n, Di]
            q_idx = self.idx_q_proj(q_lat).view(B, T, self.index_n_heads, self.index_head_dim)
            w_idx = self.idx_w_proj(hidden_states).float()
            score = (torch.relu(torch.einsum("bthd,bnd->bthn", q_idx.float(), k_idx.float())) * w_idx.unsqueeze(-1)).sum(2)
            score = score.masked_fill(~eligible, float("-inf"))
            k_sel = min(self.index_topk, n)
            top = score.topk(k_sel, dim=-1).indices
            chosen = torch.zeros(B, T, n, dtype=torch.bool, device=dev).scatter_(-1, top, True) & eligible
            s_ent = torch.einsum("bthd,bnd->bhtn", q.float(), ent.float()) * self.scaling
            s_ent = s_ent.masked_fill(~chosen.unsqueeze(1), float("-inf"))
        else:
            s_ent = s_win.new_zeros(B, H, T, 0)
        sink = self.sinks.float().view(1, H, 1, 1).expand(B, H, T, 1)
        p = torch.softmax(torch.cat((s_win, s_ent, sink), dim=-1), dim=-1)
        o = torch.einsum("bhts,bsd->bthd", p[..., :T], kv[:, :, 0].float())
        if n > 0:
            o = o + torch.einsum("bhtn,bnd->bthd", p[..., T: T + n], ent.float())
        return self.o_proj(o.reshape(B, T, H * D).to(hidden_states.dtype))
