"""Qwen3-MoE-family decoder: GQA with QK-RMSNorm and RoPE, and a sparse SwiGLU MoE feed-forward
with top-k softmax routing (renormalised), dropless expert parallelism and the load-balance
auxiliary loss. The 30B-A3B shape: 48 layers, hidden 2048, 32/4 heads of 128, 128 experts of
intermediate 768, top-8, theta 1e6, vocab 151936.

Expert weights are marked ``_tpb_expert_parallel`` (each rank holds ``num_experts / world`` of
them); attention, norms, router and embeddings are sharded by the training engine like any other
parameter. The reference can only run this family single-GPU through a HuggingFace import alias
(benchmark/bench_qwen3_moe_e2e.py:163-200).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist
from torch import Tensor, nn

from .. import ops
from ..parallel.moe import MoEWorkspace, expert_parallel_ffn, topk_route
from .llama import _embedding


@dataclass
class Qwen3MoEConfig:
    vocab_size: int = 151936
    hidden_size: int = 2048
    num_layers: int = 48
    num_heads: int = 32
    num_kv_heads: int = 4
    head_dim: int = 128
    num_experts: int = 128
    moe_intermediate: int = 768
    top_k: int = 8
    norm_topk_prob: bool = True
    aux_loss_coef: float = 1e-3
    rms_eps: float = 1e-6
    rope_theta: float = 1e6
    max_seq_len: int = 4096
    init_std: float = 0.02

    @staticmethod
    def qwen3_30b_a3b(**kw) -> "Qwen3MoEConfig":
        return Qwen3MoEConfig(**kw)

    @staticmethod
    def tiny(**kw) -> "Qwen3MoEConfig":
        base = dict(vocab_size=512, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=64,
                    num_experts=8, moe_intermediate=128, top_k=2, max_seq_len=256)
        base.update(kw)
        return Qwen3MoEConfig(**base)


def _qwen3_flops_per_token(self, seq_len: int, backward: bool = True, recompute: bool = False) -> float:
    """Model FLOPs per token: 2 x the matmul parameters a token activates (attention projections, router,
    ``top_k`` experts, LM head) plus causal attention, x3 with backward."""
    H, D = self.hidden_size, self.head_dim
    per_layer = (H * (self.num_heads + 2 * self.num_kv_heads) * D + self.num_heads * D * H
                 + H * self.num_experts + self.top_k * 3 * H * self.moe_intermediate)
    mm = self.num_layers * per_layer + self.vocab_size * H
    fwd = 2.0 * mm + 2.0 * 2 * self.num_layers * self.num_heads * D * seq_len / 2
    return fwd * (1.0 + (2.0 if backward else 0.0) + (1.0 if recompute else 0.0))


Qwen3MoEConfig.flops_per_token = _qwen3_flops_per_token


class _AuxLoss(torch.autograd.Function):
    """Identity on ``x`` that injects d(aux)/d(router) into backward with weight ``scale``, so the
    auxiliary loss is optimised without threading a scalar through every layer boundary."""

    @staticmethod
    def forward(ctx, x, aux, scale):
        ctx.scale = scale
        ctx.aux_shape = aux.shape
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        return g, torch.full(ctx.aux_shape, ctx.scale, dtype=torch.float32, device=g.device), None


class Qwen3MoEBlock(nn.Module):
    def __init__(self, cfg: Qwen3MoEConfig, layer_idx: int, ep_world: int = 1, device=None, dtype=None):
        super().__init__()
        kw = {"device": device, "dtype": dtype}
        H, D = cfg.hidden_size, cfg.head_dim
        self.cfg, self.layer_idx = cfg, layer_idx
        El = cfg.num_experts // ep_world
        self.attn_norm = nn.Parameter(torch.ones(H, **kw))
        self.wqkv = nn.Parameter(torch.empty((cfg.num_heads + 2 * cfg.num_kv_heads) * D, H, **kw))
        self.q_norm = nn.Parameter(torch.ones(D, **kw))
        self.k_norm = nn.Parameter(torch.ones(D, **kw))
        self.wo = nn.Parameter(torch.empty(H, cfg.num_heads * D, **kw))
        self.ffn_norm = nn.Parameter(torch.ones(H, **kw))
        self.router = nn.Parameter(torch.empty(cfg.num_experts, H, **kw))
        self.w_gate_up = nn.Parameter(torch.empty(El, 2 * cfg.moe_intermediate, H, **kw))
        self.w_down = nn.Parameter(torch.empty(El, H, cfg.moe_intermediate, **kw))
        self.w_gate_up._tpb_expert_parallel = True
        self.w_down._tpb_expert_parallel = True
        self.workspace: Optional[MoEWorkspace] = None
        self.ep_group = None
        self.loss_scale = 1.0

    def reset_parameters(self, generator=None):
        for w in (self.wqkv, self.wo, self.router, self.w_gate_up, self.w_down):
            nn.init.normal_(w, std=self.cfg.init_std, generator=generator)

    def forward(self, x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
        cfg = self.cfg
        B, T, H = x.shape
        Hq, Hkv, D = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        h = ops.rms_norm(x, self.attn_norm, cfg.rms_eps)
        qkv = ops.linear(h, self.wqkv).view(B, T, Hq + 2 * Hkv, D)
        q = ops.rms_norm(qkv[:, :, :Hq], self.q_norm, cfg.rms_eps).view(B, T, Hq, D)
        k = ops.rms_norm(qkv[:, :, Hq:Hq + Hkv], self.k_norm, cfg.rms_eps).view(B, T, Hkv, D)
        q = ops.apply_rope(q, cos, sin)
        k = ops.apply_rope(k, cos, sin)
        a = ops.flash_attention(q, k, qkv[:, :, Hq + Hkv:], causal=True)
        a = ops.linear(a.reshape(B, T, Hq * D), self.wo)
        h, x = ops.rms_norm(a, self.ffn_norm, cfg.rms_eps, residual=x)
        flat = h.reshape(B * T, H)
        logits = ops.linear(flat, self.router)
        idx, w, aux = topk_route(logits, cfg.top_k, cfg.norm_topk_prob)
        y = expert_parallel_ffn(flat, idx, w.to(flat.dtype), self.w_gate_up, self.w_down, self.workspace,
                                cfg.num_experts, self.ep_group,
                                result_is_region_output=getattr(self, "_tpb_region_is_layer", False))
        if cfg.aux_loss_coef and torch.is_grad_enabled():
            y = _AuxLoss.apply(y, aux, cfg.aux_loss_coef * self.loss_scale)
        return x + y.view(B, T, H)


class Qwen3MoE(nn.Module):
    def __init__(self, cfg: Qwen3MoEConfig, ep_group=None, device=None, dtype=None):
        super().__init__()
        kw = {"device": device, "dtype": dtype}
        self.cfg = cfg
        self.ep_group = ep_group
        self.ep_world = dist.get_world_size(ep_group) if dist.is_initialized() else 1
        self.embed = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, **kw))
        self.layers = nn.ModuleList([Qwen3MoEBlock(cfg, i, self.ep_world, **kw) for i in range(cfg.num_layers)])
        self.final_norm = nn.Parameter(torch.ones(cfg.hidden_size, **kw))
        self.lm_head = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, **kw))
        self._rope = None
        for l in self.layers:
            l.ep_group = ep_group

    def reset_parameters(self, seed: Optional[int] = None) -> None:
        gen = None
        if seed is not None:
            gen = torch.Generator(device=self.embed.device)
            gen.manual_seed(seed)
        nn.init.normal_(self.embed, std=self.cfg.init_std, generator=gen)
        nn.init.normal_(self.lm_head, std=self.cfg.init_std, generator=gen)
        for l in self.layers:
            l.reset_parameters(gen)

    def attach_workspace(self, tokens_per_rank: int, capacity_factor: float = 2.0) -> MoEWorkspace:
        """Allocate the shared expert-parallel buffers (collective; CUDA only)."""
        ws = MoEWorkspace(tokens_per_rank, self.cfg.top_k, self.cfg.hidden_size, self.cfg.num_experts,
                          group=self.ep_group, capacity_factor=capacity_factor)
        for l in self.layers:
            l.workspace = ws
        return ws

    def rope_tables(self, n: int, device):
        if self._rope is None or self._rope[0].shape[0] < n or self._rope[0].device != torch.device(device):
            self._rope = ops.rope_tables(max(n, self.cfg.max_seq_len), self.cfg.head_dim, self.cfg.rope_theta,
                                         device=device)
        return self._rope

    def layer_extra_args(self, tokens: Tensor):
        return self.rope_tables(tokens.shape[1], tokens.device)

    def embed_tokens(self, tokens: Tensor) -> Tensor:
        return _embedding(tokens, self.embed)

    def head(self, x: Tensor, targets: Optional[Tensor] = None) -> Tensor:
        h = ops.rms_norm(x, self.final_norm, self.cfg.rms_eps)
        logits = ops.linear(h, self.lm_head)
        if targets is None:
            return logits
        return ops.cross_entropy(logits.view(-1, logits.shape[-1]), targets.reshape(-1))

    def forward(self, tokens: Tensor, targets: Optional[Tensor] = None, position_ids=None,
                past_key_values=None) -> Tensor:
        cos, sin = self.rope_tables(tokens.shape[1], tokens.device)
        x = self.embed_tokens(tokens)
        for layer in self.layers:
            x = layer(x, cos, sin)
        return self.head(x, targets)
