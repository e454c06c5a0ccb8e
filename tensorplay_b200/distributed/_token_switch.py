"""``TokenSwitch``: MoE token routing with expert parallelism. ``create_routing`` / ``dispatch`` /
``combine`` keep the reference's call shape (tensorplay/distributed/_token_switch.py:43-132) but
run the peer-memory kernels of ``tensorplay_b200.parallel.moe`` on CUDA; on CPU they permute
locally (single rank) like the reference does."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..parallel.moe import MoEWorkspace, topk_route


@dataclass
class Routing:
    topk_idx: torch.Tensor
    topk_weight: torch.Tensor
    dst_rank: Optional[torch.Tensor] = None
    dst_row: Optional[torch.Tensor] = None
    offsets: Optional[torch.Tensor] = None
    order: Optional[torch.Tensor] = None


class TokenSwitch:
    def __init__(self, num_experts: int, top_k: int, hidden: int, tokens: int, group=None,
                 capacity_factor: float = 2.0):
        self.E, self.k, self.H, self.T = num_experts, top_k, hidden, tokens
        self.ws = None
        if torch.cuda.is_available():
            self.ws = MoEWorkspace(tokens, top_k, hidden, num_experts, group=group, capacity_factor=capacity_factor)

    def create_routing(self, router_logits: torch.Tensor, renormalize: bool = True) -> Routing:
        idx, w, _ = topk_route(router_logits, self.k, renormalize)
        r = Routing(idx, w)
        if self.ws is not None and router_logits.is_cuda:
            r.dst_rank, r.dst_row, r.offsets = self.ws.route(idx)
        else:
            flat = idx.reshape(-1)
            r.order = torch.argsort(flat, stable=True)
            counts = torch.bincount(flat, minlength=self.E)
            r.offsets = torch.cat((counts.new_zeros(1), counts.cumsum(0)))
        return r

    def dispatch(self, x: torch.Tensor, routing: Routing) -> torch.Tensor:
        """Expert-sorted token rows (on CUDA: this rank's expert buffer, 128-row padded segments)."""
        if routing.dst_row is not None:
            self.ws.dispatch(x, routing.dst_rank, routing.dst_row, self.ws.xbuf)
            return self.ws.xbuf
        rows = x.repeat_interleave(self.k, dim=0)
        return rows[routing.order]

    def combine(self, expert_out: torch.Tensor, routing: Routing) -> torch.Tensor:
        if routing.dst_row is not None:
            if expert_out.data_ptr() != self.ws.ybuf.data_ptr():
                self.ws.ybuf[: expert_out.shape[0]].copy_(expert_out)
            out, _ = self.ws.combine(self.ws.ybuf, routing.dst_rank, routing.dst_row,
                                     w=routing.topk_weight.reshape(-1).float().contiguous())
            return out
        T = routing.topk_idx.shape[0]
        rows = torch.empty_like(expert_out)
        rows[routing.order] = expert_out
        return (rows.view(T, self.k, -1).float() * routing.topk_weight[..., None].float()).sum(1).to(expert_out.dtype)


TokenSwitchNCCL = TokenSwitch
