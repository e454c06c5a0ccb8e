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
        """Expert-sorted token rows (on CUDA: a copy of this rank's expert buffer, 128-row padded
        segments). Differentiable: the gradient of the rows is combined back onto the tokens."""
        if routing.dst_row is not None:
            return _DispatchFn.apply(x, self, routing)
        rows = x.repeat_interleave(self.k, dim=0)
        return rows[routing.order]

    def combine(self, expert_out: torch.Tensor, routing: Routing) -> torch.Tensor:
        """``out[t] = sum_k w[t, k] * expert_out[row(t, k)]``. Differentiable with respect to the
        expert outputs (the scaled gradient rows are dispatched to the experts' owners) and to the
        routing weights (dot products of the token gradient with the rows)."""
        if routing.dst_row is not None:
            return _CombineFn.apply(expert_out, routing.topk_weight, self, routing)
        T = routing.topk_idx.shape[0]
        rows = torch.empty_like(expert_out)
        rows[routing.order] = expert_out
        return (rows.view(T, self.k, -1).float() * routing.topk_weight[..., None].float()).sum(1).to(expert_out.dtype)


class _DispatchFn(torch.autograd.Function):
    """Rows to their experts' owners; backward = unweighted combine of the row gradients
    (tensorplay/distributed/_token_switch.py:43-84 gives dispatch / combine autograd on one process)."""

    @staticmethod
    def forward(ctx, x, switch: "TokenSwitch", routing: Routing):
        ws = switch.ws
        ws.dispatch(x.contiguous(), routing.dst_rank, routing.dst_row, ws.xbuf)
        ws.generation += 1
        ctx.switch, ctx.routing, ctx.tokens = switch, routing, x.shape[0]
        return ws.xbuf.clone()

    @staticmethod
    def backward(ctx, d_rows):
        ws, r = ctx.switch.ws, ctx.routing
        ws.ybuf.copy_(d_rows)
        ws.generation += 1
        dx, _ = ws.combine(ws.ybuf, r.dst_rank, r.dst_row, tokens=ctx.tokens)
        return dx, None, None


class _CombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, expert_out, topk_weight, switch: "TokenSwitch", routing: Routing):
        ws = switch.ws
        if expert_out.data_ptr() != ws.ybuf.data_ptr():
            ws.ybuf[: expert_out.shape[0]].copy_(expert_out)
        ws.generation += 1
        wf = topk_weight.reshape(-1).float().contiguous()
        out, _ = ws.combine(ws.ybuf, routing.dst_rank, routing.dst_row, w=wf)
        ctx.save_for_backward(expert_out, wf)
        ctx.switch, ctx.routing, ctx.wshape, ctx.wdtype = switch, routing, topk_weight.shape, topk_weight.dtype
        return out

    @staticmethod
    def backward(ctx, dy):
        expert_out, wf = ctx.saved_tensors
        ws, r = ctx.switch.ws, ctx.routing
        dy = dy.contiguous()
        T = dy.shape[0]
        d_w = None
        if ctx.needs_input_grad[1]:
            # the rows of this forward, back in the buffer that the peers read
            ws.ybuf[: expert_out.shape[0]].copy_(expert_out)
            _, dots = ws.combine(ws.ybuf, r.dst_rank, r.dst_row, tokens=T, g=dy, want_out=False)
            d_w = dots.view(ctx.wshape).to(ctx.wdtype)
        ws.dispatch(dy, r.dst_rank, r.dst_row, ws.dbuf, scale=wf)
        ws.generation += 1
        return ws.dbuf[: expert_out.shape[0]].clone(), d_w, None, None


TokenSwitchNCCL = TokenSwitch
