"""One pipeline stage: runs a sub-module on micro-batches, keeps what backward needs, and talks
to its neighbours with p2p ops that the schedules batch."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.distributed as dist
from torch import nn

_DT = [torch.float32, torch.bfloat16, torch.float16, torch.float64, torch.int64, torch.int32]


class PipelineStage:
    def __init__(self, submodule: nn.Module, stage_index: int, num_stages: int, device=None, group=None,
                 input_args=None, output_args=None):
        self.submod = submodule
        self.stage_index, self.num_stages = stage_index, num_stages
        self.device = torch.device(device) if device is not None else next(submodule.parameters()).device
        self.group = group
        self.group_size = dist.get_world_size(group) if dist.is_initialized() else 1
        self.group_rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.is_first = stage_index == 0
        self.is_last = stage_index == num_stages - 1
        # stage s lives on group rank s % group_size (several stages per rank when interleaved)
        self.prev_rank = (stage_index - 1) % self.group_size
        self.next_rank = (stage_index + 1) % self.group_size
        self.fwd_cache: Dict[int, tuple] = {}
        # example tensors given up front fix the activation shapes and skip the first-step hand-shake
        self.in_meta: Optional[tuple] = self._meta_of(input_args)
        self.out_meta: Optional[tuple] = self._meta_of(output_args)
        self.grad_scale = 1.0
        self.keep_outputs = True
        self.outputs: Dict[int, torch.Tensor] = {}
        self.losses: Dict[int, torch.Tensor] = {}
        self.recv_fwd: Dict[int, torch.Tensor] = {}
        self.recv_bwd: Dict[int, torch.Tensor] = {}

    @staticmethod
    def _meta_of(example) -> Optional[tuple]:
        if example is None:
            return None
        t = example[0] if isinstance(example, (tuple, list)) else example
        return tuple(t.shape), t.dtype

    def _g(self, r: int) -> int:
        return dist.get_global_rank(self.group, r) if self.group is not None else r

    # ---------------------------------------------------------------- shape hand-shake (first step)
    def _meta_send_op(self, t: torch.Tensor) -> dist.P2POp:
        """Non-blocking header send (shape / dtype of the activations), issued once, batched with
        the first activation so that the sender never blocks on a receiver that is still busy."""
        hdr = torch.zeros(10, dtype=torch.int64)
        hdr[0], hdr[1] = t.dim(), _DT.index(t.dtype)
        hdr[2: 2 + t.dim()] = torch.tensor(list(t.shape))
        self._hdr = hdr.to(self.device) if self.device.type == "cuda" else hdr
        return dist.P2POp(dist.isend, self._hdr, self._g(self.next_rank), self.group)

    def _recv_meta(self) -> tuple:
        hdr = torch.zeros(10, dtype=torch.int64, device=self.device if self.device.type == "cuda" else "cpu")
        dist.recv(hdr, self._g(self.prev_rank), group=self.group)
        hdr = hdr.cpu()
        nd = int(hdr[0])
        return tuple(int(v) for v in hdr[2: 2 + nd]), _DT[int(hdr[1])]

    def ensure_meta_in(self) -> None:
        if not self.is_first and self.in_meta is None:
            self.in_meta = self._recv_meta()

    # ---------------------------------------------------------------- p2p op builders
    def get_fwd_recv_ops(self, mb: int) -> List[dist.P2POp]:
        if self.is_first:
            return []
        self.ensure_meta_in()
        buf = torch.empty(self.in_meta[0], dtype=self.in_meta[1], device=self.device)
        self.recv_fwd[mb] = buf
        return [dist.P2POp(dist.irecv, buf, self._g(self.prev_rank), self.group)]

    def get_fwd_send_ops(self, mb: int) -> List[dist.P2POp]:
        if self.is_last:
            return []
        out = self.outputs[mb]
        ops = []
        if self.out_meta is None:
            self.out_meta = (tuple(out.shape), out.dtype)
            ops.append(self._meta_send_op(out))
        ops.append(dist.P2POp(dist.isend, out.detach().contiguous(), self._g(self.next_rank), self.group))
        return ops

    def get_bwd_recv_ops(self, mb: int) -> List[dist.P2POp]:
        if self.is_last:
            return []
        shape, dtype = self.out_meta
        buf = torch.empty(shape, dtype=dtype, device=self.device)
        self.recv_bwd[mb] = buf
        return [dist.P2POp(dist.irecv, buf, self._g(self.next_rank), self.group)]

    def get_bwd_send_ops(self, mb: int) -> List[dist.P2POp]:
        if self.is_first:
            return []
        g = self.fwd_cache.pop(("in_grad", mb))
        return [dist.P2POp(dist.isend, g.contiguous(), self._g(self.prev_rank), self.group)]

    # ---------------------------------------------------------------- compute
    def forward_one_chunk(self, mb: int, args=(), kwargs=None, target=None, loss_fn=None):
        kwargs = kwargs or {}
        if self.is_first:
            inputs = args
        else:
            x = self.recv_fwd.pop(mb)
            if x.is_floating_point():
                x.requires_grad_()
            inputs = (x,)
        out = self.submod(*inputs, **kwargs)
        if self.keep_outputs or not self.is_last:
            self.outputs[mb] = out
        loss = None
        if self.is_last and loss_fn is not None:
            loss = loss_fn(out, target)
            self.losses[mb] = loss.detach()
        self.fwd_cache[mb] = (inputs, out, loss)
        return out

    def backward_one_chunk(self, mb: int) -> None:
        inputs, out, loss = self.fwd_cache.pop(mb)
        if self.is_last:
            if loss is None:
                raise RuntimeError("the last stage needs a loss_fn to run backward")
            (loss * self.grad_scale).backward()
        else:
            out.backward(self.recv_bwd.pop(mb))
        if not self.is_first:
            self.fwd_cache[("in_grad", mb)] = inputs[0].grad
        self.outputs.pop(mb, None) if not self.is_last else None

    def clear(self) -> None:
        self.fwd_cache.clear()
        self.recv_fwd.clear()
        self.recv_bwd.clear()


# ---------------------------------------------------------------- split backward (input / weight)
def _stage_backward_input(stage: "PipelineStage", mb: int) -> None:
    """Gradient of the micro-batch with respect to the stage's INPUT only (the part of backward
    that the previous stage waits for); the graph is kept for the weight pass
    (tensorplay/distributed/pipelining/_backward.py: ``stage_backward_input``)."""
    inputs, out, loss = stage.fwd_cache[mb]
    if stage.is_last:
        if loss is None:
            raise RuntimeError("the last stage needs a loss_fn to run backward")
        root, seed = loss * stage.grad_scale, None
    else:
        root, seed = out, stage.recv_bwd.pop(mb)
    wrt = [t for t in inputs if isinstance(t, torch.Tensor) and t.requires_grad]
    params = [p for p in stage.submod.parameters() if p.requires_grad]
    if wrt:
        grads = torch.autograd.grad(root, wrt, seed, retain_graph=bool(params), allow_unused=True)
        if not stage.is_first:
            stage.fwd_cache[("in_grad", mb)] = grads[0]
    stage.fwd_cache[("w_pending", mb)] = (root, seed)
    stage.fwd_cache[mb] = (None, None, None)   # inputs / outputs are not needed again


def _stage_backward_weight(stage: "PipelineStage", mb: int) -> None:
    """Gradient with respect to the stage's PARAMETERS, accumulated into ``.grad``
    (``stage_backward_weight``): runs whenever the schedule has a free slot."""
    root, seed = stage.fwd_cache.pop(("w_pending", mb))
    stage.fwd_cache.pop(mb, None)
    params = [p for p in stage.submod.parameters() if p.requires_grad]
    if not params:
        return
    grads = torch.autograd.grad(root, params, seed, allow_unused=True)
    for p, g in zip(params, grads):
        if g is None:
            continue
        if p.grad is None:
            p.grad = g.detach()
        else:
            p.grad.add_(g)
    stage.outputs.pop(mb, None) if not stage.is_last else None


PipelineStage.backward_input_one_chunk = _stage_backward_input
PipelineStage.backward_weight_one_chunk = _stage_backward_weight
