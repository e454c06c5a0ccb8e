"""Pipeline schedules. Gradients are scaled by 1 / n_microbatches so that a step equals the
gradient of the mean loss over the full batch."""
from __future__ import annotations

from typing import Any, Callable, List, Optional

import torch
import torch.distributed as dist

from .microbatch import merge_chunks, split_args_kwargs_into_chunks
from .stage import PipelineStage


def _run_p2p(ops: List[dist.P2POp]) -> List:
    if not ops:
        return []
    return dist.batch_isend_irecv(ops)


def _wait(works) -> None:
    for w in works:
        w.wait()


class PipelineScheduleSingle:
    """One stage per rank."""

    def __init__(self, stage: PipelineStage, n_microbatches: int, loss_fn: Optional[Callable] = None,
                 scale_grads: bool = True):
        self.stage, self.n, self.loss_fn = stage, n_microbatches, loss_fn
        stage.grad_scale = 1.0 / n_microbatches if scale_grads else 1.0
        self._wrapped = None

    def _sync_wrappers(self, enable: bool) -> None:
        """DDP- and FSDP-wrapped stages reduce only on the last micro-batch's backward (the earlier
        micro-batches accumulate locally)."""
        m = self.stage.submod
        if hasattr(m, "require_backward_grad_sync"):
            m.require_backward_grad_sync = enable
        elif hasattr(m, "set_requires_gradient_sync"):
            m.set_requires_gradient_sync(enable)
            if not m._fsdp_state.reshard_after_forward:
                # parameters kept gathered across the step's micro-batches: shard them again only
                # after the last backward
                m.set_reshard_after_backward(enable)

    def step(self, *args, target=None, losses: Optional[List] = None, return_outputs: bool = True, **kwargs):
        """``return_outputs=False``: the last stage drops each micro-batch's output once its loss
        exists (no merged copy of, say, the logits of the whole batch)."""
        st = self.stage
        st.keep_outputs = return_outputs
        a_chunks, k_chunks = split_args_kwargs_into_chunks(args, kwargs, self.n) if st.is_first else ([()] * self.n, [{}] * self.n)
        t_chunks = list(torch.chunk(target, self.n)) if (st.is_last and target is not None) else [None] * self.n
        self._step_microbatches(a_chunks, k_chunks, t_chunks)
        out = None
        if st.is_last:
            if return_outputs:
                out = merge_chunks([st.outputs[i].detach() for i in range(self.n)])
            if losses is not None:
                losses.extend(st.losses[i] for i in range(self.n))
        st.outputs.clear()
        st.clear()
        return out

    def _step_microbatches(self, a, k, t):
        raise NotImplementedError


class ScheduleGPipe(PipelineScheduleSingle):
    """All forwards, then all backwards."""

    def _step_microbatches(self, a, k, t):
        st = self.stage
        sends = []
        for i in range(self.n):
            _wait(_run_p2p(st.get_fwd_recv_ops(i)))
            st.forward_one_chunk(i, a[i], k[i], t[i], self.loss_fn)
            sends += _run_p2p(st.get_fwd_send_ops(i))
        _wait(sends)
        sends = []
        for i in range(self.n):
            self._sync_wrappers(i == self.n - 1)
            _wait(_run_p2p(st.get_bwd_recv_ops(i)))
            st.backward_one_chunk(i)
            sends += _run_p2p(st.get_bwd_send_ops(i))
        _wait(sends)
        self._sync_wrappers(True)


class Schedule1F1B(PipelineScheduleSingle):
    """Warm-up forwards, steady one-forward-one-backward, cool-down backwards. In the steady
    state the send of an activation is batched with the receive of a gradient (and vice versa)
    so that neighbours never block each other."""

    def _step_microbatches(self, a, k, t):
        st, n = self.stage, self.n
        warm = min(n, st.num_stages - st.stage_index - 1)
        f = b = 0
        pending = []
        # warm-up
        for _ in range(warm):
            _wait(_run_p2p(st.get_fwd_recv_ops(f)))
            st.forward_one_chunk(f, a[f], k[f], t[f], self.loss_fn)
            pending += _run_p2p(st.get_fwd_send_ops(f))
            f += 1
        # steady state
        if f < n:
            _wait(_run_p2p(st.get_fwd_recv_ops(f)))
        while f < n:
            st.forward_one_chunk(f, a[f], k[f], t[f], self.loss_fn)
            works = _run_p2p(st.get_fwd_send_ops(f) + st.get_bwd_recv_ops(b))
            f += 1
            _wait(works)
            self._sync_wrappers(b == n - 1)
            st.backward_one_chunk(b)
            ops = st.get_bwd_send_ops(b)
            b += 1
            if f < n:
                ops += st.get_fwd_recv_ops(f)
            _wait(_run_p2p(ops))
        _wait(pending)
        # cool-down
        sends = []
        while b < n:
            self._sync_wrappers(b == n - 1)
            _wait(_run_p2p(st.get_bwd_recv_ops(b)))
            st.backward_one_chunk(b)
            sends += _run_p2p(st.get_bwd_send_ops(b))
            b += 1
        _wait(sends)
        self._sync_wrappers(True)


class PipelineScheduleMulti:
    """Several stages per rank (interleaved / looped placements)."""

    def __init__(self, stages: List[PipelineStage], n_microbatches: int, loss_fn: Optional[Callable] = None,
                 scale_grads: bool = True):
        self.stages, self.n, self.loss_fn = stages, n_microbatches, loss_fn
        for s in stages:
            s.grad_scale = 1.0 / n_microbatches if scale_grads else 1.0

    def step(self, *args, target=None, losses: Optional[List] = None, **kwargs):
        first = next((s for s in self.stages if s.is_first), None)
        last = next((s for s in self.stages if s.is_last), None)
        a, k = split_args_kwargs_into_chunks(args, kwargs, self.n) if first is not None else ([()] * self.n, [{}] * self.n)
        t = list(torch.chunk(target, self.n)) if (last is not None and target is not None) else [None] * self.n
        self._step_microbatches(a, k, t)
        out = None
        if last is not None:
            out = merge_chunks([last.outputs[i].detach() for i in range(self.n)])
            if losses is not None:
                losses.extend(last.losses[i] for i in range(self.n))
        for s in self.stages:
            s.outputs.clear()
            s.clear()
        return out


class ScheduleLoopedBFS(PipelineScheduleMulti):
    """Looped placement (stage s on rank s % world), breadth-first: all micro-batch forwards of local
    stage 0, then of local stage 1, ...; backwards in reverse. Simple and deadlock-free with plain
    batched p2p, but every micro-batch's activations are alive at the turn: the depth-first
    :class:`ScheduleInterleaved1F1B` (runtime.py) bounds them."""

    def _step_microbatches(self, a, k, t):
        for st in self.stages:
            sends = []
            for i in range(self.n):
                _wait(_run_p2p(st.get_fwd_recv_ops(i)))
                st.forward_one_chunk(i, a[i] if st.is_first else (), k[i] if st.is_first else {},
                                     t[i] if st.is_last else None, self.loss_fn)
                sends += _run_p2p(st.get_fwd_send_ops(i))
            _wait(sends)
        for st in reversed(self.stages):
            sends = []
            for i in range(self.n):
                _wait(_run_p2p(st.get_bwd_recv_ops(i)))
                st.backward_one_chunk(i)
                sends += _run_p2p(st.get_bwd_send_ops(i))
            _wait(sends)
