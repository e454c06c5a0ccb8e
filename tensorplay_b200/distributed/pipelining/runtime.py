"""Schedule runtime: executes per-rank lists of compute actions (F forward, B full backward, I
input-gradient backward, W weight-gradient backward) for any placement of stages on ranks, and the
schedules built on it: depth-first interleaved 1F1B, interleaved zero bubble, the V-shaped zero
bubble placements, and schedules loaded from a CSV file.

How it runs. Every rank derives the same global table by simulating all ranks: time advances in
ticks, a rank executes its next action when what the action needs was produced in an earlier tick
(otherwise it idles, or - zero-bubble schedules - fills the slot with a pending W). After a tick
the activations and gradients produced in it are exchanged in ONE batched isend / irecv per rank;
both sides order the transfers of a batch by the same key, so matching never depends on timing
and no send waits behind an unposted receive.

Counterparts in the reference: ``_PipelineScheduleRuntime`` (CSV-driven, schedules.py:1277),
``ScheduleInterleaved1F1B`` :1636, ``ScheduleInterleavedZeroBubble`` :1723,
``ScheduleZBVZeroBubble`` :1886, ``ScheduleDualPipeV`` :2057, split backward in ``_backward.py``.
"""
from __future__ import annotations

import csv
import re
from typing import Callable, Dict, List, NamedTuple, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from .microbatch import merge_chunks, split_args_kwargs_into_chunks
from .stage import PipelineStage


class Action(NamedTuple):
    stage: int
    kind: str  # "F", "B", "I", "W"
    mb: int

    def __str__(self) -> str:
        return f"{self.stage}{self.kind}{self.mb}"


_ACTION_RE = re.compile(r"^\s*(\d+)\s*([FBIW])\s*(\d+)\s*$")


def parse_action(text: str) -> Optional[Action]:
    """``"2F0"`` -> ``Action(2, "F", 0)``; communication / FSDP entries of a CSV (``SEND_F`` ...) are
    not compute actions and return ``None`` (the runtime derives the transfers itself)."""
    m = _ACTION_RE.match(text)
    return Action(int(m.group(1)), m.group(2), int(m.group(3))) if m else None


# ------------------------------------------------------------------------------------------ placements
def loop_placement(world: int) -> Callable[[int], int]:
    return lambda s: s % world


def v_placement(world: int) -> Callable[[int], int]:
    """Stage s on rank s for the first ``world`` stages, then back down: rank r holds stages r and
    2 * world - 1 - r (the last and the first stage share rank 0's neighbour-free end)."""
    return lambda s: s if s < world else 2 * world - 1 - s


# ------------------------------------------------------------------------------------------ simulation
class Tick(NamedTuple):
    actions: Dict[int, Action]                       # rank -> action of this tick
    transfers: List[Tuple[int, int, str, int, int]]  # (src rank, dst rank, "act" | "grad", consumer stage, mb)


def simulate(order: Dict[int, List[Action]], num_stages: int, rank_of: Callable[[int], int],
             fill_with_weight: bool = False, max_pending_w: int = 1 << 30) -> List[Tick]:
    """Assign ticks to the ordered per-rank action lists. ``fill_with_weight``: the lists hold F and
    I only; each I leaves a W behind that runs when the rank would otherwise idle (or when more than
    ``max_pending_w`` are waiting), and the rest is flushed at the end."""
    ranks = sorted(order)
    pos = {r: 0 for r in ranks}
    pending_w: Dict[int, List[Action]] = {r: [] for r in ranks}
    done_at: Dict[Tuple[int, str, int], int] = {}
    ticks: List[Tick] = []
    last = num_stages - 1

    def ready(a: Action, t: int) -> bool:
        def before(key):
            return key in done_at and done_at[key] < t
        if a.kind == "F":
            return a.stage == 0 or before((a.stage - 1, "F", a.mb))
        if a.kind in ("B", "I"):
            if not before((a.stage, "F", a.mb)):
                return False
            return a.stage == last or before((a.stage + 1, "B", a.mb)) or before((a.stage + 1, "I", a.mb))
        return before((a.stage, "I", a.mb))  # W

    t = 0
    guard = sum(len(v) for v in order.values()) * 4 + 64
    while any(pos[r] < len(order[r]) or pending_w[r] for r in ranks):
        acts: Dict[int, Action] = {}
        for r in ranks:
            nxt = order[r][pos[r]] if pos[r] < len(order[r]) else None
            must_w = fill_with_weight and len(pending_w[r]) > max_pending_w
            if nxt is not None and ready(nxt, t) and not must_w:
                acts[r] = nxt
                pos[r] += 1
                if fill_with_weight and nxt.kind == "I":
                    pending_w[r].append(Action(nxt.stage, "W", nxt.mb))
            elif pending_w[r] and ready(pending_w[r][0], t):
                acts[r] = pending_w[r].pop(0)
        transfers = []
        for r, a in acts.items():
            done_at[(a.stage, a.kind, a.mb)] = t
            if a.kind == "F" and a.stage < last and rank_of(a.stage + 1) != r:
                transfers.append((r, rank_of(a.stage + 1), "act", a.stage + 1, a.mb))
            if a.kind in ("B", "I") and a.stage > 0 and rank_of(a.stage - 1) != r:
                transfers.append((r, rank_of(a.stage - 1), "grad", a.stage - 1, a.mb))
        ticks.append(Tick(acts, sorted(transfers)))
        t += 1
        if t > guard:
            stuck = {r: str(order[r][pos[r]]) for r in ranks if pos[r] < len(order[r])}
            raise RuntimeError(f"the schedule cannot make progress (dependency cycle); waiting actions: {stuck}")
    return ticks


# ------------------------------------------------------------------------------------------ runtime
class PipelineScheduleRuntime:
    """Runs a table of compute actions on this rank's stages.

    ``stages``: this rank's :class:`PipelineStage` objects; ``order``: rank -> ordered actions of
    EVERY rank (each rank simulates the whole pipeline); ``rank_of``: stage -> rank."""

    def __init__(self, stages: Sequence[PipelineStage], n_microbatches: int, loss_fn: Optional[Callable] = None,
                 order: Optional[Dict[int, List[Action]]] = None, rank_of: Optional[Callable[[int], int]] = None,
                 scale_grads: bool = True, fill_with_weight: bool = False, max_pending_w: int = 1 << 30):
        self.stages = {s.stage_index: s for s in stages}
        first = stages[0]
        self.group = first.group
        self.world = first.group_size
        self.rank = first.group_rank
        self.num_stages = first.num_stages
        self.n, self.loss_fn = n_microbatches, loss_fn
        self.rank_of = rank_of or loop_placement(self.world)
        for s in stages:
            s.grad_scale = 1.0 / n_microbatches if scale_grads else 1.0
            if self.rank_of(s.stage_index) != self.rank:
                raise ValueError(f"stage {s.stage_index} is placed on rank {self.rank_of(s.stage_index)}, not {self.rank}")
        self.fill_with_weight, self.max_pending_w = fill_with_weight, max_pending_w
        self.order = order
        self._ticks: Optional[List[Tick]] = None
        self._meta: Dict[int, Tuple[tuple, torch.dtype]] = {}   # stage -> (shape, dtype) of its INPUT activation

    # ---- table
    def ticks(self) -> List[Tick]:
        if self._ticks is None:
            if self.order is None:
                raise ValueError("no action order given")
            self._ticks = simulate(self.order, self.num_stages, self.rank_of, self.fill_with_weight, self.max_pending_w)
        return self._ticks

    def bubble_fraction(self) -> float:
        """Idle share of the simulated table (every action one tick)."""
        t = self.ticks()
        busy = sum(len(x.actions) for x in t)
        return 1.0 - busy / (len(t) * len(self.order))

    def dump_csv(self, path: str) -> None:
        """One row per rank, one cell per tick (empty = idle), cells spelled like ``2F0``."""
        t = self.ticks()
        with open(path, "w", newline="") as f:
            w = csv.writer(f)
            for r in sorted(self.order):
                w.writerow([str(x.actions[r]) if r in x.actions else "" for x in t])

    @staticmethod
    def load_csv(path: str) -> Dict[int, List[Action]]:
        """Rank r = row r; cells that are not compute actions (transfers, UNSHARD / RESHARD /
        REDUCE_GRAD, empty) are skipped: the runtime places transfers and FSDP switches itself."""
        order: Dict[int, List[Action]] = {}
        with open(path, newline="") as f:
            for r, row in enumerate(csv.reader(f)):
                order[r] = [a for a in (parse_action(c) for c in row) if a is not None]
        return order

    # ---- activation shapes (first step)
    def _g(self, r: int) -> int:
        return dist.get_global_rank(self.group, r) if self.group is not None else r

    def _ensure_meta(self, first_inputs) -> None:
        if self._meta or self.num_stages == 1:
            return
        # stages given example tensors need no probing
        if all(st.in_meta is not None or st.is_first for st in self.stages.values()) and self.world == 1:
            for st in self.stages.values():
                if st.in_meta is not None:
                    self._meta[st.stage_index] = st.in_meta
            return
        # one pass over the stages: the owner runs its module once without recording a graph and tells
        # everybody the shape of what it produces (stochastic layers see one extra call)
        meta = None
        for s in range(self.num_stages - 1):
            owner = self.rank_of(s)
            box = [None]
            if owner == self.rank:
                st = self.stages[s]
                if st.out_meta is not None:
                    box[0] = st.out_meta
                else:
                    with torch.no_grad():
                        if s == 0:
                            out = st.submod(*first_inputs[0], **first_inputs[1])
                        else:
                            shape, dtype = self._meta[s]
                            out = st.submod(torch.zeros(shape, dtype=dtype, device=st.device))
                    box[0] = (tuple(out.shape), out.dtype)
            if self.world > 1:
                dist.broadcast_object_list(box, src=self._g(owner), group=self.group)
            meta = box[0]
            self._meta[s + 1] = meta

    # ---- one step
    def step(self, *args, target=None, losses: Optional[List] = None, return_outputs: bool = True, **kwargs):
        n = self.n
        first = self.stages.get(0)
        last = self.stages.get(self.num_stages - 1)
        a_chunks, k_chunks = split_args_kwargs_into_chunks(args, kwargs, n) if first is not None else ([()] * n, [{}] * n)
        t_chunks = list(torch.chunk(target, n)) if (last is not None and target is not None) else [None] * n
        self._ensure_meta((a_chunks[0], k_chunks[0]))
        for st in self.stages.values():
            st.keep_outputs = return_outputs or not st.is_last
        remaining_b = {s: n for s in self.stages}
        handed: Dict[Tuple[str, int, int], torch.Tensor] = {}
        pending_sends = []
        for tick in self.ticks():
            a = tick.actions.get(self.rank)
            if a is not None:
                st = self.stages[a.stage]
                if a.kind == "F":
                    if not st.is_first:
                        st.recv_fwd[a.mb] = handed.pop(("act", a.stage, a.mb))
                    st.forward_one_chunk(a.mb, a_chunks[a.mb] if st.is_first else (), k_chunks[a.mb] if st.is_first else {},
                                         t_chunks[a.mb] if st.is_last else None, self.loss_fn)
                    if not st.is_last and self.rank_of(a.stage + 1) == self.rank:
                        handed[("act", a.stage + 1, a.mb)] = st.outputs[a.mb].detach()   # neighbour stage on this rank
                elif a.kind in ("B", "I"):
                    if not st.is_last:
                        st.recv_bwd[a.mb] = handed.pop(("grad", a.stage, a.mb))
                    if a.kind == "B":
                        remaining_b[a.stage] -= 1
                        self._sync_wrappers(st, remaining_b[a.stage] == 0)
                        st.backward_one_chunk(a.mb)
                    else:
                        st.backward_input_one_chunk(a.mb)
                    if not st.is_first and self.rank_of(a.stage - 1) == self.rank:
                        handed[("grad", a.stage - 1, a.mb)] = st.fwd_cache.pop(("in_grad", a.mb))
                else:
                    remaining_b[a.stage] -= 1
                    self._sync_wrappers(st, remaining_b[a.stage] == 0)
                    st.backward_weight_one_chunk(a.mb)
            # transfers of this tick that touch this rank, both directions in one batch
            ops, recvs = [], []
            for src, dst, kind, stage, mb in tick.transfers:
                if src == self.rank:
                    producer = self.stages[stage - 1] if kind == "act" else self.stages[stage + 1]
                    t = producer.outputs[mb].detach() if kind == "act" else producer.fwd_cache.pop(("in_grad", mb))
                    ops.append(dist.P2POp(dist.isend, t.contiguous(), self._g(dst), self.group))
                elif dst == self.rank:
                    shape, dtype = self._meta[stage] if kind == "act" else self._meta[stage + 1]
                    buf = torch.empty(shape, dtype=dtype, device=self.stages[stage].device)
                    recvs.append(((kind, stage, mb), buf))
                    ops.append(dist.P2POp(dist.irecv, buf, self._g(src), self.group))
            if ops:
                works = dist.batch_isend_irecv(ops)
                for w in works:
                    w.wait()
                for key, buf in recvs:
                    if key[0] == "act" and buf.is_floating_point():
                        buf.requires_grad_()
                    handed[key] = buf
        for st in self.stages.values():
            self._sync_wrappers(st, True)
        out = None
        if last is not None:
            if return_outputs:
                out = merge_chunks([last.outputs[i].detach() for i in range(n)])
            if losses is not None:
                losses.extend(last.losses[i] for i in range(n))
        for st in self.stages.values():
            st.outputs.clear()
            st.losses.clear()
            st.clear()
        return out

    @staticmethod
    def _sync_wrappers(st: PipelineStage, enable: bool) -> None:
        """DDP- and FSDP-wrapped stages reduce only with their last backward of the step."""
        m = st.submod
        if hasattr(m, "require_backward_grad_sync"):
            m.require_backward_grad_sync = enable
        elif hasattr(m, "set_requires_gradient_sync"):
            m.set_requires_gradient_sync(enable)
            if not m._fsdp_state.reshard_after_forward:
                m.set_reshard_after_backward(enable)


# ------------------------------------------------------------------------------------------ orders
def interleaved_1f1b_order(world: int, local_stages: int, n_microbatches: int, split_backward: bool = False
                           ) -> Dict[int, List[Action]]:
    """Depth-first interleaved 1F1B for the looped placement (stage = chunk * world + rank):
    micro-batches advance in rounds of ``world``; a rank warms up with
    ``2 (world - rank - 1) + (local_stages - 1) world`` forwards, then alternates one forward with one
    backward, so at most that many micro-batch activations (plus one) are alive per rank - not the
    whole batch as in a breadth-first order. ``split_backward``: emit I instead of B."""
    if n_microbatches % world:
        raise ValueError(f"interleaved 1F1B needs the number of micro-batches ({n_microbatches}) to be a multiple of "
                         f"the pipeline size ({world})")
    total = n_microbatches * local_stages
    bk = "I" if split_backward else "B"

    def fwd(k, r):
        chunk = (k // world) % local_stages
        mb = (k // (world * local_stages)) * world + k % world
        return Action(chunk * world + r, "F", mb)

    def bwd(k, r):
        chunk = local_stages - 1 - (k // world) % local_stages
        mb = (k // (world * local_stages)) * world + k % world
        return Action(chunk * world + r, bk, mb)

    order = {}
    for r in range(world):
        warm = min(total, 2 * (world - r - 1) + (local_stages - 1) * world)
        acts = [fwd(k, r) for k in range(warm)]
        for i in range(total - warm):
            acts.append(fwd(warm + i, r))
            acts.append(bwd(i, r))
        acts += [bwd(i, r) for i in range(total - warm, total)]
        order[r] = acts
    return order


def greedy_zero_bubble_order(num_stages: int, rank_of: Callable[[int], int], n_microbatches: int,
                             max_inflight: int, max_pending_w: int) -> Dict[int, List[Action]]:
    """Split-backward order for ANY placement, found by simulating the pipeline with one rule per
    rank and tick: run an input-gradient pass if one is ready (oldest micro-batch first, the stage
    nearest the loss first), else a forward if fewer than ``max_inflight`` micro-batch activations
    are alive on the rank (the stage nearest the loss first, so that work drains toward the loss),
    else a waiting weight-gradient pass; a backlog of more than ``max_pending_w`` weight passes is
    worked off first. Every rank computes the same table."""
    ranks = sorted({rank_of(s) for s in range(num_stages)})
    local = {r: [s for s in range(num_stages) if rank_of(s) == r] for r in ranks}
    next_f = {s: 0 for s in range(num_stages)}
    next_i = {s: 0 for s in range(num_stages)}
    pend_w: Dict[int, List[Action]] = {r: [] for r in ranks}
    done_at: Dict[Tuple[int, str, int], int] = {}
    order: Dict[int, List[Action]] = {r: [] for r in ranks}
    last, n = num_stages - 1, n_microbatches
    t = 0
    while any(next_i[s] < n for s in range(num_stages)) or any(pend_w[r] for r in ranks):
        chosen: Dict[int, Action] = {}
        for r in ranks:
            def before(key):
                return key in done_at and done_at[key] < t
            inflight = sum(next_f[s] - next_i[s] for s in local[r])
            cand_i = [Action(s, "I", next_i[s]) for s in local[r]
                      if next_i[s] < next_f[s] and before((s, "F", next_i[s])) and
                      (s == last or before((s + 1, "I", next_i[s])))]
            cand_f = [Action(s, "F", next_f[s]) for s in local[r]
                      if next_f[s] < n and (s == 0 or before((s - 1, "F", next_f[s])))]
            if len(pend_w[r]) > max_pending_w:
                chosen[r] = pend_w[r].pop(0)
            elif cand_i:
                chosen[r] = min(cand_i, key=lambda a: (a.mb, -a.stage))
            elif cand_f and inflight < max_inflight:
                chosen[r] = max(cand_f, key=lambda a: (a.stage, -a.mb))
            elif pend_w[r]:
                chosen[r] = pend_w[r].pop(0)
        for r, a in chosen.items():
            done_at[(a.stage, a.kind, a.mb)] = t
            order[r].append(a)
            if a.kind == "F":
                next_f[a.stage] += 1
            elif a.kind == "I":
                next_i[a.stage] += 1
                pend_w[r].append(Action(a.stage, "W", a.mb))
        t += 1
        if t > 16 * num_stages * n + 64:
            raise RuntimeError("the greedy schedule search does not terminate")
    return order


# ------------------------------------------------------------------------------------------ schedules
class ScheduleInterleaved1F1B(PipelineScheduleRuntime):
    """Looped placement, depth-first: see :func:`interleaved_1f1b_order`."""

    def __init__(self, stages, n_microbatches, loss_fn=None, scale_grads=True):
        st = stages[0]
        super().__init__(stages, n_microbatches, loss_fn, scale_grads=scale_grads,
                         order=interleaved_1f1b_order(st.group_size, st.num_stages // st.group_size, n_microbatches))


class ScheduleInterleavedZeroBubble(PipelineScheduleRuntime):
    """Interleaved 1F1B with the backward split: input gradients keep the order of the 1F1B
    backwards (they are what the neighbour waits for), weight gradients fill the slots in which the
    rank would wait, at most ``max_pending_w`` of them outstanding."""

    def __init__(self, stages, n_microbatches, loss_fn=None, scale_grads=True, max_pending_w: Optional[int] = None):
        st = stages[0]
        world, local = st.group_size, st.num_stages // st.group_size
        super().__init__(stages, n_microbatches, loss_fn, scale_grads=scale_grads,
                         order=interleaved_1f1b_order(world, local, n_microbatches, split_backward=True),
                         fill_with_weight=True, max_pending_w=max_pending_w if max_pending_w is not None else 2 * world)


class ScheduleZBVZeroBubble(PipelineScheduleRuntime):
    """Two stages per rank in a V; split backward, weight gradients in the idle slots; at most
    ``2 * world`` micro-batch activations alive per rank (the memory of 1F1B)."""

    def __init__(self, stages, n_microbatches, loss_fn=None, scale_grads=True, max_pending_w: Optional[int] = None):
        st = stages[0]
        world = st.group_size
        if st.num_stages != 2 * world:
            raise ValueError("the V placement needs exactly two stages per rank")
        place = v_placement(world)
        super().__init__(stages, n_microbatches, loss_fn, scale_grads=scale_grads, rank_of=place,
                         order=greedy_zero_bubble_order(2 * world, place, n_microbatches, max_inflight=2 * world,
                                                        max_pending_w=max_pending_w if max_pending_w is not None else 2 * world))


class ScheduleDualPipeV(ScheduleZBVZeroBubble):
    """The V placement with the weight-gradient backlog kept at one pass: every input-gradient pass
    is followed by a weight-gradient pass unless an input is already waiting, which pairs a forward
    of one leg with the backward of the other in neighbouring slots (the reference's DualPipeV
    overlaps such a pair inside one step; here they run back to back)."""

    def __init__(self, stages, n_microbatches, loss_fn=None, scale_grads=True):
        super().__init__(stages, n_microbatches, loss_fn, scale_grads, max_pending_w=1)


class ScheduleFromCSV(PipelineScheduleRuntime):
    """Executes the compute actions of a CSV file (row = rank, cells like ``1F0``, ``1I0``, ``1W0``,
    ``1B0``); ``rank_of`` defaults to the looped placement."""

    def __init__(self, stages, n_microbatches, loss_fn=None, csv_path: str = "", rank_of=None, scale_grads=True):
        super().__init__(stages, n_microbatches, loss_fn, scale_grads=scale_grads, rank_of=rank_of,
                         order=PipelineScheduleRuntime.load_csv(csv_path))
