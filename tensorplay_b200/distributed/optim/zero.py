"""ZeRO stage 1: every rank keeps the optimizer state of a slice of the parameters only, steps that
slice and receives the other slices' updated values.

After tensorplay/distributed/optim/zero_redundancy_optimizer.py (``ZeroRedundancyOptimizer`` :262,
``consolidate_state_dict`` :422, ``_partition_parameters`` :522, ``step`` :865, ``state_dict`` :944). The
reference broadcasts each owner's parameters one bucket per owner and device after the step; here the owned
parameters of each rank live in one flat buffer per dtype (the parameters are views into it), all flat buffers
have the same padded length, and the exchange after the step is ONE all-gather per dtype into a buffer whose
rank-``r`` slice the parameters of rank ``r`` alias: no per-tensor copies on either side.
"""
from __future__ import annotations

import copy
from typing import Any, Dict, List, Optional, Type

import torch
import torch.distributed as dist
from ..algorithms.join import Join, Joinable, JoinHook
from torch.optim import Optimizer


class _ZeroJoinHook(JoinHook):
    """A rank that ran out of inputs still owns a slice of the parameters: it steps that slice with the
    gradients that the data-parallel wrapper's shadow reduction left in ``.grad`` (list the wrapper before the
    optimizer in ``Join([...])``) and takes part in the exchange."""

    def __init__(self, zero: "ZeroRedundancyOptimizer"):
        self.zero = zero

    def main_hook(self):
        with torch.no_grad():
            self.zero._sync_hyperparameters()
            self.zero.optim.step()
            self.zero._exchange()


class ZeroRedundancyOptimizer(Optimizer, Joinable):
    def __init__(self, params, optimizer_class: Type[Optimizer], process_group=None,
                 parameters_as_bucket_view: bool = True, overlap_with_ddp: bool = False, **defaults: Any):
        if overlap_with_ddp:
            raise NotImplementedError(
                "overlap_with_ddp: the fused path of this package's DistributedDataParallel (fused_adamw=...) "
                "shards the optimizer state and steps inside the reduction; use it instead")
        params = list(params)
        if not params:
            raise ValueError("ZeroRedundancyOptimizer got an empty parameter list")
        if all(isinstance(p, torch.Tensor) for p in params):
            groups = [{"params": params}]
        elif all(isinstance(p, dict) for p in params):
            groups = [dict(g, params=list(g["params"])) for g in params]
        else:
            raise TypeError("params must be an iterable of tensors or of dicts")
        Optimizer.__init__(self, groups, defaults)
        Joinable.__init__(self)
        self.process_group = process_group if process_group is not None else dist.group.WORLD
        self.world_size = dist.get_world_size(self.process_group)
        self.rank = dist.get_rank(self.process_group)
        self._optim_class, self._defaults = optimizer_class, defaults
        self.parameters_as_bucket_view = parameters_as_bucket_view
        self._all_states: Optional[List[dict]] = None   # filled on the target rank by consolidate_state_dict
        self.initialized = False
        self._build()

    # ------------------------------------------------------------------ partition
    def _all_params(self) -> List[torch.Tensor]:
        return [p for g in self.param_groups for p in g["params"]]

    def _partition(self) -> List[List[Dict[str, Any]]]:
        """Per rank, a list of parameter groups holding that rank's parameters. Largest parameter first onto
        the lightest rank; ties go to the lower rank, so every rank computes the same assignment."""
        load = [0] * self.world_size
        per_rank: List[List[Dict[str, Any]]] = [[] for _ in range(self.world_size)]
        self._owner: Dict[int, int] = {}
        for g in self.param_groups:
            mine: List[List[torch.Tensor]] = [[] for _ in range(self.world_size)]
            order = sorted(range(len(g["params"])), key=lambda i: -g["params"][i].numel())
            for i in order:
                p = g["params"][i]
                r = min(range(self.world_size), key=lambda k: (load[k], k))
                load[r] += p.numel()
                mine[r].append((i, p))
                self._owner[id(p)] = r
            for r in range(self.world_size):
                sub = {k: v for k, v in g.items() if k != "params"}
                sub["params"] = [p for _, p in sorted(mine[r], key=lambda t: t[0])]
                per_rank[r].append(sub)
        return per_rank

    def _build(self) -> None:
        self._per_rank = self._partition()
        # flat exchange buffers: per (dtype, device), [world, padded] with rank r's parameters packed in row r
        self._flat: Dict[Any, torch.Tensor] = {}
        self._rows: Dict[Any, List[List[torch.Tensor]]] = {}
        by_key: Dict[Any, List[List[torch.Tensor]]] = {}
        for r in range(self.world_size):
            for g in self._per_rank[r]:
                for p in g["params"]:
                    by_key.setdefault((p.dtype, p.device), [[] for _ in range(self.world_size)])[r].append(p)
        for key, rows in by_key.items():
            padded = max(sum(p.numel() for p in row) for row in rows)
            padded = (padded + 127) // 128 * 128
            flat = torch.zeros(self.world_size, padded, dtype=key[0], device=key[1])
            for r, row in enumerate(rows):
                off = 0
                for p in row:
                    v = flat[r, off: off + p.numel()].view(p.shape)
                    v.copy_(p.data)
                    if self.parameters_as_bucket_view:
                        p.data = v
                    off += p.numel()
            self._flat[key] = flat
            self._rows[key] = rows
        local_groups = [g for g in self._per_rank[self.rank]]
        if not any(g["params"] for g in local_groups):
            # an optimizer needs at least one parameter: a rank without any holds a dummy one
            self._dummy = torch.zeros(1, requires_grad=True)
            local_groups = [dict(local_groups[0], params=[self._dummy])] + local_groups[1:]
        self.optim = self._optim_class([g for g in local_groups if g["params"]] or local_groups, **self._defaults)
        self._local_groups = local_groups
        self.state = self.optim.state
        self.initialized = True

    def add_param_group(self, param_group: dict) -> None:
        """Before the first build it is the base class collecting the groups; afterwards the partition and the
        flat buffers are rebuilt (optimizer state gathered so far is kept for the parameters that stay)."""
        if not getattr(self, "initialized", False):
            return Optimizer.add_param_group(self, param_group)
        old_state = {id(p): s for p, s in self.optim.state.items()}
        Optimizer.add_param_group(self, param_group)
        self._build()
        for p in [q for g in self.optim.param_groups for q in g["params"]]:
            if id(p) in old_state:
                self.optim.state[p] = old_state[id(p)]

    # ------------------------------------------------------------------ step
    def _sync_hyperparameters(self) -> None:
        # the local optimizer holds the groups that own parameters on this rank (all of them when none does), in
        # order: pair them with the outer groups by position, never by comparing group dictionaries
        keep = [i for i, g in enumerate(self._local_groups) if g["params"]] or list(range(len(self._local_groups)))
        for local, i in zip(self.optim.param_groups, keep):
            glob = self.param_groups[i]
            for k, v in glob.items():
                if k != "params":
                    local[k] = v

    def _exchange(self) -> None:
        for key, flat in self._flat.items():
            if not self.parameters_as_bucket_view:
                off = 0
                for p in self._rows[key][self.rank]:
                    flat[self.rank, off: off + p.numel()].copy_(p.data.reshape(-1))
                    off += p.numel()
            if flat.device.type == "cuda":
                dist.all_gather_into_tensor(flat.view(-1), flat[self.rank].clone(), group=self.process_group)
            else:
                dist.all_gather(list(flat.unbind(0)), flat[self.rank].clone(), group=self.process_group)
            if not self.parameters_as_bucket_view:
                for r, row in enumerate(self._rows[key]):
                    off = 0
                    for p in row:
                        if r != self.rank:
                            p.data.copy_(flat[r, off: off + p.numel()].view(p.shape))
                        off += p.numel()

    @torch.no_grad()
    def step(self, closure=None, **kwargs):
        Join.notify_join_context(self)
        self._sync_hyperparameters()
        if closure is not None:
            with torch.enable_grad():
                loss = self.optim.step(closure=closure, **kwargs)
        else:
            loss = self.optim.step(**kwargs)
        self._exchange()
        self._all_states = None
        return loss

    # ------------------------------------------------------------------ Joinable
    def join_hook(self, **kwargs) -> JoinHook:
        return _ZeroJoinHook(self)

    @property
    def join_device(self) -> torch.device:
        return self._all_params()[0].device

    @property
    def join_process_group(self):
        return self.process_group

    # ------------------------------------------------------------------ state dicts
    def _param_index(self) -> Dict[int, int]:
        return {id(p): i for i, p in enumerate(self._all_params())}

    def _local_state_by_global_index(self) -> Dict[int, dict]:
        idx = self._param_index()
        return {idx[id(p)]: s for p, s in self.optim.state.items() if id(p) in idx}

    def consolidate_state_dict(self, to: int = 0) -> None:
        """Collect every rank's slice of the optimizer state on rank ``to`` (as CPU tensors)."""
        def cpu(o):
            if isinstance(o, torch.Tensor):
                return o.detach().cpu()
            if isinstance(o, dict):
                return {k: cpu(v) for k, v in o.items()}
            return copy.deepcopy(o)
        mine = cpu(self._local_state_by_global_index())
        out = [None] * self.world_size if self.rank == to else None
        dist.gather_object(mine, out, dst=dist.get_global_rank(self.process_group, to)
                           if self.process_group is not dist.group.WORLD else to, group=self.process_group)
        self._all_states = out

    def state_dict(self) -> Dict[str, Any]:
        """The state of the WHOLE optimizer in the layout of an unsharded one; valid on the rank that
        ``consolidate_state_dict`` targeted, after that call."""
        if self._all_states is None:
            raise RuntimeError("Optimizer state has not been consolidated on this rank. "
                               "Call consolidate_state_dict(to=rank) on all ranks first.")
        state: Dict[int, dict] = {}
        for part in self._all_states:
            state.update(part)
        groups, off = [], 0
        for g in self.param_groups:
            d = {k: v for k, v in g.items() if k != "params"}
            d["params"] = list(range(off, off + len(g["params"])))
            off += len(g["params"])
            groups.append(d)
        return {"state": dict(sorted(state.items())), "param_groups": groups}

    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        """Takes an unsharded state dict (every rank passes the same one) and keeps this rank's slice."""
        params = self._all_params()
        for g, sg in zip(self.param_groups, state_dict["param_groups"]):
            for k, v in sg.items():
                if k != "params":
                    g[k] = v
        self.optim.state.clear()
        for i, s in state_dict["state"].items():
            p = params[int(i)]
            if self._owner[id(p)] == self.rank:
                self.optim.state[p] = {k: (v.to(p.device) if isinstance(v, torch.Tensor) else copy.deepcopy(v))
                                       for k, v in s.items()}
        self._sync_hyperparameters()
        self._all_states = None

