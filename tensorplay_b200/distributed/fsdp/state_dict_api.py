"""State-dict types, their configurations, the optimizer-state helpers and the sharded gradient scaler of the
wrapper class ``FullyShardedDataParallel``.

After tensorplay/distributed/fsdp/api.py (``StateDictType``, the ``*StateDictConfig`` / ``*OptimStateDictConfig``
dataclasses, ``StateDictSettings``), fully_sharded_data_parallel.py (``set_state_dict_type`` :595,
``state_dict_type`` :705, ``optim_state_dict`` :1790, ``optim_state_dict_to_load`` :1889) and
sharded_grad_scaler.py. The work is done by ``distributed.checkpoint.state_dict``: a FULL state dict gathers
every sharded tensor (and every optimizer state tensor shaped like its parameter) over the shard group, a
SHARDED / LOCAL one keeps this rank's rows with their global offsets; loading accepts either and keeps the
rows of this rank.
"""
from __future__ import annotations

import contextlib
from dataclasses import dataclass, field
from enum import Enum, auto
from typing import Any, Dict, Optional

import torch
import torch.distributed as dist
from torch import nn


class StateDictType(Enum):
    FULL_STATE_DICT = auto()
    LOCAL_STATE_DICT = auto()
    SHARDED_STATE_DICT = auto()


@dataclass
class StateDictConfig:
    offload_to_cpu: bool = False


@dataclass
class FullStateDictConfig(StateDictConfig):
    rank0_only: bool = False


@dataclass
class LocalStateDictConfig(StateDictConfig):
    pass


@dataclass
class ShardedStateDictConfig(StateDictConfig):
    _use_dtensor: bool = False


@dataclass
class OptimStateDictConfig:
    offload_to_cpu: bool = True


@dataclass
class FullOptimStateDictConfig(OptimStateDictConfig):
    rank0_only: bool = False


@dataclass
class LocalOptimStateDictConfig(OptimStateDictConfig):
    offload_to_cpu: bool = False


@dataclass
class ShardedOptimStateDictConfig(OptimStateDictConfig):
    _use_dtensor: bool = False


@dataclass
class StateDictSettings:
    state_dict_type: StateDictType = StateDictType.FULL_STATE_DICT
    state_dict_config: StateDictConfig = field(default_factory=FullStateDictConfig)
    optim_state_dict_config: OptimStateDictConfig = field(default_factory=FullOptimStateDictConfig)


_DEFAULT_CFG = {StateDictType.FULL_STATE_DICT: (FullStateDictConfig, FullOptimStateDictConfig),
                StateDictType.LOCAL_STATE_DICT: (LocalStateDictConfig, LocalOptimStateDictConfig),
                StateDictType.SHARDED_STATE_DICT: (ShardedStateDictConfig, ShardedOptimStateDictConfig)}


def _wrappers(module: nn.Module):
    from .api import FullyShardedDataParallel
    return [m for m in module.modules() if isinstance(m, FullyShardedDataParallel)]


class StateDictMixin:
    """Methods of ``FullyShardedDataParallel`` that deal with model and optimizer state dicts."""

    _sd_settings: StateDictSettings

    # ---------------------------------------------------------------- settings
    @staticmethod
    def set_state_dict_type(module: nn.Module, state_dict_type: StateDictType,
                            state_dict_config: Optional[StateDictConfig] = None,
                            optim_state_dict_config: Optional[OptimStateDictConfig] = None) -> StateDictSettings:
        """Set the kind of state dict that ``state_dict()`` / ``load_state_dict()`` of every wrapper below
        ``module`` produce and accept; returns the previous settings."""
        sd_cls, osd_cls = _DEFAULT_CFG[state_dict_type]
        sd_cfg = state_dict_config if state_dict_config is not None else sd_cls()
        osd_cfg = optim_state_dict_config if optim_state_dict_config is not None else osd_cls()
        if not isinstance(sd_cfg, sd_cls) or not isinstance(osd_cfg, osd_cls):
            raise RuntimeError(f"{state_dict_type} expects {sd_cls.__name__} and {osd_cls.__name__}")
        ws = _wrappers(module)
        if not ws:
            raise ValueError("set_state_dict_type: no FullyShardedDataParallel wrapper below this module")
        prev = ws[0]._sd_settings
        for w in ws:
            w._sd_settings = StateDictSettings(state_dict_type, sd_cfg, osd_cfg)
        return prev

    @staticmethod
    def get_state_dict_type(module: nn.Module) -> StateDictSettings:
        ws = _wrappers(module)
        if not ws:
            raise ValueError("get_state_dict_type: no FullyShardedDataParallel wrapper below this module")
        first = ws[0]._sd_settings
        if any(w._sd_settings.state_dict_type != first.state_dict_type for w in ws):
            raise RuntimeError("the wrappers below this module disagree on their state-dict type")
        return first

    @staticmethod
    @contextlib.contextmanager
    def state_dict_type(module: nn.Module, state_dict_type: StateDictType,
                        state_dict_config: Optional[StateDictConfig] = None,
                        optim_state_dict_config: Optional[OptimStateDictConfig] = None):
        prev = StateDictMixin.set_state_dict_type(module, state_dict_type, state_dict_config, optim_state_dict_config)
        try:
            yield
        finally:
            StateDictMixin.set_state_dict_type(module, prev.state_dict_type, prev.state_dict_config,
                                               prev.optim_state_dict_config)

    # ---------------------------------------------------------------- model state
    def _rank(self) -> int:
        return dist.get_rank() if dist.is_initialized() else 0

    def state_dict(self, *args, destination=None, prefix: str = "", keep_vars: bool = False) -> Dict[str, Any]:
        from ..checkpoint.state_dict import StateDictOptions, get_model_state_dict
        s = self._sd_settings
        full = s.state_dict_type == StateDictType.FULL_STATE_DICT
        sd = get_model_state_dict(self, options=StateDictOptions(full_state_dict=full,
                                                                 cpu_offload=s.state_dict_config.offload_to_cpu))
        if full and getattr(s.state_dict_config, "rank0_only", False) and self._rank() != 0:
            sd = {}   # every rank took part in the gathers; only rank 0 keeps the result
        out = destination if destination is not None else {}
        for k, v in sd.items():
            out[prefix + k] = v
        return out

    def load_state_dict(self, state_dict: Dict[str, Any], strict: bool = True, assign: bool = False):
        """Accepts full tensors (every rank keeps its rows) or this rank's shards, whatever the current type."""
        from ..checkpoint.state_dict import StateDictOptions, set_model_state_dict
        missing, unexpected = set_model_state_dict(self, state_dict, options=StateDictOptions(strict=strict))
        return torch.nn.modules.module._IncompatibleKeys(missing, unexpected)

    # ---------------------------------------------------------------- optimizer state
    @staticmethod
    def optim_state_dict(model: nn.Module, optim: torch.optim.Optimizer, optim_state_dict: Optional[Dict] = None,
                         group=None) -> Dict[str, Any]:
        """The optimizer's state keyed by parameter names, in the form that the model's state-dict type says:
        full tensors (gathered; on rank 0 only with ``rank0_only``) or this rank's shards."""
        from ..checkpoint.state_dict import StateDictOptions, get_optimizer_state_dict
        s = StateDictMixin.get_state_dict_type(model)
        full = s.state_dict_type == StateDictType.FULL_STATE_DICT
        osd = get_optimizer_state_dict(model, optim, options=StateDictOptions(
            full_state_dict=full, cpu_offload=s.optim_state_dict_config.offload_to_cpu))
        if full and getattr(s.optim_state_dict_config, "rank0_only", False) and dist.is_initialized() \
                and dist.get_rank() != 0:
            return {}
        return osd

    @staticmethod
    def optim_state_dict_to_load(model: nn.Module, optim: torch.optim.Optimizer, optim_state_dict: Dict[str, Any],
                                 is_named_optimizer: bool = False, load_directly: bool = False, group=None):
        """Turn a state dict made by :meth:`optim_state_dict` (full or sharded, keyed by names) into one that
        ``optim.load_state_dict`` takes on this rank: parameter ids as keys, tensors cut to this rank's rows."""
        from ..checkpoint.api import ShardedTensor
        from ..checkpoint.state_dict import _named_params
        if getattr(StateDictMixin.get_state_dict_type(model).optim_state_dict_config, "rank0_only", False) \
                and dist.is_initialized():
            box = [optim_state_dict if dist.get_rank() == 0 else None]
            dist.broadcast_object_list(box, src=0, group=group)
            optim_state_dict = box[0]
        by_name = dict(_named_params(model))
        ids, k = {}, 0
        for g in optim.param_groups:
            for p in g["params"]:
                ids[id(p)] = k
                k += 1
        name_of = {id(p): n for n, p in by_name.items()}
        state = {}
        for fqn, st in optim_state_dict.get("state", {}).items():
            p = by_name.get(fqn)
            if p is None or id(p) not in ids:
                continue
            entry = {}
            info, fst = getattr(p, "_fsdp_info", None), getattr(p, "_fsdp_state", None)
            for key, v in st.items():
                if isinstance(v, ShardedTensor):
                    v = v.local
                per_param = isinstance(v, torch.Tensor) and key != "step"   # "step" is the one scalar state
                if per_param and info is not None and tuple(v.shape) != tuple(p.shape):
                    # a full tensor (also of a 0-dim parameter, kept as one row): this rank's rows
                    v = v.reshape((info.n0,) + info.rest)[fst.rank * info.chunk: fst.rank * info.chunk + info.local_rows]
                    v = v.reshape(p.shape)
                if per_param:
                    entry[key] = v.detach().clone().to(p.device)
                else:   # scalars are cloned too: optimizers advance "step" in place
                    entry[key] = v.detach().clone() if isinstance(v, torch.Tensor) else v
            state[ids[id(p)]] = entry
        groups = []
        saved = {tuple(g["params"]): g for g in optim_state_dict.get("param_groups", [])}
        for g in optim.param_groups:
            names = tuple(name_of[id(p)] for p in g["params"] if id(p) in name_of)
            src = saved.get(names, g)
            groups.append({**{kk: vv for kk, vv in src.items() if kk != "params"}, "params": [ids[id(p)] for p in g["params"]]})
        out = {"state": state, "param_groups": groups}
        if load_directly:
            optim.load_state_dict(out)
        return out

    @staticmethod
    def full_optim_state_dict(model: nn.Module, optim: torch.optim.Optimizer, optim_input=None, rank0_only: bool = True,
                              group=None) -> Dict[str, Any]:
        with StateDictMixin.state_dict_type(model, StateDictType.FULL_STATE_DICT, FullStateDictConfig(),
                                            FullOptimStateDictConfig(rank0_only=rank0_only)):
            return StateDictMixin.optim_state_dict(model, optim, group=group)

    @staticmethod
    def sharded_optim_state_dict(model: nn.Module, optim: torch.optim.Optimizer, group=None) -> Dict[str, Any]:
        with StateDictMixin.state_dict_type(model, StateDictType.SHARDED_STATE_DICT):
            return StateDictMixin.optim_state_dict(model, optim, group=group)

    @staticmethod
    def shard_full_optim_state_dict(full_optim_state_dict: Dict[str, Any], model: nn.Module, optim_input=None,
                                    optim: Optional[torch.optim.Optimizer] = None) -> Dict[str, Any]:
        if optim is None:
            raise ValueError("shard_full_optim_state_dict needs optim=")
        with StateDictMixin.state_dict_type(model, StateDictType.FULL_STATE_DICT):
            return StateDictMixin.optim_state_dict_to_load(model, optim, full_optim_state_dict)


class ShardedGradScaler:
    """Gradient scaler for sharded parameters: every rank sees only its shards' gradients, so the non-finite
    flags are combined over the process group before the step is taken or skipped and before the scale moves
    (tensorplay/distributed/fsdp/sharded_grad_scaler.py). Built on this package's ``amp.GradScaler`` (device-side
    unscale + check, device-side scale update)."""

    def __new__(cls, device: str = "cuda", init_scale: float = 2.0 ** 16, backoff_factor: float = 0.5,
                growth_factor: float = 2.0, growth_interval: int = 2000, enabled: bool = True, process_group=None):
        from ...amp import GradScaler

        class _Sharded(GradScaler):
            def _unscale_grads_(self, optimizer, inv_scale, found_inf, allow_fp16):
                out = super()._unscale_grads_(optimizer, inv_scale, found_inf, allow_fp16)
                if not out:   # a rank without gradients still takes part in the exchange
                    out = {found_inf.device: found_inf}
                if dist.is_initialized() and dist.get_world_size(self._pg) > 1:
                    for fi in out.values():
                        t = fi if fi.is_cuda or dist.get_backend(self._pg) != "nccl" else fi.cuda()
                        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self._pg)
                        if t is not fi:
                            fi.copy_(t)
                return out

        obj = _Sharded(device, init_scale=init_scale, growth_factor=growth_factor, backoff_factor=backoff_factor,
                       growth_interval=growth_interval, enabled=enabled)
        obj._pg = process_group
        return obj
