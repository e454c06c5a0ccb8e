"""State dicts of wrapped models and their optimizers, by fully-qualified parameter name.

``get_model_state_dict`` / ``get_optimizer_state_dict`` / ``get_state_dict`` and the matching
``set_*`` look through ``DistributedDataParallel`` and ``FullyShardedDataParallel`` wrappers (their
``module.`` prefixes never appear in keys) and understand ``fully_shard`` units: a sharded parameter
is returned either as this rank's ``ShardedTensor`` window (default; what :func:`save` writes
without gathering) or, with ``StateDictOptions(full_state_dict=True)``, as the gathered full tensor
(optionally on the CPU, optionally on rank 0 only). Optimizer state is keyed by parameter name, so
a checkpoint loads into a differently ordered or differently sharded optimizer
(tensorplay/distributed/checkpoint/state_dict.py: ``StateDictOptions`` and the six functions).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Iterable, List, Optional, Tuple

import torch
import torch.distributed as dist
from torch import nn

from .api import ShardedTensor


@dataclass
class StateDictOptions:
    full_state_dict: bool = False
    cpu_offload: bool = False
    ignore_frozen_params: bool = False
    keep_submodule_prefixes: bool = True
    strict: bool = True
    broadcast_from_rank0: bool = False
    flatten_optimizer_state_dict: bool = False


def _unwrap(model: nn.Module) -> nn.Module:
    from ..ddp import DistributedDataParallel
    from ..fsdp.api import FullyShardedDataParallel
    while isinstance(model, (DistributedDataParallel, FullyShardedDataParallel, nn.parallel.DistributedDataParallel)):
        model = model.module
    return model


def _named_params(model: nn.Module) -> List[Tuple[str, torch.Tensor]]:
    return list(_unwrap(model).named_parameters(remove_duplicate=False))


def _gather_full(p: torch.Tensor) -> torch.Tensor:
    info = p._fsdp_info
    st = p._fsdp_state
    pad = torch.zeros((info.chunk,) + info.rest, dtype=p.dtype, device=st.device)
    pad[: info.local_rows].copy_(p.detach().to(st.device))
    if st.world > 1:
        out = torch.empty((st.world * info.chunk,) + info.rest, dtype=p.dtype, device=st.device)
        dist.all_gather_into_tensor(out, pad, group=st.group)
    else:
        out = pad
    return out[: info.n0].reshape(info.full_shape)


def _export(t: torch.Tensor, opts: StateDictOptions, like: Optional[torch.Tensor] = None):
    """A parameter or a same-shaped state tensor in checkpoint form."""
    ref = like if like is not None else t
    info = getattr(ref, "_fsdp_info", None)
    if info is None:
        out = t.detach()
        return out.cpu() if opts.cpu_offload else out
    if opts.full_state_dict:
        if like is not None and t.shape == ref.shape:
            # state shaped like the sharded parameter: gather it the same way
            carrier = t.detach().clone()
            carrier._fsdp_info, carrier._fsdp_state = ref._fsdp_info, ref._fsdp_state
            full = _gather_full(carrier)
        else:
            full = _gather_full(ref) if like is None else t.detach()
        return full.cpu() if opts.cpu_offload else full
    if like is not None and t.shape != ref.shape:
        return t.detach()   # scalar state such as the step count
    st = ref._fsdp_state
    shape = info.full_shape if info.full_shape else (1,)
    offs = (st.rank * info.chunk,) + (0,) * (len(shape) - 1)
    return ShardedTensor(t.detach(), tuple(shape), offs)


def get_model_state_dict(model: nn.Module, *, submodules=None, options: Optional[StateDictOptions] = None) -> Dict[str, Any]:
    opts = options or StateDictOptions()
    root = _unwrap(model)
    keep = None
    if submodules:
        keep = tuple(n + "." for n, m in root.named_modules() if m in set(submodules))
    out: Dict[str, Any] = {}
    for name, p in root.named_parameters(remove_duplicate=False):
        if opts.ignore_frozen_params and not p.requires_grad:
            continue
        if keep is not None and not name.startswith(keep):
            continue
        out[name] = _export(p, opts)
    for name, b in root.named_buffers(remove_duplicate=False):
        if keep is not None and not name.startswith(keep):
            continue
        if name.rsplit(".", 1)[-1] in getattr(root.get_submodule(name.rsplit(".", 1)[0]) if "." in name else root,
                                                "_non_persistent_buffers_set", ()):
            continue
        out[name] = b.detach().cpu() if opts.cpu_offload else b.detach()
    return out


def _import(dst: torch.Tensor, src, opts: StateDictOptions) -> None:
    info = getattr(dst, "_fsdp_info", None)
    if isinstance(src, ShardedTensor):
        src = src.local
    if info is None or tuple(src.shape) == tuple(dst.shape):
        dst.data.copy_(src.to(dst.device))
        return
    st = dst._fsdp_state
    full = src.reshape((info.n0,) + info.rest)
    rows = full[st.rank * info.chunk: st.rank * info.chunk + info.local_rows]
    dst.data.copy_(rows.to(dst.device))


def set_model_state_dict(model: nn.Module, model_state_dict: Dict[str, Any], *, options: Optional[StateDictOptions] = None):
    opts = options or StateDictOptions()
    root = _unwrap(model)
    targets = dict(root.named_parameters(remove_duplicate=False))
    targets.update(dict(root.named_buffers(remove_duplicate=False)))
    missing = [k for k in targets if k not in model_state_dict]
    unexpected = [k for k in model_state_dict if k not in targets]
    if opts.strict and (unexpected or [k for k in missing if k in dict(root.named_parameters())]):
        raise RuntimeError(f"set_model_state_dict: missing {missing[:5]}, unexpected {unexpected[:5]}")
    with torch.no_grad():
        for k, v in model_state_dict.items():
            if k in targets:
                _import(targets[k], v, opts)
    return missing, unexpected


def get_optimizer_state_dict(model: nn.Module, optimizers, *, options: Optional[StateDictOptions] = None) -> Dict[str, Any]:
    """``{"state": {fqn: {...}}, "param_groups": [{..., "params": [fqn, ...]}]}`` merged over the
    given optimizers."""
    opts = options or StateDictOptions()
    optimizers = [optimizers] if isinstance(optimizers, torch.optim.Optimizer) else list(optimizers)
    name_of = {id(p): n for n, p in _named_params(model)}
    out = {"state": {}, "param_groups": []}
    for opt in optimizers:
        for g in opt.param_groups:
            names = [name_of[id(p)] for p in g["params"] if id(p) in name_of]
            out["param_groups"].append({**{k: v for k, v in g.items() if k != "params"}, "params": names})
            for p in g["params"]:
                if id(p) not in name_of or p not in opt.state:
                    continue
                out["state"][name_of[id(p)]] = {k: (_export(v, opts, like=p) if isinstance(v, torch.Tensor) else v)
                                                for k, v in opt.state[p].items()}
    if opts.flatten_optimizer_state_dict:
        flat = {}
        for fqn, st in out["state"].items():
            for k, v in st.items():
                flat[f"state.{fqn}.{k}"] = v
        for gi, g in enumerate(out["param_groups"]):
            for k, v in g.items():
                flat[f"param_groups.{gi}.{k}"] = v
        return flat
    return out


def set_optimizer_state_dict(model: nn.Module, optimizers, optim_state_dict: Dict[str, Any], *,
                             options: Optional[StateDictOptions] = None) -> None:
    opts = options or StateDictOptions()
    optimizers = [optimizers] if isinstance(optimizers, torch.optim.Optimizer) else list(optimizers)
    by_name = dict(_named_params(model))
    groups = {tuple(g["params"]): g for g in optim_state_dict.get("param_groups", [])}
    name_of = {id(p): n for n, p in by_name.items()}
    for opt in optimizers:
        for g in opt.param_groups:
            names = tuple(name_of[id(p)] for p in g["params"] if id(p) in name_of)
            saved = groups.get(names)
            if saved is not None:
                for k, v in saved.items():
                    if k != "params":
                        g[k] = v
            for p in g["params"]:
                fqn = name_of.get(id(p))
                st = optim_state_dict["state"].get(fqn) if fqn is not None else None
                if st is None:
                    continue
                dst = opt.state[p]
                for k, v in st.items():
                    if isinstance(v, (torch.Tensor, ShardedTensor)):
                        src = v.local if isinstance(v, ShardedTensor) else v
                        if k in dst and isinstance(dst[k], torch.Tensor) and dst[k].shape == src.shape:
                            dst[k].copy_(src.to(dst[k].device))
                        elif tuple(src.shape) == tuple(p.shape) or k == "step" or getattr(p, "_fsdp_info", None) is None:
                            dst[k] = src.detach().clone().to(p.device if src.dim() else src.device)
                        else:   # full tensor for a sharded parameter: keep this rank's rows
                            info, fst = p._fsdp_info, p._fsdp_state
                            rows = src.reshape((info.n0,) + info.rest)[fst.rank * info.chunk: fst.rank * info.chunk + info.local_rows]
                            dst[k] = rows.reshape(p.shape).detach().clone().to(p.device)
                    else:
                        dst[k] = v


def get_state_dict(model: nn.Module, optimizers, *, submodules=None, options: Optional[StateDictOptions] = None):
    return (get_model_state_dict(model, submodules=submodules, options=options),
            get_optimizer_state_dict(model, optimizers, options=options))


def set_state_dict(model: nn.Module, optimizers, *, model_state_dict: Dict[str, Any], optim_state_dict: Dict[str, Any],
                   options: Optional[StateDictOptions] = None):
    res = set_model_state_dict(model, model_state_dict, options=options) if model_state_dict else ([], [])
    if optim_state_dict:
        set_optimizer_state_dict(model, optimizers, optim_state_dict, options=options)
    return res
