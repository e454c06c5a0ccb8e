"""Single-process data parallelism over several devices (tensorplay/nn/parallel/data_parallel.py: ``DataParallel``,
``data_parallel``; scatter_gather.py: ``scatter``, ``gather``).

The batch is cut along ``dim`` into one piece per device; each piece runs through the SAME module object with its
parameters and buffers replaced, for that call only, by copies on the piece's device (``torch.func.functional_call``),
and the outputs are concatenated on ``output_device``. The device copies are differentiable, so the gradients of all
pieces flow back into the one set of parameters and add up there: no replicas to keep in sync. The host walks the
devices one after the other; the work it queues runs concurrently, since every device has its own stream.
One process per GPU (``DistributedDataParallel``) is this framework's main path; this class exists for scripts that
drive several GPUs from one process.
"""
from __future__ import annotations

from typing import Any, List, Optional, Sequence

import torch
from torch import Tensor, nn


def _dev(d) -> torch.device:
    return torch.device("cuda", d) if isinstance(d, int) else torch.device(d)


def scatter(obj: Any, devices: Sequence, dim: int = 0) -> List[Any]:
    """Cuts every tensor inside ``obj`` (tensors, tuples, lists, dicts) into ``len(devices)`` pieces along ``dim`` and
    moves piece ``i`` to ``devices[i]``; other objects are repeated. A batch smaller than the number of devices gives
    fewer pieces."""
    devices = [_dev(d) for d in devices]
    if isinstance(obj, Tensor):
        return [c.to(d, non_blocking=True) for c, d in zip(obj.chunk(len(devices), dim), devices)]
    if isinstance(obj, (tuple, list)) and obj:
        parts = [scatter(o, devices, dim) for o in obj]
        n = min(len(p) for p in parts)
        return [type(obj)(p[i] for p in parts) for i in range(n)]
    if isinstance(obj, dict) and obj:
        parts = {k: scatter(v, devices, dim) for k, v in obj.items()}
        n = min(len(p) for p in parts.values())
        return [{k: p[i] for k, p in parts.items()} for i in range(n)]
    return [obj for _ in devices]


def gather(outputs: Sequence[Any], target_device, dim: int = 0) -> Any:
    """Inverse of :func:`scatter` for a module's outputs: tensors are concatenated along ``dim`` on ``target_device``
    (0-dim tensors are stacked), containers are gathered element-wise."""
    target = _dev(target_device)
    first = outputs[0]
    if isinstance(first, Tensor):
        moved = [o.to(target) for o in outputs]
        return torch.stack(moved) if first.dim() == 0 else torch.cat(moved, dim)
    if isinstance(first, (tuple, list)):
        return type(first)(gather([o[i] for o in outputs], target, dim) for i in range(len(first)))
    if isinstance(first, dict):
        return {k: gather([o[k] for o in outputs], target, dim) for k in first}
    return first


def data_parallel(module: nn.Module, inputs, device_ids: Optional[Sequence] = None, output_device=None, dim: int = 0,
                  module_kwargs: Optional[dict] = None):
    """Functional form: one forward pass of ``module`` over ``inputs`` split across ``device_ids``."""
    if not isinstance(inputs, tuple):
        inputs = (inputs,) if inputs is not None else ()
    if device_ids is None:
        device_ids = list(range(torch.cuda.device_count()))
    if not device_ids:
        return module(*inputs, **(module_kwargs or {}))
    devices = [_dev(d) for d in device_ids]
    output_device = devices[0] if output_device is None else _dev(output_device)
    ins = scatter(inputs, devices, dim)
    kws = scatter(module_kwargs or {}, devices, dim) if module_kwargs else [{} for _ in ins]
    state = dict(module.named_parameters(remove_duplicate=False))
    state.update(dict(module.named_buffers(remove_duplicate=False)))
    outs = []
    for piece, kw, dev in zip(ins, kws, devices):
        local = {k: (v if v.device == dev else v.to(dev, non_blocking=True)) for k, v in state.items()}
        outs.append(torch.func.functional_call(module, local, piece, kw))
    return gather(outs, output_device, dim)


class DataParallel(nn.Module):
    def __init__(self, module: nn.Module, device_ids: Optional[Sequence] = None, output_device=None, dim: int = 0):
        super().__init__()
        if device_ids is None:
            device_ids = list(range(torch.cuda.device_count()))
        self.module, self.dim = module, dim
        self.device_ids = list(device_ids)
        self.output_device = (self.device_ids[0] if self.device_ids else None) if output_device is None else output_device
        if self.device_ids:
            src = _dev(self.device_ids[0])
            for name, t in list(module.named_parameters()) + list(module.named_buffers()):
                if t.device != src:
                    raise RuntimeError(f"module must have its parameters and buffers on device {src} (device_ids[0]) "
                                       f"but found {name} on {t.device}")

    def forward(self, *inputs, **kwargs):
        if not self.device_ids:
            return self.module(*inputs, **kwargs)
        return data_parallel(self.module, inputs, self.device_ids, self.output_device, self.dim, kwargs)
