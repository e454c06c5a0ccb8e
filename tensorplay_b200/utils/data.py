"""Data loading: Dataset / DataLoader / samplers (torch.utils.data) with ``DistributedSampler``
(tensorplay/utils/data: ``DistributedSampler`` :1155) and a pinned-memory prefetcher that overlaps
the host-to-device copy of the next batch with the current step."""
from __future__ import annotations

import torch
from torch.utils.data import *  # noqa: F401,F403
from torch.utils.data import DataLoader, Dataset, DistributedSampler, Sampler, TensorDataset  # noqa: F401


class CudaPrefetcher:
    """Wraps an iterable of (nested) CPU tensors; copies batch i+1 to the device on a side stream
    while batch i is consumed."""

    def __init__(self, loader, device):
        self.loader, self.device = loader, torch.device(device)
        self.stream = torch.cuda.Stream(device=self.device) if self.device.type == "cuda" else None

    def _to(self, x):
        if isinstance(x, torch.Tensor):
            if self.stream is not None and not x.is_pinned():
                x = x.pin_memory()
            return x.to(self.device, non_blocking=True)
        if isinstance(x, (list, tuple)):
            return type(x)(self._to(v) for v in x)
        if isinstance(x, dict):
            return {k: self._to(v) for k, v in x.items()}
        return x

    def __iter__(self):
        it = iter(self.loader)
        nxt = None
        if self.stream is None:
            for b in it:
                yield self._to(b)
            return
        try:
            with torch.cuda.stream(self.stream):
                nxt = self._to(next(it))
        except StopIteration:
            return
        while nxt is not None:
            torch.cuda.current_stream().wait_stream(self.stream)
            cur = nxt
            try:
                with torch.cuda.stream(self.stream):
                    nxt = self._to(next(it))
            except StopIteration:
                nxt = None
            yield cur
