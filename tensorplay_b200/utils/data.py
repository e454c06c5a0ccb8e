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


class TokenFileLoader:
    """Batches of ``(tokens, targets)`` (int64 ``[batch, seq_len]``, targets shifted by one) from a
    flat binary file of token ids (uint16 or int32), produced by native worker threads a few batches
    ahead (``csrc/runtime/token_loader.cpp``). The sample order of an epoch is a seeded permutation
    shared by all ranks; rank ``r`` of ``world`` takes every ``world``-th sample, so ranks read disjoint
    data and yield the same number of batches. The yielded tensors are views of (pinned, when CUDA is
    available) host buffers that are reused ``depth`` batches later: copy them out (e.g. through
    :class:`CudaPrefetcher`) before asking for more than ``depth - 1`` further batches.
    """

    def __init__(self, path: str, seq_len: int, batch_size: int, *, dtype=torch.uint16, rank: int = 0, world: int = 1,
                 seed: int = 0, shuffle: bool = True, num_workers: int = 2, depth: int = 4, pin_memory=None):
        import ctypes as C

        from .. import _native
        self._C = C
        rt = _native.runtime()
        self._rt = rt
        rt.tpb_loader_open.restype = C.c_void_p
        rt.tpb_loader_open.argtypes = [C.c_char_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_ulonglong,
                                       C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.POINTER(C.c_int)]
        rt.tpb_loader_next.restype = C.c_int
        rt.tpb_loader_next.argtypes = [C.c_void_p, C.POINTER(C.c_longlong)]
        rt.tpb_loader_release.restype = None
        rt.tpb_loader_release.argtypes = [C.c_void_p, C.c_int]
        rt.tpb_loader_close.restype = None
        rt.tpb_loader_close.argtypes = [C.c_void_p]
        for fn in (rt.tpb_loader_batches_per_epoch, rt.tpb_loader_num_samples):
            fn.restype = C.c_longlong
            fn.argtypes = [C.c_void_p]
        elem = {torch.uint16: 2, torch.int16: 2, torch.int32: 4}[dtype]
        pin = torch.cuda.is_available() if pin_memory is None else pin_memory
        mk = lambda: torch.empty(batch_size, seq_len, dtype=torch.int64, pin_memory=pin)  # noqa: E731
        self._tok = [mk() for _ in range(depth)]
        self._tgt = [mk() for _ in range(depth)]
        tp = (C.c_void_p * depth)(*[t.data_ptr() for t in self._tok])
        gp = (C.c_void_p * depth)(*[t.data_ptr() for t in self._tgt])
        err = C.c_int(0)
        self._h = rt.tpb_loader_open(str(path).encode(), elem, seq_len, batch_size, rank, world, seed, int(shuffle),
                                     num_workers, depth, C.cast(tp, C.c_void_p), C.cast(gp, C.c_void_p), C.byref(err))
        if not self._h:
            raise RuntimeError(f"tpb_loader_open({path!r}) failed with code {err.value}")
        self.depth = depth
        self.batches_per_epoch = int(rt.tpb_loader_batches_per_epoch(self._h))
        self.num_samples = int(rt.tpb_loader_num_samples(self._h))
        self._held = []

    def __len__(self) -> int:
        return self.batches_per_epoch

    def next_batch(self):
        """``(tokens, targets, global_batch_number)``; the slot handed out ``depth - 1`` calls ago is
        returned to the workers."""
        while len(self._held) >= self.depth - 1:
            self._rt.tpb_loader_release(self._h, self._held.pop(0))
        n = self._C.c_longlong(0)
        slot = self._rt.tpb_loader_next(self._h, self._C.byref(n))
        if slot < 0:
            raise RuntimeError("the loader was closed")
        self._held.append(slot)
        return self._tok[slot], self._tgt[slot], int(n.value)

    def __iter__(self):
        """One epoch (continues where the previous iteration stopped)."""
        for _ in range(self.batches_per_epoch):
            tok, tgt, _ = self.next_batch()
            yield tok, tgt

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._rt.tpb_loader_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
