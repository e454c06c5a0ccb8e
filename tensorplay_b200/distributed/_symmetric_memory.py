"""Symmetric memory: peer-mapped buffers, signal pads and fused ops - implemented for real on the
NVLink arena of ``tensorplay_b200.parallel.symm`` (in the reference these names are facades over
NCCL: tensorplay/distributed/_symmetric_memory/__init__.py:118-130, 228-266, 456-471).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..parallel.symm import SymmArena
from ..parallel.tp import TPContext

_default_bytes = 1 << 30


def set_arena_bytes(nbytes: int) -> None:
    global _default_bytes
    _default_bytes = int(nbytes)


def _arena(group=None) -> SymmArena:
    return SymmArena._instance or SymmArena(_default_bytes, group=group)


class SymmetricBuffer:
    """Handle returned by ``rendezvous``: the local tensor plus access to every peer's copy."""

    def __init__(self, tensor: torch.Tensor, arena: SymmArena):
        self.tensor, self.arena = tensor, arena
        self.offset = arena.offset_of(tensor)
        self.world_size, self.rank = arena.world, arena.rank

    def get_buffer(self, peer: int, shape=None, dtype=None) -> torch.Tensor:
        """A tensor aliasing ``peer``'s copy of the buffer (peer memory, readable and writable
        from kernels and copies on this device)."""
        from ..parallel.symm import _DevMem
        nbytes = self.tensor.numel() * self.tensor.element_size()
        ptr = self.arena.raw.tpb_symm_ptr(peer, self.offset)
        t = torch.as_tensor(_DevMem(ptr, nbytes), device=self.tensor.device).view(dtype or self.tensor.dtype)
        return t.view(shape or self.tensor.shape)

    def barrier(self) -> None:
        a = self.arena
        if not hasattr(self, "_slot"):
            self._slot, self._epoch = a.slots(a.world), 0
        self._epoch += 1
        from .. import _native
        from ..ops._common import status_word, stream_ptr
        _native.check(a.raw.tpb_symm_barrier(a.pad_off, self._slot, self._epoch, 30.0,
                                             status_word(self.tensor.device).data_ptr(), stream_ptr()),
                      "tpb_symm_barrier")


def empty(*size, dtype=torch.bfloat16, device=None, group=None) -> torch.Tensor:
    """Allocate a tensor in the symmetric arena (collective: same call on every rank)."""
    shape = size[0] if len(size) == 1 and isinstance(size[0], (tuple, list)) else size
    n = 1
    for s in shape:
        n *= s
    return _arena(group).alloc(n, dtype).view(*shape)


def rendezvous(tensor: torch.Tensor, group=None) -> SymmetricBuffer:
    return SymmetricBuffer(tensor, _arena(group))


def is_symm_mem_tensor(t: torch.Tensor) -> bool:
    a = SymmArena._instance
    if a is None or not t.is_cuda:
        return False
    try:
        a.offset_of(t)
        return True
    except ValueError:
        return False


def is_nvshmem_available() -> bool:
    return False


_tp: Optional[TPContext] = None


def _ctx(group=None) -> TPContext:
    global _tp
    if _tp is None:
        _tp = TPContext(group=group, arena_bytes=_default_bytes)
    return _tp


def fused_all_gather_matmul(a_shard: torch.Tensor, b: torch.Tensor, group=None) -> torch.Tensor:
    """``all_gather(a_shard, dim=0) @ b.T`` in one kernel (``b`` is ``[N, K]``)."""
    return _ctx(group).all_gather_linear(a_shard, b)


def fused_matmul_reduce_scatter(a: torch.Tensor, b: torch.Tensor, group=None) -> torch.Tensor:
    """``reduce_scatter(a @ b.T, dim=0)`` in one kernel."""
    return _ctx(group).linear_reduce_scatter(a, b)


_backend = "ipc"            # CUDA IPC arena with P2P loads / stores (the only backend built here)
_signal_pad_size = 16384 * 4


def set_backend(name: str) -> None:
    """Select the symmetric-memory backend. Only ``"ipc"`` (CUDA IPC + peer loads / stores) exists here;
    NVSHMEM and multicast (NVLS) backends are not built."""
    if name.lower() not in ("ipc", "cuda"):
        raise ValueError(f"symmetric-memory backend {name!r} is not available (only 'ipc')")


def get_backend(device=None) -> str:
    return _backend


def set_signal_pad_size(nbytes: int) -> None:
    """Bytes of signal slots per arena; takes effect for arenas created afterwards."""
    global _signal_pad_size
    _signal_pad_size = int(nbytes)


def get_signal_pad_size() -> int:
    return _signal_pad_size


def get(tensor: torch.Tensor, group=None) -> "SymmetricBuffer":
    """Handle of an arena tensor (alias of :func:`rendezvous`)."""
    return rendezvous(tensor, group)


def get_mem_pool(device=None):
    """The process-wide arena that backs symmetric allocations (a bump allocator, not a torch MemPool)."""
    return _arena()


def reduce_scatter_offset(inp: torch.Tensor, group=None, offsets=None) -> torch.Tensor:
    """Row reduce-scatter whose shard boundaries are ``offsets`` (ascending row ends per rank; equal
    shards by default). Uneven shards take the NCCL path through padding."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    rows = inp.shape[0]
    ends = list(offsets) if offsets is not None else [rows * (r + 1) // world for r in range(world)]
    starts = [0] + ends[:-1]
    width = max(e - s for s, e in zip(starts, ends))
    padded = inp.new_zeros(world * width, *inp.shape[1:])
    for r, (s, e) in enumerate(zip(starts, ends)):
        padded[r * width: r * width + (e - s)] = inp[s:e]
    out = inp.new_empty(width, *inp.shape[1:])
    if dist.get_backend(group) == "gloo":
        dist.all_reduce(padded, group=group)
        out.copy_(padded[rank * width: (rank + 1) * width])
    else:
        dist.reduce_scatter_tensor(out, padded, group=group)
    return out[: ends[rank] - starts[rank]]


def all_to_all_nd(inp: torch.Tensor, group=None) -> torch.Tensor:
    """All-to-all of equal blocks along dimension 0 for tensors of any rank."""
    out = torch.empty_like(inp)
    dist.all_to_all_single(out, inp.contiguous(), group=group)
    return out
