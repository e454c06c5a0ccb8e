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


_signal_pad_size = 16384 * 4


def set_backend(name: str) -> None:
    """Select the allocator of arenas created afterwards: ``"vmm"`` / ``"cuda"`` (virtual-memory arena with
    an NVSwitch multicast mapping where the device supports it; the default) or ``"ipc"`` (``cudaMalloc`` +
    CUDA IPC, peer loads / stores only). NVSHMEM is not built."""
    import os
    name = name.lower()
    if name not in ("vmm", "cuda", "ipc"):
        raise ValueError(f"symmetric-memory backend {name!r} is not available ('vmm' or 'ipc')")
    os.environ["TPB_SYMM_ALLOC"] = "ipc" if name == "ipc" else "vmm"


def get_backend(device=None) -> str:
    a = SymmArena._instance
    if a is not None:
        return a.allocator
    import os
    return os.environ.get("TPB_SYMM_ALLOC", "vmm")


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


class AllToAll:
    """All-to-all(v) over peer memory: every rank copies what it sends into an arena buffer, publishes a
    table of {offset, bytes} per destination, and one kernel per rank pulls its segments from all
    sources (``csrc/kernels/symm_comm.cu`` ``all_to_all_pull_kernel``). The receiver needs no host-side
    knowledge of the counts: they are read from the sources' tables on the device and returned as a
    device tensor. The reference issues grouped NCCL send / recv here
    (p10/src/backend/cuda/NCCLContext.cpp:369-458).

    ``capacity_bytes`` bounds what a rank may send and receive per call. Construction is collective."""

    def __init__(self, capacity_bytes: int, group=None, ctas_per_peer: int = 8, wait_s: float = 30.0):
        a = _arena(group)
        self.arena, self.group = a, group
        self.capacity = (int(capacity_bytes) + 15) // 16 * 16
        self.send = a.alloc(self.capacity, torch.uint8)
        self.meta = a.alloc(2 * a.world, torch.int64)
        self.meta_host = torch.empty(2 * a.world, dtype=torch.int64).pin_memory()
        self.ready_slot = a.slots(a.world)
        self.done_slot = a.slots(a.world)
        self.counter = torch.zeros(1, dtype=torch.int32, device=a.device)
        self.recv_bytes = torch.zeros(a.world, dtype=torch.int64, device=a.device)
        self.epoch = 0
        self.ctas, self.wait_s = ctas_per_peer, wait_s

    def __call__(self, out: torch.Tensor, inp: torch.Tensor, input_split_sizes=None) -> torch.Tensor:
        """``inp`` is split along dimension 0 into ``world`` parts (``input_split_sizes`` rows each, equal
        parts by default); part ``d`` goes to rank ``d``. The parts received are packed into ``out`` in
        source order. Returns the device tensor of bytes received from each source."""
        from .. import _native
        from ..ops._common import status_word, stream_ptr
        a = self.arena
        inp = inp.contiguous()
        row_bytes = inp[0].numel() * inp.element_size() if inp.dim() > 0 and inp.shape[0] else inp.element_size()
        rows = inp.shape[0]
        splits = list(input_split_sizes) if input_split_sizes is not None else [rows // a.world] * a.world
        if sum(splits) != rows or len(splits) != a.world:
            raise ValueError("all_to_all: input_split_sizes must have one entry per rank and sum to the rows of the input")
        if row_bytes % 16:
            raise ValueError("all_to_all: a row must be a multiple of 16 bytes")
        nbytes = rows * row_bytes
        if nbytes > self.capacity:
            raise ValueError(f"all_to_all: {nbytes} bytes to send exceed the capacity of {self.capacity}")
        if not out.is_contiguous():
            raise ValueError("all_to_all: out must be contiguous")
        self.epoch += 1
        off = 0
        for d, n in enumerate(splits):
            self.meta_host[2 * d] = off
            self.meta_host[2 * d + 1] = n * row_bytes
            off += n * row_bytes
        st = status_word(a.device)
        if self.epoch > 1:
            # the previous call's readers must be done with the send buffer and the table
            _native.check(a.raw.tpb_symm_wait_slots(a.pad_off, self.done_slot, self.epoch - 1, self.wait_s,
                                                    st.data_ptr(), stream_ptr()), "tpb_symm_wait_slots")
        self.meta.copy_(self.meta_host, non_blocking=True)
        self.send[:nbytes].copy_(inp.view(-1).view(torch.uint8))
        _native.check(a.raw.tpb_symm_all_to_all(
            a.offset_of(self.send), a.offset_of(self.meta), out.data_ptr(), out.numel() * out.element_size(),
            self.recv_bytes.data_ptr(), a.pad_off, self.ready_slot, self.done_slot, self.epoch,
            self.counter.data_ptr(), self.ctas, self.wait_s, st.data_ptr(), stream_ptr()), "tpb_symm_all_to_all")
        return self.recv_bytes


_a2a: Optional[AllToAll] = None


def all_to_all_single(out: torch.Tensor, inp: torch.Tensor, output_split_sizes=None, input_split_sizes=None,
                      group=None) -> torch.Tensor:
    """``torch.distributed.all_to_all_single`` over peer memory for CUDA tensors (``output_split_sizes`` is
    not needed: the counts come from the senders' tables); NCCL / gloo otherwise."""
    global _a2a
    if not inp.is_cuda or dist.get_world_size(group) == 1:
        dist.all_to_all_single(out, inp.contiguous(), output_split_sizes, input_split_sizes, group=group)
        return out
    need = inp.numel() * inp.element_size()
    if _a2a is None:
        # first call (collective): room for four times the largest message of this call, 64 MiB at least;
        # larger exchanges construct AllToAll(capacity_bytes) themselves
        cap = torch.tensor([need], dtype=torch.int64, device=inp.device)
        dist.all_reduce(cap, op=dist.ReduceOp.MAX, group=group)
        _a2a = AllToAll(max(4 * int(cap), 64 << 20), group=group)
    _a2a(out, inp, input_split_sizes)
    return out


def all_to_all_nd(inp: torch.Tensor, group=None) -> torch.Tensor:
    """All-to-all of equal blocks along dimension 0 for tensors of any rank."""
    out = torch.empty_like(inp)
    if inp.is_cuda and inp[0].numel() * inp.element_size() % 16 == 0:
        return all_to_all_single(out, inp.contiguous(), group=group)
    dist.all_to_all_single(out, inp.contiguous(), group=group)
    return out
