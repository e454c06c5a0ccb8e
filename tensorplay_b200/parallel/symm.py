"""Symmetric memory over NVLink: arena allocation, handle exchange and the fused collectives.

Every rank allocates one device arena, exports it with CUDA IPC and maps the arenas of its
peers; buffers are carved from the arena at identical offsets on every rank, so that a kernel can
address the same buffer on any peer. This is the real counterpart of the reference's facade
``tensorplay/distributed/_symmetric_memory`` (``get_buffer(peer)`` there returns the local tensor,
__init__.py:118-130; ``rendezvous`` only all-gathers metadata, :456-467).
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Dict, Optional

import torch
import torch.distributed as dist

from .. import _native
from ..ops._common import status_word, stream_ptr

_SIGS = {
    "tpb_symm_create": [C.c_int, C.c_int, C.c_size_t, C.c_void_p],
    "tpb_symm_open": [C.c_void_p],
    "tpb_symm_destroy": [],
    "tpb_symm_allgather": [C.c_size_t, C.c_size_t, C.c_void_p, C.c_size_t, C.c_int, C.c_uint32,
                           C.c_int, C.c_double, C.c_void_p, C.c_void_p],
    "tpb_symm_rs_adamw": [C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p,
                          C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_int, C.c_float,
                          C.c_float, C.c_float, C.c_float, C.c_float, C.c_int, C.c_float, C.c_void_p,
                          C.c_size_t, C.c_int, C.c_int, C.c_uint32, C.c_void_p, C.c_int, C.c_double,
                          C.c_void_p, C.c_void_p],
    "tpb_symm_allgather_ce": [C.c_size_t, C.c_size_t, C.c_void_p, C.c_size_t, C.c_int, C.c_uint32, C.c_double,
                              C.c_void_p, C.c_void_p],
    "tpb_symm_rs_adamw_ce": [C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                             C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_float, C.c_float, C.c_float,
                             C.c_float, C.c_float, C.c_int, C.c_float, C.c_void_p, C.c_size_t, C.c_int, C.c_int,
                             C.c_uint32, C.c_int, C.c_double, C.c_void_p, C.c_void_p],
    "tpb_symm_all_to_all": [C.c_size_t, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_int, C.c_int,
                            C.c_uint32, C.c_void_p, C.c_int, C.c_double, C.c_void_p, C.c_void_p],
    "tpb_symm_set_overlap": [C.c_int, C.c_int],
    "tpb_symm_wait_slots": [C.c_size_t, C.c_int, C.c_uint32, C.c_double, C.c_void_p, C.c_void_p],
    "tpb_symm_barrier": [C.c_size_t, C.c_int, C.c_uint32, C.c_double, C.c_void_p, C.c_void_p],
    "tpb_symm_peer_copy": [C.c_int, C.c_size_t, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p],
    "tpb_symm_vmm_supported": [C.c_int],
    "tpb_symm_vmm_create": [C.c_int, C.c_int, C.c_size_t, C.POINTER(C.c_int), C.POINTER(C.c_size_t)],
    "tpb_symm_vmm_map_peer": [C.c_int, C.c_int],
    "tpb_symm_mc_create": [C.POINTER(C.c_int)],
    "tpb_symm_mc_import": [C.c_int],
    "tpb_symm_mc_add_device": [],
    "tpb_symm_mc_bind": [],
    "tpb_symm_set_multicast": [C.c_int],
    "tpb_symm_has_multicast": [],
    "tpb_symm_allgather_mc": [C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_int, C.c_int, C.c_uint32,
                              C.c_void_p, C.c_int, C.c_double, C.c_void_p, C.c_void_p],
}
NO_OFFSET = C.c_size_t(-1).value


class _DevMem:
    """Exposes a raw device range through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 2, "strides": None}


def _send_fd_to_peers(fd: int, n_receivers: int, name: str):
    """Serve ``fd`` to ``n_receivers`` connections on the abstract Unix socket ``name`` (file
    descriptors cannot travel through a key-value store; SCM_RIGHTS over a local socket can)."""
    import socket
    import threading
    srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    srv.bind("\0" + name)
    srv.listen(max(n_receivers, 1))
    srv.settimeout(120)

    def serve():
        try:
            for _ in range(n_receivers):
                c, _ = srv.accept()
                with c:
                    socket.send_fds(c, [b"f"], [fd])
        finally:
            srv.close()

    t = threading.Thread(target=serve, daemon=True)
    t.start()
    return t


def _recv_fd(name: str) -> int:
    import socket
    with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as c:
        c.settimeout(120)
        c.connect("\0" + name)
        _, fds, _, _ = socket.recv_fds(c, 1, 1)
    if not fds:
        raise RuntimeError(f"no file descriptor received on {name!r}")
    return fds[0]


class SymmArena:
    """Process-wide symmetric arena (one per process; collective to create).

    Two allocators: ``"vmm"`` (default where the device supports it) creates the arena with the CUDA
    virtual-memory API, passes its file descriptor to the peers over Unix sockets and binds all
    arenas to an NVSwitch multicast object, which gives the kernels ``multimem`` loads (reduced in
    the switch) and stores (delivered to every rank); ``"ipc"`` uses ``cudaMalloc`` + CUDA IPC and
    has peer loads / stores only. ``TPB_SYMM_ALLOC`` / ``TPB_SYMM_MULTICAST=0`` select.
    """

    _instance: Optional["SymmArena"] = None
    # one block counter per communicating unit: two launches that count into the same word may
    # only run one after the other, so units never share one
    N_COUNTERS = 1024

    def counter_ptr(self, index: int) -> int:
        if not 0 <= index < self.N_COUNTERS:
            raise IndexError(f"block counter {index} out of range (have {self.N_COUNTERS})")
        return self.counter[index:].data_ptr()

    def __init__(self, nbytes: int, group=None, pad_slots: int = 16384):
        lib = _native.kernels()
        raw = lib._lib
        _native.register_sigs(raw, _SIGS)
        raw.tpb_symm_alloc.argtypes = [C.c_size_t]
        raw.tpb_symm_alloc.restype = C.c_size_t
        raw.tpb_symm_ptr.argtypes = [C.c_int, C.c_size_t]
        raw.tpb_symm_ptr.restype = C.c_void_p
        self.lib = lib
        self.raw = raw
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = torch.device("cuda", torch.cuda.current_device())
        raw.tpb_symm_mc_ptr.argtypes = [C.c_size_t]
        raw.tpb_symm_mc_ptr.restype = C.c_void_p
        want = os.environ.get("TPB_SYMM_ALLOC", "vmm")
        self.allocator = "ipc"
        self.multicast = False
        if want == "vmm" and self._all_ranks(bool(raw.tpb_symm_vmm_supported(0))):
            nbytes = self._create_vmm(nbytes)
            self.allocator = "vmm"
        else:
            handle = (C.c_char * 64)()
            _native.check(raw.tpb_symm_create(self.world, self.rank, nbytes, handle), "tpb_symm_create")
            if self.world > 1:
                gathered = [None] * self.world
                dist.all_gather_object(gathered, bytes(handle.raw), group=group)
                blob = b"".join(gathered)
                buf = (C.c_char * len(blob)).from_buffer_copy(blob)
                _native.check(raw.tpb_symm_open(buf), "tpb_symm_open")
        self.nbytes = nbytes
        self._offsets: Dict[int, int] = {}
        self.canaries = [] if os.environ.get("TPB_SYMM_CANARY", "0") == "1" else None
        if self.canaries is not None:
            import atexit
            atexit.register(self._check_at_exit)
        self.pad_slots = pad_slots
        self.pad_off = self._alloc_bytes(pad_slots * 4)
        self._next_slot = 0
        self.counter = torch.zeros(self.N_COUNTERS, dtype=torch.int32, device=self.device)
        if self.world > 1:
            dist.barrier(group=group)
        SymmArena._instance = self

    def _all_ranks(self, flag: bool) -> bool:
        """True when ``flag`` holds on every rank (collective)."""
        if self.world == 1:
            return flag
        got = [None] * self.world
        dist.all_gather_object(got, bool(flag), group=self.group)
        return all(got)

    def _create_vmm(self, nbytes: int) -> int:
        raw, w, r = self.raw, self.world, self.rank
        fd, size = C.c_int(-1), C.c_size_t(0)
        _native.check(raw.tpb_symm_vmm_create(w, r, nbytes, C.byref(fd), C.byref(size)), "tpb_symm_vmm_create")
        if w == 1:
            os.close(fd.value)
            return size.value
        tag = [f"tpb_symm_{os.getpid()}_{int.from_bytes(os.urandom(4), 'little')}"]
        dist.broadcast_object_list(tag, src=dist.get_global_rank(self.group, 0) if self.group is not None else 0,
                                   group=self.group)
        tag = tag[0]
        server = _send_fd_to_peers(fd.value, w - 1, f"{tag}_{r}")
        dist.barrier(group=self.group)  # every rank is listening
        for p in range(w):
            if p != r:
                pfd = _recv_fd(f"{tag}_{p}")
                try:
                    _native.check(raw.tpb_symm_vmm_map_peer(p, pfd), "tpb_symm_vmm_map_peer")
                finally:
                    os.close(pfd)
        server.join()
        os.close(fd.value)
        dist.barrier(group=self.group)
        want_mc = os.environ.get("TPB_SYMM_MULTICAST", "1") != "0"
        if want_mc and self._all_ranks(bool(raw.tpb_symm_vmm_supported(1))):
            if r == 0:
                mfd = C.c_int(-1)
                _native.check(raw.tpb_symm_mc_create(C.byref(mfd)), "tpb_symm_mc_create")
                server = _send_fd_to_peers(mfd.value, w - 1, f"{tag}_mc")
                dist.barrier(group=self.group)
                server.join()
                os.close(mfd.value)
            else:
                dist.barrier(group=self.group)
                mfd = _recv_fd(f"{tag}_mc")
                try:
                    _native.check(raw.tpb_symm_mc_import(mfd), "tpb_symm_mc_import")
                finally:
                    os.close(mfd)
            dist.barrier(group=self.group)
            _native.check(raw.tpb_symm_mc_add_device(), "tpb_symm_mc_add_device")
            dist.barrier(group=self.group)  # every device joined before any memory is bound
            _native.check(raw.tpb_symm_mc_bind(), "tpb_symm_mc_bind")
            dist.barrier(group=self.group)
            self.multicast = True
        return size.value

    def multicast_ptr(self, t: torch.Tensor) -> int:
        """Multicast address of an arena tensor (0 without a multicast mapping)."""
        return int(self.raw.tpb_symm_mc_ptr(self.offset_of(t)) or 0) if self.multicast else 0

    def _alloc_bytes(self, nbytes: int) -> int:
        off = self.raw.tpb_symm_alloc(nbytes)
        if off == NO_OFFSET:
            raise MemoryError(f"symmetric arena exhausted (asked {nbytes} bytes of {self.nbytes})")
        return off

    # Debug aid (TPB_SYMM_CANARY=1): every allocation is followed by CANARY_BYTES of a fixed pattern
    # that no kernel may touch; check_canaries() names the allocations whose guard was overwritten
    # (a store past the end of the buffer before it, by this rank or by a peer).
    CANARY_BYTES = 256
    CANARY_BYTE = 0xA5

    def _raw_bytes(self, off: int, nbytes: int) -> torch.Tensor:
        ptr = self.raw.tpb_symm_ptr(self.rank, off)
        return torch.as_tensor(_DevMem(ptr, nbytes), device=self.device)

    def alloc(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        """Tensor backed by the arena at the same offset on every rank (call collectively)."""
        nbytes = numel * torch.empty(0, dtype=dtype).element_size()
        size = max(nbytes, 16)
        if self.canaries is not None:
            size = (size + 15) // 16 * 16
            off = self._alloc_bytes(size + self.CANARY_BYTES)
            self._raw_bytes(off + size, self.CANARY_BYTES).fill_(self.CANARY_BYTE)
            self.canaries.append((off, size))
        else:
            off = self._alloc_bytes(size)
        t = self._raw_bytes(off, size)[:nbytes].view(dtype)
        self._offsets[t.data_ptr()] = off
        return t

    def _check_at_exit(self) -> None:
        # guards on and the arena never closed: verify once at interpreter exit, fail the process loudly
        if SymmArena._instance is not self:
            return
        try:
            bad = self.check_canaries()
        except Exception:
            return
        if bad:
            import sys
            print(f"symmetric arena: guard bytes overwritten after allocations {bad}", file=sys.stderr, flush=True)
            os._exit(66)

    def check_canaries(self) -> list:
        """``[(offset, bytes), ...]`` of the allocations whose trailing guard no longer holds the pattern
        (empty when all are intact, or when guards are off). Synchronises the device."""
        if not self.canaries:
            return []
        torch.cuda.synchronize(self.device)
        bad = []
        for off, size in self.canaries:
            g = self._raw_bytes(off + size, self.CANARY_BYTES)
            if not bool((g == self.CANARY_BYTE).all()):
                bad.append((off, size))
        return bad

    def offset_of(self, t: torch.Tensor) -> int:
        """Arena offset of a tensor returned by ``alloc`` (or of a slice of one)."""
        base = self.raw.tpb_symm_ptr(self.rank, 0)
        off = t.data_ptr() - base
        if off < 0 or off >= self.nbytes:
            raise ValueError("tensor is not in the symmetric arena")
        return off

    def slots(self, n: int) -> int:
        s = self._next_slot
        if s + n > self.pad_slots:
            raise MemoryError("out of signal slots")
        self._next_slot += n
        return s

    def close(self) -> None:
        """Release the arena (collective: no rank may still read a peer's memory). With guards on, raises
        if one was overwritten."""
        torch.cuda.synchronize(self.device)
        bad = self.check_canaries()
        if self.world > 1:
            dist.barrier(group=self.group)
        self.raw.tpb_symm_destroy()
        SymmArena._instance = None
        if bad:
            raise RuntimeError(f"symmetric arena: guard bytes overwritten after allocations {bad}")


class SymmComm:
    """The engine's communication backend on peer memory: all-gather by pulls and the fused
    reduce-scatter + AdamW + bf16 parameter emit."""

    def __init__(self, engine, wait_s: float = 30.0, gather_ctas: int = 24, reduce_ctas: int = 148,
                 extra_bytes: int = 1 << 30):
        self.engine = engine
        self.world, self.rank = engine.world, engine.rank
        units = engine.units
        esz = torch.empty(0, dtype=engine.param_dtype).element_size()
        max_padded = max(u.padded for u in units)
        n_pool = (len(units) if not engine.checkpoint else 3) + 2
        total = sum(u.shard_numel for u in units) * esz + n_pool * max_padded * esz
        total += (len(units) + n_pool + 8) * 512 + (1 << 20)
        total += extra_bytes  # head-room for other users of the arena (TP plans, MoE workspaces)
        self.arena = SymmArena(total, group=engine.group)
        self.wait_s = wait_s
        # CTAs of the communication kernels: enough to keep NVLink busy, few enough to leave the SMs
        # to the GEMMs they overlap with (TPB_GATHER_CTAS / TPB_REDUCE_CTAS override for tuning)
        self.gather_ctas = int(os.environ.get("TPB_GATHER_CTAS", gather_ctas))
        self.reduce_ctas = int(os.environ.get("TPB_REDUCE_CTAS", reduce_ctas))
        w = self.world
        self.slot_gather = {u.index: self.arena.slots(w) for u in units}
        self.slot_gather_done = {u.index: self.arena.slots(w) for u in units}
        self.slot_ready = {u.index: self.arena.slots(w) for u in units}
        self.slot_done = {u.index: self.arena.slots(w) for u in units}
        self.epoch_gather = {u.index: 0 for u in units}
        self.epoch_reduce = {u.index: 0 for u in units}
        self.grad_slot_last = {}  # grad pool slot -> (unit index, epoch) whose readers must finish
        self.status = status_word(engine.device)
        # "ce": bulk transfers by the copy engines (no SM time; the fused reduce + AdamW kernel then
        # reads local memory only); "sm": kernels that load from peer memory themselves (with a
        # multicast mapping the reduce + AdamW kernel takes its slice through one in-switch reducing
        # load per 16 bytes); "mc": as "sm", and the all-gather is a multicast push (every rank
        # stores its shard once, the switch delivers it to all ranks).
        spec = os.environ.get("TPB_REDUCE_OVERLAP", "")  # "threads,max_shared" for the reduce + AdamW kernel
        if spec:
            th, ms = (int(x) for x in spec.split(","))
            _native.check(self.arena.raw.tpb_symm_set_overlap(th, ms), "tpb_symm_set_overlap")
        self.transport = os.environ.get("TPB_COMM_TRANSPORT", "ce")
        if self.transport == "mc" and not self.arena.multicast:
            raise RuntimeError("TPB_COMM_TRANSPORT=mc needs the virtual-memory arena with a multicast mapping")
        self.staging = None
        if self.transport == "ce":
            shard_max = max(u.shard_numel for u in units)
            self.staging = torch.empty(self.world * shard_max, dtype=engine.param_dtype, device=engine.device)

    def alloc_shard(self, u) -> torch.Tensor:
        t = self.arena.alloc(u.shard_numel, self.engine.param_dtype)
        u._shard_off = self.arena.offset_of(t)
        return t

    def alloc_full(self, numel: int) -> torch.Tensor:
        return self.arena.alloc(numel, self.engine.param_dtype)

    def all_gather(self, u, buf: torch.Tensor) -> None:
        self.epoch_gather[u.index] += 1
        if self.transport == "ce":
            code = self.arena.raw.tpb_symm_allgather_ce(
                u._shard_off, u.shard_numel * buf.element_size(), buf.data_ptr(), self.arena.pad_off,
                self.slot_gather[u.index], self.epoch_gather[u.index], self.wait_s, self.status.data_ptr(),
                stream_ptr())
            _native.launch_count += 1
            _native.check(code, "tpb_symm_allgather_ce")
            return
        if self.transport == "mc":
            ep = self.epoch_gather[u.index]
            code = self.arena.raw.tpb_symm_allgather_mc(
                u.shard.data_ptr(), u.shard_numel * buf.element_size(), self.arena.offset_of(buf), self.arena.pad_off,
                self.slot_gather[u.index], self.slot_gather_done[u.index], ep, self.arena.counter_ptr(512 + u.index),
                self.gather_ctas, self.wait_s, self.status.data_ptr(), stream_ptr())
            _native.check(code, "tpb_symm_allgather_mc")
            code = self.arena.raw.tpb_symm_wait_slots(self.arena.pad_off, self.slot_gather_done[u.index], ep,
                                                      self.wait_s, self.status.data_ptr(), stream_ptr())
            _native.launch_count += 2
            _native.check(code, "tpb_symm_wait_slots")
            return
        code = self.arena.raw.tpb_symm_allgather(
            u._shard_off, u.shard_numel * buf.element_size(), buf.data_ptr(), self.arena.pad_off,
            self.slot_gather[u.index], self.epoch_gather[u.index], self.gather_ctas, self.wait_s,
            self.status.data_ptr(), stream_ptr())
        _native.launch_count += 1
        _native.check(code, "tpb_symm_allgather")

    def reduce_scatter_adamw(self, u, g: torch.Tensor, adam: dict) -> None:
        self.epoch_reduce[u.index] += 1
        ep = self.epoch_reduce[u.index]
        lo, hi = u.shard_range()
        if self.transport == "ce":
            code = self.arena.raw.tpb_symm_rs_adamw_ce(
                self.arena.offset_of(g), lo, hi - lo, self.staging.data_ptr(), u.master.data_ptr(),
                u.exp_avg.data_ptr(), u.exp_avg_sq.data_ptr(), u.shard.data_ptr(), None, None, 0, adam["lr"],
                adam["beta1"], adam["beta2"], adam["eps"], adam["weight_decay"], int(adam["step"]),
                1.0 / self.world, None, self.arena.pad_off, self.slot_ready[u.index], self.slot_done[u.index],
                ep, self.reduce_ctas, self.wait_s, self.status.data_ptr(), stream_ptr())
            _native.launch_count += 3
            _native.check(code, "tpb_symm_rs_adamw_ce")
            self.grad_slot_last[u._grad_slot] = (u.index, ep)
            return
        code = self.arena.raw.tpb_symm_rs_adamw(
            self.arena.offset_of(g), lo, hi - lo, u.master.data_ptr(), u.exp_avg.data_ptr(),
            u.exp_avg_sq.data_ptr(), u.shard.data_ptr(), NO_OFFSET, None, None, 0, adam["lr"],
            adam["beta1"], adam["beta2"], adam["eps"], adam["weight_decay"], int(adam["step"]),
            1.0 / self.world, None, self.arena.pad_off, self.slot_ready[u.index],
            self.slot_done[u.index], ep, self.arena.counter_ptr(u.index),
            self.reduce_ctas, self.wait_s, self.status.data_ptr(), stream_ptr())
        _native.launch_count += 1
        _native.check(code, "tpb_symm_rs_adamw")
        self.grad_slot_last[u._grad_slot] = (u.index, ep)

    def reduce_scatter_only(self, u, g: torch.Tensor, red_out: torch.Tensor, sumsq: torch.Tensor) -> None:
        """Reduce-scatter (mean) of the bf16 gradient into ``red_out`` (fp32 shard) and add its squared
        norm to ``sumsq``: phase 1 of a clipped step."""
        self.epoch_reduce[u.index] += 1
        ep = self.epoch_reduce[u.index]
        lo, hi = u.shard_range()
        if self.transport == "ce":
            code = self.arena.raw.tpb_symm_rs_adamw_ce(
                self.arena.offset_of(g), lo, hi - lo, self.staging.data_ptr(), None, None, None, None,
                red_out.data_ptr(), sumsq.data_ptr(), 1, 0.0, 0.9, 0.999, 1e-8, 0.0, 1, 1.0 / self.world, None,
                self.arena.pad_off, self.slot_ready[u.index], self.slot_done[u.index], ep, self.reduce_ctas,
                self.wait_s, self.status.data_ptr(), stream_ptr())
            _native.launch_count += 3
            _native.check(code, "tpb_symm_rs_adamw_ce")
            self.grad_slot_last[u._grad_slot] = (u.index, ep)
            return
        code = self.arena.raw.tpb_symm_rs_adamw(
            self.arena.offset_of(g), lo, hi - lo, None, None, None, None, NO_OFFSET, red_out.data_ptr(),
            sumsq.data_ptr(), 1, 0.0, 0.9, 0.999, 1e-8, 0.0, 1, 1.0 / self.world, None, self.arena.pad_off,
            self.slot_ready[u.index], self.slot_done[u.index], ep,
            self.arena.counter_ptr(u.index), self.reduce_ctas, self.wait_s,
            self.status.data_ptr(), stream_ptr())
        _native.launch_count += 1
        _native.check(code, "tpb_symm_rs_adamw")
        self.grad_slot_last[u._grad_slot] = (u.index, ep)

    def before_grad_reuse(self, slot: int) -> None:
        """Order the current stream after every peer's reads of gradient buffer ``slot``."""
        last = self.grad_slot_last.get(slot)
        if last is None:
            return
        uidx, ep = last
        code = self.arena.raw.tpb_symm_wait_slots(self.arena.pad_off, self.slot_done[uidx], ep,
                                                  self.wait_s, self.status.data_ptr(), stream_ptr())
        _native.launch_count += 1
        _native.check(code, "tpb_symm_wait_slots")
