"""Bounded device-side waits: a wait that nothing satisfies runs out after its budget, the kernel
returns, the host reads the status word as ``DeviceWaitTimeout`` and the context stays usable.

The failure is made on the host side only: the test asks for an epoch that no rank ever signals
and gives the wait a budget of a few hundredths of a second. Nothing faults, traps or hangs.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _arena():
    from tensorplay_b200.parallel.symm import SymmArena
    return SymmArena._instance or SymmArena(64 << 20)


def _wait(arena, slot, epoch, wait_s):
    from tensorplay_b200 import _native
    from tensorplay_b200.ops._common import status_word, stream_ptr
    st = status_word(arena.device)
    _native.check(arena.raw.tpb_symm_wait_slots(arena.pad_off, slot, epoch, wait_s, st.data_ptr(), stream_ptr()),
                  "tpb_symm_wait_slots")


def test_wait_on_unsignalled_slot_times_out_and_context_survives():
    import tensorplay_b200.ops as ops
    from tensorplay_b200.ops._common import DeviceWaitTimeout
    arena = _arena()
    slot = arena.slots(arena.world)
    ops.check_status()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    _wait(arena, slot, 7, 0.05)  # epoch 7 of a slot that was never written
    t1.record()
    torch.cuda.synchronize()
    assert 20.0 < t0.elapsed_time(t1) < 2000.0  # gave up after about the budget, not at once and not never
    with pytest.raises(DeviceWaitTimeout) as e:
        ops.check_status()
    assert "site 23" in str(e.value)
    ops.check_status()  # the word was reset
    # the next kernels run normally
    x = torch.randn(64, 512, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(512, device="cuda", dtype=torch.bfloat16)
    y = ops.rms_norm(x, w, 1e-5)
    ref = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-5)
    assert (y.float() - ref).abs().max().item() < 0.05
    ops.check_status()


def test_timed_out_handshake_leaves_optimizer_state_untouched():
    """Copy-engine reduce + AdamW after a hand-shake that ran out of time: master weights and moments
    keep their values; after the status word is cleared the same call updates them."""
    import tensorplay_b200.ops as ops
    from tensorplay_b200 import _native
    from tensorplay_b200.ops._common import DeviceWaitTimeout, status_word, stream_ptr
    arena = _arena()
    n = 8192
    dev = arena.device
    g = arena.alloc(n, torch.bfloat16)
    g.copy_(torch.randn(n, device=dev).to(torch.bfloat16))
    staging = torch.empty(arena.world * n, dtype=torch.bfloat16, device=dev)
    master = torch.randn(n, device=dev)
    m = torch.zeros(n, device=dev)
    v = torch.zeros(n, device=dev)
    shard = master.to(torch.bfloat16)
    keep = (master.clone(), m.clone(), v.clone(), shard.clone())
    ready, done = arena.slots(arena.world), arena.slots(arena.world)
    dead = arena.slots(arena.world)
    st = status_word(dev)

    def call(epoch):
        code = arena.raw.tpb_symm_rs_adamw_ce(
            arena.offset_of(g), 0, n, staging.data_ptr(), master.data_ptr(), m.data_ptr(), v.data_ptr(),
            shard.data_ptr(), None, None, 0, 1e-2, 0.9, 0.95, 1e-8, 0.0, 1, 1.0, None, arena.pad_off, ready, done,
            epoch, 8, 0.05, st.data_ptr(), stream_ptr())
        _native.check(code, "tpb_symm_rs_adamw_ce")

    ops.check_status()
    _wait(arena, dead, 3, 0.03)  # runs out: status word set
    call(1)
    torch.cuda.synchronize()
    for a, b in zip((master, m, v, shard), keep):
        assert torch.equal(a, b)
    with pytest.raises(DeviceWaitTimeout):
        ops.check_status()
    call(2)
    torch.cuda.synchronize()
    ops.check_status()
    assert not torch.equal(master, keep[0])
    assert (m - 0.1 * g.float()).abs().max().item() < 1e-6


def test_virtual_memory_arena_on_one_gpu():
    """The arena of a single rank comes from the virtual-memory allocator (no peers, no multicast
    object): tensors carved from it are ordinary device memory at 256-byte aligned offsets."""
    arena = _arena()
    assert arena.allocator == "vmm" and not arena.multicast
    a = arena.alloc(1000, torch.float32)
    b = arena.alloc(7, torch.bfloat16)
    assert arena.offset_of(a) % 256 == 0 and arena.offset_of(b) % 256 == 0
    assert arena.offset_of(b) >= arena.offset_of(a) + 4000
    a.copy_(torch.arange(1000, device=a.device, dtype=torch.float32))
    b.fill_(3.0)
    torch.cuda.synchronize()
    assert float(a.sum()) == 999 * 1000 / 2 and float(b.float().sum()) == 21.0
    assert arena.multicast_ptr(a) == 0
