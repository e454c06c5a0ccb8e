"""torchrun worker: the symmetric-memory collectives against NCCL on integer patterns.

Small integers are exact in bf16 and so are their sums over <= 8 ranks, whatever the order of the
additions: the all-gather, the reduce-scatter (reduce-only mode of the fused kernel) and the
all-reduce must match NCCL bit for bit, with the multicast (in-switch) forms and with plain peer
loads and stores. A second part checks the reduce-scatter on random bf16 data within the tolerance
of one bf16 rounding of the sum.
"""
import ctypes as C
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import tensorplay_b200.ops as O  # noqa: E402
from tensorplay_b200 import _native  # noqa: E402
from tensorplay_b200.ops._common import status_word, stream_ptr  # noqa: E402
from tensorplay_b200.parallel.symm import NO_OFFSET, SymmArena  # noqa: E402


def main():
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    arena = SymmArena(256 << 20)
    raw = arena.raw
    st = status_word(dev)
    res = {"rank": rank, "allocator": arena.allocator, "multicast": arena.multicast, "checks": []}
    n = 1 << 20                      # elements per rank
    assert n % (8 * world) == 0
    gen = torch.Generator(device="cpu").manual_seed(100 + rank)
    mine = torch.randint(-8, 9, (n,), generator=gen).to(torch.bfloat16).to(dev)
    epoch = 0

    def check(name, a, b):
        same = bool(torch.equal(a, b))
        res["checks"].append((name, same))
        if not same:
            raise AssertionError(f"rank {rank}: {name} differs from NCCL ({(a.float() - b.float()).abs().max().item()})")

    # ---------------------------------------------------------------- all-gather
    shard = arena.alloc(n, torch.bfloat16)
    full = arena.alloc(n * world, torch.bfloat16)
    shard.copy_(mine)
    ref = torch.empty(n * world, dtype=torch.bfloat16, device=dev)
    dist.all_gather_into_tensor(ref, mine)
    s_ready, s_done = arena.slots(world), arena.slots(world)
    for kind in ("pull", "ce") + (("mc",) if arena.multicast else ()):
        epoch += 1
        full.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        if kind == "pull":
            code = raw.tpb_symm_allgather(arena.offset_of(shard), n * 2, full.data_ptr(), arena.pad_off, s_ready, epoch, 8,
                                          10.0, st.data_ptr(), stream_ptr())
        elif kind == "ce":
            code = raw.tpb_symm_allgather_ce(arena.offset_of(shard), n * 2, full.data_ptr(), arena.pad_off, s_ready,
                                             epoch, 10.0, st.data_ptr(), stream_ptr())
        else:
            code = raw.tpb_symm_allgather_mc(shard.data_ptr(), n * 2, arena.offset_of(full), arena.pad_off, s_ready,
                                             s_done, epoch, arena.counter_ptr(0), 16, 10.0, st.data_ptr(), stream_ptr())
            _native.check(code, "allgather_mc")
            code = raw.tpb_symm_wait_slots(arena.pad_off, s_done, epoch, 10.0, st.data_ptr(), stream_ptr())
        _native.check(code, f"allgather {kind}")
        torch.cuda.synchronize()
        O.check_status()
        check(f"all_gather/{kind}", full, ref)
        dist.barrier()

    # ---------------------------------------------------------------- reduce-scatter and all-reduce
    grads = arena.alloc(n, torch.bfloat16)
    grads.copy_(mine)
    per = n // world
    ref_rs = torch.empty(per, dtype=torch.bfloat16, device=dev)
    dist.reduce_scatter_tensor(ref_rs, mine.clone(), op=dist.ReduceOp.SUM)
    ref_ar = mine.clone()
    dist.all_reduce(ref_ar)
    r_ready, r_done = arena.slots(world), arena.slots(world)
    work = arena.alloc(n, torch.bfloat16)
    for mc in ((1, 0) if arena.multicast else (0,)):
        raw.tpb_symm_set_multicast(mc)
        tag = "multimem" if mc else "peer loads"
        # reduce-scatter: mode 1 writes the reduced fp32 slice
        epoch += 1
        red = torch.zeros(per, dtype=torch.float32, device=dev)
        sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        torch.cuda.synchronize()
        dist.barrier()
        code = raw.tpb_symm_rs_adamw(arena.offset_of(grads), rank * per, per, None, None, None, None, NO_OFFSET,
                                     red.data_ptr(), sumsq.data_ptr(), 1, 0.0, 0.9, 0.999, 1e-8, 0.0, 1, 1.0, None,
                                     arena.pad_off, r_ready, r_done, epoch, arena.counter_ptr(1), 32, 10.0,
                                     st.data_ptr(), stream_ptr())
        _native.check(code, "rs")
        code = raw.tpb_symm_wait_slots(arena.pad_off, r_done, epoch, 10.0, st.data_ptr(), stream_ptr())
        _native.check(code, "rs wait")
        torch.cuda.synchronize()
        O.check_status()
        check(f"reduce_scatter/{tag}", red.to(torch.bfloat16), ref_rs)
        # all-reduce in place: mode 2 puts the reduced slice into every rank's buffer
        epoch += 1
        work.copy_(mine)
        torch.cuda.synchronize()
        dist.barrier()
        code = raw.tpb_symm_rs_adamw(arena.offset_of(work), rank * per, per, None, None, None, None,
                                     arena.offset_of(work), None, None, 2, 0.0, 0.9, 0.999, 1e-8, 0.0, 1, 1.0, None,
                                     arena.pad_off, r_ready, r_done, epoch, arena.counter_ptr(1), 32, 10.0,
                                     st.data_ptr(), stream_ptr())
        _native.check(code, "ar")
        code = raw.tpb_symm_wait_slots(arena.pad_off, r_done, epoch, 10.0, st.data_ptr(), stream_ptr())
        _native.check(code, "ar wait")
        torch.cuda.synchronize()
        O.check_status()
        check(f"all_reduce/{tag}", work, ref_ar)
        dist.barrier()

    # ---------------------------------------------------------------- random data: one bf16 rounding of the sum
    gen.manual_seed(500 + rank)
    rnd = torch.randn(n, generator=gen).to(torch.bfloat16).to(dev)
    grads.copy_(rnd)
    exact = rnd.float()
    dist.all_reduce(exact)
    exact = exact[rank * per:(rank + 1) * per]
    for mc in ((1, 0) if arena.multicast else (0,)):
        raw.tpb_symm_set_multicast(mc)
        epoch += 1
        red = torch.zeros(per, dtype=torch.float32, device=dev)
        sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        torch.cuda.synchronize()
        dist.barrier()
        code = raw.tpb_symm_rs_adamw(arena.offset_of(grads), rank * per, per, None, None, None, None, NO_OFFSET,
                                     red.data_ptr(), sumsq.data_ptr(), 1, 0.0, 0.9, 0.999, 1e-8, 0.0, 1, 1.0, None,
                                     arena.pad_off, r_ready, r_done, epoch, arena.counter_ptr(1), 32, 10.0,
                                     st.data_ptr(), stream_ptr())
        _native.check(code, "rs random")
        code = raw.tpb_symm_wait_slots(arena.pad_off, r_done, epoch, 10.0, st.data_ptr(), stream_ptr())
        _native.check(code, "rs wait")
        torch.cuda.synchronize()
        O.check_status()
        err = ((red - exact).abs() / (exact.abs() + 1.0)).max().item()
        res["checks"].append((f"reduce_scatter random/{'multimem' if mc else 'peer loads'} rel err {err:.2e}", err < 8e-3))
        assert err < 8e-3, err
        dist.barrier()
    raw.tpb_symm_set_multicast(1)

    # ---------------------------------------------------------------- all-to-all(v) against NCCL
    from tensorplay_b200.distributed._symmetric_memory import AllToAll
    a2a = AllToAll(8 << 20)
    width = 64                        # bf16: 128-byte rows
    for trial in range(3):            # repeated calls reuse the send buffer: exercises the done hand-shake
        g2 = torch.Generator(device="cpu").manual_seed(900 + trial)
        counts = torch.randint(0, 400, (world, world), generator=g2)   # counts[s][d]: rows from s to d
        if trial == 2:
            counts[:, 0] = 0          # a rank that receives nothing
        send_rows = int(counts[rank].sum())
        recv_rows = int(counts[:, rank].sum())
        x = (torch.arange(send_rows * width, dtype=torch.float32) % 251 + rank).to(torch.bfloat16).to(dev).view(send_rows, width)
        out = torch.zeros(max(recv_rows, 1), width, dtype=torch.bfloat16, device=dev)
        ref = torch.zeros(max(recv_rows, 1), width, dtype=torch.bfloat16, device=dev)
        dist.all_to_all_single(ref[:recv_rows], x, counts[:, rank].tolist(), counts[rank].tolist())
        got_bytes = a2a(out, x, counts[rank].tolist())
        torch.cuda.synchronize()
        O.check_status()
        check(f"all_to_all_v trial {trial}", out[:recv_rows], ref[:recv_rows])
        assert got_bytes.tolist() == [int(c) * width * 2 for c in counts[:, rank]], got_bytes.tolist()
        dist.barrier()
    print("RESULT " + json.dumps(res), flush=True)
    arena.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
