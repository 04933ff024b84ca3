"""The chunked, double-buffered transport protocol and the plan-level pair
order on CPU ranks (gloo, world_size 2 and 4). The bytes are packed and
unpacked by the oracle here; on a GPU the same functions are driven by the
CUDA library (tests/test_gpu_multi.py)."""
import os
import socket
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from elasticmm_b200.engine.v0.transport import (MigrationPlan, Transfer, plan_chunks, pipelined_recv,
                                                pipelined_send)
from oracle import kv_oracle


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _init(rank, world, port):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)


GEOM = dict(L=6, NB=48, BS=4, H=2, D=8)


def _pool(seed, guard=False):
    return kv_oracle.make_pool(GEOM["L"], GEOM["NB"], GEOM["BS"], GEOM["H"], GEOM["D"], torch.float16, seed,
                               fill="guard" if guard else "normal")


def _page_bytes():
    return GEOM["BS"] * GEOM["H"] * GEOM["D"] * 2


def _send(pool, ids, dst, target_bytes):
    n = len(ids)
    chunks = plan_chunks(GEOM["L"], n, _page_bytes(), target_bytes)
    slots = {}

    def buffer_for(slot, count):
        shape = (count, 2, n, GEOM["BS"], GEOM["H"], GEOM["D"])
        if slot not in slots or slots[slot].shape != shape:
            slots[slot] = torch.empty(shape, dtype=torch.float16)
        return slots[slot]

    def pack(buf, begin, count):
        buf.copy_(kv_oracle.extract_kv_blocks(pool[begin:begin + count], ids))

    return pipelined_send(chunks, buffer_for, pack, lambda buf: dist.isend(buf, dst=dst))


def _recv(pool, ids, src, target_bytes):
    n = len(ids)
    chunks = plan_chunks(GEOM["L"], n, _page_bytes(), target_bytes)
    slots = {}

    def buffer_for(slot, count):
        shape = (count, 2, n, GEOM["BS"], GEOM["H"], GEOM["D"])
        if slot not in slots or slots[slot].shape != shape:
            slots[slot] = torch.empty(shape, dtype=torch.float16)
        return slots[slot]

    def unpack(buf, begin, count):
        kv_oracle.write_kv_blocks(pool[begin:begin + count], ids, buf)

    return pipelined_recv(chunks, buffer_for, lambda buf: dist.irecv(buf, src=src), unpack)


def _pair_worker(rank, world, port, out_dir, target_bytes):
    _init(rank, world, port)
    g = torch.Generator().manual_seed(3)
    src_ids = torch.randperm(GEOM["NB"], generator=g)[:19].tolist()
    dst_ids = torch.randperm(GEOM["NB"], generator=g)[:19].tolist()
    if rank == 0:
        msgs = _send(_pool(41), src_ids, 1, target_bytes)
    else:
        pool = _pool(0, guard=True)
        msgs = _recv(pool, dst_ids, 0, target_bytes)
        want = _pool(0, guard=True)
        kv_oracle.write_kv_blocks(want, dst_ids, kv_oracle.extract_kv_blocks(_pool(41), src_ids))
        ok = all(kv_oracle.bit_equal(a, b) for a, b in zip(pool, want))
        torch.save({"ok": ok, "msgs": msgs}, os.path.join(out_dir, "r1.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("target_bytes", [1, 19 * 2 * 128 * 2, 1 << 30])
def test_pipelined_pair_transfer_is_bit_exact(target_bytes):
    """One layer per message, two layers per message, and the two-chunk minimum."""
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_pair_worker, args=(2, _free_port(), d, target_bytes), nprocs=2, join=True)
        res = torch.load(os.path.join(d, "r1.pt"))
    assert res["ok"]
    assert res["msgs"] == len(plan_chunks(GEOM["L"], 19, _page_bytes(), target_bytes)) >= 2


def _plan(world_sources, world_sinks, seed):
    g = torch.Generator().manual_seed(seed)
    plan = MigrationPlan()
    next_dst = {d: 0 for d in world_sinks}
    for s in world_sources:
        free = torch.randperm(GEOM["NB"], generator=g).tolist()
        for r in range(5):
            n = int(torch.randint(1, 6, (1,), generator=g))
            dst = world_sinks[int(torch.randint(0, len(world_sinks), (1,), generator=g))]
            src_blocks, free = free[:n], free[n:]
            dst_blocks = list(range(next_dst[dst], next_dst[dst] + n))
            next_dst[dst] += n
            plan.add(Transfer(f"s{s}r{r}", s, dst, tuple(src_blocks), tuple(dst_blocks)))
    return plan


def _plan_worker(rank, world, port, out_dir):
    _init(rank, world, port)
    plan = _plan([0, 1], [2, 3], seed=8)
    plan.validate(lambda r: GEOM["NB"])
    pool = _pool(60 + rank) if rank < 2 else _pool(0, guard=True)
    for s, d in plan.ordered_pairs():
        if s == rank:
            _send(pool, plan.tables(s, d)[0], d, 4096)
        elif d == rank:
            _recv(pool, plan.tables(s, d)[1], s, 4096)
    if rank >= 2:
        want = _pool(0, guard=True)
        for s in plan.incoming(rank):
            si, di = plan.tables(s, rank)
            kv_oracle.write_kv_blocks(want, di, kv_oracle.extract_kv_blocks(_pool(60 + s), si))
        ok = all(kv_oracle.bit_equal(a, b) for a, b in zip(pool, want))
        torch.save({"ok": ok}, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_plan_level_migration_two_sources_two_sinks():
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_plan_worker, args=(4, _free_port(), d), nprocs=4, join=True)
        assert torch.load(os.path.join(d, "r2.pt"))["ok"]
        assert torch.load(os.path.join(d, "r3.pt"))["ok"]


def _absent_peer_worker(rank, world, port, out_dir):
    """Failure detection on the host: the source never sends; the sink's
    receive must end with an error within the group's timeout."""
    import datetime

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    if rank == 1:
        err = None
        try:
            _recv(_pool(0, guard=True), [1, 2, 3], 0, 1 << 30)
        except Exception as e:  # gloo reports the timeout as a RuntimeError
            err = type(e).__name__
        torch.save({"err": err}, os.path.join(out_dir, "r1.pt"))
    else:
        import time
        time.sleep(5)
    try:
        dist.destroy_process_group()
    except Exception:
        pass


def test_receive_from_a_silent_peer_times_out_on_the_host():
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_absent_peer_worker, args=(2, _free_port(), d), nprocs=2, join=True)
        assert torch.load(os.path.join(d, "r1.pt"))["err"] is not None
