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


class _StubPool:
    """Stands in for KVPool on a CPU rank: only the host-side id checks are needed."""

    def __init__(self, num_blocks):
        self.num_blocks = num_blocks

    def _validated(self, host, unique=False):
        import numpy as np

        from elasticmm_b200 import _lib

        host = np.asarray(host)
        if host.size and (host.min() < 0 or host.max() >= self.num_blocks):
            raise _lib.EmmError(_lib.ERR_ID_RANGE, f"block id outside [0, {self.num_blocks})")
        if unique and np.unique(host).size != host.size:
            raise _lib.EmmError(_lib.ERR_DUPLICATE, "duplicate destination block id")
        return host

    def block_bytes(self):
        return 1024


def _host_worker(rank, mapped_peers, pushes):
    """A V0Worker without a GPU: the constructor is bypassed, device waits are no-ops and the push
    'kernel' records what it was asked to move. Everything else of migrate() is the product code."""
    from elasticmm_b200.engine.v0.worker import V0Worker

    class HostOnlyWorker(V0Worker):
        def _own_stream_sync(self):
            pass

        def _device_error(self, what):
            return None

        def p2p_push_kv(self, dst_rank, src_blocks, dst_blocks):
            pushes.append((dst_rank, len(src_blocks)))
            return {"bytes": len(src_blocks) * 1024, "blocks": len(src_blocks)}

    w = object.__new__(HostOnlyWorker)
    w.device = torch.device("cpu")
    w.process_group = None
    w.global_rank = rank
    w.pool = _StubPool(GEOM["NB"])
    w.peer_pools = {p: _StubPool(GEOM["NB"]) for p in mapped_peers}
    w._nccl_comm = None
    return w


def _agreement_worker(rank, world, port, out_dir):
    import datetime

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    plan = MigrationPlan([Transfer("a", 0, 2, (1, 2, 3), (4, 5, 6)), Transfer("b", 1, 2, (7,), (9,)),
                          Transfer("c", 1, 3, (8, 9), (0, 1))])
    results = {}
    # 1. rank 1 has not mapped the pool of rank 3: every rank must return an error, and nothing is pushed
    pushes = []
    mapped = {0: [2], 1: [2], 2: [], 3: []}[rank]
    results["unmapped"] = (_host_worker(rank, mapped, pushes).migrate(plan, method="push"), list(pushes))
    # 2. a destination block used twice on rank 2 (seen by rank 2 only)
    bad = MigrationPlan([Transfer("a", 0, 2, (1, 2), (4, 5)), Transfer("b", 1, 2, (7,), (5,))])
    pushes = []
    results["duplicate"] = (_host_worker(rank, {0: [2], 1: [2, 3], 2: [], 3: []}[rank], pushes).migrate(bad, "push"),
                            list(pushes))
    # 3. all-to-all without a communicator fails on every rank before any exchange
    results["no_comm"] = (_host_worker(rank, [], []).migrate(plan, method="alltoall"), [])
    # 4. the good case
    pushes = []
    results["ok"] = (_host_worker(rank, {0: [2], 1: [2, 3], 2: [], 3: []}[rank], pushes).migrate(plan, "push"),
                     list(pushes))
    torch.save(results, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_every_rank_returns_the_error_when_one_rank_fails_a_host_check():
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_agreement_worker, args=(4, _free_port(), d), nprocs=4, join=True)
        res = [torch.load(os.path.join(d, f"r{r}.pt")) for r in range(4)]
    for r in range(4):
        for case in ("unmapped", "duplicate", "no_comm"):
            out, pushes = res[r][case]
            assert "error" in out and out["bytes"] == 0 and pushes == [], (r, case, out)
    assert "not mapped" in res[1]["unmapped"][0]["error"]
    assert "another rank" in res[0]["unmapped"][0]["error"]
    assert "duplicate" in res[2]["duplicate"][0]["error"]
    assert all("init_native_nccl" in res[r]["no_comm"][0]["error"] for r in range(4))
    assert res[0]["ok"] == ({"bytes": 3 * 1024, "blocks": 3}, [(2, 3)])
    assert res[1]["ok"] == ({"bytes": 3 * 1024, "blocks": 3}, [(2, 1), (3, 2)]) or \
        res[1]["ok"] == ({"bytes": 3 * 1024, "blocks": 3}, [(3, 2), (2, 1)])
    assert res[2]["ok"][0] == {"bytes": 0, "blocks": 0} and res[3]["ok"][0] == {"bytes": 0, "blocks": 0}
