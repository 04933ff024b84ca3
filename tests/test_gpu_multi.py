"""Prefill -> decode migration between GPUs (one process per GPU, NCCL + peer-mapped pools).
The NCCL cases need two or four GPUs. The direct-load path (the default migration path) is
also run as two processes sharing ONE GPU, with a gloo group for the host-side agreement and
CUDA IPC between the processes, so that a single-GPU box still checks plan-level pulls, waves
without a barrier and the all-ranks error agreement against the oracle."""
import os
import socket
import tempfile

import pytest
import torch

pytestmark = pytest.mark.gpu

GEOM = dict(L=28, NB=512, BS=16, H=4, D=128)   # Qwen2.5-VL-7B-shaped pages on a reduced pool


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _requests(seed):
    g = torch.Generator().manual_seed(seed)
    sperm = torch.randperm(GEOM["NB"], generator=g).tolist()
    dperm = torch.randperm(GEOM["NB"], generator=g).tolist()
    out, pos = [], 0
    for i in range(6):
        tokens = 576 + int(torch.randint(32, 1025, (1,), generator=g))
        n = -(-tokens // GEOM["BS"])
        if pos + n > GEOM["NB"]:
            break
        out.append((f"r{i}", sperm[pos:pos + n], dperm[pos:pos + n]))
        pos += n
    return out


def _worker_main(rank, world, port, out_dir):
    import torch.distributed as dist

    from elasticmm_b200.engine.v0 import MigrationPlan, Transfer, TransferMethod, V0KVTransferManager, V0Worker
    from oracle import kv_oracle

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    dev = torch.device("cuda", rank)

    def fresh(seed, guard):
        cpu = kv_oracle.make_pool(GEOM["L"], GEOM["NB"], GEOM["BS"], GEOM["H"], GEOM["D"], torch.bfloat16, seed,
                                  fill="guard" if guard else "normal")
        w = V0Worker(worker_id=rank, dtype="bfloat16", device=dev, global_rank=rank, world_size=world,
                     kv_cache=[t.to(dev) for t in cpu])
        assert w.init_global_nccl()
        return w, cpu

    def expect(reqs):
        src_cpu = kv_oracle.make_pool(GEOM["L"], GEOM["NB"], GEOM["BS"], GEOM["H"], GEOM["D"], torch.bfloat16, 70)
        want = kv_oracle.make_pool(GEOM["L"], GEOM["NB"], GEOM["BS"], GEOM["H"], GEOM["D"], torch.bfloat16, 0,
                                   fill="guard")
        for _, s, d in reqs:
            kv_oracle.write_kv_blocks(want, d, kv_oracle.extract_kv_blocks(src_cpu, s))
        return want

    def same(w, want):
        return all(kv_oracle.bit_equal(a.cpu(), b) for a, b in zip(w.kv_cache, want))

    results = {}
    reqs = _requests(3)

    # 1. staged NCCL, request by request, through the manager (source sends, sink receives)
    w, _ = fresh(70 if rank == 0 else 0, guard=rank != 0)
    mgr = V0KVTransferManager(transfer_method=TransferMethod.NCCL)
    mgr.register_worker(rank, w, "prefill" if rank == 0 else "decoding")
    oks = [mgr.transfer_kv_cache_sync(rid, 0, 1, s, d) for rid, s, d in reqs]
    results["nccl_ok"] = all(oks)
    if rank == 1:
        results["nccl_exact"] = same(w, expect(reqs))
        results["nccl_bytes"] = mgr.last_result["bytes"]
    dist.barrier()

    # 1b. the same through a communicator owned by the C library (pipelines run inside the library)
    w, _ = fresh(70 if rank == 0 else 0, guard=rank != 0)
    results["native_init_ok"] = w.init_native_nccl()
    mgr = V0KVTransferManager(transfer_method=TransferMethod.NCCL)
    mgr.register_worker(rank, w, "prefill" if rank == 0 else "decoding")
    before = w.ctx.launch_count
    oks = [mgr.transfer_kv_cache_sync(rid, 0, 1, s, d) for rid, s, d in reqs]
    results["native_nccl_ok"] = all(oks) and w.ctx.launch_count > before
    if rank == 1:
        results["native_nccl_exact"] = same(w, expect(reqs))
    # raw entries: one message each way, then both ways in one grouped exchange
    comm = w._nccl_comm
    mine = torch.full((1 << 20,), float(rank + 1), dtype=torch.float32, device=dev)
    theirs = torch.zeros_like(mine)
    if rank == 0:
        w.ctx.send_packed(comm, mine, 1)
        w.ctx.recv_packed(comm, theirs, 1)
    else:
        w.ctx.recv_packed(comm, theirs, 0)
        w.ctx.send_packed(comm, mine, 0)
    torch.cuda.synchronize()
    results["packed_exact"] = bool(torch.all(theirs == float(2 - rank)))
    theirs.zero_()
    w.ctx.exchange(comm, [(True, mine, 1 - rank), (False, theirs, 1 - rank)])
    torch.cuda.synchronize()
    results["exchange_packed_exact"] = bool(torch.all(theirs == float(2 - rank)))
    dist.barrier()

    # 1c. per-layer pipelined all-to-all over the same communicator: one direction, then both at once
    wa, _ = fresh(70 if rank == 0 else 0, guard=rank != 0)
    wa.init_native_nccl()
    plan_a = MigrationPlan([Transfer(rid, 0, 1, tuple(s), tuple(d)) for rid, s, d in reqs])
    res = wa.migrate(plan_a, method="alltoall")
    results["alltoall_ok"] = "error" not in res
    if rank == 1:
        results["alltoall_exact"] = same(wa, expect(reqs))
    dist.barrier()
    wb2, _ = fresh(70, guard=False)          # every rank holds source data in the lower half of its pool ...
    wb2.init_native_nccl()
    half = GEOM["NB"] // 2
    both = MigrationPlan([Transfer(f"x{src}", src, 1 - src, tuple(range(src, half, 2)),
                                   tuple(range(half + src, GEOM["NB"], 2))) for src in (0, 1)])
    before_cpu = kv_oracle.make_pool(GEOM["L"], GEOM["NB"], GEOM["BS"], GEOM["H"], GEOM["D"], torch.bfloat16, 70)
    res = wb2.migrate(both, method="alltoall")  # ... and receives the peer's blocks into its upper half
    results["alltoall_both_ok"] = "error" not in res and res["blocks"] == 2 * len(range(0, half, 2))
    src_ids, dst_ids = both.tables(1 - rank, rank)
    kv_oracle.write_kv_blocks(before_cpu, dst_ids, kv_oracle.extract_kv_blocks(
        kv_oracle.make_pool(GEOM["L"], GEOM["NB"], GEOM["BS"], GEOM["H"], GEOM["D"], torch.bfloat16, 70), src_ids))
    results["alltoall_both_exact"] = same(wb2, before_cpu)
    dist.barrier()

    # 2. direct peer stores: map the sink's pool into the source, one launch per request
    w, _ = fresh(70 if rank == 0 else 0, guard=rank != 0)
    handles = [None] * world
    dist.all_gather_object(handles, (w.get_ipc_handles(), w.get_pool_desc()))
    for peer in range(world):
        if peer != rank:
            w.attach_peer_pool(peer, handles[peer][0], handles[peer][1])
    for direction in ("pull", "push"):
        if direction == "push":
            w, _ = fresh(70 if rank == 0 else 0, guard=rank != 0)
            handles = [None] * world
            dist.all_gather_object(handles, (w.get_ipc_handles(), w.get_pool_desc()))
            for peer in range(world):
                if peer != rank:
                    w.attach_peer_pool(peer, handles[peer][0], handles[peer][1])
        mgr = V0KVTransferManager(transfer_method=TransferMethod.B200_PEER, peer_direction=direction)
        mgr.register_worker(rank, w, "prefill" if rank == 0 else "decoding")
        launches = w.ctx.launch_count
        oks = [mgr.transfer_kv_cache_sync(rid, 0, 1, s, d) for rid, s, d in reqs]
        results[f"peer_{direction}_ok"] = all(oks)
        active = 1 if direction == "pull" else 0
        results[f"peer_{direction}_launches_ok"] = (w.ctx.launch_count - launches) == (len(reqs) if rank == active else 0)
        dist.barrier()
        if rank == 1:
            results[f"peer_{direction}_exact"] = same(w, expect(reqs))
        dist.barrier()

    # 3. plan level, both methods, all requests as one table per pair
    for method in ("pull", "push", "nccl"):
        w2, _ = fresh(70 if rank == 0 else 0, guard=rank != 0)
        if method != "nccl":
            h2 = [None] * world
            dist.all_gather_object(h2, (w2.get_ipc_handles(), w2.get_pool_desc()))
            for peer in range(world):
                if peer != rank:
                    w2.attach_peer_pool(peer, h2[peer][0], h2[peer][1])
        plan = MigrationPlan([Transfer(rid, 0, 1, tuple(s), tuple(d)) for rid, s, d in reqs])
        res = w2.migrate(plan, method=method)
        results[f"plan_{method}_ok"] = "error" not in res
        dist.barrier()
        if rank == 1:
            results[f"plan_{method}_exact"] = same(w2, expect(reqs))
        dist.barrier()

    # 3b. broadcast form (the reference's collective_transfer_kv)
    wb, _ = fresh(70 if rank == 0 else 0, guard=rank != 0)
    rid, s_ids, d_ids = reqs[0]
    shape = (GEOM["L"], 2, len(s_ids), GEOM["BS"], GEOM["H"], GEOM["D"])
    res = wb.collective_transfer_kv(None, 0, s_ids if rank == 0 else d_ids, shape, "torch.bfloat16",
                                    "send" if rank == 0 else "recv")
    results["broadcast_ok"] = res["bytes"] == 2 * len(s_ids) * GEOM["L"] * GEOM["BS"] * GEOM["H"] * GEOM["D"] * 2
    if rank == 1:
        results["broadcast_exact"] = same(wb, expect(reqs[:1]))
    dist.barrier()

    # 4. exchange: both ranks are source and sink at once; each pulls from the other's source pool
    w3, _ = fresh(70, guard=False)
    sink_cpu = kv_oracle.make_pool(GEOM["L"], GEOM["NB"], GEOM["BS"], GEOM["H"], GEOM["D"], torch.bfloat16, 0,
                                   fill="guard")
    sink = V0Worker(worker_id=rank, dtype="bfloat16", device=dev, global_rank=rank, world_size=world,
                    kv_cache=[t.to(dev) for t in sink_cpu])
    sink.init_global_nccl()
    h3 = [None] * world
    dist.all_gather_object(h3, (w3.get_ipc_handles(), w3.get_pool_desc()))
    for peer in range(world):
        if peer != rank:
            sink.attach_peer_pool(peer, h3[peer][0], h3[peer][1])
    plan = MigrationPlan([Transfer(f"{rid}-{src}", src, 1 - src, tuple(s), tuple(d))
                          for src in (0, 1) for rid, s, d in _requests(3 + src)])
    res = sink.migrate(plan, method="pull")
    results["exchange_ok"] = "error" not in res and res["blocks"] > 0
    dist.barrier()
    mine = [(rid, s, d) for rid, s, d in _requests(3 + (1 - rank))]
    results["exchange_exact"] = same(sink, expect(mine))
    dist.barrier()

    results.update(_waves_and_agreement(rank, world, dev, fresh))
    torch.save(results, os.path.join(out_dir, f"r{rank}.pt"))
    dist.destroy_process_group()


def _wave_plans(n_waves, seed):
    """Rank 0 -> rank 1 in waves that alternate between the halves of both pools."""
    from elasticmm_b200.engine.v0 import MigrationPlan, Transfer

    g = torch.Generator().manual_seed(seed)
    half = GEOM["NB"] // 2
    plans = []
    for wv in range(n_waves):
        base = (wv % 2) * half
        sperm = (torch.randperm(half, generator=g) + base).tolist()
        dperm = (torch.randperm(half, generator=g) + base).tolist()
        plan, pos = MigrationPlan(), 0
        for r in range(3):
            n = int(torch.randint(5, 70, (1,), generator=g))
            plan.add(Transfer(f"w{wv}r{r}", 0, 1, tuple(sperm[pos:pos + n]), tuple(dperm[pos:pos + n])))
            pos += n
        plans.append(plan)
    return plans


def _waves_and_agreement(rank, world, dev, fresh):
    """Shared by the two-GPU run and the two-processes-on-one-GPU run: direct-load migration per plan,
    waves two deep without a barrier, and a host-side failure on one rank reported by all."""
    import torch.distributed as dist

    from elasticmm_b200.engine.v0 import MigrationPlan, Transfer
    from elasticmm_b200.engine.v0.transport import WaveLedger
    from oracle import kv_oracle

    results = {}
    store = dist.distributed_c10d._get_default_store()

    def mapped(seed, guard):
        w, cpu = fresh(seed, guard)
        hs = [None] * world
        dist.all_gather_object(hs, (w.get_ipc_handles(), w.get_pool_desc()))
        for peer in range(world):
            if peer != rank:
                w.attach_peer_pool(peer, hs[peer][0], hs[peer][1])
        return w, cpu

    src_cpu = kv_oracle.make_pool(GEOM["L"], GEOM["NB"], GEOM["BS"], GEOM["H"], GEOM["D"], torch.bfloat16, 70)

    def same(w, want):
        return all(kv_oracle.bit_equal(a.cpu(), b) for a, b in zip(w.kv_cache, want))

    # waves two deep, no barrier between them; every landed wave is checked while the next ones run
    plans = _wave_plans(5, seed=21)
    w, _ = mapped(70 if rank == 0 else 0, guard=rank != 0)
    checked = []

    def on_wave_landed(wv):
        for t in plans[wv].transfers:
            got = w.extract_kv_blocks(list(t.dst_blocks)).cpu()
            checked.append(kv_oracle.bit_equal(got, kv_oracle.extract_kv_blocks(src_cpu, list(t.src_blocks))))

    res = w.migrate_waves(plans, WaveLedger(store, "test/waves"), depth=2,
                          on_wave_landed=on_wave_landed if rank == 1 else None)
    results["waves_ok"] = "error" not in res and res["blocks"] == (sum(p.total_blocks() for p in plans) if rank == 1 else 0)
    if rank == 1:
        want = kv_oracle.make_pool(GEOM["L"], GEOM["NB"], GEOM["BS"], GEOM["H"], GEOM["D"], torch.bfloat16, 0, fill="guard")
        for plan in plans:
            for t in plan.transfers:
                kv_oracle.write_kv_blocks(want, list(t.dst_blocks), kv_oracle.extract_kv_blocks(src_cpu, list(t.src_blocks)))
        results["waves_exact"] = same(w, want) and len(checked) == 15 and all(checked) and len(res["wave_ms"]) == 5
    else:
        ledger = WaveLedger(store, "test/waves")
        # every wave that a later wave had to wait for was posted (the last two are covered by the exit agreement)
        results["waves_exact"] = all(ledger.count(wv, 0) == 1 for wv in range(3))
    dist.barrier()

    # the same tables resident on the device
    w2, _ = mapped(70 if rank == 0 else 0, guard=rank != 0)
    tables = [{0: tuple(w2.pool.upload_ids(t) for t in plan.tables(0, 1))} if rank == 1 else {} for plan in plans]
    res = w2.migrate_waves(plans, WaveLedger(store, "test/waves_dev"), depth=2, tables=tables)
    results["waves_device_tables_ok"] = "error" not in res
    if rank == 1:
        results["waves_device_tables_exact"] = same(w2, want)
    dist.barrier()

    # a rank whose peer pool is not mapped: every rank returns the error, nobody hangs, nothing is written
    w3, _ = fresh(70 if rank == 0 else 0, guard=rank != 0)   # no attach_peer_pool on any rank
    res = w3.migrate(MigrationPlan([Transfer("r", 0, 1, (1, 2, 3), (4, 5, 6))]), method="pull")
    results["unmapped_error_on_every_rank_ok"] = "error" in res and res["bytes"] == 0
    res = w3.migrate_waves(plans, WaveLedger(store, "test/waves_err"))
    results["unmapped_waves_error_on_every_rank_ok"] = "error" in res
    bad = MigrationPlan([Transfer("r", 0, 1, (1, 2), (4, GEOM["NB"]))])   # destination id outside the sink's pool
    res = w.migrate(bad, method="pull")
    results["bad_id_error_on_every_rank_ok"] = "error" in res
    if rank == 1:
        guard = kv_oracle.make_pool(GEOM["L"], GEOM["NB"], GEOM["BS"], GEOM["H"], GEOM["D"], torch.bfloat16, 0, fill="guard")
        results["unmapped_nothing_written_exact"] = same(w3, guard)
    dist.barrier()
    return results


def _one_gpu_worker_main(rank, world, port, out_dir):
    """Two processes on cuda:0. gloo carries the host-side agreement (NCCL refuses two ranks on one GPU);
    the pools are shared through CUDA IPC exactly as between GPUs, and the sink's kernel loads from the
    source process's pool. The kernels never wait for one another, so sharing the GPU is safe."""
    import torch.distributed as dist

    from elasticmm_b200.engine.v0 import MigrationPlan, Transfer, TransferMethod, V0KVTransferManager, V0Worker
    from oracle import kv_oracle

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    dist.init_process_group("gloo", rank=rank, world_size=world)

    def fresh(seed, guard):
        cpu = kv_oracle.make_pool(GEOM["L"], GEOM["NB"], GEOM["BS"], GEOM["H"], GEOM["D"], torch.bfloat16, seed,
                                  fill="guard" if guard else "normal")
        w = V0Worker(worker_id=rank, dtype="bfloat16", device=dev, global_rank=rank, world_size=world,
                     kv_cache=[t.to(dev) for t in cpu])
        assert w.init_global_nccl()
        return w, cpu

    results = _waves_and_agreement(rank, world, dev, fresh)

    # plan level through the manager (transfer_many -> migrate -> one direct-load kernel on the sink)
    reqs = _requests(3)
    w, _ = fresh(70 if rank == 0 else 0, guard=rank != 0)
    hs = [None] * world
    dist.all_gather_object(hs, (w.get_ipc_handles(), w.get_pool_desc()))
    w.attach_peer_pool(1 - rank, hs[1 - rank][0], hs[1 - rank][1])
    mgr = V0KVTransferManager(transfer_method=TransferMethod.B200_PEER)
    mgr.register_worker(rank, w, "prefill" if rank == 0 else "decoding")
    plan = MigrationPlan([Transfer(rid, 0, 1, tuple(s), tuple(d)) for rid, s, d in reqs])
    launches = w.ctx.launch_count
    results["transfer_many_ok"] = mgr.transfer_many(plan) and (w.ctx.launch_count - launches) == (1 if rank == 1 else 0)
    if rank == 1:
        src_cpu = kv_oracle.make_pool(GEOM["L"], GEOM["NB"], GEOM["BS"], GEOM["H"], GEOM["D"], torch.bfloat16, 70)
        want = kv_oracle.make_pool(GEOM["L"], GEOM["NB"], GEOM["BS"], GEOM["H"], GEOM["D"], torch.bfloat16, 0, fill="guard")
        for _, s, d in reqs:
            kv_oracle.write_kv_blocks(want, d, kv_oracle.extract_kv_blocks(src_cpu, s))
        results["transfer_many_exact"] = all(kv_oracle.bit_equal(a.cpu(), b) for a, b in zip(w.kv_cache, want))
    dist.barrier()
    # push direction and the request-by-request form of the reference's manager call
    for direction in ("pull", "push"):
        w, _ = fresh(70 if rank == 0 else 0, guard=rank != 0)
        hs = [None] * world
        dist.all_gather_object(hs, (w.get_ipc_handles(), w.get_pool_desc()))
        w.attach_peer_pool(1 - rank, hs[1 - rank][0], hs[1 - rank][1])
        mgr = V0KVTransferManager(transfer_method=TransferMethod.B200_PEER, peer_direction=direction)
        mgr.register_worker(rank, w, "prefill" if rank == 0 else "decoding")
        dist.barrier()
        results[f"per_request_{direction}_ok"] = all(mgr.transfer_kv_cache_sync(rid, 0, 1, s, d) for rid, s, d in reqs)
        dist.barrier()
        if rank == 1:
            results[f"per_request_{direction}_exact"] = all(kv_oracle.bit_equal(a.cpu(), b) for a, b in zip(w.kv_cache, want))
        dist.barrier()
    torch.save(results, os.path.join(out_dir, f"r{rank}.pt"))
    dist.destroy_process_group()


def test_two_ranks_sharing_one_gpu_pull_migration_is_bit_exact():
    import torch.multiprocessing as mp

    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_one_gpu_worker_main, args=(2, _free_port(), d), nprocs=2, join=True)
        r0, r1 = torch.load(os.path.join(d, "r0.pt")), torch.load(os.path.join(d, "r1.pt"))
    assert len(r1) >= 14
    for r in (r0, r1):
        for k, v in r.items():
            assert v is True, f"{k} failed: {r}"


def _one_gpu_four_ranks_main(rank, world, port, out_dir):
    """Four processes on cuda:0: ranks 0, 1 are sources, ranks 2, 3 sinks (the 2 -> 2 rebalancing pattern).
    Every sink pulls from both sources side by side with capped grids, in three waves two deep; then one plan
    through the manager. gloo carries the agreement, CUDA IPC the pools."""
    import torch.distributed as dist

    from elasticmm_b200.engine.v0 import MigrationPlan, TransferMethod, V0KVTransferManager, V0Worker
    from elasticmm_b200.engine.v0.transport import WaveLedger
    from oracle import kv_oracle

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    geom = dict(GEOM, L=6, NB=256)
    is_src = rank < 2

    def pool_cpu(r):
        return kv_oracle.make_pool(geom["L"], geom["NB"], geom["BS"], geom["H"], geom["D"], torch.bfloat16,
                                   80 + r if r < 2 else 0, fill="normal" if r < 2 else "guard")

    def fresh():
        w = V0Worker(worker_id=rank, dtype="bfloat16", device=dev, global_rank=rank, world_size=world,
                     kv_cache=[t.to(dev) for t in pool_cpu(rank)])
        w.init_global_nccl()
        hs = [None] * world
        dist.all_gather_object(hs, (w.get_ipc_handles(), w.get_pool_desc()))
        for peer in range(world):
            if peer != rank:
                w.attach_peer_pool(peer, hs[peer][0], hs[peer][1])
        return w

    g = torch.Generator().manual_seed(17)
    plan = MigrationPlan()
    used = {2: 0, 3: 0}
    dperm = {d: torch.randperm(geom["NB"], generator=g).tolist() for d in (2, 3)}
    for s in (0, 1):
        sperm = torch.randperm(geom["NB"], generator=g).tolist()
        pos = 0
        for r in range(9):
            n = int(torch.randint(3, 25, (1,), generator=g))
            d = 2 + int(torch.randint(0, 2, (1,), generator=g))
            from elasticmm_b200.engine.v0 import Transfer
            plan.add(Transfer(f"s{s}r{r}", s, d, tuple(sperm[pos:pos + n]), tuple(dperm[d][used[d]:used[d] + n])))
            pos += n
            used[d] += n
    plan.validate(lambda r: geom["NB"])

    def expected():
        want = pool_cpu(rank)
        for s in plan.incoming(rank):
            si, di = plan.tables(s, rank)
            kv_oracle.write_kv_blocks(want, di, kv_oracle.extract_kv_blocks(pool_cpu(s), si))
        return want

    results = {}
    w = fresh()
    waves = [MigrationPlan(plan.transfers[k::3]) for k in range(3)]
    res = w.migrate_waves(waves, WaveLedger(dist.distributed_c10d._get_default_store(), "test1x4/waves"), depth=2)
    results["waves_ok"] = "error" not in res and (is_src or len(res["wave_ms"]) == 3)
    if not is_src:
        results["waves_exact"] = all(kv_oracle.bit_equal(a.cpu(), b) for a, b in zip(w.kv_cache, expected()))
    dist.barrier()
    w = fresh()
    mgr = V0KVTransferManager(transfer_method=TransferMethod.B200_PEER)
    mgr.register_worker(rank, w, "prefill" if is_src else "decoding")
    launches = w.ctx.launch_count
    results["plan_ok"] = mgr.transfer_many(plan) and (w.ctx.launch_count - launches) == (0 if is_src else 2)
    if not is_src:
        results["plan_exact"] = all(kv_oracle.bit_equal(a.cpu(), b) for a, b in zip(w.kv_cache, expected()))
    dist.barrier()
    torch.save(results, os.path.join(out_dir, f"r{rank}.pt"))
    dist.destroy_process_group()


def test_four_ranks_sharing_one_gpu_two_sources_two_sinks_is_bit_exact():
    import torch.multiprocessing as mp

    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_one_gpu_four_ranks_main, args=(4, _free_port(), d), nprocs=4, join=True)
        for r in range(4):
            res = torch.load(os.path.join(d, f"r{r}.pt"))
            assert len(res) == (2 if r < 2 else 4) and all(v is True for v in res.values()), f"rank {r}: {res}"


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_migration_is_bit_exact():
    import torch.multiprocessing as mp

    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_worker_main, args=(2, _free_port(), d), nprocs=2, join=True)
        r0, r1 = torch.load(os.path.join(d, "r0.pt")), torch.load(os.path.join(d, "r1.pt"))
    for r in (r0, r1):
        for k, v in r.items():
            if k.endswith("_ok") or k.endswith("_exact"):  # includes *_launches_ok
                assert v, f"{k} failed: {r}"
    assert r1["nccl_bytes"] > 0


def _plan4(seed):
    """Two sources (ranks 0, 1) -> two sinks (ranks 2, 3), unequal request sizes."""
    from elasticmm_b200.engine.v0 import MigrationPlan, Transfer

    g = torch.Generator().manual_seed(seed)
    plan = MigrationPlan()
    used = {2: 0, 3: 0}
    dperm = {d: torch.randperm(GEOM["NB"], generator=g).tolist() for d in (2, 3)}
    for s in (0, 1):
        sperm = torch.randperm(GEOM["NB"], generator=g).tolist()
        pos = 0
        for r in range(6):
            n = int(torch.randint(3, 60, (1,), generator=g))
            d = 2 + int(torch.randint(0, 2, (1,), generator=g))
            plan.add(Transfer(f"s{s}r{r}", s, d, tuple(sperm[pos:pos + n]), tuple(dperm[d][used[d]:used[d] + n])))
            pos += n
            used[d] += n
    return plan


def _worker4_main(rank, world, port, out_dir):
    import torch.distributed as dist

    from elasticmm_b200.engine.v0 import TransferMethod, V0KVTransferManager, V0Worker
    from oracle import kv_oracle

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    plan = _plan4(11)
    plan.validate(lambda r: GEOM["NB"])
    results = {}
    for method in ("pull", "push", "nccl", "alltoall", "waves"):
        is_src = rank < 2
        cpu = kv_oracle.make_pool(GEOM["L"], GEOM["NB"], GEOM["BS"], GEOM["H"], GEOM["D"], torch.bfloat16,
                                  80 + rank if is_src else 0, fill="normal" if is_src else "guard")
        w = V0Worker(worker_id=rank, dtype="bfloat16", device=dev, global_rank=rank, world_size=world,
                     kv_cache=[t.to(dev) for t in cpu])
        w.init_global_nccl()
        if method == "alltoall":
            w.init_native_nccl()
        if method not in ("nccl", "alltoall"):
            hs = [None] * world
            dist.all_gather_object(hs, (w.get_ipc_handles(), w.get_pool_desc()))
            for peer in range(world):
                if peer != rank:
                    w.attach_peer_pool(peer, hs[peer][0], hs[peer][1])
        if method == "pull":   # through the manager, as a role switch would call it
            mgr = V0KVTransferManager(transfer_method=TransferMethod.B200_PEER)
            mgr.register_worker(rank, w, "prefill" if is_src else "decoding")
            results[f"{method}_ok"] = mgr.transfer_many(plan)
        elif method == "waves":  # the plan's transfers as three waves over disjoint blocks, two in flight
            from elasticmm_b200.engine.v0 import MigrationPlan
            from elasticmm_b200.engine.v0.transport import WaveLedger

            ledger = WaveLedger(dist.distributed_c10d._get_default_store(), "test4/waves")
            waves = [MigrationPlan(plan.transfers[k::3]) for k in range(3)]
            results[f"{method}_ok"] = "error" not in w.migrate_waves(waves, ledger, depth=2)
        else:
            results[f"{method}_ok"] = "error" not in w.migrate(plan, method=method)
        dist.barrier()
        if not is_src:
            want = kv_oracle.make_pool(GEOM["L"], GEOM["NB"], GEOM["BS"], GEOM["H"], GEOM["D"], torch.bfloat16, 0,
                                       fill="guard")
            for s in plan.incoming(rank):
                si, di = plan.tables(s, rank)
                src_cpu = kv_oracle.make_pool(GEOM["L"], GEOM["NB"], GEOM["BS"], GEOM["H"], GEOM["D"],
                                              torch.bfloat16, 80 + s)
                kv_oracle.write_kv_blocks(want, di, kv_oracle.extract_kv_blocks(src_cpu, si))
            results[f"{method}_exact"] = all(kv_oracle.bit_equal(a.cpu(), b) for a, b in zip(w.kv_cache, want))
        dist.barrier()
    torch.save(results, os.path.join(out_dir, f"r{rank}.pt"))
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs four GPUs")
def test_four_gpu_two_sources_two_sinks_is_bit_exact():
    import torch.multiprocessing as mp

    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_worker4_main, args=(4, _free_port(), d), nprocs=4, join=True)
        for r in range(4):
            res = torch.load(os.path.join(d, f"r{r}.pt"))
            assert res and all(res.values()), f"rank {r}: {res}"


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("direction", ["pull", "push"])
def test_one_process_two_gpus(direction):
    """One process driving two GPUs: the manager maps the other worker's pool by pointer and moves
    the blocks with one direct kernel (loads or stores over NVLink); p2p_copy and staged_copy too."""
    from elasticmm_b200.engine.v0 import TransferMethod, V0KVTransferManager, V0Worker
    from oracle import kv_oracle

    geom = dict(L=4, NB=64, BS=16, H=4, D=128)
    src_cpu = kv_oracle.make_pool(geom["L"], geom["NB"], geom["BS"], geom["H"], geom["D"], torch.bfloat16, 5)
    g = torch.Generator().manual_seed(1)
    sperm, dperm = torch.randperm(geom["NB"], generator=g).tolist(), torch.randperm(geom["NB"], generator=g).tolist()
    reqs = [(f"r{i}", sperm[i * 12:(i + 1) * 12], dperm[i * 12:(i + 1) * 12]) for i in range(3)]
    for method in (TransferMethod.B200_PEER, TransferMethod.P2P_COPY, TransferMethod.STAGED_COPY):
        dst_cpu = kv_oracle.make_pool(geom["L"], geom["NB"], geom["BS"], geom["H"], geom["D"], torch.bfloat16, 0,
                                      fill="guard")
        src = V0Worker(worker_id=0, dtype="bfloat16", device="cuda:0", kv_cache=[t.to("cuda:0") for t in src_cpu])
        dst = V0Worker(worker_id=1, dtype="bfloat16", device="cuda:1", kv_cache=[t.to("cuda:1") for t in dst_cpu])
        mgr = V0KVTransferManager(transfer_method=method, peer_direction=direction)
        mgr.register_worker(0, src, "prefill")
        mgr.register_worker(1, dst, "decoding")
        for rid, s, d in reqs:
            assert mgr.transfer_kv_cache_sync(rid, 0, 1, s, d), mgr.last_result
            kv_oracle.write_kv_blocks(dst_cpu, d, kv_oracle.extract_kv_blocks(src_cpu, s))
        assert all(kv_oracle.bit_equal(a.cpu(), b) for a, b in zip(dst.kv_cache, dst_cpu)), method
        if method == TransferMethod.B200_PEER:
            # The source pool is rewritten by work still queued on the source GPU's stream when the transfer
            # is requested: the sink's kernel must be ordered after it (no synchronisation in between).
            new_cpu = kv_oracle.make_pool(geom["L"], geom["NB"], geom["BS"], geom["H"], geom["D"], torch.bfloat16, 6)
            staged = [t.to("cuda:0") for t in new_cpu]
            busy = torch.empty(256 << 20, dtype=torch.uint8, device="cuda:0")
            torch.cuda.synchronize()
            with torch.cuda.device("cuda:0"):
                for _ in range(20):
                    busy.add_(1)                              # keeps the source stream busy for a while
                for layer, new in zip(src.kv_cache, staged):
                    layer.copy_(new, non_blocking=True)       # the "prefill" that produces the blocks
            rid, s, d = reqs[0]
            assert mgr.transfer_kv_cache_sync("late", 0, 1, s, d), mgr.last_result
            kv_oracle.write_kv_blocks(dst_cpu, d, kv_oracle.extract_kv_blocks(new_cpu, s))
            assert all(kv_oracle.bit_equal(a.cpu(), b) for a, b in zip(dst.kv_cache, dst_cpu)), "pull not ordered"
