"""Host-side logic (block tables, rank map, manager bookkeeping, planners)
against traces recorded from the reference's own classes."""
import asyncio
import json
import os

import numpy as np
import pytest

import cases
from elasticmm_b200 import EmmError, _lib, compact_plan
from elasticmm_b200.engine.v0 import (MigrationPlan, NCCLCoordinator, Request, Transfer, TransferMethod,
                                      V0BlockManager, V0KVTransferManager, V0VisionBlockManager)
from elasticmm_b200.engine.v0.transport import plan_chunks
from oracle import kv_oracle

HOST = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "host_golden.json")))


def snapshot(bm):
    return {
        "tables": {k: list(v) for k, v in bm.block_table.items()},
        "free_gpu": bm.free_gpu_blocks_list,
        "free_cpu": bm.free_cpu_blocks_list,
        "swapping_gpu": bm.swapping_gpu_blocks_list,
        "swapping_cpu": bm.swapping_cpu_blocks_list,
        "locations": {k: v.value for k, v in bm.request_location.items()},
        "avail_gpu": bm.get_num_avail_gpu_blocks(),
    }


@pytest.mark.parametrize("script", cases.BLOCK_MANAGER_SCRIPTS, ids=lambda s: s["name"])
def test_block_manager_follows_reference_trace(script):
    golden = next(t for t in HOST["block_manager"] if t["name"] == script["name"])["steps"]
    bm = V0BlockManager("prefill", script["gpu_blocks"], script["cpu_blocks"], script["block_size"])
    reqs = {}
    for op, want in zip(script["ops"], golden):
        kind = op[0]
        if kind == "alloc":
            reqs[op[1]] = Request.of_length(op[1], op[2])
            bm.allocate_blocks(reqs[op[1]])
        elif kind == "alloc_n":
            reqs[op[1]] = Request.of_length(op[1], op[2])
            bm.allocate_blocks(reqs[op[1]], op[3])
        elif kind == "grow":
            reqs[op[1]].output_token_ids.extend([0] * op[2])
            bm.append_blocks(reqs[op[1]])
        elif kind == "expand":
            bm.expand_blocks_for_seq_len(op[1], op[2])
        elif kind == "free":
            bm.free_blocks(op[1])
        elif kind == "swap_out":
            bm.swap_out_requests(list(op[1]))
        elif kind == "swap_in":
            bm.swap_in_requests(list(op[1]))
        assert snapshot(bm) == want, f"after {op}"


def test_block_manager_errors_match_reference_behaviour():
    bm = V0BlockManager("decoding", 4, 2, 16)
    bm.allocate_blocks(Request.of_length("a", 48))
    with pytest.raises(AssertionError, match="Not enough free blocks on GPU, requested 2, available 1"):
        bm.allocate_blocks(Request.of_length("b", 32))
    with pytest.raises(AssertionError, match="not allocated"):
        bm.free_blocks("zz")
    with pytest.raises(ValueError, match="not allocated"):
        bm.expand_blocks_for_seq_len("zz", 5)
    assert bm.get_block_table("zz") == []
    assert not bm.can_allocate(Request.of_length("b", 32)) and bm.can_allocate(Request.of_length("b", 16))
    vis = V0VisionBlockManager("encoding", 100, 0, 16)
    r = Request(request_id="v", images=[object(), object()])
    assert vis.get_num_blocks_needed(r) == 2 * 36 and vis.get_num_blocks_needed(Request("t")) == 0


def test_slot_mapping_and_compact_on_block_manager():
    bm = V0BlockManager("decoding", 32, 0, 4)
    lens = {"a": 10, "b": 30, "c": 7, "d": 21, "e": 12}
    for k, n in lens.items():
        bm.allocate_blocks(Request.of_length(k, n))
    bm.free_blocks("b")
    bm.free_blocks("d")
    bm.allocate_blocks(Request.of_length("f", 50))
    assert bm.get_slot_mapping("f", [0, 4, 49]) == kv_oracle.slot_mapping_from_table(
        bm.get_block_table("f"), [0, 4, 49], 4)
    before = {k: list(v) for k, v in bm.block_table.items()}
    flat = [b for v in before.values() for b in v]
    want_new, want_src, want_dst = kv_oracle.compact_plan(flat, 32)
    src, dst = bm.compact()
    assert (src, dst) == (want_src, want_dst)
    after = [b for v in bm.block_table.values() for b in v]
    assert after == want_new and sorted(after) == list(range(len(flat)))
    assert bm.free_gpu_blocks_list == list(range(len(flat), 32))
    assert bm.compact() == ([], [])


def test_compact_plan_library_matches_oracle_and_rejects_bad_tables():
    rng = np.random.default_rng(4)
    for nb, live in [(8192, 4870), (100, 100), (5, 0), (64, 1)]:
        ids = rng.permutation(nb)[:live].tolist()
        new, src, dst = compact_plan(ids, nb)
        o_new, o_src, o_dst = kv_oracle.compact_plan(ids, nb)
        assert new.tolist() == o_new and src.tolist() == o_src and dst.tolist() == o_dst
    with pytest.raises(EmmError) as e:
        compact_plan([1, 2, 2], 8)
    assert e.value.status == _lib.ERR_DUPLICATE
    with pytest.raises(EmmError) as e:
        compact_plan([1, 9], 8)
    assert e.value.status == _lib.ERR_ID_RANGE
    with pytest.raises(EmmError) as e:
        compact_plan([0, 1, 2], 2)
    assert e.value.status == _lib.ERR_LENGTH


def test_coordinator_follows_reference_trace():
    coord = NCCLCoordinator()
    for op, want in zip(cases.COORDINATOR_SCRIPT, HOST["coordinator"]):
        kind = op[0]
        if kind == "register":
            res = coord.register_worker(op[1], op[2])
        elif kind == "unregister":
            res = coord.unregister_worker(op[1], op[2])
        elif kind == "switch":
            res = coord.update_worker_role(op[1], op[2], op[3])
        else:
            res = coord.get_rank(op[1], op[2])
        got = {"result": res, "world": coord.get_world_size(),
               "ranks": sorted([s, w, r] for (s, w), r in coord.get_all_workers().items()),
               "init_method": coord.get_init_method()}
        assert got == want, f"after {op}"
    with pytest.raises(KeyError):
        coord.get_worker(99)


class FakeWorker:
    """CPU stand-in with the two methods the manager's copy path calls."""

    def __init__(self, pool):
        import torch

        self.pool_tensors = pool
        self.device = torch.device("cpu")

    def extract_kv_blocks(self, ids):
        return kv_oracle.extract_kv_blocks(self.pool_tensors, ids)

    def write_kv_blocks(self, ids, data):
        kv_oracle.write_kv_blocks(self.pool_tensors, ids, data)


def test_manager_bookkeeping_follows_reference_trace(monkeypatch):
    import hashlib
    import torch

    monkeypatch.setattr(torch.cuda, "synchronize", lambda *a, **k: None)
    golden = HOST["manager"]
    case = cases.MANAGER_CASE
    src_pool, dst_pool = cases.build_pools(case)
    calls = []
    mgr = V0KVTransferManager(transfer_method=TransferMethod.P2P_COPY,
                              metrics_callback=lambda transfer_time_sec, num_blocks: calls.append(num_blocks))
    mgr.register_worker(0, FakeWorker(src_pool), "prefill")
    mgr.register_worker(1, FakeWorker(dst_pool), "decoding")
    results = [asyncio.run(mgr.transfer_kv_cache(rid, s, d, si, di))
               for rid, si, di, s, d in case["transfers"]]
    assert results == golden["results"]
    assert calls == golden["callback_blocks"]
    assert mgr.get_stats()["transfer_count"] == golden["transfer_count"]
    mgr.update_worker_stage(0, "DECODING")
    assert mgr.rank_to_stage[0] == golden["stage_after_switch"]
    whole = torch.stack(dst_pool, 0)
    assert hashlib.sha256(kv_oracle.bits(whole).numpy().tobytes()).hexdigest() == golden["dst_pool_sha256"]
    assert set(golden["methods"]) <= {m.value for m in TransferMethod}
    mgr.unregister_worker(0)
    assert 0 not in mgr.worker_registry
    assert not asyncio.run(mgr.transfer_kv_cache("x", 0, 1, [1], [2]))
    assert not asyncio.run(mgr.transfer_kv_cache("y", 1, 1, [1, 2], [2]))  # count mismatch
    mgr.reset_stats()
    assert mgr.get_stats() == {"transfer_count": 0, "total_transfer_time": 0.0,
                               "total_bytes_transferred": 0, "avg_transfer_time": 0.0}


def test_chunk_schedule():
    page = 16 * 4 * 128 * 2
    assert plan_chunks(28, 69, page) == [(b, 14) for b in (0, 14)]          # small request: two halves
    big = plan_chunks(28, 8900, page)
    assert big == [(l, 1) for l in range(28)]                                 # one layer per message
    assert plan_chunks(1, 5, page) == [(0, 1)] and plan_chunks(4, 0, page) == []
    for L, n in [(32, 1), (40, 300), (80, 7), (5, 100000)]:
        ch = plan_chunks(L, n, page)
        assert ch[0][0] == 0 and sum(c for _, c in ch) == L
        assert all(a[0] + a[1] == b[0] for a, b in zip(ch, ch[1:]))
        assert len(ch) >= 2
        tp = plan_chunks(L, n, page, target_bytes=1 << 30, taper=True)      # short first and last chunk
        assert tp[0][0] == 0 and sum(c for _, c in tp) == L and all(c > 0 for _, c in tp)
        assert all(a[0] + a[1] == b[0] for a, b in zip(tp, tp[1:]))
        if max(c for _, c in tp) > 1:
            assert tp[0][1] == 1 and tp[-1][1] == 1


def test_migration_plan_grouping_and_order():
    plan = MigrationPlan()
    sinks = [2, 3, 4, 5, 6, 7]
    for i in range(24):
        src = i % 2
        dst = sinks[(i * 5 + 1) % 6]
        plan.add(Transfer(f"r{i}", src, dst, (i, i + 100), (2 * i, 2 * i + 1)))
    assert plan.total_blocks() == 48
    s, d = plan.tables(0, plan.outgoing(0)[0])
    assert len(s) == len(d) and len(s) % 2 == 0
    order = plan.ordered_pairs()
    assert sorted(order) == plan.pairs()
    # in every step of the rotation the two sources address different sinks
    by_src = {0: [d for s, d in order if s == 0], 1: [d for s, d in order if s == 1]}
    full = MigrationPlan([Transfer(f"q{s}{d}", s, d, (1,), (1,)) for s in (0, 1) for d in sinks])
    o = full.ordered_pairs()
    for step in range(6):
        a, b = o[2 * step], o[2 * step + 1]
        assert a[0] != b[0] and a[1] != b[1]
    with pytest.raises(ValueError, match="Block count mismatch"):
        Transfer("bad", 0, 1, (1, 2), (3,))
    with pytest.raises(ValueError, match="both"):
        plan.add(Transfer("self", 1, 1, (1,), (2,)))
    plan.validate(lambda r: 1000)
    with pytest.raises(ValueError, match="outside"):
        plan.validate(lambda r: 50)
    dup = MigrationPlan([Transfer("a", 0, 2, (1,), (5,)), Transfer("b", 1, 2, (1,), (5,))])
    with pytest.raises(ValueError, match="assigned twice"):
        dup.validate(lambda r: 10)


def test_metrics_feed_the_gain_cost_file(tmp_path):
    """KV-transfer samples -> the keys the reference's calibration writes and GainCostConfig reads."""
    from elasticmm_b200.engine.v0 import KVTransferMetrics

    m = KVTransferMetrics("decoding", block_bytes=1 << 20)
    assert m.gain_cost_params() == {} and "kv_transfer" not in m.get_stats()
    for t, n in [(0.002, 15), (0.004, 45), (0.003, 30)]:
        m.record_kv_transfer(transfer_time_sec=t, num_blocks=n)
    kv = m.get_stats()["kv_transfer"]
    assert kv["avg_time_sec"] == pytest.approx(0.003) and kv["avg_blocks"] == 30
    assert kv["bandwidth_blocks_per_sec"] == pytest.approx(90 / 0.009)
    assert kv["bandwidth_gb_per_sec"] == pytest.approx(90 * (1 << 20) / 0.009 / 1e9)
    path = tmp_path / "gain_cost_params.json"
    path.write_text(json.dumps({"preemption_penalty": 0.004, "migration_cost": 0.1}))
    merged = m.update_gain_cost_file(str(path))
    assert merged == json.loads(path.read_text())
    assert merged["migration_cost"] == pytest.approx(0.003) and merged["preemption_penalty"] == 0.004
    assert merged["kv_transfer_bandwidth"] == pytest.approx(10000.0)


def test_pull_and_push_orders_spread_the_first_flows():
    sinks = [2, 3, 4, 5, 6, 7]
    plan = MigrationPlan([Transfer(f"q{s}{d}", s, d, (1,), (1,)) for s in (0, 1) for d in sinks])
    firsts = [plan.pull_order(d)[0] for d in sinks]
    assert firsts.count(0) == 3 and firsts.count(1) == 3            # sources loaded evenly from the start
    assert all(sorted(plan.pull_order(d)) == [0, 1] for d in sinks)
    assert plan.push_order(0)[0] != plan.push_order(1)[0]            # sources start at different sinks
    assert sorted(plan.push_order(0)) == sinks and plan.pull_order(0) == [] and plan.push_order(5) == []
    lone = MigrationPlan([Transfer("a", 0, 1, (1,), (2,))])
    assert lone.pull_order(1) == [0] and lone.push_order(0) == [1]


def test_manager_batching_merges_a_pair_into_one_transfer():
    """enable_batching: requests of one (source, sink) pair are queued and moved as one merged table."""

    class Recorder:
        def __init__(self):
            self.calls = []
            self.peer_pools = {0: object()}
            self.device = None

        def p2p_pull_kv(self, src_rank, src_blocks, dst_blocks):
            self.calls.append((src_rank, list(src_blocks), list(dst_blocks)))
            return {"bytes": 100 * len(src_blocks), "blocks": len(src_blocks)}

    sink = Recorder()
    seen = []
    mgr = V0KVTransferManager(TransferMethod.B200_PEER, enable_batching=True, batch_size=3, batch_timeout=3600.0,
                              metrics_callback=lambda transfer_time_sec, num_blocks: seen.append(num_blocks))
    mgr.register_worker(1, sink, "decoding")
    import torch

    real_sync = torch.cuda.synchronize
    torch.cuda.synchronize = lambda *a, **k: None
    sink.ctx = type("C", (), {"status": staticmethod(lambda: (0, 0))})()
    try:
        assert mgr.transfer_kv_cache_sync("a", 0, 1, [1, 2], [7, 8]) and sink.calls == []
        assert mgr.transfer_kv_cache_sync("b", 0, 1, [3], [9]) and sink.calls == []
        assert mgr.transfer_kv_cache_sync("c", 0, 1, [4, 5], [0, 1])                 # third request: flush
        assert sink.calls == [(0, [1, 2, 3, 4, 5], [7, 8, 9, 0, 1])]
        assert mgr.transfer_kv_cache_sync("d", 0, 1, [6], [2]) and len(sink.calls) == 1  # queued again
        assert not mgr.transfer_kv_cache_sync("bad", 0, 1, [6, 7], [2])               # count mismatch refused
        assert mgr.flush() and sink.calls[-1] == (0, [6], [2])
        assert mgr.flush() and len(sink.calls) == 2                                    # nothing left
    finally:
        torch.cuda.synchronize = real_sync
    assert seen == [5, 1]                       # one metrics sample per merged transfer
    assert mgr.get_stats()["transfer_count"] == 1   # the first (cold) merged transfer is not averaged


def test_kv_cache_config_mirrors_the_reference_fields():
    from elasticmm_b200.engine.v0 import DEFAULT_V0_KV_CONFIG, V0KVCacheConfig
    d = DEFAULT_V0_KV_CONFIG
    d.validate()
    # defaults of the shared fields are the reference's (elasticmm/engine/v0/config.py:25-35)
    assert (d.block_size, d.max_num_gpu_blocks, d.max_num_cpu_blocks, d.dtype, d.kv_transfer_method) == \
        (16, 5000, 1000, "float16", "p2p_copy")
    assert d.transfer_method is TransferMethod.P2P_COPY
    # a dictionary written for the reference's V0EngineConfig loads; its other fields are ignored
    ref_style = {"model_path": "m", "num_prefill_workers": 4, "block_size": 32, "max_num_gpu_blocks": 100,
                 "max_num_cpu_blocks": 0, "dtype": "bfloat16", "tensor_parallel_size": 1,
                 "gpu_memory_utilization": 0.9, "kv_transfer_method": "nccl"}
    c = V0KVCacheConfig.from_dict(ref_style)
    c.validate()
    assert c.block_size == 32 and c.transfer_method is TransferMethod.NCCL
    assert V0KVCacheConfig.from_dict(c.to_dict()) == c
    with pytest.raises(TypeError, match="unexpected configuration keys"):
        V0KVCacheConfig.from_dict({"blok_size": 16})
    for bad in (dict(kv_transfer_method="rdma"), dict(block_size=0), dict(layout="dhn"), dict(dtype="int4"),
                dict(peer_direction="both")):
        with pytest.raises(AssertionError):
            V0KVCacheConfig(**bad).validate()
    V0KVCacheConfig(kv_transfer_method="b200_peer", peer_direction="push").validate()
    # sizes: Llama-7B shape, 16-token blocks, fp16 -> 128 KiB pages, 8 MiB per block id
    assert d.page_bytes == 128 * 1024 and d.block_bytes == 8 << 20
    assert d.pool_bytes(8192) == 64 << 30
    assert d.blocks_for_bytes(10 << 30) == 1280 and d.blocks_for_bytes(1 << 50) == 5000
    assert d.blocks_for_tokens(2048) == 128 and d.blocks_for_tokens(2049) == 129
