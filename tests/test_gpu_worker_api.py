"""The engine/v0 call surface on a GPU: worker methods, manager methods, swap."""
import asyncio

import pytest
import torch

from elasticmm_b200 import get_context
from elasticmm_b200.engine.v0 import (EngineStage, KVTransferMetrics, Request, TransferMethod, V0BlockManager, V0KVTransferManager, V0Worker)
from gpu_util import assert_clean, configure, pools_equal, to_gpu
from oracle import kv_oracle

pytestmark = pytest.mark.gpu
GEOM = dict(L=4, NB=64, BS=16, H=4, D=128)


def make_worker(seed, guard=False, dtype=torch.bfloat16, **kw):
    cpu = kv_oracle.make_pool(GEOM["L"], GEOM["NB"], GEOM["BS"], GEOM["H"], GEOM["D"], dtype, seed,
                              fill="guard" if guard else "normal")
    w = V0Worker(dtype=str(dtype).split(".")[-1], device="cuda:0", kv_cache=to_gpu(cpu), **kw)
    return w, cpu


def test_extract_write_layout_like_the_reference():
    configure(get_context(0))
    src, src_cpu = make_worker(1)
    dst, dst_cpu = make_worker(0, guard=True)
    assert src.get_kv_cache_layout() == {"num_layers": 4, "block_size": 16, "num_heads": 4, "head_size": 128,
                                         "dtype": "bfloat16"}
    bm_src = V0BlockManager("prefill", GEOM["NB"], 0, GEOM["BS"])
    bm_dst = V0BlockManager("decoding", GEOM["NB"], 0, GEOM["BS"])
    for i, tokens in enumerate([234, 17, 600]):
        r = Request.of_length(f"req{i}", tokens)
        bm_src.allocate_blocks(r)
        bm_dst.allocate_blocks(Request.of_length("pad", 16 * (i + 1)))  # shifts the sink's ids
        bm_dst.allocate_blocks(r)
        s, d = bm_src.get_block_table(r.request_id), bm_dst.get_block_table(r.request_id)
        data = src.extract_kv_blocks(s)
        assert data.shape == (4, 2, len(s), 16, 4, 128) and data.is_contiguous()
        dst.write_kv_blocks(d, data)
        kv_oracle.write_kv_blocks(dst_cpu, d, kv_oracle.extract_kv_blocks(src_cpu, s))
        bm_dst.free_blocks("pad")
    assert_clean(src.ctx)
    assert pools_equal(dst.kv_cache, dst_cpu)
    with pytest.raises(AssertionError, match="Block count mismatch"):
        dst.write_kv_blocks([1, 2, 3], data)
    empty = V0Worker(device="cuda:0")
    assert empty.get_kv_cache_layout() == {}
    with pytest.raises(RuntimeError, match="KV cache not initialized"):
        empty.extract_kv_blocks([0])
    assert empty.p2p_send_kv(1, [0]) == {"error": "Global NCCL not initialized", "bytes": 0, "blocks": 0}
    assert empty.p2p_recv_kv(1, [0])["error"] == "Global NCCL not initialized"
    with pytest.raises(RuntimeError, match="Global NCCL not initialized"):
        empty.p2p_coordinated_transfer_kv(None, 0, [1], [1])
    assert empty.get_global_rank() == -1 and empty.init_global_nccl() is False
    assert empty.switch_role(EngineStage.DECODING) and empty.get_stage() == EngineStage.DECODING


@pytest.mark.parametrize("method", [TransferMethod.P2P_COPY, TransferMethod.B200_PEER, TransferMethod.CUDA_IPC,
                                    TransferMethod.STAGED_COPY])
def test_transfer_manager_in_process(method):
    src, src_cpu = make_worker(2)
    dst, dst_cpu = make_worker(0, guard=True)
    metrics = KVTransferMetrics("decoding", block_bytes=src.pool.block_bytes())
    mgr = V0KVTransferManager(transfer_method=method, metrics_callback=metrics.record_kv_transfer)
    mgr.register_worker(0, src, "prefill")
    mgr.register_worker(1, dst, "decoding")
    g = torch.Generator().manual_seed(4)
    sperm, dperm = torch.randperm(64, generator=g).tolist(), torch.randperm(64, generator=g).tolist()
    pos = 0
    for i, n in enumerate([15, 1, 30, 7]):
        s, d = sperm[pos:pos + n], dperm[pos:pos + n]
        assert asyncio.run(mgr.transfer_kv_cache(f"r{i}", 0, 1, s, d))
        kv_oracle.write_kv_blocks(dst_cpu, d, kv_oracle.extract_kv_blocks(src_cpu, s))
        pos += n
    assert pools_equal(dst.kv_cache, dst_cpu)
    assert not asyncio.run(mgr.transfer_kv_cache("bad", 0, 1, [1, 2], [3]))
    assert not asyncio.run(mgr.transfer_kv_cache("bad", 0, 1, [1, 999], [3, 4]))
    assert not asyncio.run(mgr.transfer_kv_cache("bad", 7, 8, [1], [3]))
    stats = mgr.get_stats()
    assert stats["transfer_count"] == (4 if method == TransferMethod.P2P_COPY else 3)
    kv = metrics.get_stats()["kv_transfer"]
    assert kv["avg_blocks"] == 53 / 4 and kv["bandwidth_blocks_per_sec"] > 0 and kv["bandwidth_gb_per_sec"] > 0
    assert pools_equal(dst.kv_cache, dst_cpu)  # failed transfers wrote nothing


def test_swap_out_and_in_through_pinned_host_pool():
    w, cpu = make_worker(6)
    host_cpu = kv_oracle.make_pool(GEOM["L"], 32, GEOM["BS"], GEOM["H"], GEOM["D"], torch.bfloat16, 0, fill="guard")
    w.bind_kv_swap([t.clone().pin_memory() for t in host_cpu])
    bm = V0BlockManager("decoding", GEOM["NB"], 32, GEOM["BS"],
                        engine_remote_call_all_workers_async=lambda name, *a: getattr(w, name)(*a))
    reqs = [Request.of_length(f"r{i}", n) for i, n in enumerate([100, 40, 250])]
    for r in reqs:
        bm.allocate_blocks(r)
    before = {r.request_id: kv_oracle.extract_kv_blocks(cpu, bm.get_block_table(r.request_id)) for r in reqs}
    src_ids, tgt_ids = bm.swap_out_requests(["r0", "r2"])
    w.wait_for_all_swap_out()
    kv_oracle.swap_blocks(cpu, host_cpu, src_ids, tgt_ids, is_swap_in=False)
    assert all(kv_oracle.bit_equal(a, b) for a, b in zip(w.kv_swap, host_cpu))
    # overwrite the vacated GPU blocks, then bring the requests back to new ids
    junk = Request.of_length("junk", 16 * bm.get_num_avail_gpu_blocks())
    bm.allocate_blocks(junk)
    w.write_kv_blocks(bm.get_block_table("junk"),
                      torch.zeros((GEOM["L"], 2, len(bm.get_block_table("junk")), 16, 4, 128),
                                  dtype=torch.bfloat16, device="cuda"))
    bm.free_blocks("junk")
    bm.swap_in_requests(["r2", "r0"])
    w.wait_for_all_swap_in()
    assert_clean(w.ctx)
    for r in reqs:
        assert kv_oracle.bit_equal(w.extract_kv_blocks(bm.get_block_table(r.request_id)).cpu(), before[r.request_id])
    w.clear_request_resource("r0")
    assert "r0" not in w.swap_event_table


def test_reshape_and_cache_via_worker_and_block_manager_slots():
    w, cpu = make_worker(8)
    bm = V0BlockManager("decoding", GEOM["NB"], 0, GEOM["BS"])
    lens = [33, 16, 200, 1]
    reqs = [Request.of_length(f"r{i}", n) for i, n in enumerate(lens)]
    for r in reqs:
        bm.allocate_blocks(r)
    # one decode step: each request appends the token at position len-1; one padded entry
    slots = [bm.get_slot_mapping(r.request_id, [n - 1])[0] for r, n in zip(reqs, lens)] + [-1]
    slots_t = torch.tensor(slots)
    g = torch.Generator().manual_seed(3)
    key = torch.randn(GEOM["L"], 5, GEOM["H"], GEOM["D"], generator=g).to(torch.bfloat16)
    value = torch.randn(GEOM["L"], 5, GEOM["H"], GEOM["D"], generator=g).to(torch.bfloat16)
    for l in range(GEOM["L"]):
        w.reshape_and_cache(key[l].cuda(), value[l].cuda(), slots_t.cuda(), l)
        kv_oracle.reshape_and_cache(key[l], value[l], cpu[l], slots_t)
    assert_clean(w.ctx)
    assert pools_equal(w.kv_cache, cpu)
    w2, cpu2 = make_worker(8)
    w2.reshape_and_cache_all_layers(key.cuda(), value.cuda(), slots_t.cuda())
    assert pools_equal(w2.kv_cache, cpu)


@pytest.mark.parametrize("method", [TransferMethod.P2P_COPY, TransferMethod.B200_PEER])
def test_manager_batching_on_gpu(method):
    """enable_batching: queued requests of a pair move together (one launch per direction for
    p2p_copy, one merged direct copy for b200_peer) and land exactly where the serial calls put them."""
    src, src_cpu = make_worker(3)
    dst, dst_cpu = make_worker(0, guard=True)
    mgr = V0KVTransferManager(transfer_method=method, enable_batching=True, batch_size=4, batch_timeout=3600.0)
    mgr.register_worker(0, src, "prefill")
    mgr.register_worker(1, dst, "decoding")
    g = torch.Generator().manual_seed(6)
    sperm, dperm = torch.randperm(64, generator=g).tolist(), torch.randperm(64, generator=g).tolist()
    pos = 0
    launches = src.ctx.launch_count
    for i, n in enumerate([5, 1, 9, 3, 7, 2]):
        s, d = sperm[pos:pos + n], dperm[pos:pos + n]
        assert asyncio.run(mgr.transfer_kv_cache(f"r{i}", 0, 1, s, d))
        kv_oracle.write_kv_blocks(dst_cpu, d, kv_oracle.extract_kv_blocks(src_cpu, s))
        pos += n
    assert src.ctx.launch_count - launches == (2 if method == TransferMethod.P2P_COPY else 1)  # first four flushed
    assert mgr.flush()                                                                          # the last two
    assert src.ctx.launch_count - launches == (4 if method == TransferMethod.P2P_COPY else 2)
    assert pools_equal(dst.kv_cache, dst_cpu)


@pytest.mark.parametrize("layout", ["nhd", "hnd"])
def test_worker_and_manager_from_config(layout):
    from elasticmm_b200.engine.v0 import V0KVCacheConfig
    cfg = V0KVCacheConfig(block_size=16, max_num_gpu_blocks=48, max_num_cpu_blocks=8, dtype="bfloat16",
                          kv_transfer_method="b200_peer", num_layers=3, num_kv_heads=4, head_size=64,
                          layout=layout)
    src = V0Worker.from_config(cfg, worker_id=0, stage=EngineStage.PREFILL, device="cuda:0", global_rank=0)
    dst = V0Worker.from_config(cfg, worker_id=1, stage=EngineStage.DECODING, device="cuda:0", global_rank=1)
    assert len(src.kv_cache) == 3 and tuple(src.kv_cache[0].shape) == (2, 48, 16, 4, 64)
    assert src.kv_cache[0].is_contiguous() == (layout == "nhd")
    assert len(src.kv_swap) == 3 and tuple(src.kv_swap[0].shape) == (2, 8, 16, 4, 64)
    assert sum(t.numel() * t.element_size() for t in src.kv_cache) == cfg.pool_bytes()
    src_cpu = kv_oracle.make_pool(3, 48, 16, 4, 64, torch.bfloat16, 21)
    dst_cpu = kv_oracle.make_pool(3, 48, 16, 4, 64, torch.bfloat16, 0, fill="guard")
    for w, cpu in ((src, src_cpu), (dst, dst_cpu)):
        for t, c in zip(w.kv_cache, cpu):
            t.copy_(c)
    # append through the slot mapping, then move the request with the configured method
    g = torch.Generator().manual_seed(5)
    key = torch.randn(20, 4, 64, generator=g).to(torch.bfloat16)
    value = torch.randn(20, 4, 64, generator=g).to(torch.bfloat16)
    table = [7, 40]
    slots = torch.tensor(kv_oracle.slot_mapping_from_table(table, range(20), 16))
    for layer in range(3):
        src.reshape_and_cache(key.cuda(), value.cuda(), slots.cuda(), layer)
        kv_oracle.reshape_and_cache(key, value, src_cpu[layer], slots)
    mgr = V0KVTransferManager.from_config(cfg)
    assert mgr.transfer_method == TransferMethod.B200_PEER and mgr.peer_direction == "pull"
    mgr.register_worker(0, src, "prefill")
    mgr.register_worker(1, dst, "decoding")
    assert mgr.transfer_kv_cache_sync("r", 0, 1, table, [3, 4])
    kv_oracle.copy_blocks(src_cpu, dst_cpu, table, [3, 4])
    # and a swap out of the sink's new blocks into its pinned pool
    dst.swap_blocks(["r"], [3, 4], [0, 5], False)
    dst.wait_for_all_swap_out()
    assert_clean(src.ctx)
    assert pools_equal(src.kv_cache, src_cpu) and pools_equal(dst.kv_cache, dst_cpu)
    for layer in range(3):
        assert kv_oracle.bit_equal(dst.kv_swap[layer][:, [0, 5]], dst_cpu[layer][:, [3, 4]])
