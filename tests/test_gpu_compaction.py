"""Eviction + defragmentation: host plan, one block-copy launch, rewritten tables."""
import pytest
import torch

from elasticmm_b200 import get_context
from elasticmm_b200.engine.v0 import Request, V0BlockManager, V0Worker
from gpu_util import BULK_DEFAULT, LDG_DEFAULT, assert_clean, configure, pools_equal, to_gpu, vid
from oracle import kv_oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("opts", [BULK_DEFAULT, LDG_DEFAULT], ids=vid)
def test_evict_then_compact_matches_oracle(opts):
    """70B-shaped pages (8 KV heads, bf16) on a reduced pool: fill to ~85 %,
    evict the 30 % least recently used requests, compact."""
    ctx = get_context(0)
    configure(ctx, **opts)
    L, NB, BS, H, D = 5, 160, 16, 8, 128
    g = torch.Generator().manual_seed(5)
    pool_cpu = kv_oracle.make_pool(L, NB, BS, H, D, torch.bfloat16, 9)
    worker = V0Worker(dtype="bfloat16", device="cuda:0", kv_cache=to_gpu(pool_cpu))
    bm = V0BlockManager("decoding", NB, 0, BS)
    # a randomly permuted free list stands for a pool fragmented by earlier traffic
    perm = torch.randperm(NB, generator=g).tolist()
    bm._free[next(iter(bm._free))].clear()
    bm._free[next(iter(bm._free))].extend(perm)
    stamps = {}
    i = 0
    while bm.get_num_avail_gpu_blocks() > 0.15 * NB:
        tokens = int(torch.randint(16, 400, (1,), generator=g))
        r = Request.of_length(f"r{i}", tokens)
        if not bm.can_allocate(r):
            break
        bm.allocate_blocks(r)
        stamps[r.request_id] = float(torch.rand(1, generator=g))
        i += 1
    victims = sorted(stamps, key=stamps.get)[: max(1, int(0.3 * len(stamps)))]
    for rid in victims:
        bm.free_blocks(rid)
    survivors = {rid: list(t) for rid, t in bm.block_table.items()}
    contents = {rid: kv_oracle.extract_kv_blocks(pool_cpu, t) for rid, t in survivors.items()}
    flat = [b for t in survivors.values() for b in t]
    want_new, want_src, want_dst = kv_oracle.compact_plan(flat, NB)
    move_src, move_dst = bm.compact()
    assert (move_src, move_dst) == (want_src, want_dst) and len(move_src) > 0
    res = worker.compact_blocks(move_src, move_dst)
    assert res["blocks"] == len(move_src) and res["bytes"] == len(move_src) * 2 * L * BS * H * D * 2
    assert_clean(ctx)
    kv_oracle.compact(pool_cpu, want_src, want_dst)
    assert pools_equal(worker.kv_cache, pool_cpu)
    n_live = len(flat)
    for rid, table in bm.block_table.items():
        assert all(b < n_live for b in table)
        assert kv_oracle.bit_equal(worker.extract_kv_blocks(table).cpu(), contents[rid])
    assert bm.compact() == ([], [])
    configure(ctx)
