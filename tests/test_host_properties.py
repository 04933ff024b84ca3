"""Property tests of the host-side logic (no GPU): compaction plans, chunk
schedules, migration-plan orders, block-manager invariants and the staged
transport's buffer-reuse protocol, on inputs drawn by hypothesis."""
import numpy as np
import pytest
from hypothesis import given, settings, strategies as st

from elasticmm_b200 import EmmError, compact_plan
from elasticmm_b200.engine.v0 import MigrationPlan, Request, Transfer, V0BlockManager
from elasticmm_b200.engine.v0.transport import pipelined_recv, pipelined_send, plan_chunks
from oracle import kv_oracle

FAST = settings(max_examples=150, deadline=None)


@st.composite
def live_tables(draw):
    num_blocks = draw(st.integers(1, 200))
    n_live = draw(st.integers(0, num_blocks))
    ids = draw(st.permutations(range(num_blocks)))[:n_live]
    return list(ids), num_blocks


@FAST
@given(live_tables())
def test_compact_plan_is_minimal_disjoint_and_equals_the_oracle(case):
    ids, num_blocks = case
    new_ids, src, dst = compact_plan(ids, num_blocks)
    want_new, want_src, want_dst = kv_oracle.compact_plan(ids, num_blocks)
    assert (new_ids.tolist(), src.tolist(), dst.tolist()) == (want_new, want_src, want_dst)
    n = len(ids)
    assert sorted(new_ids.tolist()) == list(range(n))                 # dense prefix, each id once
    assert len(src) == sum(1 for b in ids if b >= n)                  # only blocks outside the prefix move
    assert not set(src.tolist()) & set(dst.tolist())                  # one launch may run it in place
    assert all(a == b for a, b in zip(ids, new_ids) if a < n)          # blocks inside the prefix stay put
    again, src2, _ = compact_plan(new_ids, num_blocks)                # idempotent
    assert again.tolist() == new_ids.tolist() and len(src2) == 0


@FAST
@given(st.lists(st.integers(-3, 40), min_size=1, max_size=30), st.integers(1, 32))
def test_compact_plan_refuses_what_is_not_a_table(ids, num_blocks):
    ok = len(set(ids)) == len(ids) and all(0 <= b < num_blocks for b in ids)
    if ok:
        compact_plan(ids, num_blocks)
    else:
        with pytest.raises(EmmError):
            compact_plan(ids, num_blocks)


@FAST
@given(st.integers(1, 96), st.integers(1, 5000), st.sampled_from([120, 4096, 16384, 131072, 163840]),
       st.sampled_from([1 << 20, 16 << 20, 64 << 20]))
def test_chunk_schedule_covers_the_layers_once_and_overlaps(num_layers, n_blocks, page, target):
    chunks = plan_chunks(num_layers, n_blocks, page, target)
    assert [b for b, _ in chunks] == list(np.cumsum([0] + [c for _, c in chunks[:-1]]))
    assert sum(c for _, c in chunks) == num_layers and all(c >= 1 for _, c in chunks)
    if num_layers >= 2:
        assert len(chunks) >= 2                                       # packing can overlap the wire
    layer_bytes = 2 * n_blocks * page
    assert all(c == 1 or c * layer_bytes <= target for _, c in chunks)


class _Work:
    def __init__(self, log, what):
        self.log, self.what, self.done = log, what, False

    def wait(self):
        self.done = True
        self.log.append(("done", self.what))


@FAST
@given(st.integers(1, 40), st.integers(1, 9), st.integers(1, 4))
def test_staged_pipeline_never_reuses_a_slot_still_on_the_wire(num_layers, per_chunk, depth):
    chunks = [(b, min(per_chunk, num_layers - b)) for b in range(0, num_layers, per_chunk)]
    log, in_flight = [], {}

    def buffer_for(slot, count):
        return slot

    def pack(slot, begin, count):
        assert slot not in in_flight or in_flight[slot].done, "packed over a message still being sent"
        log.append(("pack", begin, count))

    def isend(slot):
        in_flight[slot] = _Work(log, ("send", slot))
        return in_flight[slot]

    assert pipelined_send(chunks, buffer_for, pack, isend, depth=depth) == len(chunks)
    assert [e[1:] for e in log if e[0] == "pack"] == chunks
    assert all(w.done for w in in_flight.values())

    log.clear()
    landed, posted_now = {}, {}

    def irecv(slot):
        assert slot not in posted_now, "posted a receive into a slot not yet unpacked"
        posted_now[slot] = True
        return _Work(log, ("recv", slot))

    def unpack(slot, begin, count):
        posted_now.pop(slot)
        landed[begin] = count

    assert pipelined_recv(chunks, buffer_for, irecv, unpack, depth=depth) == len(chunks)
    assert sorted(landed.items()) == chunks and not posted_now


@st.composite
def plans(draw):
    n_src = draw(st.integers(1, 4))
    n_dst = draw(st.integers(1, 6))
    sources, sinks = list(range(n_src)), list(range(n_src, n_src + n_dst))
    transfers = []
    for k in range(draw(st.integers(1, 24))):
        n = draw(st.integers(0, 5))
        transfers.append(Transfer(f"r{k}", draw(st.sampled_from(sources)), draw(st.sampled_from(sinks)),
                                  tuple(range(k * 8, k * 8 + n)), tuple(range(k * 8 + 1, k * 8 + 1 + n))))
    return MigrationPlan(transfers)


@FAST
@given(plans())
def test_plan_orders_are_permutations_every_rank_agrees_on(plan):
    pairs = plan.pairs()
    assert sorted(plan.ordered_pairs()) == pairs
    # one global order restricted to a rank gives that rank's own order: no circular wait
    order = {p: k for k, p in enumerate(plan.ordered_pairs())}
    ranks = {r for p in pairs for r in p}
    for r in ranks:
        mine = [p for p in plan.ordered_pairs() if r in p]
        assert [order[p] for p in mine] == sorted(order[p] for p in mine)
        assert sorted(plan.pull_order(r)) == sorted(plan.incoming(r))
        assert sorted(plan.push_order(r)) == sorted(plan.outgoing(r))
    # tables hold every request's blocks once, in plan order
    assert sum(len(plan.tables(s, d)[0]) for s, d in pairs) == plan.total_blocks()
    for s, d in pairs:
        src, dst = plan.tables(s, d)
        want = [b for t in plan.transfers if (t.src_rank, t.dst_rank) == (s, d) for b in t.src_blocks]
        assert src == want and len(dst) == len(src)
        a, b = plan.tables_np(s, d)
        assert a.tolist() == src and b.tolist() == dst and a.dtype == np.int64
    plan.validate(lambda rank: 10_000)
    if plan.total_blocks():
        with pytest.raises(ValueError, match="outside"):
            plan.validate(lambda rank: 0)


@FAST
@given(st.lists(st.tuples(st.sampled_from(["alloc", "grow", "free", "compact"]), st.integers(0, 7),
                          st.integers(1, 70)), min_size=1, max_size=40))
def test_block_manager_never_loses_or_shares_a_block(ops):
    nb, bs = 24, 16
    bm = V0BlockManager("decoding", nb, 0, bs)
    lens = {}
    for op, k, tokens in ops:
        rid = f"r{k}"
        if op == "alloc" and rid not in lens:
            r = Request.of_length(rid, tokens)
            if bm.can_allocate(r):
                bm.allocate_blocks(r)
                lens[rid] = tokens
        elif op == "grow" and rid in lens:
            need = -(-(lens[rid] + tokens) // bs) - bm.get_allocated_num_blocks(rid)
            if need <= bm.get_num_avail_gpu_blocks():
                lens[rid] += tokens
                bm.expand_blocks_for_seq_len(rid, lens[rid])
        elif op == "free" and rid in lens:
            bm.free_blocks(rid)
            del lens[rid]
        elif op == "compact":
            before = {r: bm.get_block_table(r)[:] for r in lens}
            src, dst = bm.compact()
            live = sum(len(t) for t in before.values())
            assert all(b < live for r in lens for b in bm.get_block_table(r))
            moved = dict(zip(src, dst))
            for r in lens:
                assert bm.get_block_table(r) == [moved.get(b, b) for b in before[r]]
        tables = [b for r in lens for b in bm.get_block_table(r)]
        assert len(tables) == len(set(tables))                                  # no block in two tables
        assert sorted(tables + bm.free_gpu_blocks_list) == list(range(nb))      # none lost
        for r, n in lens.items():
            assert bm.get_allocated_num_blocks(r) == -(-n // bs)
            pos = list(range(n))
            slots = bm.get_slot_mapping(r, pos)
            assert slots == kv_oracle.slot_mapping_from_table(bm.get_block_table(r), pos, bs)
