"""The barrier-free wave protocol on the host: WaveLedger over a key-value store and the
run_waves driver, with threads standing in for ranks and the oracle standing in for the
copy kernels. Checks the ordering rule (wave w of a source starts only after every sink
has finished wave w - depth of it), the result, and that a failed rank releases the others."""
import random
import threading
import time

import pytest
import torch
import torch.distributed as dist

from elasticmm_b200.engine.v0.transport import MigrationPlan, Transfer, WaveLedger, run_waves
from oracle import kv_oracle

GEOM = dict(L=2, NB=32, BS=4, H=2, D=8)
SOURCES, SINKS = [0, 1], [2, 3, 4]
HALF = GEOM["NB"] // 2


def _pool(seed, guard=False):
    return kv_oracle.make_pool(GEOM["L"], GEOM["NB"], GEOM["BS"], GEOM["H"], GEOM["D"], torch.float16, seed,
                               fill="guard" if guard else "normal")


def _plans(n_waves, seed):
    """Waves alternate between the two halves of every pool (blocks are reused two waves later)."""
    g = torch.Generator().manual_seed(seed)
    plans = []
    for w in range(n_waves):
        base = (w % 2) * HALF
        plan = MigrationPlan()
        dst_free = {d: (torch.randperm(HALF, generator=g) + base).tolist() for d in SINKS}
        for s in SOURCES:
            src_free = (torch.randperm(HALF, generator=g) + base).tolist()
            for r in range(4):
                n = int(torch.randint(1, 4, (1,), generator=g))
                d = SINKS[int(torch.randint(0, len(SINKS), (1,), generator=g))]
                if w == 1 and s == 1 and d == 4:
                    continue  # a wave in which one pair has nothing to move
                plan.add(Transfer(f"w{w}s{s}r{r}", s, d, tuple(src_free[:n]), tuple(dst_free[d][:n])))
                src_free, dst_free[d] = src_free[n:], dst_free[d][n:]
        plans.append(plan)
    return plans


def test_ledger_counts_and_times_out():
    ledger = WaveLedger(dist.HashStore(), "m0", timeout_s=0.2)
    assert ledger.count(0, 1) == 0
    assert ledger.post(0, 1) == 1 and ledger.post(0, 1) == 2
    ledger.wait(0, 1, 2)
    ledger.wait(5, 1, 0)  # nothing expected: returns at once
    with pytest.raises(TimeoutError, match="1 of 3|2 of 3"):
        ledger.wait(0, 1, 3)
    assert ledger.failed() is None
    ledger.mark_failed("sink 3: pool of rank 0 is not mapped")
    with pytest.raises(RuntimeError, match="not mapped"):
        WaveLedger(ledger.store, "m0", timeout_s=5.0).wait(1, 0, 1)


@pytest.mark.parametrize("depth", [1, 2])
def test_waves_without_barrier_are_ordered_and_bit_exact(depth):
    n_waves = 6
    plans = _plans(n_waves, seed=depth)
    store = dist.HashStore()
    src_pools = {s: _pool(10 + s) for s in SOURCES}
    dst_pools = {d: _pool(0, guard=True) for d in SINKS}
    want = {d: _pool(0, guard=True) for d in SINKS}
    landed = {d: [] for d in SINKS}
    violations, errors = [], []
    rng = random.Random(depth)
    delays = {(w, d): rng.uniform(0.0, 0.004) for w in range(n_waves) for d in SINKS}

    def rank_main(rank):
        ledger = WaveLedger(store, "epoch0", timeout_s=20.0)

        def launch(w, source, earlier):
            if w >= depth:
                need = len(plans[w - depth].outgoing(source))
                if ledger.count(w - depth, source) < need:
                    violations.append((rank, w, source))
            for h in earlier:
                if not h["done"]:
                    violations.append(("own", rank, w))
            time.sleep(delays[(w, rank)])  # sinks progress at different speeds
            si, di = plans[w].tables(source, rank)
            kv_oracle.write_kv_blocks(dst_pools[rank], di, kv_oracle.extract_kv_blocks(src_pools[source], si))
            return {"done": False, "ms": delays[(w, rank)] * 1e3}

        def wait_done(h):
            h["done"] = True
            return h["ms"]

        def on_landed(w):
            # what this sink holds for wave w is intact although later waves are already in flight
            for s in plans[w].incoming(rank):
                si, di = plans[w].tables(s, rank)
                got = kv_oracle.extract_kv_blocks(dst_pools[rank], di)
                if not kv_oracle.bit_equal(got, kv_oracle.extract_kv_blocks(src_pools[s], si)):
                    errors.append((rank, w, s))
            landed[rank].append(w)

        try:
            ms = run_waves(plans, rank, ledger, depth, launch, wait_done, on_landed if rank in SINKS else None)
            if rank in SINKS:
                assert len(ms) == len(plans)
            else:
                assert ms == []
        except Exception as e:  # pragma: no cover - reported below
            errors.append((rank, repr(e)))

    threads = [threading.Thread(target=rank_main, args=(r,)) for r in SOURCES + SINKS]
    for t in threads:
        t.start()
    for t in threads:
        t.join(60)
    assert not any(t.is_alive() for t in threads), "a rank is still waiting"
    assert not errors and not violations, (errors, violations)
    for d in SINKS:
        assert landed[d] == list(range(n_waves))
        for plan in plans:
            for s in plan.incoming(d):
                si, di = plan.tables(s, d)
                kv_oracle.write_kv_blocks(want[d], di, kv_oracle.extract_kv_blocks(src_pools[s], si))
        assert all(kv_oracle.bit_equal(a, b) for a, b in zip(dst_pools[d], want[d]))
    ledger = WaveLedger(store, "epoch0")
    for w, plan in enumerate(plans):
        for s in SOURCES:
            assert ledger.count(w, s) == len(plan.outgoing(s))


def test_a_failed_rank_releases_the_ranks_that_wait_for_it():
    plans = _plans(4, seed=3)
    store = dist.HashStore()
    outcome = {}

    def rank_main(rank):
        ledger = WaveLedger(store, "epoch1", timeout_s=20.0)

        def launch(w, source, earlier):
            if rank == 3 and w == 1:
                raise RuntimeError("sink 3 lost its mapping")
            return w

        try:
            run_waves(plans, rank, ledger, 2, launch, lambda h: 0.0)
            outcome[rank] = None
        except Exception as e:
            outcome[rank] = f"{type(e).__name__}: {e}"
            ledger.mark_failed(outcome[rank])

    threads = [threading.Thread(target=rank_main, args=(r,)) for r in SOURCES + SINKS]
    t0 = time.monotonic()
    for t in threads:
        t.start()
    for t in threads:
        t.join(30)
    assert not any(t.is_alive() for t in threads)
    assert time.monotonic() - t0 < 10, "the others waited for the timeout instead of the failure mark"
    assert "lost its mapping" in outcome[3]
    assert all(outcome[r] is not None for r in SOURCES), outcome  # the sources learn that their blocks were not all read
