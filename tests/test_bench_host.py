"""Host-side pieces of bench.py: seeded workload generation and wave packing (no GPU)."""
import importlib.util
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_request_lengths_follow_the_configs(bench):
    w1 = bench.WORKLOADS["llama7b_cfg1"]
    c1 = bench.request_blocks(w1, 1)
    assert len(c1) == 64 and min(c1) >= 8 and max(c1) <= 128            # 128..2048 tokens, 16 per block
    assert c1 == bench.request_blocks(w1, 1)                             # seeded
    w3 = bench.WORKLOADS["qwen25vl7b_cfg3"]
    c3 = bench.request_blocks(w3, 4)
    assert len(c3) == 128 and min(c3) >= (576 + 32) // 16 and max(c3) <= -(-(576 + 1024) // 16)
    w4 = bench.WORKLOADS["llava13b_cfg4"]
    c4 = bench.request_blocks(w4, 4)
    assert len(c4) == 512 and min(c4) >= 16 and max(c4) <= 512           # 256..8192 tokens
    # log-uniform: the median sits near the geometric mean (1448 tokens = 91 blocks), far below the mean
    assert 60 <= sorted(c4)[256] <= 130 < sum(c4) / 512
    assert bench.block_bytes(w1) == 8 << 20 and bench.block_bytes(w4) == int(12.5 * (1 << 20))
    assert bench.page_bytes(w3) == 16 << 10


def test_waves_respect_the_pool(bench):
    w1 = bench.WORKLOADS["llama7b_cfg1"]
    counts = bench.request_blocks(w1, 1)
    waves = bench.make_waves(counts, w1["NB"])
    assert sum(counts) > w1["NB"] and len(waves) >= 2                    # the requests exceed the pool
    assert [i for wave in waves for i in wave] == list(range(64))        # every request once, in order
    assert all(sum(counts[i] for i in wave) <= w1["NB"] for wave in waves)
    assert bench.make_waves([5000], 2048) == [[0]]                        # an oversize request still gets a wave


def test_measured_peak_fallback(bench, monkeypatch, tmp_path):
    monkeypatch.setattr(bench, "ROOT", str(tmp_path))
    assert bench.measured_peak() == (6650.0, "fallback")
    (tmp_path / "MEASURED_PEAKS.json").write_text('{"hbm_gbs": 6553.3}')
    assert bench.measured_peak() == (6553.3, "measured")


def test_build_requests_is_seeded_and_tables_do_not_repeat_within_a_wave(bench):
    w1 = bench.WORKLOADS["llama7b_cfg1"]
    counts, waves, reqs = bench.build_requests(w1, 1)
    assert (counts, waves, reqs) == bench.build_requests(w1, 1)
    assert len(reqs) == 64 and [len(s) for s, _ in reqs] == [counts[i] for wave in waves for i in wave]
    pos = 0
    for wave in waves:
        src = [b for s, _ in reqs[pos:pos + len(wave)] for b in s]
        dst = [b for _, d in reqs[pos:pos + len(wave)] for b in d]
        assert len(set(src)) == len(src) and len(set(dst)) == len(dst)
        assert all(len(s) == len(d) for s, d in reqs[pos:pos + len(wave)])
        pos += len(wave)


@pytest.mark.parametrize("sources,sinks", [([0, 1], [2, 3]), ([0, 1], [2, 3, 4, 5, 6, 7])])
def test_wave_plans_use_half_pools_alternately_and_balance_the_sinks(bench, sources, sinks):
    w = bench.WORKLOADS["llava13b_cfg4"]
    plans = bench.build_wave_plans(w, sources, sinks)
    counts = bench.request_blocks(w, 4)
    half = w["NB"] // 2
    seen = sorted(int(t.request_id[3:]) for p in plans for t in p.transfers)
    assert seen == list(range(len(counts)))                               # every request exactly once
    for k, plan in enumerate(plans):
        lo, hi = (k % 2) * half, (k % 2) * half + half
        plan.validate(lambda r: w["NB"])                                   # ranges, no destination block twice
        for s in sources:
            used = [b for t in plan.transfers if t.src_rank == s for b in t.src_blocks]
            assert len(set(used)) == len(used) <= half and all(lo <= b < hi for b in used)
        for d in sinks:
            used = [b for t in plan.transfers if t.dst_rank == d for b in t.dst_blocks]
            assert len(used) <= half and all(lo <= b < hi for b in used)
    # full waves: all but the tail use nearly all of every source's half pool, and no sink has to take in more
    # per wave than a source sends out (a sink's link then never limits the wave)
    for k, plan in enumerate(plans[:-1]):
        for s in sources:
            used = sum(len(t.src_blocks) for t in plan.transfers if t.src_rank == s)
            assert used > (0.9 if k < len(plans) - 3 else 0.75) * half
        for d in sinks:
            assert sum(len(t.src_blocks) for t in plan.transfers if t.dst_rank == d) <= half
    # the sinks' shares of a wave are proportional to what they still have to receive: before the tail no
    # sink takes more than 1.3 times the mean share
    for plan in plans[: len(plans) - 6]:
        shares = [sum(len(t.src_blocks) for t in plan.transfers if t.dst_rank == d) for d in sinks]
        assert max(shares) <= 1.3 * sum(shares) / len(shares)
