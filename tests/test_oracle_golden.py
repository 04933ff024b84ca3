"""The CPU oracle (torch restatement and C restatement) against the fixtures
generated from the reference's own extract_kv_blocks / write_kv_blocks."""
import hashlib
import os

import numpy as np
import pytest
import torch

import cases
from oracle import kv_oracle, kv_oracle_c

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "kv_golden.npz"))


def sha(t: torch.Tensor) -> bytes:
    return hashlib.sha256(kv_oracle.bits(t).numpy().tobytes()).digest()


@pytest.mark.parametrize("case", cases.KV_CASES, ids=lambda c: c["name"])
@pytest.mark.parametrize("impl", ["torch", "c"])
def test_gather_scatter_matches_reference(case, impl):
    src, dst = cases.build_pools(case)
    name = case["name"]
    if impl == "torch":
        packed = kv_oracle.extract_kv_blocks(src, case["src_ids"])
    else:
        packed = kv_oracle_c.gather(src, case["src_ids"], threads=3)
    assert tuple(packed.shape) == tuple(GOLDEN[f"{name}/packed_shape"])
    assert sha(packed) == GOLDEN[f"{name}/packed_sha256"].tobytes()
    if case["store"] == "full":
        assert np.array_equal(kv_oracle.bits(packed).numpy(), GOLDEN[f"{name}/packed"])
    if case["dst_ids"] is None:
        return
    if impl == "torch":
        kv_oracle.write_kv_blocks(dst, case["dst_ids"], packed)
    else:
        kv_oracle_c.scatter(dst, case["dst_ids"], packed, threads=2)
    whole = torch.stack(dst, dim=0)
    assert sha(whole) == GOLDEN[f"{name}/dst_pool_sha256"].tobytes()
    if case["store"] == "full":
        assert np.array_equal(kv_oracle.bits(whole).numpy(), GOLDEN[f"{name}/dst_pool"])


def test_restated_variants_equal_gather_scatter():
    """The 6-D single-tensor transfer, the per-layer send/recv payload and
    the per-block swap copy all move the same bytes as extract -> write."""
    case = cases.KV_CASES[0]
    src, dst_a = cases.build_pools(case)
    _, dst_b = cases.build_pools(case)
    _, dst_c = cases.build_pools(case)
    _, dst_d = cases.build_pools(case)
    s, d = case["src_ids"], case["dst_ids"]
    kv_oracle.write_kv_blocks(dst_a, d, kv_oracle.extract_kv_blocks(src, s))
    six_src, six_dst = torch.stack(src, 0), torch.stack(dst_b, 0)
    kv_oracle.transfer_blocks_6d(six_src, six_dst, s, d)
    assert kv_oracle.bit_equal(torch.stack(dst_a, 0), six_dst)
    nbytes = kv_oracle.send_recv_per_layer(src, dst_c, s, d)
    assert nbytes == len(s) * 2 * case["L"] * case["BS"] * case["H"] * case["D"] * 2
    assert kv_oracle.bit_equal(torch.stack(dst_a, 0), torch.stack(dst_c, 0))
    kv_oracle.swap_blocks(dst_d, src, s, d, is_swap_in=True)
    assert kv_oracle.bit_equal(torch.stack(dst_a, 0), torch.stack(dst_d, 0))
    kv_oracle_c.copy_blocks(src, dst_b, s, d, threads=2)
    assert kv_oracle.bit_equal(torch.stack(dst_a, 0), torch.stack(dst_b, 0))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_append_restatements_agree(dtype):
    g = torch.Generator().manual_seed(5)
    pool = kv_oracle.make_pool(2, 9, 4, 3, 8, dtype, 7)
    key = torch.randn(11, 3, 8, generator=g).to(dtype)
    value = torch.randn(11, 3, 8, generator=g).to(dtype)
    slots = torch.randperm(36, generator=g)[:11]
    slots[2] = -1
    slots[7] = -1
    a, b = pool[0].clone(), pool[0].clone()
    kv_oracle.reshape_and_cache(key, value, a, slots)
    kv_oracle_c.append(b, key, value, slots)
    assert kv_oracle.bit_equal(a, b)
    # by hand: row t sits at block s // BS, offset s % BS; padding rows untouched
    for t, s in enumerate(slots.tolist()):
        if s < 0:
            continue
        assert kv_oracle.bit_equal(a[0, s // 4, s % 4], key[t])
        assert kv_oracle.bit_equal(a[1, s // 4, s % 4], value[t])
    touched = {s for s in slots.tolist() if s >= 0}
    for s in range(36):
        if s not in touched:
            assert kv_oracle.bit_equal(a[:, s // 4, s % 4], pool[0][:, s // 4, s % 4])


def test_compact_plan_properties():
    g = torch.Generator().manual_seed(9)
    for nb, live in [(10, 5), (64, 40), (64, 64), (7, 0), (33, 1)]:
        ids = torch.randperm(nb, generator=g)[:live].tolist()
        new, src, dst = kv_oracle.compact_plan(ids, nb)
        assert kv_oracle_c.compact_plan(ids, nb) == (new, src, dst)
        assert sorted(new) == list(range(live))              # dense prefix
        assert all(s >= live for s in src) and all(d < live for d in dst)
        assert not set(src) & set(dst)
        assert len(src) == sum(1 for b in ids if b >= live)  # minimal: only outsiders move
        assert all(n == o for n, o in zip(new, ids) if o < live)
        assert kv_oracle.compact_plan(new, nb)[1] == []      # idempotent


def test_compaction_preserves_request_contents():
    pool = kv_oracle.make_pool(2, 16, 4, 2, 8, torch.float16, 3)
    tables = {"a": [9, 2, 14], "b": [0, 11], "c": [7, 15, 1, 12]}
    flat = [b for t in tables.values() for b in t]
    before = {k: kv_oracle.extract_kv_blocks(pool, t) for k, t in tables.items()}
    new, src, dst = kv_oracle.compact_plan(flat, 16)
    kv_oracle.compact(pool, src, dst)
    pos = 0
    for k, t in tables.items():
        after = kv_oracle.extract_kv_blocks(pool, new[pos:pos + len(t)])
        assert kv_oracle.bit_equal(after, before[k])
        pos += len(t)


def test_block_tables_restatement_fragments_like_the_reference():
    bt = kv_oracle.BlockTables(12, 4)
    bt.allocate("a", 10)
    bt.allocate("b", 4)
    bt.allocate("c", 9)
    bt.release("a")
    bt.allocate("d", 30)
    assert bt.table["d"] == [7, 8, 9, 10, 11, 0, 1, 2]  # tail first, then the freed ids
    assert kv_oracle.slot_mapping_from_table(bt.table["d"], [0, 5, 21], 4) == [28, 33, 1]


def test_vision_block_transfer_restatement():
    g = torch.Generator().manual_seed(2)
    src = torch.randn(12, 4, 8, generator=g).to(torch.bfloat16)
    dst = torch.zeros(9, 4, 8, dtype=torch.bfloat16)
    recv = kv_oracle.transfer_vision_blocks(src, dst, [7, 0, 11], [2, 8, 5])
    assert recv.shape == (3, 4, 8)
    for s, d in zip([7, 0, 11], [2, 8, 5]):
        assert kv_oracle.bit_equal(dst[d], src[s])
    assert torch.count_nonzero(dst[[0, 1, 3, 4, 6, 7]]) == 0


APPEND_GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "append_golden.npz"))


@pytest.mark.parametrize("case", cases.APPEND_CASES, ids=lambda c: c["name"])
@pytest.mark.parametrize("impl", ["torch", "c"])
def test_append_matches_vllm_cache_op(case, impl):
    """reshape_and_cache of both restatements against pools written by vLLM's own
    reshape_and_cache_flash (the op behind the reference's model_runner.execute_model,
    elasticmm/engine/v0/worker_steps.py:281,438), recorded by tests/golden/make_append_golden.py."""
    pool, key, value, slots = cases.build_append_inputs(case)
    for l in range(case["L"]):
        if impl == "torch":
            kv_oracle.reshape_and_cache(key[l], value[l], pool[l], slots)
        else:
            kv_oracle_c.append(pool[l], key[l], value[l], slots)
    whole = torch.stack(pool, dim=0)
    name = case["name"]
    assert sha(whole) == APPEND_GOLDEN[f"{name}/pool_sha256"].tobytes()
    if case["store"] == "full":
        assert np.array_equal(kv_oracle.bits(whole).numpy(), APPEND_GOLDEN[f"{name}/pool"])


def test_append_fixture_names_the_vllm_version_that_made_it():
    assert bytes(APPEND_GOLDEN["vllm_version"]).decode().startswith("0.")
