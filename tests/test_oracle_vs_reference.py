"""Live cross-check of the oracle against the reference's own functions.

Runs only where the reference tree is present (it does not exist on a GPU
box); the same comparison is frozen into tests/golden/ for everywhere else.
"""
import contextlib
import io

import pytest
import torch

from oracle import kv_oracle, kv_oracle_c, ref_loader

pytestmark = pytest.mark.skipif(not ref_loader.reference_available(), reason="reference tree not present")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_random_round_trips(dtype, seed):
    g = torch.Generator().manual_seed(100 + seed)
    L, NB, BS, H, D = 4, 40, 16, 4, 32
    src = kv_oracle.make_pool(L, NB, BS, H, D, dtype, seed)
    dst_ref = kv_oracle.make_pool(L, NB, BS, H, D, dtype, 0, fill="guard")
    dst_orc = [t.clone() for t in dst_ref]
    dst_c = [t.clone() for t in dst_ref]
    n = int(torch.randint(1, NB, (1,), generator=g))
    s = torch.randperm(NB, generator=g)[:n].tolist()
    d = torch.randperm(NB, generator=g)[:n].tolist()
    ref_src, ref_dst = ref_loader.make_worker(src), ref_loader.make_worker(dst_ref)
    packed_ref = ref_src.extract_kv_blocks(s)
    assert kv_oracle.bit_equal(packed_ref, kv_oracle.extract_kv_blocks(src, s))
    assert kv_oracle.bit_equal(packed_ref, kv_oracle_c.gather(src, s, threads=4))
    ref_dst.write_kv_blocks(d, packed_ref)
    kv_oracle.write_kv_blocks(dst_orc, d, packed_ref)
    kv_oracle_c.scatter(dst_c, d, packed_ref, threads=4)
    for a, b, c in zip(dst_ref, dst_orc, dst_c):
        assert kv_oracle.bit_equal(a, b) and kv_oracle.bit_equal(a, c)
    assert ref_src.get_kv_cache_layout() == {"num_layers": L, "block_size": BS, "num_heads": H,
                                             "head_size": D, "dtype": str(dtype).split(".")[-1]}


def test_block_tables_random_walk():
    g = torch.Generator().manual_seed(7)
    with contextlib.redirect_stdout(io.StringIO()):
        ref = ref_loader.make_block_manager("prefill", 64, 0, 16)
        orc = kv_oracle.BlockTables(64, 16)
        live = {}
        for step in range(200):
            if live and (len(live) > 6 or torch.rand(1, generator=g).item() < 0.4):
                rid = sorted(live)[int(torch.randint(0, len(live), (1,), generator=g))]
                ref.free_blocks(rid)
                orc.release(rid)
                del live[rid]
            else:
                tokens = int(torch.randint(1, 120, (1,), generator=g))
                if ref.get_num_avail_gpu_blocks() < -(-tokens // 16):
                    continue
                rid = f"r{step}"
                live[rid] = tokens
                ref.allocate_blocks(ref_loader.make_request(rid, tokens))
                orc.allocate(rid, tokens)
            assert {k: list(v) for k, v in ref.block_table.items()} == orc.table
            assert list(ref.free_gpu_blocks_list) == orc.free
