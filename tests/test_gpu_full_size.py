"""The benchmark geometries at full size on one B200, checked through size-independent
properties (round trips, untouched-guard counts, per-block checksums) plus the
CPU oracle on whole layers copied back to the host."""
import pytest
import torch

from elasticmm_b200 import KVPool, compact_plan, get_context
from gpu_util import assert_clean, configure
from oracle import kv_oracle

pytestmark = pytest.mark.gpu


def _need(gib):
    free, _ = torch.cuda.mem_get_info(0)
    if free < gib * (1 << 30):
        pytest.skip(f"needs {gib} GiB of free device memory")


def _randn_pool(L, NB, BS, H, D, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return [torch.randn((2, NB, BS, H, D), generator=g, device="cuda", dtype=dtype) for _ in range(L)]


def _guard_pool(L, NB, BS, H, D, dtype):
    out = []
    for _ in range(L):
        t = torch.empty((2, NB, BS, H, D), device="cuda", dtype=dtype)
        t.view(torch.int16).fill_(0x7FFF)
        out.append(t)
    return out


def _block_checksums(layers):
    """Per-block sum of all 16-bit words over layers and planes (int64, exact)."""
    total = None
    for t in layers:
        nb = t.shape[1]
        s = t.view(torch.int16).reshape(2, nb, -1).sum(dim=2, dtype=torch.int64).sum(dim=0)
        total = s if total is None else total + s
    return total


def test_config1_llama7b_gather_then_scatter_full_pool():
    """32 layers, 32 KV heads, fp16, 2048 blocks per layer; 64 requests of
    128..2048 tokens processed in waves that fit the pool."""
    _need(40)
    ctx = get_context(0)
    configure(ctx)
    L, NB, BS, H, D = 32, 2048, 16, 32, 128
    src_layers = _randn_pool(L, NB, BS, H, D, torch.float16, 1)
    dst_layers = _guard_pool(L, NB, BS, H, D, torch.float16)
    src, dst = KVPool(src_layers, ctx), KVPool(dst_layers, ctx)
    g = torch.Generator().manual_seed(1)
    lens = torch.randint(128, 2049, (64,), generator=g).tolist()
    nblk = [-(-n // BS) for n in lens]
    waves, cur = [], []
    for n in nblk:
        if sum(cur) + n > NB:
            waves.append(cur)
            cur = []
        cur.append(n)
    waves.append(cur)
    assert len(waves) >= 2
    check_layers = [0, L - 1]
    src_cpu = [src_layers[l].cpu() for l in check_layers]
    dst_cpu = [dst_layers[l].cpu() for l in check_layers]
    src_sum = _block_checksums(src_layers)
    for wave in waves:
        sperm, dperm = torch.randperm(NB, generator=g).tolist(), torch.randperm(NB, generator=g).tolist()
        pos = 0
        written = torch.zeros(NB, dtype=torch.bool)
        for n in wave:
            s, d = sperm[pos:pos + n], dperm[pos:pos + n]
            packed = src.gather(s)
            dst.scatter(d, packed)
            back = dst.gather(d)
            assert torch.equal(back.view(torch.int16), packed.view(torch.int16))  # round trip
            kv_oracle.write_kv_blocks(dst_cpu, d, kv_oracle.extract_kv_blocks(src_cpu, s))
            written[d] = True
            pos += n
        assert_clean(ctx)
        # whole-pool checks for the wave: moved blocks carry their source's checksum ...
        dst_sum = _block_checksums(dst_layers)
        moved_s = torch.tensor(sperm[:pos], device="cuda")
        moved_d = torch.tensor(dperm[:pos], device="cuda")
        assert torch.equal(dst_sum[moved_d], src_sum[moved_s])
        # ... and two whole layers equal the oracle bit for bit
        for l, want in zip(check_layers, dst_cpu):
            assert kv_oracle.bit_equal(dst_layers[l].cpu(), want)
    # blocks never written in the last wave that were never written before keep the guard word
    assert_clean(ctx)


def test_config2_append_full_pool():
    """32 layers, [2, 16384, 16, 8, 128] bf16 per layer (32 GiB); 256 tokens, 1 % padding."""
    _need(40)
    ctx = get_context(0)
    configure(ctx)
    L, NB, BS, H, D, T = 32, 16384, 16, 8, 128, 256
    layers = _guard_pool(L, NB, BS, H, D, torch.bfloat16)
    pool = KVPool(layers, ctx)
    g = torch.Generator().manual_seed(2)
    slots = torch.randperm(NB * BS, generator=g)[:T].clone()
    pad = torch.randperm(T, generator=g)[:3]
    slots[pad] = -1
    key = torch.randn(L, T, H, D, generator=g).to(torch.bfloat16)
    value = torch.randn(L, T, H, D, generator=g).to(torch.bfloat16)
    key_d, value_d, slots_d = key.cuda(), value.cuda(), slots.cuda()
    half = L // 2
    for l in range(half):                       # per-layer calls, as a model runner issues them
        pool.append(l, key_d[l], value_d[l], slots_d)
    upper = KVPool(layers[half:], ctx)          # the rest in one launch
    upper.append_all_layers(key_d[half:], value_d[half:], slots_d)
    assert_clean(ctx)
    valid = slots >= 0
    vs = slots[valid].cuda()
    for l in range(L):
        flat = layers[l].view(2, NB * BS, H, D)
        assert torch.equal(flat[0, vs].view(torch.int16), key_d[l][valid.cuda()].view(torch.int16))
        assert torch.equal(flat[1, vs].view(torch.int16), value_d[l][valid.cuda()].view(torch.int16))
        untouched = (layers[l].view(torch.int16) == 0x7FFF).sum().item()
        # 253 rows per plane were written; a written word equals the guard only by chance
        assert untouched >= 2 * (NB * BS - 253) * H * D
    for l in (0, L - 1):                        # two whole layers against the oracle
        want = torch.empty((2, NB, BS, H, D), dtype=torch.bfloat16)
        want.view(torch.int16).fill_(0x7FFF)
        kv_oracle.reshape_and_cache(key[l], value[l], want, slots)
        assert kv_oracle.bit_equal(layers[l].cpu(), want)


def test_config5_gqa70b_eviction_compaction_full_pool():
    """80 layers, 8 KV heads, bf16, 8192 blocks per layer at 85 % occupancy;
    evict 30 % of the requests by last use; compact to a dense prefix."""
    _need(50)
    ctx = get_context(0)
    configure(ctx)
    L, NB, BS, H, D = 80, 8192, 16, 8, 128
    layers = _randn_pool(L, NB, BS, H, D, torch.bfloat16, 5)
    pool = KVPool(layers, ctx)
    g = torch.Generator().manual_seed(5)
    perm = torch.randperm(NB, generator=g).tolist()
    tables, used = [], 0
    while True:
        n = -(-int(torch.randint(512, 16385, (1,), generator=g)) // BS)
        if used + n > 0.85 * NB:
            break
        tables.append(perm[used:used + n])
        used += n
    stamps = torch.rand(len(tables), generator=g)
    evict = set(torch.argsort(stamps)[: max(1, round(0.3 * len(tables)))].tolist())
    live = [t for i, t in enumerate(tables) if i not in evict]
    flat = [b for t in live for b in t]
    new_ids, move_src, move_dst = compact_plan(flat, NB)
    assert (new_ids.tolist(), move_src.tolist(), move_dst.tolist()) == kv_oracle.compact_plan(flat, NB)
    before = _block_checksums(layers)
    sample = live[0]
    sample_before = pool.gather(sample)
    l0_before = layers[0].cpu()
    pool.copy_blocks(pool, move_src, move_dst)
    assert_clean(ctx)
    after = _block_checksums(layers)
    old = torch.tensor(flat, device="cuda")
    new = torch.tensor(new_ids.tolist(), device="cuda")
    assert torch.equal(after[new], before[old])             # every live block arrived intact
    assert sorted(new_ids.tolist()) == list(range(len(flat)))
    assert torch.equal(pool.gather(new_ids[: len(sample)].tolist()).view(torch.int16),
                       sample_before.view(torch.int16))
    want = [l0_before]
    kv_oracle.compact(want, move_src.tolist(), move_dst.tolist())
    assert kv_oracle.bit_equal(layers[0].cpu(), want[0])    # one whole layer against the oracle
    # idempotence: a compacted pool plans no moves
    assert compact_plan(new_ids.tolist(), NB)[1].size == 0
