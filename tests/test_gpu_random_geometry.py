"""Seeded random pool geometries (odd sizes, all element widths, both page orders) through every
whole-block entry, bit-exact against the oracle."""
import pytest
import torch

from elasticmm_b200 import KVPool, get_context
from gpu_util import BULK_DEFAULT, LDG_DEFAULT, assert_clean, configure, pools_equal, vid
from oracle import kv_oracle

pytestmark = pytest.mark.gpu
DTYPES = [torch.float16, torch.bfloat16, torch.float32, torch.uint8, torch.float64]


def _random_pool(g, L, NB, BS, H, D, dt, head_major):
    shape = (2, NB, H, BS, D) if head_major else (2, NB, BS, H, D)
    out = []
    for _ in range(L):
        if dt == torch.uint8:
            t = torch.randint(0, 256, shape, generator=g, dtype=torch.uint8)
        else:
            t = torch.randn(shape, generator=g, dtype=torch.float32).to(dt)
        out.append(t.permute(0, 1, 3, 2, 4) if head_major else t)
    return out


@pytest.mark.parametrize("opts", [BULK_DEFAULT, LDG_DEFAULT], ids=vid)
@pytest.mark.parametrize("seed", range(12))
def test_random_geometry(opts, seed):
    ctx = get_context(0)
    configure(ctx, **opts)
    g = torch.Generator().manual_seed(1000 + seed)
    r = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=g))
    L, NB, BS, H = r(1, 5), r(2, 70), [1, 2, 4, 8, 16, 32][r(0, 5)], r(1, 9)
    D = [1, 3, 8, 24, 64, 80, 128, 192][r(0, 7)]
    dt = DTYPES[r(0, len(DTYPES) - 1)]
    head_major = bool(r(0, 1)) and H > 1 and BS > 1
    src_cpu = _random_pool(g, L, NB, BS, H, D, dt, head_major)
    NB2 = NB + r(0, 9)
    dst_cpu = [torch.zeros_like(_random_pool(g, 1, NB2, BS, H, D, dt, head_major)[0]) for _ in range(L)]
    src = KVPool([t.cuda() if not head_major else t.permute(0, 1, 3, 2, 4).contiguous().cuda().permute(0, 1, 3, 2, 4)
                  for t in src_cpu], ctx)
    dst = KVPool([t.cuda() if not head_major else t.permute(0, 1, 3, 2, 4).contiguous().cuda().permute(0, 1, 3, 2, 4)
                  for t in dst_cpu], ctx)
    n = r(0, NB)
    s = torch.randperm(NB, generator=g)[:n].tolist()
    d = torch.randperm(NB2, generator=g)[:n].tolist()
    packed = src.gather(s)
    want = kv_oracle.extract_kv_blocks(src_cpu, s)
    assert kv_oracle.bit_equal(packed.cpu(), want), (L, NB, BS, H, D, dt, head_major, n)
    dst.scatter(d, packed)
    kv_oracle.write_kv_blocks(dst_cpu, d, want)
    assert pools_equal(dst.layers, dst_cpu)
    # a second, disjoint set of blocks by direct copy
    free_dst = [b for b in range(NB2) if b not in set(d)]
    m = min(len(free_dst), r(0, NB))
    s2 = torch.randperm(NB, generator=g)[:m].tolist()
    d2 = free_dst[:m]
    src.copy_blocks(dst, s2, d2)
    kv_oracle.copy_blocks(src_cpu, dst_cpu, s2, d2)
    assert_clean(ctx)
    assert pools_equal(dst.layers, dst_cpu) and pools_equal(src.layers, src_cpu)
    configure(ctx)
