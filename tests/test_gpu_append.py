"""Parity of the CUDA reshape_and_cache with the oracle restatement (bit-exact)."""
import pytest
import torch

from elasticmm_b200 import KVPool, _lib, get_context
from gpu_util import assert_clean, configure, pools_equal, to_gpu
from oracle import kv_oracle

pytestmark = pytest.mark.gpu


@pytest.fixture()
def ctx():
    c = get_context(0)
    configure(c)
    return c


def _slots(num_slots, T, pad_every, g):
    s = torch.randperm(num_slots, generator=g)[:T].clone()
    if pad_every:
        s[::pad_every] = -1
    return s


@pytest.mark.parametrize("geom", [
    dict(L=3, NB=64, BS=16, H=8, D=128, dtype=torch.bfloat16, T=37),   # benchmark row: 2 KiB
    dict(L=2, NB=20, BS=16, H=32, D=128, dtype=torch.float16, T=9),    # 8 KiB rows
    dict(L=2, NB=33, BS=4, H=3, D=5, dtype=torch.float16, T=21),       # 30-byte rows: 2-byte path
    dict(L=2, NB=16, BS=8, H=2, D=6, dtype=torch.float32, T=5),        # 8-byte path
    dict(L=1, NB=5, BS=16, H=1, D=64, dtype=torch.bfloat16, T=80),     # every slot of the pool
], ids=lambda g: f"H{g['H']}D{g['D']}T{g['T']}")
def test_append_per_layer_and_all_layers(ctx, geom):
    g = torch.Generator().manual_seed(geom["T"])
    L, NB, BS, H, D, dt, T = (geom[k] for k in ("L", "NB", "BS", "H", "D", "dtype", "T"))
    pool_cpu = kv_oracle.make_pool(L, NB, BS, H, D, dt, 3)
    pool_cpu2 = [t.clone() for t in pool_cpu]
    pool, pool2 = KVPool(to_gpu(pool_cpu), ctx), KVPool(to_gpu(pool_cpu2), ctx)
    key = torch.randn(L, T, H, D, generator=g).to(dt)
    value = torch.randn(L, T, H, D, generator=g).to(dt)
    slots = _slots(NB * BS, T, 7 if T < NB * BS else 0, g)
    key_d, value_d, slots_d = key.cuda(), value.cuda(), slots.cuda()
    before = ctx.launch_count
    for l in range(L):
        pool.append(l, key_d[l], value_d[l], slots_d)
        kv_oracle.reshape_and_cache(key[l], value[l], pool_cpu[l], slots)
    assert ctx.launch_count - before == L
    pool2.append_all_layers(key_d, value_d, slots_d)
    assert ctx.launch_count - before == L + 1
    pool3 = KVPool(to_gpu(pool_cpu2), ctx)          # static-buffer form: validated once, one call per layer
    bound = pool3.bind_append(key_d, value_d, slots_d)
    for l in range(L):
        bound(l)
    assert_clean(ctx)
    assert pools_equal(pool.layers, pool_cpu)
    assert pools_equal(pool2.layers, pool_cpu)
    assert pools_equal(pool3.layers, pool_cpu)


def test_append_strided_key_value_and_head_major_pool(ctx):
    """key/value as slices of a fused projection (token stride > row) into a head-major pool."""
    g = torch.Generator().manual_seed(12)
    L, NB, BS, H, D, T = 2, 12, 16, 4, 32, 19
    phys_cpu = [torch.randn(2, NB, H, BS, D, generator=g).to(torch.bfloat16) for _ in range(L)]
    logical_cpu = [p.permute(0, 1, 3, 2, 4) for p in phys_cpu]
    pool = KVPool([p.cuda().permute(0, 1, 3, 2, 4) for p in phys_cpu], ctx)
    qkv = torch.randn(L, T, (8 + 2 * H) * D, generator=g).to(torch.bfloat16)
    k_cpu = qkv[:, :, 8 * D:(8 + H) * D].unflatten(-1, (H, D))
    v_cpu = qkv[:, :, (8 + H) * D:].unflatten(-1, (H, D))
    qkv_d = qkv.cuda()
    k_d = qkv_d[:, :, 8 * D:(8 + H) * D].unflatten(-1, (H, D))
    v_d = qkv_d[:, :, (8 + H) * D:].unflatten(-1, (H, D))
    slots = _slots(NB * BS, T, 5, g)
    for l in range(L):
        pool.append(l, k_d[l], v_d[l], slots.cuda())
        kv_oracle.reshape_and_cache(k_cpu[l], v_cpu[l], logical_cpu[l], slots)
    assert_clean(ctx)
    assert pools_equal(pool.layers, logical_cpu)


def test_append_bad_slot_is_reported_and_skipped(ctx):
    L, NB, BS, H, D, T = 1, 4, 16, 2, 64, 6
    pool_cpu = kv_oracle.make_pool(L, NB, BS, H, D, torch.float16, 1)
    pool = KVPool(to_gpu(pool_cpu), ctx)
    key = torch.ones(T, H, D, dtype=torch.float16)
    value = -torch.ones(T, H, D, dtype=torch.float16)
    slots = torch.tensor([3, NB * BS, -1, 10, 1 << 40, 63])
    pool.append(0, key.cuda(), value.cuda(), slots.cuda())
    rc, detail = ctx.status()
    assert rc == _lib.ERR_ID_RANGE and detail in (NB * BS, 1 << 40)
    good = torch.tensor([3, -1, -1, 10, -1, 63])
    kv_oracle.reshape_and_cache(key, value, pool_cpu[0], good)
    assert pools_equal(pool.layers, pool_cpu)
    with pytest.raises(ValueError):
        pool.append(0, key.cuda(), value.cuda(), slots[:3].cuda())
    with pytest.raises(ValueError):
        pool.append(0, key.cuda().to(torch.bfloat16), value.cuda().to(torch.bfloat16), slots.cuda())
    with pytest.raises(Exception):
        pool.append(1, key.cuda(), value.cuda(), slots.cuda())  # layer out of range
