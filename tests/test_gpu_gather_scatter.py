"""Parity of the CUDA gather / scatter / block copy with the reference fixtures and the oracle."""
import hashlib
import os

import numpy as np
import pytest
import torch

import cases
from elasticmm_b200 import EmmError, KVPool, _lib, get_context
from gpu_util import BULK_DEFAULT, LDG_DEFAULT, VARIANTS, assert_clean, configure, pools_equal, to_gpu, vid
from oracle import kv_oracle

pytestmark = pytest.mark.gpu
GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "kv_golden.npz"))


def sha(t: torch.Tensor) -> bytes:
    return hashlib.sha256(kv_oracle.bits(t.cpu()).numpy().tobytes()).digest()


@pytest.fixture()
def ctx():
    c = get_context(0)
    configure(c)
    yield c
    configure(c)


@pytest.mark.parametrize("case", cases.KV_CASES, ids=lambda c: c["name"])
@pytest.mark.parametrize("opts", VARIANTS, ids=vid)
def test_golden_cases(ctx, case, opts):
    """extract_kv_blocks / write_kv_blocks fixtures, every kernel variant, host-list ids."""
    configure(ctx, **opts)
    src_cpu, dst_cpu = cases.build_pools(case)
    src, dst = KVPool(to_gpu(src_cpu), ctx), KVPool(to_gpu(dst_cpu), ctx)
    name = case["name"]
    packed = src.gather(case["src_ids"])
    assert_clean(ctx)
    assert tuple(packed.shape) == tuple(GOLDEN[f"{name}/packed_shape"])
    assert sha(packed) == GOLDEN[f"{name}/packed_sha256"].tobytes()
    if case["store"] == "full":
        assert np.array_equal(kv_oracle.bits(packed.cpu()).numpy(), GOLDEN[f"{name}/packed"])
    if case["dst_ids"] is None:
        return
    dst.scatter(case["dst_ids"], packed)
    assert_clean(ctx)
    whole = torch.stack(dst.layers, 0)
    assert sha(whole) == GOLDEN[f"{name}/dst_pool_sha256"].tobytes()
    # the source pool is read-only for both operations
    assert pools_equal(src.layers, src_cpu)


@pytest.mark.parametrize("case", [cases.KV_CASES[0], cases.KV_CASES[4], cases.KV_CASES[10]], ids=lambda c: c["name"])
@pytest.mark.parametrize("opts", [BULK_DEFAULT, LDG_DEFAULT], ids=vid)
def test_device_tables_layer_ranges_and_block_copy(ctx, case, opts):
    configure(ctx, **opts)
    src_cpu, dst_cpu = cases.build_pools(case)
    src, dst = KVPool(to_gpu(src_cpu), ctx), KVPool(to_gpu(dst_cpu), ctx)
    s_ids, d_ids = case["src_ids"], case["dst_ids"]
    s_dev, d_dev = src.upload_ids(s_ids), dst.upload_ids(d_ids)
    want_packed = kv_oracle.extract_kv_blocks(src_cpu, s_ids)
    assert kv_oracle.bit_equal(src.gather(s_dev).cpu(), want_packed)
    # per-layer-range messages, as the staged transport sends them
    L = case["L"]
    for begin, count in [(0, 1), (L - 1, 1), (1, L - 1)]:
        part = src.gather(s_dev, layer_begin=begin, layer_count=count)
        assert kv_oracle.bit_equal(part.cpu(), want_packed[begin:begin + count])
        dst.scatter(d_dev, part, layer_begin=begin, layer_count=count)
    kv_oracle.write_kv_blocks(dst_cpu, d_ids, want_packed)
    assert_clean(ctx)
    assert pools_equal(dst.layers, dst_cpu)
    # direct block copy into a fresh guard pool == extract -> write
    _, dst2_cpu = cases.build_pools(case)
    dst2 = KVPool(to_gpu(dst2_cpu), ctx)
    src.copy_blocks(dst2, s_dev, d_dev)
    src.copy_blocks(dst2, s_ids, d_ids)  # host-list form, same result
    assert_clean(ctx)
    assert pools_equal(dst2.layers, dst_cpu)


@pytest.mark.parametrize("opts", [BULK_DEFAULT, LDG_DEFAULT], ids=vid)
def test_head_major_pool_and_single_6d_tensor(ctx, opts):
    configure(ctx, **opts)
    L, NB, BS, H, D = 3, 10, 16, 4, 32
    g = torch.Generator().manual_seed(2)
    ids, dids = [7, 0, 3, 9], [1, 2, 8, 4]
    # head-major allocation [2, NB, H, BS, D] seen through its logical [2, NB, BS, H, D] view
    phys = [torch.randn(2, NB, H, BS, D, generator=g).to(torch.bfloat16) for _ in range(L)]
    logical_cpu = [p.permute(0, 1, 3, 2, 4) for p in phys]
    pool = KVPool([p.cuda().permute(0, 1, 3, 2, 4) for p in phys], ctx)
    assert pool.head_major
    packed = pool.gather(ids)
    assert kv_oracle.bit_equal(packed.cpu(), kv_oracle.extract_kv_blocks(logical_cpu, ids))
    sink_cpu = [torch.zeros(2, NB, H, BS, D, dtype=torch.bfloat16).permute(0, 1, 3, 2, 4) for _ in range(L)]
    sink = KVPool([torch.zeros(2, NB, H, BS, D, dtype=torch.bfloat16, device="cuda").permute(0, 1, 3, 2, 4)
                   for _ in range(L)], ctx)
    sink.scatter(dids, packed)
    kv_oracle.write_kv_blocks(sink_cpu, dids, kv_oracle.extract_kv_blocks(logical_cpu, ids))
    assert pools_equal(sink.layers, sink_cpu)
    # one [L, 2, NB, BS, H, D] tensor (the legacy transfer manager's view of the pool)
    six_cpu = torch.randn(L, 2, NB, BS, H, D, generator=g).to(torch.float16)
    six_dst_cpu = torch.zeros_like(six_cpu)
    six, six_dst = six_cpu.cuda(), six_dst_cpu.cuda()
    a, b = KVPool(list(six.unbind(0)), ctx), KVPool(list(six_dst.unbind(0)), ctx)
    a.copy_blocks(b, ids, dids)
    kv_oracle.transfer_blocks_6d(six_cpu, six_dst_cpu, ids, dids)
    assert_clean(ctx)
    assert kv_oracle.bit_equal(six_dst.cpu(), six_dst_cpu)


def test_errors_are_status_codes_not_faults(ctx):
    case = cases.KV_CASES[0]
    src_cpu, dst_cpu = cases.build_pools(case)
    src, dst = KVPool(to_gpu(src_cpu), ctx), KVPool(to_gpu(dst_cpu), ctx)
    with pytest.raises(EmmError) as e:
        src.gather([0, 12])
    assert e.value.status == _lib.ERR_ID_RANGE
    with pytest.raises(EmmError) as e:
        src.gather([-1])
    assert e.value.status == _lib.ERR_ID_RANGE
    packed = src.gather([1, 2])
    with pytest.raises(EmmError) as e:
        dst.scatter([3, 3], packed)
    assert e.value.status == _lib.ERR_DUPLICATE
    with pytest.raises(ValueError):
        dst.scatter([3, 4, 5], packed)          # block count mismatch
    with pytest.raises(EmmError) as e:
        src.copy_blocks(src, [1, 2], [2, 5])    # block 2 is both read and written
    assert e.value.status == _lib.ERR_OVERLAP
    # device tables are checked by the kernel: the bad page is skipped, the rest is copied
    for opts in (BULK_DEFAULT, LDG_DEFAULT):
        configure(ctx, **opts)
        bad = torch.tensor([5, 99, 1, -3], dtype=torch.int32, device="cuda")
        out = torch.full((case["L"], 2, 4, case["BS"], case["H"], case["D"]), 7.0, dtype=torch.float16, device="cuda")
        src.gather(bad, out=out)
        rc, detail = ctx.status()
        assert rc == _lib.ERR_ID_RANGE and detail in (99, -3)
        want = kv_oracle.extract_kv_blocks(src_cpu, [5, 0, 1, 0])
        got = out.cpu()
        assert kv_oracle.bit_equal(got[:, :, 0], want[:, :, 0]) and kv_oracle.bit_equal(got[:, :, 2], want[:, :, 2])
        assert torch.all(got[:, :, 1] == 7.0) and torch.all(got[:, :, 3] == 7.0)
        assert ctx.status()[0] == _lib.OK       # sticky status was cleared
    assert pools_equal(src.layers, src_cpu) and pools_equal(dst.layers, dst_cpu)


def test_launch_count_is_one_per_operation(ctx):
    case = cases.KV_CASES[9]
    src_cpu, dst_cpu = cases.build_pools(case)
    src, dst = KVPool(to_gpu(src_cpu), ctx), KVPool(to_gpu(dst_cpu), ctx)
    before = ctx.launch_count
    packed = src.gather(case["src_ids"])
    dst.scatter(case["dst_ids"], packed)
    src.copy_blocks(dst, case["src_ids"], case["dst_ids"])
    src.gather([])
    assert ctx.launch_count - before == 3


def test_random_round_trips_many_requests(ctx):
    """Config-1 style: requests of random length, disjoint tables from one
    permutation, gather -> scatter into a second pool; checked against the oracle."""
    L, NB, BS, H, D = 4, 256, 16, 8, 128
    g = torch.Generator().manual_seed(1)
    src_cpu = kv_oracle.make_pool(L, NB, BS, H, D, torch.float16, 5)
    dst_cpu = kv_oracle.make_pool(L, NB, BS, H, D, torch.float16, 0, fill="guard")
    src, dst = KVPool(to_gpu(src_cpu), ctx), KVPool(to_gpu(dst_cpu), ctx)
    sperm, dperm = torch.randperm(NB, generator=g).tolist(), torch.randperm(NB, generator=g).tolist()
    pos = 0
    while pos < NB:
        n = min(int(torch.randint(1, 40, (1,), generator=g)), NB - pos)
        s, d = sperm[pos:pos + n], dperm[pos:pos + n]
        dst.scatter(d, src.gather(s))
        kv_oracle.write_kv_blocks(dst_cpu, d, kv_oracle.extract_kv_blocks(src_cpu, s))
        pos += n
    assert_clean(ctx)
    assert pools_equal(dst.layers, dst_cpu)


def test_device_table_entries_replay_from_a_cuda_graph(ctx):
    """gather -> scatter -> block copy captured once and replayed with new table contents."""
    case = cases.KV_CASES[12]   # 32 KiB pages
    src_cpu, dst_cpu = cases.build_pools(case)
    src, dst = KVPool(to_gpu(src_cpu), ctx), KVPool(to_gpu(dst_cpu), ctx)
    n = len(case["src_ids"])
    s_dev, d_dev = src.upload_ids(case["src_ids"]), dst.upload_ids(case["dst_ids"])
    packed = src.new_packed(n)
    src.gather(s_dev, out=packed)          # first use outside capture (sets the kernel's shared-memory limit)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            src.gather(s_dev, out=packed)
            dst.scatter(d_dev, packed)
    for trial in range(2):
        g = torch.Generator().manual_seed(trial)
        s_ids = torch.randperm(case["NB"], generator=g)[:n].tolist()
        d_ids = torch.randperm(case["NB"], generator=g)[:n].tolist()
        s_dev.copy_(torch.tensor(s_ids, dtype=torch.int32))
        d_dev.copy_(torch.tensor(d_ids, dtype=torch.int32))
        graph.replay()
        kv_oracle.write_kv_blocks(dst_cpu, d_ids, kv_oracle.extract_kv_blocks(src_cpu, s_ids))
    assert_clean(ctx)
    assert pools_equal(dst.layers, dst_cpu)


@pytest.mark.parametrize("opts", [BULK_DEFAULT, LDG_DEFAULT], ids=vid)
@pytest.mark.parametrize("case", [cases.KV_CASES[0], cases.KV_CASES[4], cases.KV_CASES[10]], ids=lambda c: c["name"])
def test_many_requests_in_one_launch(ctx, opts, case):
    """gather_many / scatter_many: one launch, one contiguous tensor per request, same bytes as the
    per-request calls (and as the reference's per-request functions)."""
    from elasticmm_b200.engine.v0 import V0Worker

    configure(ctx, **opts)
    src_cpu, dst_cpu = cases.build_pools(case)
    src = V0Worker(dtype=case["dtype"], device="cuda:0", kv_cache=to_gpu(src_cpu))
    dst = V0Worker(dtype=case["dtype"], device="cuda:0", kv_cache=to_gpu(dst_cpu))
    g = torch.Generator().manual_seed(3)
    sperm = torch.randperm(case["NB"], generator=g).tolist()
    dperm = torch.randperm(case["dst_NB"], generator=g).tolist()
    sizes, pos, s_lists, d_lists = [], 0, [], []
    while pos < min(case["NB"], case["dst_NB"]):
        n = min(int(torch.randint(0, 6, (1,), generator=g)), min(case["NB"], case["dst_NB"]) - pos)
        s_lists.append(sperm[pos:pos + n])
        d_lists.append(dperm[pos:pos + n])
        pos += max(n, 1) if n else 1
    before = ctx.launch_count
    parts = src.extract_kv_blocks_many(s_lists)
    assert ctx.launch_count - before == 1 and len(parts) == len(s_lists)
    for ids, part in zip(s_lists, parts):
        assert part.shape[2] == len(ids)
        assert kv_oracle.bit_equal(part.cpu(), kv_oracle.extract_kv_blocks(src_cpu, ids))
    dst.write_kv_blocks_many(d_lists, parts)
    assert ctx.launch_count - before == 2
    for ids, d_ids in zip(s_lists, d_lists):
        kv_oracle.write_kv_blocks(dst_cpu, d_ids, kv_oracle.extract_kv_blocks(src_cpu, ids))
    assert_clean(ctx)
    assert pools_equal(dst.kv_cache, dst_cpu)
    with pytest.raises(EmmError):
        src.extract_kv_blocks_many([[0], [case["NB"]]])
    with pytest.raises(EmmError):
        dst.write_kv_blocks_many([[1], [1]], src.extract_kv_blocks_many([[0], [1]]))


def test_two_contexts_on_one_device_share_the_kernel_shared_memory_limit():
    """The dynamic shared-memory limit belongs to the kernel and the device, not
    to a context: a second context with a small ring must not lower it under
    the first one's 128 KiB launches."""
    from elasticmm_b200.kv_pool import Context
    first = get_context(0)
    configure(first, **BULK_DEFAULT)
    second = Context(0)
    second.configure(variant=_lib.COPY_BULK, chunk_bytes=4096, stages=2, warps=1)
    cpu = kv_oracle.make_pool(2, 24, 16, 32, 128, torch.float16, 9)      # 128 KiB pages
    gpu = to_gpu(cpu)
    ids = [5, 0, 23, 11, 12]
    want = kv_oracle.extract_kv_blocks(cpu, ids)
    for ctx in (first, second, first, second):
        got = KVPool(gpu, ctx).gather(ids)
        assert_clean(ctx)
        assert kv_oracle.bit_equal(got.cpu(), want)


def test_a_pool_may_be_destroyed_after_its_context():
    from elasticmm_b200.kv_pool import Context
    ctx = Context(0)
    cpu = kv_oracle.make_pool(2, 8, 4, 2, 8, torch.float16, 3)
    pool = KVPool(to_gpu(cpu), ctx)
    assert kv_oracle.bit_equal(pool.gather([1, 6]).cpu(), kv_oracle.extract_kv_blocks(cpu, [1, 6]))
    torch.cuda.synchronize()
    ctx.close()
    pool.close()      # frees the pool's device array without touching the closed context
    pool.close()      # and closing twice is harmless
