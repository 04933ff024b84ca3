"""The ways a block table reaches the kernels, and the launch attributes of the copy kernels.

Host lists of up to 128 ids travel in the kernel arguments, longer ones through the pinned staging
ring; tables kept on the device are uploaded once with emm_upload_ids; several peers' blocks are
packed per peer for a layer range (the packed side of an all-to-all). Every form must give what
the reference's extract_kv_blocks / write_kv_blocks give (elasticmm/engine/v0/worker.py:578-633)."""

import numpy as np
import pytest
import torch

from elasticmm_b200 import EmmError, KVPool, _lib, get_context
from gpu_util import BULK_DEFAULT, LDG_DEFAULT, assert_clean, configure, pools_equal, to_gpu, vid
from oracle import kv_oracle

pytestmark = pytest.mark.gpu
GEOM = dict(L=5, NB=200, BS=16, H=4, D=64)


@pytest.fixture()
def ctx():
    c = get_context(0)
    configure(c)
    yield c
    configure(c)
    c.set_option(_lib.OPT_PDL, 1)


def _pools(ctx, dtype=torch.bfloat16):
    src_cpu = kv_oracle.make_pool(GEOM["L"], GEOM["NB"], GEOM["BS"], GEOM["H"], GEOM["D"], dtype, 31)
    dst_cpu = kv_oracle.make_pool(GEOM["L"], GEOM["NB"], GEOM["BS"], GEOM["H"], GEOM["D"], dtype, 0, fill="guard")
    return src_cpu, dst_cpu, KVPool(to_gpu(src_cpu), ctx), KVPool(to_gpu(dst_cpu), ctx)


@pytest.mark.parametrize("n", [1, 127, 128, 129, 180])
@pytest.mark.parametrize("opts", [BULK_DEFAULT, LDG_DEFAULT], ids=vid)
def test_host_lists_on_both_sides_of_the_inline_limit(ctx, n, opts):
    """128 ids ride in the kernel arguments, 129 go through the staging ring: same bytes either way."""
    configure(ctx, **opts)
    src_cpu, dst_cpu, src, dst = _pools(ctx)
    g = torch.Generator().manual_seed(n)
    s_ids = torch.randperm(GEOM["NB"], generator=g)[:n].tolist()
    d_ids = torch.randperm(GEOM["NB"], generator=g)[:n].tolist()
    packed = src.gather(s_ids)
    want = kv_oracle.extract_kv_blocks(src_cpu, s_ids)
    assert kv_oracle.bit_equal(packed.cpu(), want)
    dst.scatter(d_ids, packed)
    kv_oracle.write_kv_blocks(dst_cpu, d_ids, want)
    assert pools_equal(dst.layers, dst_cpu)
    # block copy with both tables as host lists, into the blocks the scatter left untouched
    free = [b for b in range(GEOM["NB"]) if b not in set(d_ids)][:min(n, GEOM["NB"] - n)]
    src.copy_blocks(dst, s_ids[:len(free)], free)
    kv_oracle.write_kv_blocks(dst_cpu, free, kv_oracle.extract_kv_blocks(src_cpu, s_ids[:len(free)]))
    assert_clean(ctx)
    assert pools_equal(dst.layers, dst_cpu)
    with pytest.raises(EmmError):
        src.gather(s_ids[:-1] + [GEOM["NB"]])          # a bad id is refused on the host on either path
    with pytest.raises(EmmError):
        dst.scatter(d_ids[:-1] + [d_ids[0]] if n > 1 else [-1], packed)


def test_upload_ids_goes_through_the_pinned_ring_and_checks_values(ctx):
    _, _, src, _ = _pools(ctx)
    for n in (0, 1, 5000, 70000):                           # grows the ring slot on the way
        ids = (np.arange(n, dtype=np.int64) * 7919) % (1 << 31)
        dev = src.upload_ids(ids)
        assert dev.dtype == torch.int32 and dev.numel() == n
        assert np.array_equal(dev.cpu().numpy().astype(np.int64), ids)
    lib = _lib.load()
    out = torch.empty(2, dtype=torch.int32, device="cuda")
    bad = np.array([3, 1 << 31], dtype=np.int64)
    assert lib.emm_upload_ids(ctx._h, bad.ctypes.data, 2, out.data_ptr(), None) == _lib.ERR_ID_RANGE
    assert lib.emm_upload_ids(ctx._h, None, 2, out.data_ptr(), None) == _lib.ERR_BAD_ARG


@pytest.mark.parametrize("opts", [BULK_DEFAULT, LDG_DEFAULT], ids=vid)
def test_per_peer_segments_of_a_layer_range(ctx, opts):
    """gather_segments lays a chunk of layers out as [peer][layer][plane][n_peer][page]; each peer's share is
    one contiguous run equal to extract_kv_blocks of that layer range; scatter_segments is its inverse."""
    configure(ctx, **opts)
    src_cpu, dst_cpu, src, dst = _pools(ctx)
    g = torch.Generator().manual_seed(5)
    perm = torch.randperm(GEOM["NB"], generator=g).tolist()
    peers = [perm[0:17], perm[17:18], [], perm[18:90]]       # unequal shares, one empty
    dperm = torch.randperm(GEOM["NB"], generator=g).tolist()
    dsts = [dperm[0:17], dperm[17:18], [], dperm[18:90]]
    s_tab = src.many_tables(peers)
    d_tab = dst.many_tables(dsts, unique=True)
    total = sum(len(p) for p in peers)
    for begin, count in ((0, 2), (2, 3), (4, 1)):
        flat = torch.empty(src.packed_bytes(total, count) // 2, dtype=torch.bfloat16, device="cuda")
        src.gather_segments(s_tab, flat, begin, count)
        per_block = src.packed_bytes(1, count) // 2
        pos = 0
        for ids in peers:
            piece = flat[pos * per_block:(pos + len(ids)) * per_block].view(src.packed_shape(len(ids), count))
            want = kv_oracle.extract_kv_blocks(src_cpu[begin:begin + count], ids) if ids else piece.cpu()
            assert kv_oracle.bit_equal(piece.cpu(), want)
            pos += len(ids)
        dst.scatter_segments(d_tab, flat, begin, count)
        for s_ids, d_ids in zip(peers, dsts):
            if s_ids:
                kv_oracle.write_kv_blocks(dst_cpu[begin:begin + count], d_ids,
                                          kv_oracle.extract_kv_blocks(src_cpu[begin:begin + count], s_ids))
    assert_clean(ctx)
    assert pools_equal(dst.layers, dst_cpu)
    lib = _lib.load()
    assert lib.emm_gather_many_layers(src._h, 4, 2, None, None, 1, 1, None, 0, None) == _lib.ERR_BAD_ARG  # past L


@pytest.mark.parametrize("pdl", [1, 0])
def test_dependent_back_to_back_launches_with_and_without_programmatic_launch(ctx, pdl):
    """Each copy reads what the previous copy in the stream wrote (scatter into B, gather from B, scatter into
    C, ...): with programmatic stream serialisation the next kernel starts early but must not read early."""
    ctx.set_option(_lib.OPT_PDL, pdl)
    assert ctx.get_option(_lib.OPT_PDL) == pdl
    src_cpu, guard_cpu, a, b = _pools(ctx)
    c = KVPool(to_gpu(guard_cpu), ctx)
    g = torch.Generator().manual_seed(3)
    tabs = [a.upload_ids(torch.randperm(GEOM["NB"], generator=g)[:120].tolist()) for _ in range(12)]
    hosts = [t.cpu().tolist() for t in tabs]
    buf = a.new_packed(120)
    pools, cpu = [a, b, c], [src_cpu, [t.clone() for t in guard_cpu], [t.clone() for t in guard_cpu]]
    for k in range(11):                                      # no synchronisation anywhere in the chain
        s, d = pools[k % 3], pools[(k + 1) % 3]
        s.gather(tabs[k], out=buf)
        d.scatter(tabs[k + 1], buf)
    for k in range(11):
        kv_oracle.write_kv_blocks(cpu[(k + 1) % 3], hosts[k + 1], kv_oracle.extract_kv_blocks(cpu[k % 3], hosts[k]))
    assert_clean(ctx)
    for p, want in zip(pools, cpu):
        assert pools_equal(p.layers, want)


def test_bound_append_raw_call_reports_a_bad_layer(ctx):
    _, _, pool, _ = _pools(ctx)
    T = 9
    key = torch.randn(GEOM["L"], T, GEOM["H"], GEOM["D"], device="cuda").to(torch.bfloat16)
    slots = torch.arange(T, device="cuda", dtype=torch.int64)
    bound = pool.bind_append(key, key, slots)
    stream = torch.cuda.current_stream().cuda_stream
    assert bound.raw(0, stream) == _lib.OK
    assert bound.raw(GEOM["L"], stream) == _lib.ERR_BAD_ARG
    with pytest.raises(EmmError):
        bound(-1)
    torch.cuda.synchronize()
    assert torch.equal(pool.layers[0][0, 0, :T].view(torch.int16), key[0].view(torch.int16))
    bound.release()
