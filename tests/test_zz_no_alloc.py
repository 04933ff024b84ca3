"""The allocation-free gather entry point against the ordinary one.

Some callers of this library cannot allocate device memory on the KV path: a
serving process whose own caching allocator already owns almost all of HBM, or
a section that cannot tolerate the device-wide synchronisation a cudaMalloc or
cudaFree implies. `emm_gather_noalloc` serves them from a fixed scratch array
inside the library. This file is collected last on purpose, so a run that
stops at the first failure has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from elasticmm_b200 import KVPool, _lib, get_context
from gpu_util import BULK_DEFAULT, configure
from oracle import kv_oracle

pytestmark = pytest.mark.gpu


def _noalloc_gather(pool: KVPool, ids, out: torch.Tensor) -> int:
    lib = _lib.load()
    host = np.ascontiguousarray(ids, dtype=np.int64)
    ptrs = (C.c_void_p * pool.num_layers)(*pool.layer_ptrs)
    stream = torch.cuda.current_stream(pool.device).cuda_stream
    return lib.emm_gather_noalloc(pool.device.index, C.byref(pool.desc), ptrs, host.ctypes.data_as(C.c_void_p),
                                  len(host), C.c_void_p(out.data_ptr()), out.numel() * out.element_size(),
                                  C.c_void_p(stream))


@pytest.mark.parametrize("geom", [
    dict(L=4, NB=96, BS=16, H=8, D=128, dtype=torch.bfloat16),   # 32 KiB pages: bulk-copy kernel
    dict(L=3, NB=40, BS=4, H=3, D=5, dtype=torch.float16),       # 120-byte pages: register kernel
], ids=["pages_32KiB", "pages_120B"])
def test_two_calls_in_a_row_match_the_allocating_entry(geom):
    ctx = get_context(0)
    cpu = kv_oracle.make_pool(geom["L"], geom["NB"], geom["BS"], geom["H"], geom["D"], geom["dtype"], 17)
    pool = KVPool([t.cuda() for t in cpu], ctx)
    g = torch.Generator().manual_seed(3)
    first = torch.randperm(geom["NB"], generator=g)[:29].tolist()
    second = torch.randperm(geom["NB"], generator=g)[:11].tolist()   # shorter: stale table entries must not matter
    for ids in (first, second):
        want = pool.gather(ids)                       # emm_gather_h
        got = torch.full_like(want, 7.0)
        assert _noalloc_gather(pool, ids, got) == _lib.OK, _lib.last_error()
        torch.cuda.synchronize()
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))    # bit-exact, as every parity test here
        assert kv_oracle.bit_equal(got.cpu(), kv_oracle.extract_kv_blocks(cpu, ids))
    assert ctx.status()[0] == _lib.OK


def test_a_warm_call_allocates_nothing_and_the_largest_table_fits():
    """Free device memory is the same before and after a warm call (the caller owns the
    output), also at the largest table the fixed array holds."""
    ctx = get_context(0)
    cpu = kv_oracle.make_pool(2, 8, 4, 2, 8, torch.float16, 2)             # 128-byte pages
    pool = KVPool([t.cuda() for t in cpu], ctx)
    n = _lib.NOALLOC_MAX_IDS
    ids = (torch.arange(n) * 5 % 8).tolist()                                # repeats are fine for a gather
    out = pool.new_packed(n)
    assert _noalloc_gather(pool, ids[:7], out[:, :, :7].contiguous()) == _lib.OK   # first call on the device: set-up
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(0)
    assert _noalloc_gather(pool, ids, out) == _lib.OK, _lib.last_error()
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info(0)
    assert free_after == free_before
    want = kv_oracle.extract_kv_blocks(cpu, ids)
    assert kv_oracle.bit_equal(out.cpu(), want)


def test_a_capturing_stream_is_refused():
    """The table is uploaded from host memory at call time, so the entry refuses a stream under capture."""
    ctx = get_context(0)
    cpu = kv_oracle.make_pool(2, 8, 4, 2, 8, torch.float16, 3)
    pool = KVPool([t.cuda() for t in cpu], ctx)
    out = pool.new_packed(2)
    assert _noalloc_gather(pool, [1, 2], out) == _lib.OK                    # set-up outside any capture
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            rc = _noalloc_gather(pool, [1, 2], out)
            out.add_(0)                                                     # keep the captured graph non-empty
    assert rc == _lib.ERR_BAD_ARG
    assert b"capturing" in _lib.load().emm_last_error()
    torch.cuda.synchronize()
    assert _noalloc_gather(pool, [3, 4], out) == _lib.OK
    torch.cuda.synchronize()
    assert kv_oracle.bit_equal(out.cpu(), kv_oracle.extract_kv_blocks(cpu, [3, 4]))


def test_a_small_ring_here_leaves_the_larger_launches_of_a_context_working():
    """Both entry points launch the same kernel, whose shared-memory limit is
    per device: a 16 KiB-page call here (96 KiB ring) between two 128 KiB-ring
    gathers of a context must not make the second one fail."""
    ctx = get_context(0)
    configure(ctx, **BULK_DEFAULT)
    big_cpu = kv_oracle.make_pool(2, 16, 16, 32, 128, torch.float16, 4)      # 128 KiB pages
    small_cpu = kv_oracle.make_pool(2, 16, 16, 4, 128, torch.float16, 5)     # 16 KiB pages
    big, small = KVPool([t.cuda() for t in big_cpu], ctx), KVPool([t.cuda() for t in small_cpu], ctx)
    ids = [3, 9, 1]
    assert kv_oracle.bit_equal(big.gather(ids).cpu(), kv_oracle.extract_kv_blocks(big_cpu, ids))
    got = small.new_packed(len(ids))
    assert _noalloc_gather(small, ids, got) == _lib.OK, _lib.last_error()
    assert kv_oracle.bit_equal(got.cpu(), kv_oracle.extract_kv_blocks(small_cpu, ids))
    assert kv_oracle.bit_equal(big.gather(ids).cpu(), kv_oracle.extract_kv_blocks(big_cpu, ids))
    assert ctx.status()[0] == _lib.OK


def test_limits_and_bad_arguments_are_refused_with_a_message():
    ctx = get_context(0)
    cpu = kv_oracle.make_pool(2, 8, 4, 2, 8, torch.float16, 1)
    pool = KVPool([t.cuda() for t in cpu], ctx)
    out = pool.new_packed(3)
    lib = _lib.load()
    too_many = list(range(8)) * ((_lib.NOALLOC_MAX_IDS // 8) + 1)
    big = torch.empty(1, dtype=torch.float16, device="cuda")
    assert _noalloc_gather(pool, too_many, big) == _lib.ERR_TOO_LARGE
    assert b"exceed the fixed maximum" in lib.emm_last_error()
    assert _noalloc_gather(pool, [0, 1, 8], out) == _lib.ERR_ID_RANGE
    assert _noalloc_gather(pool, [0, 1], out) == _lib.ERR_LENGTH
    assert _noalloc_gather(pool, [], pool.new_packed(0)) == _lib.OK
    layers = _lib.PoolDesc.from_buffer_copy(pool.desc)
    layers.num_layers = _lib.NOALLOC_MAX_LAYERS + 1
    ptrs = (C.c_void_p * (layers.num_layers))(*([pool.layer_ptrs[0]] * layers.num_layers))
    host = np.array([0], dtype=np.int64)
    rc = lib.emm_gather_noalloc(0, C.byref(layers), ptrs, host.ctypes.data_as(C.c_void_p), 1,
                                C.c_void_p(out.data_ptr()), 0, None)
    assert rc == _lib.ERR_TOO_LARGE
