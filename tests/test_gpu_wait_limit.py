"""The bounded device-side wait of the bulk-copy kernel, made to run out.

No GPU fault, trap or endless loop is involved: a test-only entry over-counts
the bytes each load is expected to deliver, so the kernel's waits cannot
complete; with the limit set to one millisecond every lane gives up, records
EMM_ERR_TIMEOUT and returns, and the context keeps working. The reference's
counterpart is its host-side poll with a deadline
(elasticmm/engine/v0/worker.py:806-812).
"""
import ctypes as C
import time

import pytest
import torch

from elasticmm_b200 import KVPool, _lib, get_context
from gpu_util import BULK_DEFAULT, configure
from oracle import kv_oracle

pytestmark = pytest.mark.gpu


def test_wait_runs_out_status_is_timeout_and_the_context_stays_usable():
    ctx = get_context(0)
    configure(ctx, **BULK_DEFAULT)
    default_limit = ctx.get_option(_lib.OPT_WAIT_LIMIT_NS)
    assert default_limit == 2_000_000_000
    cpu = kv_oracle.make_pool(2, 16, 16, 8, 128, torch.bfloat16, 9)       # 32 KiB pages
    pool = KVPool([t.cuda() for t in cpu], ctx)
    ids = [5, 2, 11]
    table = pool.upload_ids(ids)
    out = pool.new_packed(len(ids))
    ptr, nbytes = pool._packed_ptr(out, len(ids), pool.num_layers)
    lib = _lib.load()
    ctx.set_option(_lib.OPT_WAIT_LIMIT_NS, 1_000_000)                      # 1 ms
    try:
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        rc = lib.emm_test_gather_expect_overcount(pool._h, C.c_void_p(table.data_ptr()), len(ids), C.c_void_p(ptr),
                                                  nbytes, 16, C.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert rc == _lib.OK, _lib.last_error()
        status, detail = ctx.status()                                       # synchronises: the kernel has RETURNED
        elapsed = time.perf_counter() - t0
        assert status == _lib.ERR_TIMEOUT
        assert 0 <= detail < 2 * 2 * len(ids) * 8                           # the chunk index a lane was waiting for
        assert elapsed < 1.0, f"kernel took {elapsed:.3f} s with a 1 ms limit"
        assert ctx.status()[0] == _lib.OK                                   # sticky status was cleared by the read
    finally:
        ctx.set_option(_lib.OPT_WAIT_LIMIT_NS, default_limit)
    # the next ordinary gather and scatter are bit-exact
    got = pool.gather(ids)
    assert kv_oracle.bit_equal(got.cpu(), kv_oracle.extract_kv_blocks(cpu, ids))
    assert ctx.status()[0] == _lib.OK


def test_wait_limit_option_is_range_checked():
    ctx = get_context(0)
    lib = _lib.load()
    assert lib.emm_ctx_set_option(ctx._h, _lib.OPT_WAIT_LIMIT_NS, 10) == _lib.ERR_BAD_ARG
    assert lib.emm_ctx_set_option(ctx._h, _lib.OPT_WAIT_LIMIT_NS, 10 ** 12) == _lib.ERR_BAD_ARG
    assert ctx.get_option(_lib.OPT_WAIT_LIMIT_NS) == 2_000_000_000
