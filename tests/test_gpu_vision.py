"""Vision-embedding hand-off (encode -> prefill): block cache [blocks, tokens, dim] and request-keyed store."""
import asyncio

import pytest
import torch

from elasticmm_b200 import EmmError, KVPool, get_context
from elasticmm_b200.engine.v0 import NCCLCoordinator, TransferMethod, V0KVTransferManager, V0Worker
from gpu_util import BULK_DEFAULT, LDG_DEFAULT, assert_clean, configure, vid
from oracle import kv_oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("opts", [BULK_DEFAULT, LDG_DEFAULT], ids=vid)
@pytest.mark.parametrize("shape", [(40, 16, 3584, torch.bfloat16), (17, 9, 100, torch.float16), (8, 3, 5, torch.float32)],
                         ids=["qwen_16x3584", "odd_9x100", "tiny_fp32"])
def test_block_cache_gather_scatter_copy(opts, shape):
    ctx = get_context(0)
    configure(ctx, **opts)
    nb, t, e, dt = shape
    g = torch.Generator().manual_seed(nb)
    src_cpu = torch.randn(nb, t, e, generator=g).to(dt)
    dst_cpu = torch.zeros(nb + 3, t, e, dtype=dt)
    n = max(1, nb // 3)
    s = torch.randperm(nb, generator=g)[:n].tolist()
    d = torch.randperm(nb + 3, generator=g)[:n].tolist()
    src, dst = V0Worker(device="cuda:0"), V0Worker(device="cuda:0")
    src.bind_ve_block_cache(src_cpu.cuda())
    dst.bind_ve_block_cache(dst_cpu.cuda())
    data = src.extract_ve_blocks(s)
    want = kv_oracle.transfer_vision_blocks(src_cpu, dst_cpu, s, d)
    assert kv_oracle.bit_equal(data.cpu(), want)
    dst.write_ve_blocks(d, data)
    assert_clean(ctx)
    assert kv_oracle.bit_equal(dst.ve_blocks.cpu(), dst_cpu)
    # direct block copy between the two caches
    dst2 = KVPool([torch.zeros(nb + 3, t, e, dtype=dt, device="cuda")], ctx)
    src.ve_pool.copy_blocks(dst2, s, d)
    assert kv_oracle.bit_equal(dst2.layers[0].cpu(), dst_cpu)
    with pytest.raises(EmmError):
        src.ve_pool.copy_blocks(KVPool([torch.zeros(2, nb, t, 1, e, dtype=dt, device="cuda")], ctx), s, d)  # KV pool: planes differ
    with pytest.raises(Exception):
        src.ve_pool.append(0, data, data, torch.zeros(n, dtype=torch.int64, device="cuda"))
    configure(ctx)


def test_manager_hands_over_embeddings_by_request_and_by_block():
    coord = NCCLCoordinator()
    enc, pre = V0Worker(device="cuda:0"), V0Worker(device="cuda:0")
    mgr = V0KVTransferManager(TransferMethod.P2P_COPY, nccl_coordinator=coord)
    mgr.register_worker(coord.register_worker("encoding", 0), enc, "encoding")
    mgr.register_worker(coord.register_worker("prefill", 0), pre, "prefill")
    enc.init_ve_cache()
    emb = torch.randn(216, 3584, dtype=torch.bfloat16, device="cuda")
    enc.write_vision_blocks("req-1", emb)
    assert enc.get_ve_shape("req-1") == (216, 3584) and enc.get_ve_cache_keys() == ["req-1"]
    assert asyncio.run(mgr.transfer_vision_embeddings("req-1", "encoding", 0, [], "prefill", 0, []))
    assert torch.equal(pre.extract_vision_blocks("req-1"), emb)
    with pytest.raises(KeyError):
        pre.extract_vision_blocks("nope")
    # block form
    src_cpu = torch.randn(30, 16, 256).to(torch.float16)
    dst_cpu = torch.zeros(30, 16, 256, dtype=torch.float16)
    enc.bind_ve_block_cache(src_cpu.cuda())
    pre.bind_ve_block_cache(dst_cpu.cuda())
    assert asyncio.run(mgr.transfer_vision_embeddings("req-2", "encoding", 0, [3, 29, 7], "prefill", 0, [0, 1, 2]))
    kv_oracle.transfer_vision_blocks(src_cpu, dst_cpu, [3, 29, 7], [0, 1, 2])
    assert kv_oracle.bit_equal(pre.ve_blocks.cpu(), dst_cpu)
    assert not asyncio.run(mgr.transfer_vision_embeddings("req-3", "encoding", 0, [1, 2], "prefill", 0, [0]))
    assert not asyncio.run(mgr.transfer_vision_embeddings("req-3", "decoding", 5, [1], "prefill", 0, [0]))
