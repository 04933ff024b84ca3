"""The CUDA append against the third-party op the reference actually runs.

In the reference the new-token K/V rows are written inside
model_runner.execute_model (elasticmm/engine/v0/worker_steps.py:281,438) by
vLLM's reshape_and_cache_flash on the pool bound at
elasticmm/engine/v0/worker.py:380-412. When that op loads on the machine,
these tests run it and emm_append / emm_append_all_layers on identical seeded
inputs and compare whole pools bit for bit; the CPU oracle is compared with the
op as well. When it does not load, every test here skips with the import error
as the reason. Collected after the other GPU tests because importing vLLM is
slow and registers its own operators in the process.
"""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))

import cases  # noqa: E402
from elasticmm_b200 import KVPool, get_context  # noqa: E402
from gpu_util import assert_clean, configure  # noqa: E402
from oracle import kv_oracle  # noqa: E402

pytestmark = pytest.mark.gpu

_OP = {}


def vllm_op():
    """vllm._custom_ops.reshape_and_cache_flash, or skip with the reason it is unavailable."""
    if "fn" not in _OP:
        try:
            import make_append_golden

            _OP["fn"], _OP["version"] = make_append_golden.load_vllm_op()
        except BaseException as e:  # vLLM's import can raise anything, SystemExit included
            _OP["fn"], _OP["error"] = None, f"{type(e).__name__}: {e}"
    if _OP["fn"] is None:
        pytest.skip(f"vLLM's reshape_and_cache_flash is not usable here: {_OP['error']}")
    return _OP["fn"]


def run_vllm(op, layers, key, value, slots):
    one = torch.ones(1, dtype=torch.float32, device=key.device)
    for l, layer in enumerate(layers):
        op(key[l], value[l], layer[0], layer[1], slots, "auto", one, one)


def pools_bit_equal(a_layers, b_layers):
    return all(torch.equal(kv_oracle.bits(a), kv_oracle.bits(b)) for a, b in zip(a_layers, b_layers))


@pytest.mark.parametrize("case", cases.APPEND_CASES, ids=lambda c: c["name"])
def test_append_equals_vllm_cache_op(case):
    op = vllm_op()
    ctx = get_context(0)
    configure(ctx)
    pool_cpu, key, value, slots = cases.build_append_inputs(case)
    key_d, value_d, slots_d = key.cuda(), value.cuda(), slots.cuda()
    want = [t.cuda() for t in pool_cpu]
    run_vllm(op, want, key_d, value_d, slots_d)
    torch.cuda.synchronize()

    per_layer = KVPool([t.cuda() for t in pool_cpu], ctx)
    for l in range(case["L"]):
        per_layer.append(l, key_d[l], value_d[l], slots_d)
    all_layers = KVPool([t.cuda() for t in pool_cpu], ctx)
    all_layers.append_all_layers(key_d, value_d, slots_d)
    bound_pool = KVPool([t.cuda() for t in pool_cpu], ctx)
    bound = bound_pool.bind_append(key_d, value_d, slots_d)
    for l in range(case["L"]):
        bound(l)
    assert_clean(ctx)
    assert pools_bit_equal(per_layer.layers, want), "emm_append differs from vLLM's op"
    assert pools_bit_equal(all_layers.layers, want), "emm_append_all_layers differs from vLLM's op"
    assert pools_bit_equal(bound_pool.layers, want), "bound per-layer append differs from vLLM's op"

    # and the CPU restatement the other append tests use as their oracle
    for l in range(case["L"]):
        kv_oracle.reshape_and_cache(key[l], value[l], pool_cpu[l], slots)
    assert all(kv_oracle.bit_equal(w.cpu(), o) for w, o in zip(want, pool_cpu)), "oracle differs from vLLM's op"


def test_append_config2_full_pool_equals_vllm_cache_op():
    """BASELINE config 2 at full size: 32 layers, 16384 blocks, [256, 8, 128] bf16 per layer, 1 % padding."""
    op = vllm_op()
    free, _ = torch.cuda.mem_get_info(0)
    if free < 72 * (1 << 30):
        pytest.skip("needs 72 GiB of free device memory (two 32 GiB pools)")
    ctx = get_context(0)
    configure(ctx)
    L, NB, BS, H, D, T = 32, 16384, 16, 8, 128, 256
    gd = torch.Generator(device="cuda").manual_seed(2)
    ours = [torch.randn((2, NB, BS, H, D), generator=gd, device="cuda", dtype=torch.bfloat16) for _ in range(L)]
    theirs = [t.clone() for t in ours]
    g = torch.Generator().manual_seed(2)
    pool = KVPool(ours, ctx)
    for step in range(3):  # three decode steps, per-layer calls then the all-layers call on fresh slots
        key = torch.randn(L, T, H, D, generator=gd, device="cuda", dtype=torch.bfloat16)
        value = torch.randn(L, T, H, D, generator=gd, device="cuda", dtype=torch.bfloat16)
        slots = torch.randperm(NB * BS, generator=g)[:T].clone()
        slots[torch.randperm(T, generator=g)[:3]] = -1
        slots_d = slots.cuda()
        run_vllm(op, theirs, key, value, slots_d)
        if step % 2 == 0:
            for l in range(L):
                pool.append(l, key[l], value[l], slots_d)
        else:
            pool.append_all_layers(key, value, slots_d)
    assert_clean(ctx)
    assert pools_bit_equal(ours, theirs)
