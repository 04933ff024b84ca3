"""Input definitions shared by the fixture generator and the tests.

Every KV case is rebuilt from its seed: the source pool is N(0,1) cast to the
case dtype, the destination pool is filled with the guard word 0x7FFF so that
bytes no write touched stay recognisable.
"""
from __future__ import annotations

import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from oracle import kv_oracle  # noqa: E402

_DT = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}


def _perm(n: int, seed: int, k: int) -> list:
    g = torch.Generator().manual_seed(seed)
    return torch.randperm(n, generator=g)[:k].tolist()


def _case(name, L, NB, BS, H, D, dtype, seed, src_ids, dst_ids, dst_NB=None, store="full"):
    return dict(name=name, L=L, NB=NB, BS=BS, H=H, D=D, dtype=dtype, seed=seed, src_ids=src_ids,
                dst_ids=dst_ids, dst_NB=dst_NB or NB, store=store)


KV_CASES = [
    _case("fp16_basic", 3, 12, 4, 2, 8, "float16", 11, [5, 1, 7, 10], [0, 3, 2, 9]),
    _case("bf16_single", 2, 8, 16, 4, 16, "bfloat16", 12, [6], [1]),
    _case("all_blocks_permuted", 2, 16, 4, 2, 8, "float16", 13, _perm(16, 1, 16), _perm(16, 2, 16)),
    _case("gather_duplicates", 2, 8, 4, 2, 8, "float16", 14, [3, 3, 0, 3], None),
    _case("odd_page_120B", 3, 9, 4, 3, 5, "float16", 15, [8, 0, 4], [2, 7, 1]),
    _case("odd_page_6B", 2, 7, 1, 3, 1, "bfloat16", 16, [6, 2, 5, 0], [1, 0, 4, 3]),
    _case("fp32", 2, 10, 4, 2, 8, "float32", 17, [9, 4, 2], [0, 5, 7]),
    _case("empty", 2, 6, 4, 2, 8, "float16", 18, [], []),
    _case("different_pool_sizes", 2, 12, 4, 2, 8, "bfloat16", 19, [11, 2, 6], [1, 19, 0], dst_NB=20),
    # Page sizes of the benchmark geometries (only digests are stored).
    _case("llama7b_page_128KiB", 2, 24, 16, 32, 128, "float16", 21, _perm(24, 3, 9), _perm(24, 4, 9), store="sha"),
    _case("qwen25vl_page_16KiB", 3, 40, 16, 4, 128, "bfloat16", 22, _perm(40, 5, 17), _perm(40, 6, 17), store="sha"),
    _case("llava13b_page_160KiB", 2, 12, 16, 40, 128, "float16", 23, _perm(12, 7, 5), _perm(12, 8, 5), store="sha"),
    _case("gqa70b_page_32KiB", 4, 32, 16, 8, 128, "bfloat16", 24, _perm(32, 9, 13), _perm(32, 10, 13), store="sha"),
]


# Per-token append (reshape_and_cache). The expected pools come from vLLM's own cache op
# (vllm._custom_ops.reshape_and_cache_flash, the op behind the reference's
# model_runner.execute_model, elasticmm/engine/v0/worker_steps.py:281,438) run by
# make_append_golden.py on a CUDA machine. pad_every > 0 sets every pad_every-th slot to -1.
# Every head row here is a multiple of 16 bytes: vLLM's kernel copies 16-byte vectors and raised
# "misaligned address" on 10-byte head rows, so odd head sizes are covered by the oracle-only tests.
def _append_case(name, L, NB, BS, H, D, dtype, seed, T, pad_every, store="full"):
    return dict(name=name, L=L, NB=NB, BS=BS, H=H, D=D, dtype=dtype, seed=seed, T=T, pad_every=pad_every,
                store=store)


APPEND_CASES = [
    _append_case("gqa8_row_2KiB", 3, 12, 16, 8, 128, "bfloat16", 41, 37, 7, store="sha"),
    _append_case("mha32_row_8KiB", 2, 6, 16, 32, 128, "float16", 42, 9, 4, store="sha"),
    _append_case("hd64_row_384B", 2, 9, 4, 3, 64, "float16", 43, 21, 5),
    _append_case("fp32_hd32_row_256B", 2, 6, 8, 2, 32, "float32", 44, 5, 0),
    _append_case("every_slot", 1, 5, 16, 1, 64, "bfloat16", 45, 80, 0),
    _append_case("all_padding", 1, 4, 16, 2, 64, "float16", 46, 6, 1),
    # BASELINE config 2's shape (256 tokens, 8 KV heads, head_dim 128, bf16, 32 layers, 1 % padding) on a
    # pool cut to 128 blocks per layer; only the digest of the resulting pool is stored.
    _append_case("cfg2_decode_batch_256", 32, 128, 16, 8, 128, "bfloat16", 47, 256, 100, store="sha"),
]


def build_append_inputs(case):
    """(pool, key [L,T,H,D], value [L,T,H,D], slot_mapping [T] int64), all CPU tensors rebuilt from the seed."""
    dt = _DT[case["dtype"]]
    L, NB, BS, H, D, T = (case[k] for k in ("L", "NB", "BS", "H", "D", "T"))
    pool = kv_oracle.make_pool(L, NB, BS, H, D, dt, case["seed"])
    g = torch.Generator().manual_seed(case["seed"] + 1000)
    key = torch.randn(L, T, H, D, generator=g).to(dt)
    value = torch.randn(L, T, H, D, generator=g).to(dt)
    slots = torch.randperm(NB * BS, generator=g)[:T].clone()
    if case["pad_every"]:
        slots[::case["pad_every"]] = -1
    return pool, key, value, slots


def build_pools(case):
    """(source pool, guard-filled destination pool) as lists of CPU tensors."""
    dt = _DT[case["dtype"]]
    src = kv_oracle.make_pool(case["L"], case["NB"], case["BS"], case["H"], case["D"], dt, case["seed"])
    if dt == torch.float32:
        dst = [torch.full((2, case["dst_NB"], case["BS"], case["H"], case["D"]), -7.5, dtype=dt)
               for _ in range(case["L"])]
    else:
        dst = kv_oracle.make_pool(case["L"], case["dst_NB"], case["BS"], case["H"], case["D"], dt, 0, fill="guard")
    return src, dst


BLOCK_MANAGER_SCRIPTS = [
    dict(name="fifo_fragmentation", gpu_blocks=24, cpu_blocks=8, block_size=4, ops=[
        ("alloc", "a", 10), ("alloc", "b", 4), ("alloc", "c", 17), ("free", "b"), ("alloc", "d", 9),
        ("grow", "a", 7), ("free", "a"), ("alloc", "e", 20), ("expand", "d", 14), ("free", "c"),
        ("alloc_n", "f", 3, 4),
    ]),
    dict(name="swap_round_trip", gpu_blocks=18, cpu_blocks=12, block_size=16, ops=[
        ("alloc", "r0", 40), ("alloc", "r1", 70), ("alloc", "r2", 16), ("swap_out", ("r1",)),
        ("alloc", "r3", 33), ("swap_out", ("r0", "r2")), ("swap_in", ("r1",)), ("alloc", "r4", 100),
        ("free", "r3"), ("swap_in", ("r2", "r0")), ("free", "r1"),
    ]),
]

COORDINATOR_SCRIPT = [
    ("register", "encoding", 0), ("register", "prefill", 0), ("register", "prefill", 1),
    ("register", "decoding", 0), ("register", "prefill", 1), ("rank", "prefill", 1),
    ("switch", 1, "prefill", "decoding"), ("rank", "decoding", 1), ("rank", "prefill", 1),
    ("unregister", "encoding", 0), ("register", "encoding", 3), ("rank", "missing", 9),
    ("switch", 7, "prefill", "decoding"),
]

MANAGER_CASE = dict(
    name="manager_p2p_copy", L=2, NB=16, BS=4, H=2, D=8, dtype="float16", seed=31, dst_NB=16,
    transfers=[
        ("req-0", [3, 9, 1], [0, 1, 2], 0, 1),
        ("req-1", [4], [7], 0, 1),
        ("req-2", [5, 6], [9, 8], 0, 1),
        ("req-3", [0], [3], 5, 1),  # unknown source rank: must report failure
    ],
)
