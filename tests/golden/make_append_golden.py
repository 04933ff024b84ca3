"""Generates the append fixture from vLLM's own cache op.

    python tests/golden/make_append_golden.py [--out tests/golden/append_golden.npz]

The reference never writes new-token K/V itself: the write happens inside
model_runner.execute_model (elasticmm/engine/v0/worker_steps.py:281,438), which
calls vLLM's reshape_and_cache_flash on the pool bound at
elasticmm/engine/v0/worker.py:380-412 (one tensor [2, NB, BS, H, D] per layer,
K plane = t[0], V plane = t[1]). This script runs that op
(vllm._custom_ops.reshape_and_cache_flash, kv_cache_dtype "auto") on the seeded
inputs of cases.APPEND_CASES and stores the resulting pools, so that the CPU
oracle and the CUDA kernel can be checked against the third-party op's own
output where vLLM cannot load. It needs a CUDA device and a loadable vLLM
extension; it exits with a message otherwise.
"""
from __future__ import annotations

import argparse
import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)

from oracle import kv_oracle  # noqa: E402
import cases  # noqa: E402


def load_vllm_op():
    """The op, or raises with the reason it cannot be used here."""
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device")
    import vllm  # noqa: F401
    import vllm._custom_ops as ops

    torch.ops._C_cache_ops.reshape_and_cache_flash  # AttributeError when the extension did not load
    return ops.reshape_and_cache_flash, vllm.__version__


def run_vllm(op, pool_cpu, key, value, slots, device="cuda:0"):
    """Applies the op layer by layer to a device copy of the pool; returns the pool on the CPU."""
    pool = [t.to(device) for t in pool_cpu]
    one = torch.ones(1, dtype=torch.float32, device=device)
    key_d, value_d, slots_d = key.to(device), value.to(device), slots.to(device)
    for l, layer in enumerate(pool):
        op(key_d[l], value_d[l], layer[0], layer[1], slots_d, "auto", one, one)
    torch.cuda.synchronize()
    return [t.cpu() for t in pool]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.join(HERE, "append_golden.npz"))
    args = ap.parse_args()
    try:
        op, version = load_vllm_op()
    except Exception as e:
        raise SystemExit(f"vLLM's cache op is not usable here: {type(e).__name__}: {e}")
    out = {"vllm_version": np.frombuffer(version.encode(), dtype=np.uint8)}
    for case in cases.APPEND_CASES:
        pool, key, value, slots = cases.build_append_inputs(case)
        after = torch.stack(run_vllm(op, pool, key, value, slots), dim=0)
        bits = kv_oracle.bits(after).numpy()
        if case["store"] == "full":
            out[f"{case['name']}/pool"] = bits.copy()
        out[f"{case['name']}/pool_sha256"] = np.frombuffer(hashlib.sha256(bits.tobytes()).digest(), dtype=np.uint8)
        print(case["name"], tuple(after.shape), hashlib.sha256(bits.tobytes()).hexdigest()[:16])
    np.savez_compressed(args.out, **out)
    print("wrote", args.out, os.path.getsize(args.out), "bytes; vLLM", version)


if __name__ == "__main__":
    main()
