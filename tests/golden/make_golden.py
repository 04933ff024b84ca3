"""Generates the golden fixtures from the reference's own code.

    python tests/golden/make_golden.py

Runs only where the reference tree is present (see oracle/ref_loader.py). It
imports the reference's V0Worker, V0BlockManager, NCCLCoordinator and
V0KVTransferManager unmodified, drives them on seeded CPU inputs and writes
  tests/golden/kv_golden.npz    bit images of extract_kv_blocks / write_kv_blocks results
  tests/golden/host_golden.json block-table, rank-map and manager-statistics traces
The case list (geometry, dtype, seeds, ids) lives in tests/golden/cases.py so
the tests rebuild the identical inputs.
"""
from __future__ import annotations

import asyncio
import contextlib
import hashlib
import io
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)

from oracle import kv_oracle, ref_loader  # noqa: E402
import cases  # noqa: E402


def bits_np(t: torch.Tensor) -> np.ndarray:
    return kv_oracle.bits(t).numpy().copy()


def digest(t: torch.Tensor) -> str:
    return hashlib.sha256(bits_np(t).tobytes()).hexdigest()


def kv_cases() -> dict:
    out = {}
    for case in cases.KV_CASES:
        pool, dst = cases.build_pools(case)
        worker = ref_loader.make_worker(pool)
        packed = worker.extract_kv_blocks(case["src_ids"])
        if case["store"] == "full":
            out[f"{case['name']}/packed"] = bits_np(packed)
        out[f"{case['name']}/packed_sha256"] = np.frombuffer(bytes.fromhex(digest(packed)), dtype=np.uint8)
        out[f"{case['name']}/packed_shape"] = np.array(packed.shape, dtype=np.int64)
        if case["dst_ids"] is not None:
            sink = ref_loader.make_worker(dst)
            sink.write_kv_blocks(case["dst_ids"], packed)
            whole = torch.stack(dst, dim=0)
            if case["store"] == "full":
                out[f"{case['name']}/dst_pool"] = bits_np(whole)
            out[f"{case['name']}/dst_pool_sha256"] = np.frombuffer(bytes.fromhex(digest(whole)), dtype=np.uint8)
    return out


def block_manager_traces() -> list:
    traces = []
    for script in cases.BLOCK_MANAGER_SCRIPTS:
        with contextlib.redirect_stdout(io.StringIO()):
            bm = ref_loader.make_block_manager("prefill", script["gpu_blocks"], script["cpu_blocks"],
                                               script["block_size"])
            reqs = {}
            steps = []
            for op in script["ops"]:
                kind = op[0]
                if kind == "alloc":
                    _, rid, tokens = op
                    reqs[rid] = ref_loader.make_request(rid, tokens)
                    bm.allocate_blocks(reqs[rid])
                elif kind == "alloc_n":
                    _, rid, tokens, n = op
                    reqs[rid] = ref_loader.make_request(rid, tokens)
                    bm.allocate_blocks(reqs[rid], n)
                elif kind == "grow":
                    _, rid, extra = op
                    reqs[rid].output_token_ids.extend([0] * extra)
                    bm.append_blocks(reqs[rid])
                elif kind == "expand":
                    _, rid, seq_len = op
                    bm.expand_blocks_for_seq_len(rid, seq_len)
                elif kind == "free":
                    bm.free_blocks(op[1])
                elif kind == "swap_out":
                    bm.swap_out_requests(list(op[1]))
                elif kind == "swap_in":
                    bm.swap_in_requests(list(op[1]))
                else:
                    raise ValueError(kind)
                steps.append({
                    "tables": {k: list(v) for k, v in bm.block_table.items()},
                    "free_gpu": list(bm.free_gpu_blocks_list),
                    "free_cpu": list(bm.free_cpu_blocks_list),
                    "swapping_gpu": list(bm.swapping_gpu_blocks_list),
                    "swapping_cpu": list(bm.swapping_cpu_blocks_list),
                    "locations": {k: v.value for k, v in bm.request_location.items()},
                    "avail_gpu": bm.get_num_avail_gpu_blocks(),
                })
        traces.append({"name": script["name"], "steps": steps})
    return traces


def coordinator_trace() -> list:
    with contextlib.redirect_stdout(io.StringIO()):
        coord = ref_loader.load("nccl_coordinator").NCCLCoordinator()
        steps = []
        for op in cases.COORDINATOR_SCRIPT:
            kind = op[0]
            if kind == "register":
                res = coord.register_worker(op[1], op[2])
            elif kind == "unregister":
                res = coord.unregister_worker(op[1], op[2])
            elif kind == "switch":
                res = coord.update_worker_role(op[1], op[2], op[3])
            elif kind == "rank":
                res = coord.get_rank(op[1], op[2])
            else:
                raise ValueError(kind)
            steps.append({"result": res, "world": coord.get_world_size(),
                          "ranks": sorted([s, w, r] for (s, w), r in coord.get_all_workers().items()),
                          "init_method": coord.get_init_method()})
    return steps


class _Remote:
    """Actor-method stand-in: `.remote(...)` runs the bound method and returns an awaitable."""

    def __init__(self, fn):
        self._fn = fn

    def remote(self, *a, **k):
        async def run():
            return self._fn(*a, **k)
        return run()


class _Handle:
    def __init__(self, worker):
        self.extract_kv_blocks = _Remote(worker.extract_kv_blocks)
        self.write_kv_blocks = _Remote(worker.write_kv_blocks)


def manager_trace() -> dict:
    """V0KVTransferManager on its default p2p_copy path with in-process workers."""
    case = cases.MANAGER_CASE
    src_pool, dst_pool = cases.build_pools(case)
    kt = ref_loader.load("kv_transfer")
    calls = []
    with contextlib.redirect_stdout(io.StringIO()):
        mgr = kt.V0KVTransferManager(transfer_method=kt.TransferMethod.P2P_COPY,
                                     metrics_callback=lambda transfer_time_sec, num_blocks: calls.append(num_blocks))
        mgr.register_worker(0, _Handle(ref_loader.make_worker(src_pool)), "prefill")
        mgr.register_worker(1, _Handle(ref_loader.make_worker(dst_pool)), "decoding")
        results = []
        for rid, src_ids, dst_ids, src_rank, dst_rank in case["transfers"]:
            ok = asyncio.run(mgr.transfer_kv_cache(rid, src_rank, dst_rank, src_ids, dst_ids))
            results.append(bool(ok))
        stats = mgr.get_stats()
        mgr.update_worker_stage(0, "DECODING")
        stage_after = mgr.rank_to_stage[0]
    return {
        "results": results,
        "callback_blocks": calls,
        "transfer_count": stats["transfer_count"],
        "stage_after_switch": stage_after,
        "dst_pool_sha256": digest(torch.stack(dst_pool, dim=0)),
        "methods": sorted(m.value for m in kt.TransferMethod),
    }


def main() -> None:
    if not ref_loader.reference_available():
        raise SystemExit("reference tree not present; fixtures can only be generated beside it")
    np.savez_compressed(os.path.join(HERE, "kv_golden.npz"), **kv_cases())
    host = {
        "block_manager": block_manager_traces(),
        "coordinator": coordinator_trace(),
        "manager": manager_trace(),
        "torch": torch.__version__,
    }
    with open(os.path.join(HERE, "host_golden.json"), "w") as f:
        json.dump(host, f, indent=1, sort_keys=True)
    print("wrote kv_golden.npz and host_golden.json")


if __name__ == "__main__":
    main()
