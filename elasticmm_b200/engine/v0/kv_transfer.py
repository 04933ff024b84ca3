"""KV transfer orchestration with the reference's manager surface.

Mirrors V0KVTransferManager (elasticmm/engine/v0/kv_transfer.py): a registry
of workers keyed by global rank that survives role switches (:114-174),
`transfer_kv_cache(request_id, src_rank, dst_rank, src_blocks, dst_blocks)
-> bool` (:224-262), byte/time counters that leave out the first (cold)
transfer (:506-515, :843-859) and a metrics callback called as
`metrics_callback(transfer_time_sec=..., num_blocks=...)` for every transfer
(:518-519).

The reference's manager lives in a driver process and reaches workers through
Ray actor handles. Here a manager lives in each worker process (one process
per GPU): it holds the local worker object(s) and knows the other ranks only
by number. A transfer whose source and sink are both local runs entirely in
this process; otherwise this process performs its half (send or push on the
source, receive on the sink) and the peer process performs the other half by
making the same call.

Added: TransferMethod.B200_PEER (direct loads from / stores into a peer-mapped pool)
and `transfer_many(plan)`, which moves all requests of a role switch as one
table per (source, sink) pair instead of one call per request
(the reference serialises them, elasticmm/engine/v0/backend.py:674-718).
"""
from __future__ import annotations

import time
from enum import Enum
from typing import Any, Callable, Dict, List, Optional, Sequence

import torch

from .transport import MigrationPlan, Transfer


class TransferMethod(Enum):
    CUDA_IPC = "cuda_ipc"      # accepted as an alias of B200_PEER
    NCCL = "nccl"              # staged: pack -> NCCL send/recv -> unpack, pipelined by layer chunk
    P2P_COPY = "p2p_copy"      # extract on the source, write on the sink (both workers in this process)
    STAGED_COPY = "staged_copy"  # gather -> pinned host buffer -> scatter (a sleep stub in the reference)
    B200_PEER = "b200_peer"    # one kernel over peer-mapped pools: the sink loads (default) or the source stores


class V0KVTransferManager:
    def __init__(self, transfer_method: TransferMethod = TransferMethod.P2P_COPY, nccl_coordinator=None,
                 enable_batching: bool = False, batch_size: int = 3, batch_timeout: float = 0.005,
                 metrics_callback: Optional[Callable[..., None]] = None, peer_direction: str = "pull"):
        if peer_direction not in ("pull", "push"):
            raise ValueError("peer_direction must be 'pull' or 'push'")
        self.peer_direction = peer_direction  # B200_PEER: the sink loads (default) or the source stores
        self.transfer_method = transfer_method
        self.nccl_coordinator = nccl_coordinator
        self.enable_batching = enable_batching  # queue transfers per (source, sink) pair; see flush()
        self.metrics_callback = metrics_callback
        self.worker_registry: Dict[int, Any] = {}
        self.rank_to_stage: Dict[int, str] = {}
        self.ipc_mem_handles: Dict[str, Dict[int, Dict[str, Any]]] = {}
        self.transfer_count = 0
        self.total_transfer_time = 0.0
        self.total_bytes_transferred = 0
        self.first_transfer_done = False
        self.last_result: Dict[str, Any] = {}  # what the most recent transfer returned (bytes, blocks or error)
        self._host_stage: Optional[torch.Tensor] = None  # pinned buffer of the staged_copy method
        # batching: small transfers of one (source, sink) pair are merged into one table
        self._transfer_queue: Dict[tuple, List[tuple]] = {}
        self._last_flush_time: Dict[tuple, float] = {}
        self._batch_flush_threshold = batch_size
        self._batch_flush_timeout = batch_timeout

    @classmethod
    def from_config(cls, config, nccl_coordinator=None, **kwargs) -> "V0KVTransferManager":
        """A manager using the transfer method and peer direction of a
        V0KVCacheConfig (the reference passes `kv_transfer_method` as a string,
        elasticmm/engine/v0/config.py:35)."""
        config.validate()
        return cls(transfer_method=config.transfer_method, nccl_coordinator=nccl_coordinator,
                   peer_direction=config.peer_direction, **kwargs)

    # -- registry --------------------------------------------------------------
    @staticmethod
    def _normalize_stage(stage: Any) -> str:
        return str(getattr(stage, "value", stage)).lower()

    def register_worker(self, global_rank: int, worker: Any, stage: str) -> None:
        self.worker_registry[global_rank] = worker
        self.rank_to_stage[global_rank] = self._normalize_stage(stage)

    def register_workers(self, stage: str, workers: Sequence[Any], global_ranks: Sequence[int]) -> None:
        for worker, rank in zip(workers, global_ranks):
            if worker is not None and rank >= 0:
                self.register_worker(rank, worker, stage)

    def unregister_worker(self, global_rank: int) -> None:
        self.worker_registry.pop(global_rank, None)
        self.rank_to_stage.pop(global_rank, None)

    def update_worker_stage(self, global_rank: int, new_stage: str) -> None:
        """Role switch: only the stage label changes, the rank key stays."""
        if global_rank in self.worker_registry:
            self.rank_to_stage[global_rank] = self._normalize_stage(new_stage)

    def register_ipc_handle(self, stage: str, worker_id: int, cache_type: str, ipc_handle: Any) -> None:
        self.ipc_mem_handles.setdefault(stage, {}).setdefault(worker_id, {})[cache_type] = ipc_handle

    # -- transfers ---------------------------------------------------------------
    def _account(self, elapsed: float, nbytes: int, nblocks: int, count: int = 1) -> None:
        if self.transfer_method == TransferMethod.P2P_COPY:
            # the reference's copy path only counts transfers (kv_transfer.py:740)
            self.transfer_count += count
        elif not self.first_transfer_done:
            self.first_transfer_done = True  # cold start: not part of the averages (:506-515)
        else:
            self.transfer_count += count
            self.total_transfer_time += elapsed
            self.total_bytes_transferred += nbytes
        if self.metrics_callback:
            self.metrics_callback(transfer_time_sec=elapsed, num_blocks=nblocks)

    def _run(self, src_rank: int, dst_rank: int, src_blocks: List[int], dst_blocks: List[int]) -> Dict[str, Any]:
        src = self.worker_registry.get(src_rank)
        dst = self.worker_registry.get(dst_rank)
        method = self.transfer_method
        if method == TransferMethod.CUDA_IPC:
            method = TransferMethod.B200_PEER
        if src is None and dst is None:
            return {"error": f"neither rank {src_rank} nor rank {dst_rank} is local", "bytes": 0, "blocks": 0}
        if len(src_blocks) != len(dst_blocks):
            return {"error": f"Block count mismatch: src={len(src_blocks)}, dst={len(dst_blocks)}",
                    "bytes": 0, "blocks": 0}
        if method == TransferMethod.P2P_COPY:
            if src is None or dst is None:
                return {"error": "p2p_copy needs both workers in this process", "bytes": 0, "blocks": 0}
            data = src.extract_kv_blocks(src_blocks)
            if data.device != dst.device:
                data = data.to(dst.device, non_blocking=True)
            dst.write_kv_blocks(dst_blocks, data)
            torch.cuda.synchronize(dst.device)
            return {"bytes": data.numel() * data.element_size(), "blocks": len(src_blocks)}
        if method == TransferMethod.NCCL:
            if src is not None and dst is not None:
                return {"error": "nccl transfer needs source and sink in different processes",
                        "bytes": 0, "blocks": 0}
            if dst is not None:
                return dst.p2p_coordinated_transfer_kv(None, src_rank, src_blocks, dst_blocks, timeout=10.0)
            return src.p2p_send_kv(dst_rank, src_blocks)
        if method == TransferMethod.B200_PEER:
            if src is not None and dst is not None and src.device == dst.device:
                src.pool.copy_blocks(dst.pool, src_blocks, dst_blocks)                    # both pools on this GPU
                worker, res = src, {"bytes": len(src_blocks) * src.pool.block_bytes(), "blocks": len(src_blocks)}
            elif self.peer_direction == "pull":
                if dst is None:  # the sink does the copy; the source's half of the call is a no-op
                    return {"bytes": 0, "blocks": len(src_blocks), "passive": True}
                if src is not None and src_rank not in dst.peer_pools:
                    dst.attach_local_peer(src_rank, src)      # both workers in this process, two GPUs
                if src is not None:
                    # The sink's kernel reads the source GPU's pool: order it after whatever the source
                    # has queued on its current stream (the reference's send runs on the source's stream
                    # and is ordered after the prefill kernels in the same way).
                    ready = torch.cuda.Event()
                    ready.record(torch.cuda.current_stream(src.device))
                    torch.cuda.current_stream(dst.device).wait_event(ready)
                worker, res = dst, dst.p2p_pull_kv(src_rank, src_blocks, dst_blocks)      # sink loads over the link
            else:
                if src is None:
                    return {"bytes": 0, "blocks": len(src_blocks), "passive": True}
                if dst is not None and dst_rank not in src.peer_pools:
                    src.attach_local_peer(dst_rank, dst)
                worker, res = src, src.p2p_push_kv(dst_rank, src_blocks, dst_blocks)      # source stores over the link
            if "error" not in res:
                # The id lists were range-checked on the host before the launch, so the device status
                # word cannot hold a bad id here; waiting for the stream is all that is needed.
                torch.cuda.synchronize(worker.device)
            return res
        if method == TransferMethod.STAGED_COPY:
            # Through pinned host memory (the reference only sketches this method with a sleep,
            # elasticmm/engine/v0/kv_transfer.py:821-841): gather on the source GPU, one D2H and
            # one H2D copy of the packed buffer, scatter on the sink GPU. For pairs without a
            # peer mapping or a process group; bound by PCIe.
            if src is None or dst is None:
                return {"error": "staged_copy needs both workers in this process", "bytes": 0, "blocks": 0}
            data = src.extract_kv_blocks(src_blocks)
            nbytes = data.numel() * data.element_size()
            if self._host_stage is None or self._host_stage.numel() < nbytes:
                self._host_stage = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
            host = self._host_stage[:nbytes].view(data.dtype).view(data.shape)
            host.copy_(data, non_blocking=True)
            torch.cuda.synchronize(src.device)
            dst.write_kv_blocks(dst_blocks, host.to(dst.device, non_blocking=True))
            torch.cuda.synchronize(dst.device)
            return {"bytes": nbytes, "blocks": len(src_blocks)}
        return {"error": f"transfer method {self.transfer_method.value} is not implemented",
                "bytes": 0, "blocks": 0}

    async def transfer_kv_cache(self, request_id: str, src_rank: int, dst_rank: int,
                                src_blocks: List[int], dst_blocks: List[int]) -> bool:
        """True if the request's blocks were moved (same contract as the reference)."""
        return self.transfer_kv_cache_sync(request_id, src_rank, dst_rank, src_blocks, dst_blocks)

    def flush(self, src_rank: Optional[int] = None, dst_rank: Optional[int] = None) -> bool:
        """Moves what is queued for a pair (or for every pair) as one merged transfer per pair."""
        ok = True
        for key in [k for k in self._transfer_queue if (src_rank is None or k[0] == src_rank)
                    and (dst_rank is None or k[1] == dst_rank)]:
            queued = self._transfer_queue.pop(key, [])
            self._last_flush_time[key] = time.perf_counter()
            if not queued:
                continue
            src_all = [b for _, s, _ in queued for b in s]
            dst_all = [b for _, _, d in queued for b in d]
            start = time.perf_counter()
            try:
                src, dst = self.worker_registry.get(key[0]), self.worker_registry.get(key[1])
                if (self.transfer_method == TransferMethod.P2P_COPY and src is not None and dst is not None
                        and src.device == dst.device and hasattr(src, "extract_kv_blocks_many")):
                    # one launch per direction, one contiguous tensor per request
                    parts = src.extract_kv_blocks_many([s for _, s, _ in queued])
                    dst.write_kv_blocks_many([d for _, _, d in queued], parts)
                    torch.cuda.synchronize(dst.device)
                    res = {"bytes": sum(t.numel() * t.element_size() for t in parts), "blocks": len(src_all)}
                else:
                    res = self._run(key[0], key[1], src_all, dst_all)
            except Exception as e:
                res = {"error": f"{type(e).__name__}: {e}", "bytes": 0, "blocks": 0}
            self.last_result = res
            if "error" in res or (res.get("bytes", 0) == 0 and not res.get("passive")):
                ok = False
                continue
            self._account(time.perf_counter() - start, res.get("bytes", 0), len(src_all), count=len(queued))
        return ok

    def transfer_kv_cache_sync(self, request_id: str, src_rank: int, dst_rank: int,
                               src_blocks: List[int], dst_blocks: List[int]) -> bool:
        if self.enable_batching:
            # Merge small transfers of the same pair (the intent of the reference's batching branch,
            # elasticmm/engine/v0/kv_transfer.py:342-418,437-465): queue, and flush once `batch_size`
            # requests wait or `batch_timeout` has passed since the pair's last flush.
            if len(src_blocks) != len(dst_blocks):
                return False
            key = (src_rank, dst_rank)
            now = time.perf_counter()
            self._transfer_queue.setdefault(key, []).append((request_id, list(src_blocks), list(dst_blocks)))
            self._last_flush_time.setdefault(key, now)
            if (len(self._transfer_queue[key]) >= self._batch_flush_threshold
                    or now - self._last_flush_time[key] >= self._batch_flush_timeout):
                return self.flush(src_rank, dst_rank)
            return True  # queued; moved by a later call or by flush()
        start = time.perf_counter()
        try:
            res = self._run(src_rank, dst_rank, src_blocks, dst_blocks)
        except Exception as e:
            res = {"error": f"{type(e).__name__}: {e}", "bytes": 0, "blocks": 0}
        elapsed = time.perf_counter() - start
        self.last_result = res
        if "error" in res:
            return False
        if res.get("bytes", 0) == 0 and not res.get("passive"):
            return False  # the reference treats 0 bytes as a failed transfer
        self._account(elapsed, res.get("bytes", 0), len(src_blocks))
        return True

    async def transfer_vision_embeddings(self, request_id: str, src_stage: str, src_worker_id: int,
                                         src_blocks: List[int], dst_stage: str, dst_worker_id: int,
                                         dst_blocks: List[int]) -> bool:
        """Encode -> prefill hand-off of a request's vision embeddings, with the reference's
        stage-keyed signature (elasticmm/engine/v0/kv_transfer.py:264-300). Workers are found through
        the coordinator's (stage, worker_id) -> rank map. A request-keyed embedding is handed over
        whole (:727-730); otherwise the block lists move through the block cache
        (elasticmm/engine/v0/nccl_transfer.py:295-368)."""
        if self.nccl_coordinator is None:
            return False
        src = self.worker_registry.get(self.nccl_coordinator.get_rank(self._normalize_stage(src_stage), src_worker_id))
        dst = self.worker_registry.get(self.nccl_coordinator.get_rank(self._normalize_stage(dst_stage), dst_worker_id))
        if src is None or dst is None:
            return False
        start = time.perf_counter()
        try:
            if src.ve_cache is not None and request_id in src.ve_cache:
                data = src.extract_vision_blocks(request_id)
                if dst.ve_cache is None:
                    dst.init_ve_cache()
                dst.write_vision_blocks(request_id, data if data.device == dst.device else data.to(dst.device))
            else:
                if len(src_blocks) != len(dst_blocks):
                    return False
                data = src.extract_ve_blocks(src_blocks)
                dst.write_ve_blocks(dst_blocks, data if data.device == dst.device else data.to(dst.device))
            torch.cuda.synchronize(dst.device)
        except Exception as e:
            self.last_result = {"error": f"{type(e).__name__}: {e}", "bytes": 0, "blocks": 0}
            return False
        self.transfer_count += 1
        self.last_result = {"bytes": data.numel() * data.element_size(), "blocks": len(src_blocks),
                            "elapsed": time.perf_counter() - start}
        return True

    def transfer_kv_cache_batch(self, transfers: Sequence[Transfer]) -> bool:
        """Moves several requests at once and returns when all of them have landed: the requests of
        each (source, sink) pair travel as one merged table (one launch per direction on the copy
        path). Per-request `transfer_kv_cache` stays synchronous by default, because the reference's
        engines read the destination blocks right after awaiting it
        (elasticmm/engine/v0/stage_engine.py:1506-1566); this is the call for a caller that has
        several requests in hand (the reference's own batching branch,
        elasticmm/engine/v0/kv_transfer.py:342-418, queues them and was switched off at
        elasticmm/engine/v0/backend.py:109 because nothing flushed the queue)."""
        for t in transfers:
            self._transfer_queue.setdefault((t.src_rank, t.dst_rank), []).append(
                (t.request_id, list(t.src_blocks), list(t.dst_blocks)))
        return self.flush()

    def transfer_many(self, plan: MigrationPlan) -> bool:
        """Moves a whole plan: one table per (source, sink) pair.

        Every process that owns a rank named in the plan makes this call. With
        B200_PEER the sinks pull and all ranks meet at a barrier; with NCCL
        each pair runs the staged pipeline.
        """
        start = time.perf_counter()
        method = self.peer_direction if self.transfer_method in (TransferMethod.B200_PEER, TransferMethod.CUDA_IPC) else "nccl"
        if self.transfer_method not in (TransferMethod.B200_PEER, TransferMethod.CUDA_IPC, TransferMethod.NCCL):
            ok = all(self.transfer_kv_cache_sync(t.request_id, t.src_rank, t.dst_rank, list(t.src_blocks),
                                                 list(t.dst_blocks)) for t in plan.transfers)
            return ok
        ok = True
        nbytes = 0
        for rank, worker in self.worker_registry.items():
            res = worker.migrate(plan, method=method)
            self.last_result = res
            if "error" in res:
                ok = False
            else:
                nbytes += res["bytes"]
        if ok:
            self._account(time.perf_counter() - start, nbytes, plan.total_blocks(), count=len(plan.transfers))
        return ok

    def get_stats(self) -> Dict[str, Any]:
        return {
            "transfer_count": self.transfer_count,
            "total_transfer_time": self.total_transfer_time,
            "total_bytes_transferred": self.total_bytes_transferred,
            "avg_transfer_time": self.total_transfer_time / self.transfer_count if self.transfer_count else 0.0,
        }

    def reset_stats(self) -> None:
        self.transfer_count = 0
        self.total_transfer_time = 0.0
        self.total_bytes_transferred = 0


__all__ = ["TransferMethod", "V0KVTransferManager", "MigrationPlan", "Transfer"]
