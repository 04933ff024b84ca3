"""The worker's KV data plane, with the reference's method names.

Each public method keeps the name, argument meaning, return shape and error
convention of the V0Worker method it stands in for
(elasticmm/engine/v0/worker.py:478-1005); the device work underneath is the
CUDA library (one launch for all layers instead of one torch indexing kernel
per layer). In the reference this class is a Ray actor; here it is a plain
class owned by one process bound to one GPU, and the `@ray.remote` decoration
is left to the integrator.

Data-path errors are returned as {"error": ..., "bytes": 0, "blocks": 0}
rather than raised, precondition failures raise ValueError / RuntimeError
(elasticmm/engine/v0/worker.py:686-691,766-776).
"""
from __future__ import annotations

import contextlib
import os
import time
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ... import _lib
from ...kv_pool import Context, KVPool, _as_host_ids, get_context
from .transport import (MigrationPlan, plan_chunks, max_chunk_layers, pipelined_recv,
                        pipelined_send, run_waves, PIPELINE_DEPTH)
from .utils import EngineStage

# All-to-all migration. A rank packs about this many bytes per chunk of layers: NCCL moves one message of up
# to 256 MiB at ~550 GB/s and messages of 512 MiB and more at ~690 GB/s (measured between two B200s), so the
# chunks are large. The pack and unpack kernels are capped to the SM count minus this many CTAs: an NCCL
# point-to-point CTA needs an SM almost to itself, and with all 148 SMs held by a copy kernel the exchange that
# runs beside it fell from ~630 to ~565 GB/s.
ALLTOALL_MESSAGE_BYTES = 1 << 30
ALLTOALL_SMS_LEFT_TO_NCCL = 48

_NVTX = os.environ.get("EMM_NVTX", "0") == "1"


def _range(name: str):
    """NVTX range around a data-plane phase when EMM_NVTX=1 (for timeline tools); free otherwise."""
    return torch.cuda.nvtx.range(name) if _NVTX else contextlib.nullcontext()


_DTYPES = {"float16": torch.float16, "half": torch.float16, "bfloat16": torch.bfloat16,
           "float32": torch.float32, "float": torch.float32,
           "uint8": torch.uint8, "int8": torch.int8, "fp8": torch.uint8, "float8": torch.uint8}


class V0Worker:
    """One GPU's KV pool plus the operations that move its blocks."""

    def __init__(
        self,
        worker_id: int = 0,
        stage: EngineStage = EngineStage.PREFILL,
        block_size: int = 16,
        dtype: str = "float16",
        device: Optional[torch.device] = None,
        global_rank: Optional[int] = None,
        world_size: Optional[int] = None,
        nccl_init_method: Optional[str] = None,
        kv_cache: Optional[Sequence[torch.Tensor]] = None,
    ):
        if not torch.cuda.is_available():
            raise RuntimeError("V0Worker needs a CUDA device; the KV data plane has no CPU path")
        self.worker_id = worker_id
        self.stage = stage
        self.original_role = stage
        self.current_role = stage
        self.block_size = block_size
        self.dtype = dtype
        self.global_rank = global_rank
        self.nccl_world_size = world_size
        self.nccl_init_method = nccl_init_method
        self.nccl_pg_initialized = False
        self.process_group = None
        self.device = torch.device(device) if device is not None else torch.device(
            "cuda", torch.cuda.current_device())
        self.ctx: Context = get_context(self.device)
        self.kv_cache: Optional[List[torch.Tensor]] = None
        self.kv_swap: Optional[List[torch.Tensor]] = None
        self.pool: Optional[KVPool] = None
        self.swap_pool: Optional[KVPool] = None
        self.peer_pools: Dict[int, KVPool] = {}
        self._peer_streams: Dict[int, torch.cuda.Stream] = {}
        self._peer_keepalive: Dict[int, Any] = {}
        self.ve_cache: Optional[Dict[str, torch.Tensor]] = None
        self.ve_blocks: Optional[torch.Tensor] = None
        self.ve_pool: Optional[KVPool] = None
        self.swap_in_stream = torch.cuda.Stream(self.device)
        self.swap_out_stream = torch.cuda.Stream(self.device)
        self.swap_event_table: Dict[str, torch.cuda.Event] = {}
        self.latest_swap_in_event: Optional[torch.cuda.Event] = None
        self.latest_swap_out_event: Optional[torch.cuda.Event] = None
        self._xfer_stream = torch.cuda.Stream(self.device)
        self._staging: Optional[torch.Tensor] = None  # flat byte ring for the staged NCCL path
        self._nccl_comm: Optional[int] = None         # library-owned communicator (init_native_nccl)
        self._a2a: Optional[Dict[str, Any]] = None    # streams and staging of the all-to-all migration
        if kv_cache is not None:
            self.bind_kv_cache(kv_cache)

    # -- pool set-up -----------------------------------------------------------
    def init_kvcache(self, num_gpu_blocks: int, num_layers: int, num_kv_heads: int, head_size: int,
                     num_cpu_blocks: int = 0, layout: str = "nhd") -> None:
        """Allocates the pool: L tensors of logical shape [2, NB, BS, H, D].

        layout "nhd" is the reference's token-major allocation; "hnd" allocates
        [2, NB, H, BS, D] and binds its permuted view, so indexing stays the
        same and each head's tokens are contiguous. In the reference the
        tensors come from vLLM's CacheEngine
        (elasticmm/engine/v0/worker.py:369-394); use bind_kv_cache to adopt those.
        """
        if layout not in ("nhd", "hnd"):
            raise ValueError(f"unknown pool layout {layout!r}")
        dt = _DTYPES[self.dtype]

        def alloc(nb: int, pinned: bool) -> torch.Tensor:
            if layout == "nhd":
                shape = (2, nb, self.block_size, num_kv_heads, head_size)
            else:
                shape = (2, nb, num_kv_heads, self.block_size, head_size)
            t = torch.empty(shape, dtype=dt).pin_memory() if pinned else torch.empty(shape, dtype=dt,
                                                                                     device=self.device)
            return t if layout == "nhd" else t.permute(0, 1, 3, 2, 4)

        self.bind_kv_cache([alloc(num_gpu_blocks, False) for _ in range(num_layers)])
        if num_cpu_blocks > 0:
            self.bind_kv_swap([alloc(num_cpu_blocks, True) for _ in range(num_layers)])

    @classmethod
    def from_config(cls, config, worker_id: int = 0, stage: EngineStage = EngineStage.PREFILL,
                    device: Optional[torch.device] = None, global_rank: Optional[int] = None,
                    world_size: Optional[int] = None, num_gpu_blocks: Optional[int] = None,
                    num_cpu_blocks: Optional[int] = None) -> "V0Worker":
        """A worker with its pool allocated from a V0KVCacheConfig (block
        counts default to the configuration's maxima)."""
        config.validate()
        w = cls(worker_id=worker_id, stage=stage, block_size=config.block_size, dtype=config.dtype,
                device=device, global_rank=global_rank, world_size=world_size)
        w.init_kvcache(config.max_num_gpu_blocks if num_gpu_blocks is None else num_gpu_blocks,
                       config.num_layers, config.num_kv_heads, config.head_size,
                       num_cpu_blocks=config.max_num_cpu_blocks if num_cpu_blocks is None else num_cpu_blocks,
                       layout=config.layout)
        return w

    def bind_kv_cache(self, kv_cache: Sequence[torch.Tensor]) -> None:
        """Adopts an existing list of per-layer pool tensors (not copied)."""
        self.kv_cache = list(kv_cache)
        self.pool = KVPool(self.kv_cache, self.ctx)

    def bind_kv_swap(self, kv_swap: Sequence[torch.Tensor]) -> None:
        """Adopts a pinned host pool with the GPU pool's page geometry."""
        self.kv_swap = list(kv_swap)
        self.swap_pool = KVPool(self.kv_swap, self.ctx)

    def _require_pool(self) -> KVPool:
        if self.pool is None:
            raise RuntimeError("KV cache not initialized")
        return self.pool

    def get_stage(self) -> EngineStage:
        return self.stage

    def set_stage(self, stage: EngineStage) -> None:
        self.stage = stage

    def switch_role(self, new_stage: EngineStage) -> bool:
        """Logical role change; the pool and the global rank stay
        (elasticmm/engine/v0/worker.py:1066-1131)."""
        self.stage = new_stage
        self.current_role = new_stage
        return True

    # -- gather / scatter (elasticmm/engine/v0/worker.py:578-647) --------------
    def extract_kv_blocks(self, block_indices: List[int]) -> torch.Tensor:
        """Returns [num_layers, 2, num_blocks, block_size, num_heads, head_size]."""
        with _range("emm.extract_kv_blocks"):
            return self._require_pool().gather(block_indices)

    def write_kv_blocks(self, block_indices: List[int], kv_data: torch.Tensor) -> None:
        pool = self._require_pool()
        assert kv_data.shape[2] == len(block_indices), (
            f"Block count mismatch: {kv_data.shape[2]} vs {len(block_indices)}")
        with _range("emm.write_kv_blocks"):
            pool.scatter(block_indices, kv_data)

    def extract_kv_blocks_many(self, block_index_lists: Sequence[List[int]]) -> List[torch.Tensor]:
        """extract_kv_blocks for several requests with one kernel launch; one tensor per request."""
        with _range("emm.extract_kv_blocks_many"):
            return self._require_pool().gather_many(block_index_lists)

    def write_kv_blocks_many(self, block_index_lists: Sequence[List[int]], kv_data: Sequence[torch.Tensor]) -> None:
        """write_kv_blocks for several requests with one launch; `kv_data` as returned by
        extract_kv_blocks_many (possibly of another worker on the same GPU)."""
        for ids, data in zip(block_index_lists, kv_data):
            assert data.shape[2] == len(ids), f"Block count mismatch: {data.shape[2]} vs {len(ids)}"
        with _range("emm.write_kv_blocks_many"):
            self._require_pool().scatter_many(block_index_lists, kv_data)

    def get_kv_cache_layout(self) -> Dict[str, Any]:
        if not self.kv_cache:
            return {}
        pool = self._require_pool()
        return {
            "num_layers": pool.num_layers,
            "block_size": pool.block_size,
            "num_heads": pool.num_kv_heads,
            "head_size": pool.head_size,
            "dtype": str(pool.dtype).split(".")[-1],
        }

    # -- vision embeddings (elasticmm/engine/v0/worker.py:1007-1060) --------------
    def init_ve_cache(self) -> None:
        """Request-keyed embedding store, as the reference keeps it (a dict of tensors)."""
        self.ve_cache = {}

    def extract_vision_blocks(self, request_id: str) -> torch.Tensor:
        if self.ve_cache is None:
            raise RuntimeError("Vision embedding cache not initialized")
        if request_id not in self.ve_cache:
            raise KeyError(f"Request {request_id} not found in vision cache")
        return self.ve_cache[request_id]

    def write_vision_blocks(self, request_id: str, ve_data: torch.Tensor) -> None:
        if self.ve_cache is None:
            raise RuntimeError("Vision embedding cache not initialized")
        self.ve_cache[request_id] = ve_data

    def get_ve_cache_keys(self) -> List[str]:
        return list(self.ve_cache.keys()) if self.ve_cache else []

    def get_ve_shape(self, request_id: str):
        if self.ve_cache and request_id in self.ve_cache:
            return tuple(self.ve_cache[request_id].shape)
        return None

    def bind_ve_block_cache(self, ve_blocks: torch.Tensor) -> None:
        """Adopts a block cache [blocks, embed_tokens, embed_dim], the form the
        legacy transfer manager moves by block index
        (elasticmm/engine/v0/nccl_transfer.py:295-368)."""
        self.ve_blocks = ve_blocks
        self.ve_pool = KVPool([ve_blocks], self.ctx)

    def extract_ve_blocks(self, block_indices: List[int]) -> torch.Tensor:
        """[n, embed_tokens, embed_dim]: the stacked source blocks, one launch."""
        if self.ve_pool is None:
            raise RuntimeError("Vision embedding cache not initialized")
        n = len(block_indices)
        packed = self.ve_pool.gather(block_indices)
        return packed.view(n, self.ve_pool.block_size, self.ve_pool.head_size)

    def write_ve_blocks(self, block_indices: List[int], ve_data: torch.Tensor) -> None:
        if self.ve_pool is None:
            raise RuntimeError("Vision embedding cache not initialized")
        n = len(block_indices)
        assert ve_data.shape[0] == n, f"Block count mismatch: {ve_data.shape[0]} vs {n}"
        pool = self.ve_pool
        self.ve_pool.scatter(block_indices, ve_data.reshape(1, 1, n, pool.block_size, 1, pool.head_size))

    # -- append and compaction (no counterpart in the reference's own code) ----
    def reshape_and_cache(self, key: torch.Tensor, value: torch.Tensor,
                          slot_mapping: torch.Tensor, layer: int) -> None:
        """Writes one layer's new-token K/V rows at their slots; slot < 0 skipped."""
        self._require_pool().append(layer, key, value, slot_mapping)

    def reshape_and_cache_all_layers(self, key: torch.Tensor, value: torch.Tensor,
                                     slot_mapping: torch.Tensor) -> None:
        """Same for all layers at once; key/value are [L, T, H, D]."""
        self._require_pool().append_all_layers(key, value, slot_mapping)

    def compact_blocks(self, move_src: Sequence[int], move_dst: Sequence[int]) -> Dict[str, Any]:
        """Executes a compaction plan (V0BlockManager.compact) inside the pool."""
        pool = self._require_pool()
        try:
            pool.copy_blocks(pool, move_src, move_dst)
        except _lib.EmmError as e:
            return {"error": str(e), "bytes": 0, "blocks": 0}
        return {"bytes": len(move_src) * pool.block_bytes(), "blocks": len(move_src)}

    # -- GPU <-> CPU swap (elasticmm/engine/v0/worker.py:478-526) ---------------
    def swap_blocks(self, request_ids: List[str], source_block_ids: List[int],
                    target_block_ids: List[int], is_swap_in: bool) -> None:
        """Copies blocks between the pinned host pool and the GPU pool.

        If is_swap_in, host block source_block_ids[i] goes to GPU block
        target_block_ids[i]; otherwise the other way. One kernel launch on the
        swap stream; a request's later swap waits for its earlier one.
        """
        pool = self._require_pool()
        if self.swap_pool is None:
            raise RuntimeError("CPU swap pool not initialized")
        stream = self.swap_in_stream if is_swap_in else self.swap_out_stream
        for rid in request_ids:
            prev = self.swap_event_table.get(rid)
            if prev is not None:
                stream.wait_event(prev)
        stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(stream):
            if is_swap_in:
                self.swap_pool.copy_blocks(pool, source_block_ids, target_block_ids)
            else:
                pool.copy_blocks(self.swap_pool, source_block_ids, target_block_ids)
            event = torch.cuda.Event()
            event.record(stream)
        for rid in request_ids:
            self.swap_event_table[rid] = event
        if is_swap_in:
            self.latest_swap_in_event = event
        else:
            self.latest_swap_out_event = event

    def wait_for_all_swap_in(self) -> None:
        if self.latest_swap_in_event is not None:
            self.latest_swap_in_event.synchronize()

    def wait_for_all_swap_out(self) -> None:
        if self.latest_swap_out_event is not None:
            self.latest_swap_out_event.synchronize()

    def clear_request_resource(self, request_id: str) -> None:
        self.swap_event_table.pop(request_id, None)

    # -- process group ---------------------------------------------------------
    def init_global_nccl(self, process_group=None) -> bool:
        """True when a process group is ready for P2P transfer
        (elasticmm/engine/v0/worker.py:649-659). The group itself is created by
        the launcher (torchrun-style environment or init_process_group with the
        coordinator's init method); NVSwitch needs none of the PCIe-era NCCL
        environment overrides the reference sets."""
        if not dist.is_available() or not dist.is_initialized():
            return False
        self.process_group = process_group
        self.nccl_pg_initialized = True
        if self.global_rank is None:
            self.global_rank = dist.get_rank()
        return True

    def init_native_nccl(self) -> bool:
        """Creates a communicator owned by the C library over the ranks of the process group
        (the unique id travels through torch.distributed). With it, p2p_send_kv / p2p_recv_kv run
        their pack -> send / receive -> unpack pipelines inside the library on its own streams."""
        if not self.nccl_pg_initialized:
            return False
        world = dist.get_world_size(self.process_group)
        rank = dist.get_rank(self.process_group)
        box = [self.ctx.nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0, group=self.process_group)
        self._nccl_comm = self.ctx.nccl_comm_init(box[0], world, rank)
        return True

    def get_global_rank(self) -> int:
        return self.global_rank if self.global_rank is not None else -1

    # -- staged NCCL transfer (elasticmm/engine/v0/worker.py:665-871) -----------
    def _staging_views(self, pool: KVPool, n: int, chunks) -> List[torch.Tensor]:
        need = pool.packed_bytes(n, max_chunk_layers(chunks))
        total = need * PIPELINE_DEPTH
        if self._staging is None or self._staging.numel() < total:
            self._staging = torch.empty(total, dtype=torch.uint8, device=self.device)
        return [self._staging[i * need:(i + 1) * need] for i in range(PIPELINE_DEPTH)]

    def _buffer_for(self, pool: KVPool, n: int, slots: List[torch.Tensor]):
        def buffer_for(slot: int, layer_count: int) -> torch.Tensor:
            flat = slots[slot][: pool.packed_bytes(n, layer_count)].view(pool.dtype)
            return pool._logical(flat.view(pool.packed_shape(n, layer_count)))
        return buffer_for

    def _staged_transfer(self, sending: bool, peer: int, block_indices, checked: bool = False) -> Dict[str, Any]:
        """Common body of p2p_send_kv / p2p_recv_kv: chunk schedule, staging ring, then either the
        library's own pipeline (after init_native_nccl) or the same schedule over torch P2P."""
        what = "send" if sending else "recv"
        if not self.nccl_pg_initialized:
            return {"error": "Global NCCL not initialized", "bytes": 0, "blocks": 0}
        try:
            pool = self._require_pool()
            n = len(block_indices)
            if n == 0:
                return {"bytes": 0, "blocks": 0}
            host_ids = _as_host_ids(block_indices)
            ids = pool.upload_ids(host_ids if checked else pool._validated(host_ids, unique=not sending))
            chunks = plan_chunks(pool.num_layers, n, pool.page_bytes)
            slots = self._staging_views(pool, n, chunks)
            with _range(f"emm.p2p_{what}_kv"):
                if self._nccl_comm is not None:
                    run = pool.send_blocks if sending else pool.recv_blocks
                    run(self._nccl_comm, peer, ids, self._staging, chunks[0][1])
                else:
                    main = torch.cuda.current_stream(self.device)
                    self._xfer_stream.wait_stream(main)
                    with torch.cuda.stream(self._xfer_stream):
                        if sending:
                            pipelined_send(
                                chunks, self._buffer_for(pool, n, slots),
                                pack=lambda buf, b, c: pool.gather(ids, out=buf, layer_begin=b, layer_count=c),
                                isend=lambda buf: dist.isend(pool._logical(buf), dst=peer, group=self.process_group))
                        else:
                            pipelined_recv(
                                chunks, self._buffer_for(pool, n, slots),
                                irecv=lambda buf: dist.irecv(pool._logical(buf), src=peer, group=self.process_group),
                                unpack=lambda buf, b, c: pool.scatter(ids, buf, layer_begin=b, layer_count=c))
                    main.wait_stream(self._xfer_stream)
            torch.cuda.synchronize(self.device)
            rc, _ = self.ctx.status()
            if rc != _lib.OK:
                return {"error": f"{what} failed on device: {_lib.last_error()}", "bytes": 0, "blocks": 0}
            return {"bytes": pool.packed_bytes(n), "blocks": n}
        except Exception as e:  # data-path errors are reported, not raised
            return {"error": f"NCCL {what} failed: {type(e).__name__}: {e}", "bytes": 0, "blocks": 0}

    def p2p_send_kv(self, dst_rank: int, block_indices: List[int]) -> Dict[str, Any]:
        """Packs the blocks chunk by chunk and sends them to `dst_rank`.

        Packing of chunk c+1 overlaps the send of chunk c. The call returns
        after the device has finished, as the reference does.
        """
        return self._staged_transfer(True, dst_rank, block_indices)

    def p2p_recv_kv(self, src_rank: int, block_indices: List[int]) -> Dict[str, Any]:
        """Receives chunk by chunk and scatters into `block_indices`."""
        return self._staged_transfer(False, src_rank, block_indices)

    def p2p_coordinated_transfer_kv(self, src_worker_ref: Any, src_rank: int, src_blocks: List[int],
                                    dst_blocks: List[int], timeout: float = 10.0) -> Dict[str, Any]:
        """Called on the DESTINATION worker: triggers the source's send, then receives.

        `src_worker_ref` is an actor-style handle whose
        `p2p_send_kv.remote(dst_rank, blocks)` starts the send in the source's
        process and returns a future with `.result(timeout)`-like access via
        `get()`; pass None when the source process calls p2p_send_kv itself
        (one process per GPU, both sides following the same plan).
        """
        if not self.nccl_pg_initialized:
            raise RuntimeError("Destination worker: Global NCCL not initialized")
        if len(src_blocks) != len(dst_blocks):
            raise ValueError(f"Block count mismatch: src={len(src_blocks)}, dst={len(dst_blocks)}")
        if len(src_blocks) == 0:
            return {"bytes": 0, "blocks": 0, "error": "No blocks to transfer"}
        world = dist.get_world_size(self.process_group)
        if src_rank < 0 or src_rank >= world:
            raise ValueError(f"Invalid src_rank: {src_rank} (world_size={world})")
        start = time.time()
        send_future = None
        if src_worker_ref is not None:
            send_future = src_worker_ref.p2p_send_kv.remote(dist.get_rank(self.process_group), src_blocks)
        result = self.p2p_recv_kv(src_rank, dst_blocks)
        elapsed = time.time() - start
        if "error" in result:
            result["elapsed"] = elapsed
            return result
        if elapsed > timeout:
            return {"error": f"Transfer timeout after {timeout}s", "bytes": 0, "blocks": 0, "elapsed": elapsed}
        if send_future is not None:
            try:
                send_result = send_future.get(timeout=1.0) if hasattr(send_future, "get") else send_future
            except Exception as send_err:
                return {"error": f"Send failed: {type(send_err).__name__}: {send_err}", "bytes": 0,
                        "blocks": 0, "elapsed": elapsed}
            if isinstance(send_result, dict) and "error" in send_result:
                return {"error": f"Send error: {send_result['error']}", "bytes": 0, "blocks": 0,
                        "elapsed": elapsed}
        return {"bytes": result["bytes"], "blocks": len(dst_blocks), "elapsed": elapsed,
                "method": "coordinated_single_call"}

    def collective_transfer_kv(self, group_name: Any, root: int, block_indices: List[int],
                               tensor_shape: Sequence[int], dtype: str, mode: str) -> Dict[str, Any]:
        """Broadcast form of the transfer (elasticmm/engine/v0/worker.py:939-1005): the
        sender gathers its blocks into one flat message and broadcasts it from `root`; a
        receiver takes the broadcast and scatters it into `block_indices`. `group_name` is a
        torch.distributed process group (or None for the default group) where the reference
        passes the name of a Ray collective group.
        """
        key = dtype.replace("torch.", "").lower()
        names = {"float16": torch.float16, "half": torch.float16, "fp16": torch.float16,
                 "bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
                 "fp32": torch.float32}
        if key not in names:
            raise ValueError(f"[V0Worker] Unsupported dtype for collective transfer: {dtype}")
        group = None if isinstance(group_name, str) else group_name
        shape = tuple(int(d) for d in tensor_shape)
        if mode == "send":
            flat = self.extract_kv_blocks(block_indices).contiguous().view(-1).to(dtype=names[key])
            dist.broadcast(flat, src=root, group=group)
        elif mode == "recv":
            numel = 1
            for d in shape:
                numel *= d
            flat = torch.empty(numel, dtype=names[key], device=self.device)
            dist.broadcast(flat, src=root, group=group)
            self.write_kv_blocks(block_indices, flat.view(shape))
        else:
            raise ValueError(f"[V0Worker] Unknown collective transfer mode: {mode}")
        torch.cuda.synchronize(self.device)
        return {"bytes": flat.numel() * flat.element_size(), "mode": mode}

    def get_kv_cache_shape(self) -> tuple:
        """Shape of one layer's pool tensor (the reference calls `.shape` on its list of
        layers, which raises; this returns the per-layer shape with the layer count first)."""
        if not self.kv_cache:
            return ()
        return (len(self.kv_cache),) + tuple(self.kv_cache[0].shape)

    # -- direct peer stores (the slot the reference reserves for a CUDA-IPC
    #    extension, elasticmm/engine/v0/kv_transfer.py:303-331) ----------------
    def get_ipc_handles(self) -> List[Tuple[bytes, int]]:
        """(handle, offset) per layer for other processes on this node
        (the reference's stub returns [], elasticmm/engine/v0/worker.py:415-437)."""
        pool = self._require_pool()
        return [self.ctx.ipc_export(t) for t in pool.layers]

    def get_pool_desc(self) -> Dict[str, int]:
        d = self._require_pool().desc
        return {name: int(getattr(d, name)) for name, _ in d._fields_}

    def attach_peer_pool(self, rank: int, handles: Sequence[Tuple[bytes, int]], desc: Dict[str, int],
                         dtype: Optional[torch.dtype] = None) -> None:
        """Maps the pool of the worker with global rank `rank` into this process."""
        ptrs = [self.ctx.ipc_open(h, off) for h, off in handles]
        pd = _lib.PoolDesc(**desc)
        self.peer_pools[rank] = KVPool.from_pointers(self.ctx, pd, ptrs, dtype or self._require_pool().dtype)

    def attach_local_peer(self, rank: int, worker: "V0Worker") -> None:
        """Maps the pool of a worker that lives in THIS process on another GPU (one process
        driving several GPUs): peer access is enabled and the same device pointers are used,
        no IPC handle is needed."""
        other = worker._require_pool()
        self.ctx.enable_peer_access(worker.device)
        desc = _lib.PoolDesc.from_buffer_copy(other.desc)
        self.peer_pools[rank] = KVPool.from_pointers(self.ctx, desc, other.layer_ptrs, other.dtype)
        self._peer_keepalive[rank] = worker  # the mapped memory belongs to that worker

    def p2p_push_kv(self, dst_rank: int, src_blocks: List[int], dst_blocks: List[int]) -> Dict[str, Any]:
        """Copies blocks straight into the mapped pool of `dst_rank`: one kernel,
        local loads, stores over NVLink, no staging buffer and no NCCL call.
        Asynchronous on the current stream; the caller orders the sink's first
        read after this stream's completion (an event wait, a barrier, or any
        stream-ordered message to the sink)."""
        if dst_rank not in self.peer_pools:
            return {"error": f"pool of rank {dst_rank} is not mapped", "bytes": 0, "blocks": 0}
        if len(src_blocks) != len(dst_blocks):
            raise ValueError(f"Block count mismatch: src={len(src_blocks)}, dst={len(dst_blocks)}")
        pool = self._require_pool()
        try:
            pool.copy_blocks(self.peer_pools[dst_rank], src_blocks, dst_blocks)
        except _lib.EmmError as e:
            return {"error": str(e), "bytes": 0, "blocks": 0}
        return {"bytes": len(src_blocks) * pool.block_bytes(), "blocks": len(src_blocks)}

    def p2p_pull_kv(self, src_rank: int, src_blocks: List[int], dst_blocks: List[int],
                    max_ctas: Optional[int] = None) -> Dict[str, Any]:
        """Pull KV blocks from the worker with global rank `src_rank` into this pool.

        Same name, arguments and direction as the reference's receiver-driven
        pull (elasticmm/engine/v0/worker.py:873-910, unused there). Here it is one
        kernel on the SINK: loads over NVLink from the source's peer-mapped pool,
        stores into the local blocks; no request message, no staging buffer, no
        NCCL call. Loads over the link measured ~10 % faster than stores (785 vs
        716 GB/s per direction), so this is the default direction. Asynchronous on
        the current stream; the source may free its blocks once this stream has
        completed. `max_ctas` caps the grid when several pulls run side by side.
        """
        if src_rank not in self.peer_pools:
            return {"error": f"pool of rank {src_rank} is not mapped", "bytes": 0, "blocks": 0}
        if len(src_blocks) != len(dst_blocks):
            raise ValueError(f"Block count mismatch: src={len(src_blocks)}, dst={len(dst_blocks)}")
        pool = self._require_pool()
        try:
            with _range("emm.p2p_pull_kv"):
                self.peer_pools[src_rank].copy_blocks(pool, src_blocks, dst_blocks, max_ctas=max_ctas)
        except _lib.EmmError as e:
            return {"error": str(e), "bytes": 0, "blocks": 0}
        return {"bytes": len(src_blocks) * pool.block_bytes(), "blocks": len(src_blocks)}

    # -- plan-level migration -----------------------------------------------------
    def _agree(self, error: Optional[str]) -> Optional[str]:
        """Collective over the process group: None if no rank reports an error, else this
        rank's own message or a note that a peer failed. Every rank of a migration passes
        through the same _agree calls, so a rank that fails a host-side check never leaves the
        others waiting in an exchange or at the exit (they all return an error together)."""
        backend = dist.get_backend(self.process_group)
        flag = torch.tensor([1 if error else 0], dtype=torch.int32,
                            device=self.device if backend == "nccl" else "cpu")
        dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.process_group)
        if int(flag.item()) == 0:
            return None
        return error or "another rank of the migration reported an error; nothing was moved by this rank"

    def _post_flag(self, error: Optional[str]):
        """The non-blocking half of an agreement: starts the all-reduce of this rank's error flag on the
        current stream and returns the tensor; _read_flags turns one or more of them into an outcome. On a
        GPU group nothing here waits for the device, so kernels queued behind the all-reduce are ordered
        after every rank's arrival without the host stalling."""
        backend = dist.get_backend(self.process_group)
        flag = torch.tensor([1 if error else 0], dtype=torch.int32,
                            device=self.device if backend == "nccl" else "cpu")
        dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.process_group)
        return flag

    @staticmethod
    def _read_flags(flags, error: Optional[str]) -> Optional[str]:
        if not any(int(f.item()) for f in flags):
            return None
        return error or "another rank of the migration reported an error; this rank's part may have run"

    def _plan_error(self, plan: MigrationPlan, method: str) -> Optional[str]:
        """_check_plan_part, remembered per plan: a plan that is replayed (the waves of a long migration,
        a benchmark step) is validated on the host once."""
        key = (id(plan), len(plan.transfers), method, tuple(sorted(self.peer_pools)))
        cache = self.__dict__.setdefault("_plan_checks", {})
        if key not in cache:
            if len(cache) > 256:
                cache.clear()
            cache[key] = (plan, self._check_plan_part(plan, method))  # the plan is kept so that its id stays unique
        return cache[key][1]

    def _own_stream_sync(self) -> None:
        torch.cuda.current_stream(self.device).synchronize()

    def _device_error(self, what: str) -> Optional[str]:
        """Waits for this GPU and reads the sticky device status word."""
        torch.cuda.synchronize(self.device)
        rc, _ = self.ctx.status()
        return None if rc == _lib.OK else f"{what} failed on device: {_lib.last_error()}"

    def _check_plan_part(self, plan: MigrationPlan, method: str) -> Optional[str]:
        """Host-side validation of this rank's part of a plan, before anything is launched."""
        rank = self.get_global_rank()
        pool = self.pool
        if pool is None:
            return "KV cache not initialized"
        try:
            for peer in plan.incoming(rank):
                src_ids, dst_ids = plan.tables_np(peer, rank)
                pool._validated(dst_ids, unique=False)
                if method == "pull" and peer not in self.peer_pools:
                    return f"pool of rank {peer} is not mapped"
                if method == "pull":
                    self.peer_pools[peer]._validated(src_ids)
            incoming = [plan.tables_np(peer, rank)[1] for peer in plan.incoming(rank)]
            if incoming:
                import numpy as np

                pool._validated(np.concatenate(incoming), unique=True)
            for peer in plan.outgoing(rank):
                src_ids, dst_ids = plan.tables_np(rank, peer)
                pool._validated(src_ids)
                if method == "push" and peer not in self.peer_pools:
                    return f"pool of rank {peer} is not mapped"
                if method == "push":
                    self.peer_pools[peer]._validated(dst_ids, unique=True)
        except _lib.EmmError as e:
            return str(e)
        if method == "alltoall" and self._nccl_comm is None:
            return "alltoall migration needs init_native_nccl()"
        if method == "nccl" and plan.outgoing(rank) and plan.incoming(rank):
            return ("nccl migration needs each rank to be a pure source or a pure sink; "
                    "use the peer method for exchanges")
        return None

    def _pull_all(self, plan: MigrationPlan, tables: Optional[Dict[int, Tuple[Any, Any]]] = None):
        """Launches this sink's pulls of one wave, all sources side by side on one stream each, with the
        grids capped so that the launches together hold at most one CTA per SM: measured on NVSwitch, two
        full-size pull kernels side by side halve the rate, two half-size ones run at full link speed, and
        a flow that is left alone still saturates the link with its share of CTAs. Returns
        (error or None, blocks, [(peer, stream)])."""
        rank = self.get_global_rank()
        peers = plan.pull_order(rank)
        cap = max(24, self.ctx.sm_count // max(1, len(peers))) if len(peers) > 1 else None
        main = torch.cuda.current_stream(self.device)
        used, moved = [], 0
        for peer in peers:
            src_ids, dst_ids = tables[peer] if tables is not None else plan.tables_np(peer, rank)
            stream = self._peer_streams.get(peer)
            if stream is None:
                stream = self._peer_streams[peer] = torch.cuda.Stream(self.device)
            stream.wait_stream(main)
            with torch.cuda.stream(stream):
                res = self.p2p_pull_kv(peer, src_ids, dst_ids, max_ctas=cap)
            used.append((peer, stream))
            if "error" in res:
                return res["error"], moved, used
            moved += res["blocks"]
        return None, moved, used

    def migrate(self, plan: MigrationPlan, method: str = "pull") -> Dict[str, Any]:
        """Runs this rank's part of a migration plan; every rank of the process group calls it.

        method "pull" (default; "peer" is an alias): each sink launches one
        direct-load kernel per source, side by side with capped grids. method
        "push": each source launches one direct-store kernel per sink instead,
        one sink at a time. method "alltoall": per layer chunk, one gather for all
        sinks, one grouped NCCL exchange with one message per peer, one scatter for
        all sources, pipelined over the chunks (needs init_native_nccl). method
        "nccl": per pair, the staged pipeline of p2p_send_kv / p2p_recv_kv; every
        rank walks the pairs in the plan's one global order (sources start at
        different sinks), which rules out a circular wait.

        Ordering. A source's blocks must be final on the source's CURRENT stream
        when it calls migrate: the source waits for that stream before the entry
        agreement, and no sink reads before the agreement has completed. The call
        returns after every rank's copies have finished (the exit agreement), so a
        source may free or overwrite its blocks as soon as migrate returns.

        Errors. Host-side checks run first and all ranks agree on their outcome
        before anything is launched; device-side status is agreed on at the exit.
        If any rank fails, every rank returns {"error": ...} and none hangs.
        """
        if method == "peer":
            method = "pull"
        if method not in ("pull", "push", "alltoall", "nccl"):
            raise ValueError(f"unknown migration method {method!r}")
        rank = self.get_global_rank()
        error = self._plan_error(plan, method)
        if plan.outgoing(rank):
            self._own_stream_sync()  # what this source wrote is visible to its sinks
        error = self._agree(error)
        if error:
            return {"error": error, "bytes": 0, "blocks": 0}
        pool = self._require_pool()
        moved = 0
        if method == "pull":
            error, moved, used = self._pull_all(plan)
            main = torch.cuda.current_stream(self.device)
            for _, stream in used:
                main.wait_stream(stream)
        elif method == "push":
            # A source pushes to one sink at a time, sources starting at different sinks.
            for peer in plan.push_order(rank):
                src_ids, dst_ids = plan.tables_np(rank, peer)
                res = self.p2p_push_kv(peer, src_ids, dst_ids)
                if "error" in res:
                    error = res["error"]
                    break
                moved += res["blocks"]
        elif method == "alltoall":
            moved = self._migrate_alltoall(plan)
        else:
            for src, dst in plan.ordered_pairs():
                if src == rank:  # the plan's ids were checked above, its tables are already arrays
                    res = self._staged_transfer(True, dst, plan.tables_np(src, dst)[0], checked=True)
                elif dst == rank:
                    res = self._staged_transfer(False, src, plan.tables_np(src, dst)[1], checked=True)
                else:
                    continue
                if "error" in res:
                    error = error or res["error"]  # keep walking the pairs: the peers are in their halves
                else:
                    moved += res["blocks"]
        if not error:
            error = self._device_error(method)
        error = self._agree(error)  # also the exit meeting point: every copy of the plan has landed
        if error:
            return {"error": error, "bytes": 0, "blocks": 0}
        return {"bytes": moved * pool.block_bytes(), "blocks": moved}

    def migrate_waves(self, plans: Sequence[MigrationPlan], ledger, depth: int = 2,
                      tables: Optional[Sequence[Dict[int, Tuple[Any, Any]]]] = None,
                      on_wave_landed=None) -> Dict[str, Any]:
        """Moves a sequence of waves by direct loads with no barrier between waves.

        `plans[w]` is wave w; every rank of the process group makes the call with the
        same list. Blocks (on a source and on a sink) may be used again by wave
        w + depth: a sink launches its pull of wave w from a source only after all
        sinks have posted wave w - depth of that source in `ledger` (a WaveLedger
        over a store all ranks share), and it orders wave w on its own device after
        its wave w - depth. A sink therefore runs up to `depth` waves ahead of the
        slowest sink, and a source's link stays busy while one sink is still
        finishing. A source returns when all of its waves are complete, which is its
        signal that every block it offered may be freed.

        `tables[w][source]` optionally gives device-resident (src ids, dst ids) int32
        tensors for this sink; otherwise the plan's host lists are uploaded.
        `on_wave_landed(w)` is called on a sink after its copies of wave w have
        finished and before it posts the wave (a verification hook).

        Returns {"bytes", "blocks", "wave_ms"} with this sink's device time per wave,
        or {"error": ...} on every rank if any rank failed (a rank that failed its
        host-side checks moves nothing; the others may have moved their part).
        """
        rank = self.get_global_rank()
        pool = self.pool
        error = None
        for plan in plans:
            error = error or self._plan_error(plan, "pull")
        if any(plan.outgoing(rank) for plan in plans):
            self._own_stream_sync()
        # Entry agreement without a host stall: the flag's all-reduce sits on the current stream, the pulls
        # are ordered behind it, and its value is read together with the exit flag.
        entry = self._post_flag(error)
        if error:
            exit_flag = self._post_flag(error)
            return {"error": self._read_flags([entry, exit_flag], error), "bytes": 0, "blocks": 0}
        moved, wave_ms = [0], []
        try:
            def launch(w: int, peer: int, earlier):
                plan = plans[w]
                cap = max(24, self.ctx.sm_count // max(1, len(plan.incoming(rank)))) if len(plan.incoming(rank)) > 1 else None
                src_ids, dst_ids = tables[w][peer] if tables is not None else plan.tables_np(peer, rank)
                stream = self._peer_streams.get(peer)
                if stream is None:
                    stream = self._peer_streams[peer] = torch.cuda.Stream(self.device)
                if w < depth:  # behind the entry agreement (later waves follow their predecessors on this stream)
                    stream.wait_stream(torch.cuda.current_stream(self.device))
                for _, done in earlier:  # this sink's copies of wave w - depth, from any source, are done
                    stream.wait_event(done)
                ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                with torch.cuda.stream(stream):
                    ev0.record(stream)
                    res = self.p2p_pull_kv(peer, src_ids, dst_ids, max_ctas=cap)
                    ev1.record(stream)
                if "error" in res:
                    raise RuntimeError(res["error"])
                moved[0] += res["blocks"]
                return ev0, ev1

            def wait_done(handle) -> float:
                handle[1].synchronize()
                return handle[0].elapsed_time(handle[1])

            wave_ms = run_waves(plans, rank, ledger, depth, launch, wait_done, on_wave_landed,
                                wait_for_readers=False)  # the exit agreement below tells a source the same
            main = torch.cuda.current_stream(self.device)
            for stream in self._peer_streams.values():
                main.wait_stream(stream)
        except Exception as e:  # reported, not raised; the others stop waiting through the ledger
            error = f"{type(e).__name__}: {e}"
            try:
                ledger.mark_failed(error)
            except Exception:
                pass
        if not error:
            error = self._device_error("pull")
        error = self._read_flags([entry, self._post_flag(error)], error)
        if error:
            return {"error": error, "bytes": 0, "blocks": 0}
        return {"bytes": moved[0] * pool.block_bytes(), "blocks": moved[0], "wave_ms": wave_ms}

    def _migrate_alltoall(self, plan: MigrationPlan) -> int:
        """Per-layer pipelined all-to-all of packed pages over the library's NCCL communicator; returns
        the number of blocks this rank sent and received.

        For each chunk of layers a source packs the blocks of all its sinks with one gather laid out
        [sink][layer][plane][n_sink][page], so that each sink's share of the chunk is ONE contiguous
        message; all ranks run one grouped exchange (one ncclSend per sink, one ncclRecv per source);
        a sink unpacks [source][layer][plane][n_source][page] with one scatter. Packing chunk c+1,
        exchanging chunk c and unpacking chunk c-1 overlap on three streams with two staging slots
        per direction. A rank may be source and sink at once: its sends and receives of a chunk
        share one NCCL group.
        """
        rank = self.get_global_rank()
        pool = self._require_pool()
        page = pool.page_bytes
        sinks = sorted(plan.outgoing(rank))
        sources = sorted(plan.incoming(rank))
        n_out = [len(plan.tables_np(rank, d)[0]) for d in sinks]
        n_in = [len(plan.tables_np(s, rank)[1]) for s in sources]
        N_out, N_in = sum(n_out), sum(n_in)
        # one chunk schedule for everybody: sized by the busiest rank of the plan
        totals: Dict[Tuple[str, int], int] = {}
        for t in plan.transfers:
            totals[("o", t.src_rank)] = totals.get(("o", t.src_rank), 0) + len(t.src_blocks)
            totals[("i", t.dst_rank)] = totals.get(("i", t.dst_rank), 0) + len(t.src_blocks)
        n_ref = max(totals.values()) if totals else 0
        # a source with many sinks splits a chunk into as many messages: keep each of them large
        fan_out = max((len(plan.outgoing(s)) for s, _ in plan.pairs()), default=1)
        target = getattr(self, "alltoall_chunk_bytes", ALLTOALL_MESSAGE_BYTES * max(1, min(4, fan_out // 2)))
        chunks = plan_chunks(pool.num_layers, n_ref, page, target_bytes=target, taper=True)
        if not chunks:
            return 0
        lc_max = max_chunk_layers(chunks)

        ctx = self.ctx
        # pack and unpack leave some SMs to the NCCL kernel that runs beside them
        copy_ctas = getattr(self, "alltoall_copy_ctas", max(16, ctx.sm_count - ALLTOALL_SMS_LEFT_TO_NCCL))
        saved_cap = ctx.get_option(_lib.OPT_MAX_CTAS)
        if copy_ctas:
            ctx.set_option(_lib.OPT_MAX_CTAS, copy_ctas)
        main = torch.cuda.current_stream(self.device)
        if self._a2a is None:
            self._a2a = {"pack": torch.cuda.Stream(self.device), "wire": torch.cuda.Stream(self.device),
                         "unpack": torch.cuda.Stream(self.device), "out": None, "in": None}
        a2a = self._a2a
        need_out = 2 * pool.packed_bytes(N_out, lc_max)
        need_in = 2 * pool.packed_bytes(N_in, lc_max)
        if N_out and (a2a["out"] is None or a2a["out"].numel() < need_out):
            a2a["out"] = torch.empty(need_out, dtype=torch.uint8, device=self.device)
        if N_in and (a2a["in"] is None or a2a["in"].numel() < need_in):
            a2a["in"] = torch.empty(need_in, dtype=torch.uint8, device=self.device)
        # The segment tables of a plan are uploaded once and kept with it (a plan that is replayed, or the waves
        # of a long migration run again, pay no table work); the ids were checked by _check_plan_part.
        cache = self.__dict__.setdefault("_a2a_tables", {})
        key = (id(plan), len(plan.transfers))
        if key not in cache:
            if len(cache) > 64:
                cache.clear()
            cache[key] = (plan,
                          pool.many_tables([plan.tables_np(rank, d)[0] for d in sinks]) if N_out else None,
                          pool.many_tables([plan.tables_np(s, rank)[1] for s in sources]) if N_in else None)
        _, tab_out, tab_in = cache[key]
        for st in (a2a["pack"], a2a["wire"], a2a["unpack"]):
            st.wait_stream(main)
        ev_packed = [torch.cuda.Event(), torch.cuda.Event()]
        ev_wired = [torch.cuda.Event(), torch.cuda.Event()]
        ev_unpacked = [torch.cuda.Event(), torch.cuda.Event()]

        def slot_of(buf: torch.Tensor, slot: int) -> torch.Tensor:
            half = buf.numel() // 2
            return buf[slot * half:(slot + 1) * half]

        with _range("emm.migrate_alltoall"):
            for c, (begin, count) in enumerate(chunks):
                slot = c & 1
                per_block = count * pool.num_planes * page  # bytes one block occupies in this chunk
                ops = []
                if N_out:
                    flat_out = slot_of(a2a["out"], slot)
                    with torch.cuda.stream(a2a["pack"]):
                        if c >= 2:
                            a2a["pack"].wait_event(ev_wired[slot])       # the exchange that read this slot is done
                        pool.gather_segments(tab_out, flat_out, begin, count)
                        ev_packed[slot].record(a2a["pack"])
                    a2a["wire"].wait_event(ev_packed[slot])
                    off = 0
                    for d, n in zip(sinks, n_out):
                        ops.append((True, flat_out[off * per_block:(off + n) * per_block], d))
                        off += n
                if N_in:
                    flat_in = slot_of(a2a["in"], slot)
                    if c >= 2:
                        a2a["wire"].wait_event(ev_unpacked[slot])        # the scatter that read this slot is done
                    off = 0
                    for s_rank, n in zip(sources, n_in):
                        ops.append((False, flat_in[off * per_block:(off + n) * per_block], s_rank))
                        off += n
                with torch.cuda.stream(a2a["wire"]):
                    ctx.exchange(self._nccl_comm, ops)
                    ev_wired[slot].record(a2a["wire"])
                if N_in:
                    with torch.cuda.stream(a2a["unpack"]):
                        a2a["unpack"].wait_event(ev_wired[slot])
                        pool.scatter_segments(tab_in, flat_in, begin, count)
                        ev_unpacked[slot].record(a2a["unpack"])
        for st in (a2a["pack"], a2a["wire"], a2a["unpack"]):
            main.wait_stream(st)
        ctx.set_option(_lib.OPT_MAX_CTAS, saved_cap)
        return N_out + N_in
