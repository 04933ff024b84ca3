"""Host-side block tables: request id -> ordered list of physical block ids.

Behaviour follows elasticmm/engine/v0/block_manager.py: ids are handed out
from the head of a free list (:102-142) and freed ids go to its tail
(:247-256), so tables fragment over time; a request's table only grows
(:174-209,216-245,281-303); swapping rewrites the table to ids of the other
location and parks the old ids on a "swapping" list that is folded back into
the free list once the copies are known to be done (:118-123,305-377).

Added here, with no counterpart in the reference: `compact` (defragmentation
plan + table rewrite, planned by the C library's emm_compact_plan) and
`get_slot_mapping` (the table-to-slot arithmetic that the model runner
applies before reshape_and_cache, elasticmm/engine/v0/worker_steps.py:219,411).
"""
from __future__ import annotations

from collections import deque
from enum import Enum
from typing import Callable, Deque, Dict, Iterable, List, Optional, Sequence, Tuple

from .utils import BatchedRequests, Request


class BlockLocation(Enum):
    GPU = "gpu"
    CPU = "cpu"


class V0BlockManager:
    """Block tables and free lists for one stage's KV pool."""

    def __init__(
        self,
        stage: str,
        max_num_gpu_blocks: int,
        max_num_cpu_blocks: int,
        block_size: int,
        engine_remote_call_all_workers_async: Optional[Callable] = None,
    ):
        self.stage = stage
        self.max_num_gpu_blocks = max_num_gpu_blocks
        self.max_num_cpu_blocks = max_num_cpu_blocks
        self.block_size = block_size
        self.engine_remote_call_all_workers_async = engine_remote_call_all_workers_async
        self.block_table: Dict[str, List[int]] = {}
        self.request_location: Dict[str, BlockLocation] = {}
        self.swap_count = 0
        self._reset_free_blocks()

    # -- free lists -----------------------------------------------------------
    def _reset_free_blocks(self) -> None:
        """Re-creates the free lists after the pool size is (re)measured."""
        self._free: Dict[BlockLocation, Deque[int]] = {
            BlockLocation.GPU: deque(range(self.max_num_gpu_blocks)),
            BlockLocation.CPU: deque(range(self.max_num_cpu_blocks)),
        }
        self._swapping: Dict[BlockLocation, List[int]] = {BlockLocation.GPU: [], BlockLocation.CPU: []}

    @property
    def free_gpu_blocks_list(self) -> List[int]:
        return list(self._free[BlockLocation.GPU])

    @property
    def free_cpu_blocks_list(self) -> List[int]:
        return list(self._free[BlockLocation.CPU])

    @property
    def swapping_gpu_blocks_list(self) -> List[int]:
        return list(self._swapping[BlockLocation.GPU])

    @property
    def swapping_cpu_blocks_list(self) -> List[int]:
        return list(self._swapping[BlockLocation.CPU])

    def get_num_avail_gpu_blocks(self) -> int:
        return len(self._free[BlockLocation.GPU]) + len(self._swapping[BlockLocation.GPU])

    def get_num_avail_cpu_blocks(self) -> int:
        return len(self._free[BlockLocation.CPU]) + len(self._swapping[BlockLocation.CPU])

    def _get_free_blocks(self, num_blocks: int, location: BlockLocation) -> List[int]:
        free = self._free[location]
        parked = self._swapping[location]
        where = "GPU" if location == BlockLocation.GPU else "CPU"
        avail = len(free) + len(parked)
        assert avail >= num_blocks, (
            f"Not enough free blocks on {where}, requested {num_blocks}, available {avail}")
        if len(free) < num_blocks:
            # Parked ids become reusable only after the copies that read them finished.
            if self.engine_remote_call_all_workers_async:
                self.engine_remote_call_all_workers_async(
                    "wait_for_all_swap_out" if location == BlockLocation.GPU else "wait_for_all_swap_in")
            free.extend(parked)
            parked.clear()
        return [free.popleft() for _ in range(num_blocks)]

    # -- sizing -----------------------------------------------------------------
    def get_allocated_num_blocks(self, request_id: str) -> int:
        return len(self.block_table.get(request_id, ()))

    def get_location(self, request_id: str) -> Optional[BlockLocation]:
        return self.request_location.get(request_id)

    def get_num_blocks_needed(self, request: Request) -> int:
        return -(-request.get_total_len() // self.block_size)

    def get_num_append_blocks_needed(self, request: Request) -> int:
        assert self.request_location.get(request.request_id) == BlockLocation.GPU, (
            f"Request {request.request_id} is not on GPU")
        return max(0, self.get_num_blocks_needed(request) - len(self.block_table[request.request_id]))

    # -- allocation -------------------------------------------------------------
    def allocate_blocks(self, request: Request, num_blocks: Optional[int] = None) -> None:
        rid = request.request_id
        assert rid not in self.block_table or self.request_location.get(rid) == BlockLocation.GPU, (
            f"Request {rid} is on CPU. Migrate to GPU first.")
        needed = self.get_num_blocks_needed(request) if num_blocks is None else num_blocks
        table = self.block_table.get(rid)
        if table is None:
            self.block_table[rid] = self._get_free_blocks(needed, BlockLocation.GPU)
            self.request_location[rid] = BlockLocation.GPU
        elif len(table) < needed:
            table += self._get_free_blocks(needed - len(table), BlockLocation.GPU)

    def allocate_blocks_batched(self, batched_requests: BatchedRequests) -> None:
        for request in batched_requests:
            self.allocate_blocks(request)

    def expand_blocks_for_seq_len(self, request_id: str, expanded_seq_len: int) -> List[int]:
        if request_id not in self.block_table:
            raise ValueError(f"Request {request_id} not allocated")
        table = self.block_table[request_id]
        needed = -(-expanded_seq_len // self.block_size)
        if len(table) < needed:
            table += self._get_free_blocks(needed - len(table), BlockLocation.GPU)
        return table

    def append_blocks(self, request: Request) -> None:
        rid = request.request_id
        assert rid in self.block_table, f"Request {rid} not allocated yet"
        extra = self.get_num_append_blocks_needed(request)
        if extra > 0:
            self.block_table[rid].extend(self._get_free_blocks(extra, BlockLocation.GPU))

    def free_blocks(self, request_id: str) -> None:
        assert request_id in self.block_table, f"Request {request_id} not allocated"
        location = self.request_location.pop(request_id)
        self._free[location].extend(self.block_table.pop(request_id))

    def free_blocks_batched(self, requests: Iterable[Request]) -> None:
        for request in requests:
            if request.request_id in self.block_table:
                self.free_blocks(request.request_id)

    def get_block_table(self, request_id: str) -> List[int]:
        return self.block_table.get(request_id, [])

    def can_allocate(self, request: Request) -> bool:
        return self.get_num_avail_gpu_blocks() >= self.get_num_blocks_needed(request)

    def can_append(self, request: Request) -> bool:
        if request.request_id not in self.block_table:
            return self.can_allocate(request)
        return self.get_num_avail_gpu_blocks() >= self.get_num_append_blocks_needed(request)

    # -- swapping ---------------------------------------------------------------
    def _move(self, request_id: str, src: BlockLocation, dst: BlockLocation) -> Tuple[List[int], List[int]]:
        assert request_id in self.block_table, f"request {request_id} not allocated"
        assert self.request_location[request_id] == src, f"request {request_id} is on {dst} now"
        old_ids = self.block_table[request_id]
        new_ids = self._get_free_blocks(len(old_ids), dst)
        self._swapping[src] += old_ids
        self.block_table[request_id] = new_ids
        self.request_location[request_id] = dst
        return old_ids, new_ids

    def swap_out(self, request_id: str) -> Tuple[List[int], List[int]]:
        """Moves a request's table to CPU ids; returns (gpu_blocks, cpu_blocks)."""
        return self._move(request_id, BlockLocation.GPU, BlockLocation.CPU)

    def swap_in(self, request_id: str) -> Tuple[List[int], List[int]]:
        """Moves a request's table to GPU ids; returns (cpu_blocks, gpu_blocks)."""
        return self._move(request_id, BlockLocation.CPU, BlockLocation.GPU)

    def swap_requests(self, request_ids: Sequence[str], is_swap_in: bool) -> Tuple[List[int], List[int]]:
        """Rewrites the tables of a batch and asks the workers to copy the blocks.

        Returns (source_block_ids, target_block_ids), the flat lists passed to
        the workers' `swap_blocks`.
        """
        src = BlockLocation.CPU if is_swap_in else BlockLocation.GPU
        dst = BlockLocation.GPU if is_swap_in else BlockLocation.CPU
        source_ids: List[int] = []
        target_ids: List[int] = []
        for rid in request_ids:
            old_ids, new_ids = self._move(rid, src, dst)
            source_ids += old_ids
            target_ids += new_ids
        if self.engine_remote_call_all_workers_async:
            self.engine_remote_call_all_workers_async(
                "swap_blocks", list(request_ids), source_ids, target_ids, is_swap_in)
        self.swap_count += 1
        return source_ids, target_ids

    def swap_in_requests(self, request_ids: Sequence[str]):
        return self.swap_requests(request_ids, is_swap_in=True)

    def swap_out_requests(self, request_ids: Sequence[str]):
        return self.swap_requests(request_ids, is_swap_in=False)

    def is_all_requests_on_gpu(self, request_ids: Iterable[str]) -> bool:
        return all(self.request_location.get(rid) != BlockLocation.CPU for rid in request_ids)

    def get_block_usage(self) -> Dict[str, str]:
        used_gpu = self.max_num_gpu_blocks - self.get_num_avail_gpu_blocks()
        used_cpu = self.max_num_cpu_blocks - self.get_num_avail_cpu_blocks()
        pct = lambda n, d: round(n / d * 100) if d else 0
        return {
            "gpu": f"{pct(used_gpu, self.max_num_gpu_blocks)}% ({used_gpu}/{self.max_num_gpu_blocks})",
            "cpu": f"{pct(used_cpu, self.max_num_cpu_blocks)}% ({used_cpu}/{self.max_num_cpu_blocks})",
            "swap": f"{len(self._swapping[BlockLocation.GPU])} -> {len(self._swapping[BlockLocation.CPU])}",
            "#req": f"{len(self.block_table)}",
        }

    # -- additions --------------------------------------------------------------
    def get_slot_mapping(self, request_id: str, positions: Iterable[int]) -> List[int]:
        """slot = table[pos // BS] * BS + pos % BS for each token position."""
        table = self.block_table[request_id]
        bs = self.block_size
        return [table[p // bs] * bs + p % bs for p in positions]

    def compact(self) -> Tuple[List[int], List[int]]:
        """Plans a defragmentation of the GPU pool and rewrites the tables.

        After the call every GPU-resident request's blocks have ids below the
        number of live GPU blocks, and the free list is the ascending range
        above them. Returns (move_src, move_dst): the caller must copy those
        blocks (V0Worker.compact_blocks / KVPool.copy_blocks) before any block
        is written again. Requests with CPU tables are untouched. Blocks
        parked on the swapping list must have been drained first.
        """
        from ...kv_pool import compact_plan

        assert not self._swapping[BlockLocation.GPU], "drain pending swap-outs before compaction"
        rids = [rid for rid, loc in self.request_location.items() if loc == BlockLocation.GPU]
        flat: List[int] = []
        for rid in rids:
            flat += self.block_table[rid]
        new_ids, move_src, move_dst = compact_plan(flat, self.max_num_gpu_blocks)
        pos = 0
        for rid in rids:
            n = len(self.block_table[rid])
            self.block_table[rid] = [int(x) for x in new_ids[pos:pos + n]]
            pos += n
        self._free[BlockLocation.GPU] = deque(range(len(flat), self.max_num_gpu_blocks))
        return [int(x) for x in move_src], [int(x) for x in move_dst]


class V0VisionBlockManager(V0BlockManager):
    """Block tables for vision embeddings: a fixed block count per image.

    As in the reference (elasticmm/engine/v0/block_manager.py:526-542) an
    image is costed at `embedding_tokens_per_image` tokens (576 by default).
    """

    embedding_tokens_per_image = 576

    def get_num_blocks_needed(self, request: Request) -> int:
        if not request.images:
            return 0
        per_image = -(-self.embedding_tokens_per_image // self.block_size)
        return len(request.images) * per_image
