"""Global rank bookkeeping for the worker process group.

Same contract as elasticmm/engine/v0/nccl_coordinator.py: a worker keyed by
(stage, worker_id) gets the next free global rank on first registration
(:42-68), keeps that rank when its role changes (:91-118), and all workers
share one rendezvous address (:179-186). get_rank returns -1 for an unknown
worker, which is the behaviour of the definition that wins in the reference
(:156-168 shadows :120-137).
"""
from __future__ import annotations

from typing import Dict, Tuple

WorkerKey = Tuple[str, int]


class NCCLCoordinator:
    def __init__(self, master_addr: str = "127.0.0.1", master_port: int = 29600):
        self.master_addr = master_addr
        self.master_port = master_port
        self.worker_ranks: Dict[WorkerKey, int] = {}
        self.rank_to_worker: Dict[int, WorkerKey] = {}
        self._next_rank = 0

    def register_worker(self, stage: str, worker_id: int) -> int:
        key = (stage, worker_id)
        rank = self.worker_ranks.get(key)
        if rank is None:
            rank = self._next_rank
            self._next_rank += 1
            self.worker_ranks[key] = rank
            self.rank_to_worker[rank] = key
        return rank

    def unregister_worker(self, stage: str, worker_id: int) -> None:
        rank = self.worker_ranks.pop((stage, worker_id), None)
        if rank is not None:
            self.rank_to_worker.pop(rank, None)

    def update_worker_role(self, worker_id: int, old_stage: str, new_stage: str) -> None:
        """Re-keys a worker under its new stage; the global rank does not change."""
        rank = self.worker_ranks.pop((old_stage, worker_id), None)
        if rank is None:
            return
        self.worker_ranks[(new_stage, worker_id)] = rank
        self.rank_to_worker[rank] = (new_stage, worker_id)

    def get_rank(self, stage: str, worker_id: int) -> int:
        return self.worker_ranks.get((stage, worker_id), -1)

    def get_worker(self, global_rank: int) -> WorkerKey:
        if global_rank not in self.rank_to_worker:
            raise KeyError(f"Global rank {global_rank} not found")
        return self.rank_to_worker[global_rank]

    def get_world_size(self) -> int:
        return len(self.worker_ranks)

    def get_init_method(self) -> str:
        return f"tcp://{self.master_addr}:{self.master_port}"

    def get_all_workers(self) -> Dict[WorkerKey, int]:
        return dict(self.worker_ranks)

    def reset(self) -> None:
        self.worker_ranks.clear()
        self.rank_to_worker.clear()
        self._next_rank = 0
