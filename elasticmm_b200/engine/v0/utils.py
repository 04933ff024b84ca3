"""Small host-side types of the v0 engine that the KV path touches.

Mirrors the parts of elasticmm/engine/v0/utils.py used by the block manager and
the transfer path: EngineStage (:10-14), the length accessors of Request
(:66-76), MigratingRequest's block-index fields (:114-147) and the KV-transfer
part of StageMetrics (:244-247,292-297). Scheduling, sampling and timing fields
of the reference's Request are outside this path and omitted.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Dict, List, Optional


class EngineStage(Enum):
    ENCODING = "encoding"
    PREFILL = "prefill"
    DECODING = "decoding"


@dataclass
class Request:
    """The slice of a serving request that block accounting needs."""

    request_id: str
    prompt_token_ids: Optional[List[int]] = None
    output_token_ids: List[int] = field(default_factory=list)
    images: Optional[List[Any]] = None

    def get_input_len(self) -> int:
        return len(self.prompt_token_ids) if self.prompt_token_ids else 0

    def get_output_len(self) -> int:
        return len(self.output_token_ids)

    def get_total_len(self) -> int:
        return self.get_input_len() + self.get_output_len()

    @classmethod
    def of_length(cls, request_id: str, num_tokens: int) -> "Request":
        """A request whose prompt is `num_tokens` placeholder tokens."""
        return cls(request_id=request_id, prompt_token_ids=[0] * int(num_tokens))


@dataclass
class BatchedRequests:
    requests: List[Request] = field(default_factory=list)

    def __len__(self) -> int:
        return len(self.requests)

    def __iter__(self):
        return iter(self.requests)


@dataclass
class MigratingRequest:
    """A request handed from one stage to the next, with its source block table."""

    req: Request
    kv_block_indexes: Optional[List[int]] = None
    vision_block_indexes: Optional[List[int]] = None
    source_stage: Optional[EngineStage] = None
    source_worker_id: Optional[int] = None
    target_stage: Optional[EngineStage] = None
    target_worker_id: Optional[int] = None


class KVTransferMetrics:
    """KV-transfer samples in the two shapes the reference records.

    `record_kv_transfer(transfer_time_sec, num_blocks)` has the signature of
    StageMetrics.record_kv_transfer; `get_stats()['kv_transfer']` has the keys
    the calibration script reads (avg_time_sec, avg_blocks,
    bandwidth_blocks_per_sec). Bytes are tracked as well so GB/s can be given.
    """

    def __init__(self, stage_name: str = "decoding", block_bytes: int = 0):
        self.stage_name = stage_name
        self.block_bytes = block_bytes
        self.kv_transfer_times: List[float] = []
        self.kv_transfer_sizes: List[int] = []

    def record_kv_transfer(self, transfer_time_sec: float, num_blocks: int) -> None:
        self.kv_transfer_times.append(float(transfer_time_sec))
        self.kv_transfer_sizes.append(int(num_blocks))

    def gain_cost_params(self) -> Dict[str, float]:
        """The two keys the calibration derives from KV-transfer samples
        (examples/calibrate_gain_cost.py:612-640): `migration_cost` = mean seconds per
        transfer, `kv_transfer_bandwidth` = blocks per second."""
        kv = self.get_stats().get("kv_transfer")
        if not kv:
            return {}
        return {"migration_cost": kv["avg_time_sec"], "kv_transfer_bandwidth": kv["bandwidth_blocks_per_sec"]}

    def update_gain_cost_file(self, path: str = "gain_cost_params.json") -> Dict[str, Any]:
        """Merges the measured migration cost into the JSON file that
        GainCostConfig loads (elasticmm/core/gain_cost_config.py:58-87); other keys are kept."""
        import json
        import os

        params: Dict[str, Any] = {}
        if os.path.exists(path):
            with open(path) as f:
                params = json.load(f)
        params.update(self.gain_cost_params())
        with open(path, "w") as f:
            json.dump(params, f, indent=2, sort_keys=True)
        return params

    def get_stats(self) -> Dict[str, Any]:
        stats: Dict[str, Any] = {"stage": self.stage_name}
        if self.kv_transfer_times:
            total_t = sum(self.kv_transfer_times)
            total_b = sum(self.kv_transfer_sizes)
            n = len(self.kv_transfer_times)
            kv = {
                "avg_time_sec": total_t / n,
                "avg_blocks": total_b / n,
                "bandwidth_blocks_per_sec": total_b / total_t if total_t > 0 else 0,
            }
            if self.block_bytes:
                kv["bandwidth_gb_per_sec"] = total_b * self.block_bytes / total_t / 1e9 if total_t > 0 else 0
            stats["kv_transfer"] = kv
        return stats
