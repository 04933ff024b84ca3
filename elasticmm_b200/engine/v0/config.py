"""Configuration of the KV-cache path of the v0 engine.

Mirrors the fields of elasticmm/engine/v0/config.py:10-77 that reach the KV
data plane (block size, block counts, dtype, transfer method) and adds the
pool geometry the reference takes from vLLM's model config (layers, KV heads,
head size) so a worker's pool can be sized and allocated from one object.
Fields of the reference that configure the model runner or the schedulers are
accepted by from_dict and ignored.
"""
from __future__ import annotations

from dataclasses import dataclass, fields
from typing import Any, Dict

from .kv_transfer import TransferMethod

_ELEM_SIZE = {"float16": 2, "half": 2, "bfloat16": 2, "float32": 4, "float": 4, "float8": 1, "fp8": 1,
              "uint8": 1, "int8": 1}

# Ignored on purpose: they configure parts of the reference outside the KV path.
_FOREIGN_FIELDS = frozenset({
    "model_path", "max_model_len", "tensor_parallel_size", "trust_remote_code", "num_encoding_workers",
    "num_prefill_workers", "num_decoding_workers", "gpu_memory_utilization", "seed",
    "max_batch_size_encoding", "max_batch_size_prefill", "max_batch_size_decoding",
    "enable_chunked_prefill", "enable_prefix_caching",
})


@dataclass
class V0KVCacheConfig:
    # reference fields (same names and defaults, config.py:25-35)
    block_size: int = 16
    max_num_gpu_blocks: int = 5000
    max_num_cpu_blocks: int = 1000
    dtype: str = "float16"
    kv_transfer_method: str = "p2p_copy"
    # pool geometry (vLLM's model config in the reference)
    num_layers: int = 32
    num_kv_heads: int = 32
    head_size: int = 128
    layout: str = "nhd"          # "nhd": [2, NB, BS, H, D] (reference), "hnd": [2, NB, H, BS, D]
    # B200_PEER only: which end runs the copy kernel
    peer_direction: str = "pull"

    def to_dict(self) -> Dict[str, Any]:
        return {f.name: getattr(self, f.name) for f in fields(self)}

    @classmethod
    def from_dict(cls, config_dict: Dict[str, Any]) -> "V0KVCacheConfig":
        known = {f.name for f in fields(cls)}
        unknown = set(config_dict) - known - _FOREIGN_FIELDS
        if unknown:
            raise TypeError(f"unexpected configuration keys: {sorted(unknown)}")
        return cls(**{k: v for k, v in config_dict.items() if k in known})

    def validate(self) -> None:
        """Same assertions as config.py:65-73 for the shared fields; the
        transfer method may also be 'b200_peer'."""
        assert self.block_size > 0, "Block size must be positive"
        assert self.max_num_gpu_blocks > 0, "At least one GPU block required"
        assert self.max_num_cpu_blocks >= 0, "CPU block count must not be negative"
        assert self.kv_transfer_method in [m.value for m in TransferMethod], \
            f"Invalid KV transfer method: {self.kv_transfer_method}"
        assert self.dtype in _ELEM_SIZE, f"Unsupported KV dtype: {self.dtype}"
        assert self.layout in ("nhd", "hnd"), f"Unknown pool layout: {self.layout}"
        assert self.peer_direction in ("pull", "push"), f"Unknown peer direction: {self.peer_direction}"
        assert min(self.num_layers, self.num_kv_heads, self.head_size) > 0, "Pool geometry must be positive"

    # -- derived quantities ---------------------------------------------------

    @property
    def transfer_method(self) -> TransferMethod:
        return TransferMethod(self.kv_transfer_method)

    @property
    def elem_size(self) -> int:
        return _ELEM_SIZE[self.dtype]

    @property
    def page_bytes(self) -> int:
        """One block of one plane (K or V) of one layer."""
        return self.block_size * self.num_kv_heads * self.head_size * self.elem_size

    @property
    def block_bytes(self) -> int:
        """One block across K, V and all layers: what moving one block id costs."""
        return 2 * self.num_layers * self.page_bytes

    def pool_bytes(self, num_blocks: int | None = None) -> int:
        return (self.max_num_gpu_blocks if num_blocks is None else num_blocks) * self.block_bytes

    def blocks_for_bytes(self, budget_bytes: int) -> int:
        """Largest block count whose pool fits the budget, capped at max_num_gpu_blocks."""
        return max(0, min(self.max_num_gpu_blocks, budget_bytes // self.block_bytes))

    def blocks_for_tokens(self, num_tokens: int) -> int:
        return -(-num_tokens // self.block_size)


DEFAULT_V0_KV_CONFIG = V0KVCacheConfig()

__all__ = ["V0KVCacheConfig", "DEFAULT_V0_KV_CONFIG"]
