"""KV movement surface of the v0 engine (mirrors elasticmm/engine/v0/__init__.py
for the classes on the KV-cache path)."""
from .block_manager import BlockLocation, V0BlockManager, V0VisionBlockManager
from .config import DEFAULT_V0_KV_CONFIG, V0KVCacheConfig
from .kv_transfer import MigrationPlan, Transfer, TransferMethod, V0KVTransferManager
from .nccl_coordinator import NCCLCoordinator
from .utils import EngineStage, KVTransferMetrics, MigratingRequest, Request
from .worker import V0Worker

__all__ = [
    "BlockLocation", "V0BlockManager", "V0VisionBlockManager", "MigrationPlan", "Transfer",
    "TransferMethod", "V0KVTransferManager", "NCCLCoordinator", "EngineStage", "KVTransferMetrics",
    "MigratingRequest", "Request", "V0Worker", "V0KVCacheConfig", "DEFAULT_V0_KV_CONFIG",
]
