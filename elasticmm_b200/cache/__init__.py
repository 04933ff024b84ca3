"""KV-cache transfer API under the `cache` name.

The reference's `elasticmm/cache` package holds an image-input cache, not the
KV path; its KV block-table / send / recv surface lives in
`elasticmm/engine/v0`. This package re-exports that surface so callers that
look for a cache-transfer API find it here.
"""
from ..engine.v0 import (BlockLocation, MigrationPlan, NCCLCoordinator, Transfer, TransferMethod,
                         V0BlockManager, V0KVTransferManager, V0Worker)
from ..kv_pool import KVPool, compact_plan

__all__ = ["BlockLocation", "MigrationPlan", "NCCLCoordinator", "Transfer", "TransferMethod",
           "V0BlockManager", "V0KVTransferManager", "V0Worker", "KVPool", "compact_plan"]
