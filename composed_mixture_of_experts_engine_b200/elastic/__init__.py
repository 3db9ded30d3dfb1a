"""Elastic training: asynchronous two-tier checkpoints, liveness tracking, recovery."""

from .fault_monitor import (CHECKPOINT_SCHEMA_VERSION, AsyncCheckpointer, ClusterStateMachine, ElasticConfig,
                            ElasticTrainerHarness, LocalNVMeAdapter, ObjectStoreAdapter, S3Adapter,
                            _check_schema_compatibility, _largest_divisor_le)

__all__ = [
    "AsyncCheckpointer", "ClusterStateMachine", "ElasticTrainerHarness", "ElasticConfig", "ObjectStoreAdapter",
    "LocalNVMeAdapter", "S3Adapter", "CHECKPOINT_SCHEMA_VERSION", "_largest_divisor_le",
    "_check_schema_compatibility",
]
