"""Layers sharded over the GPUs of one node: N-split with an all-gather of outputs, K-split with
an all-reduce of fp32 partials (no counterpart in the reference, which is single-GPU)."""

from fast_kernels.dist.sharded_linear import ShardedW4A16Linear
from fast_kernels.dist.sharding import (
    activation_shard,
    check_shardable,
    column_shard_packets,
    row_shard_packets,
)

__all__ = [
    "ShardedW4A16Linear",
    "activation_shard",
    "check_shardable",
    "column_shard_packets",
    "row_shard_packets",
]
