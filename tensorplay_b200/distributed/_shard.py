"""Legacy ``ShardedTensor`` API (tensorplay/distributed/_shard): PyTorch's package, with the names of
its sub-modules (sharded tensor, sharding specs and plans, sharded optimizer) reachable at this level."""
from torch.distributed._shard import *  # noqa: F401,F403
from torch.distributed._shard import sharded_tensor, sharding_plan, sharding_spec  # noqa: F401
from torch.distributed._shard.sharded_optim import ShardedOptimizer  # noqa: F401
from torch.distributed._shard.sharded_tensor import (Shard, ShardedTensor, ShardedTensorBase, ShardedTensorMetadata,  # noqa: F401
                                                     TensorProperties, empty, full, init_from_local_shards, ones,
                                                     rand, randn, zeros)
from torch.distributed._shard.sharding_plan import ShardingPlan, ShardingPlanner  # noqa: F401
from torch.distributed._shard.sharding_spec import (ChunkShardingSpec, DevicePlacementSpec, EnumerableShardingSpec,  # noqa: F401
                                                    PlacementSpec, ShardingSpec, ShardMetadata)


# the reference has a package at this path: sub-module names without a file here resolve to PyTorch's
__path__: list = []
