"""Multi-GPU forms of the hot path: batch x heads sharding (no communication) and sequence parallelism
(state hand-off between neighbouring ranks). One process per GPU, ``torch.distributed`` for the plumbing."""
from .context_parallel import PiecePlan, context_parallel_linear_attention, plan_pieces  # noqa: F401
from .kernel_sharding import ShardPlan, plan_shards, shard_kernel_call, shard_slices  # noqa: F401
