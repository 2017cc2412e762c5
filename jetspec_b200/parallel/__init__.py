"""Multi-GPU execution: tensor parallelism with fused compute+collective kernels over NVLink
peer memory, expert parallelism for MoE layers, and their unfused NCCL baselines."""
from .tp import TensorParallel, shard_rows, shard_cols, shard_attention, shard_mlp
from .symm import SymmetricBuffer
from .ep import ExpertParallel, TokenShardedEP

__all__ = ["TensorParallel", "ExpertParallel", "TokenShardedEP", "SymmetricBuffer", "shard_rows", "shard_cols", "shard_attention", "shard_mlp"]
