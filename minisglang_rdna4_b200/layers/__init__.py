"""Model building blocks."""
from .base import BaseOP
from .linear import (
    ColumnParallelLinear, MergedColumnParallelLinear, QKVParallelLinear, ReplicatedLinear,
    RowParallelLinear,
)
from .embedding import ParallelLMHead, VocabParallelEmbedding
from .norm import RMSNorm
from .rotary import get_rope_cache
from .attention import AttentionLayer
from .activation import GatedActivation
from .moe import MoELayer

__all__ = [
    "BaseOP", "ColumnParallelLinear", "MergedColumnParallelLinear", "QKVParallelLinear",
    "ReplicatedLinear", "RowParallelLinear", "ParallelLMHead", "VocabParallelEmbedding",
    "RMSNorm", "get_rope_cache", "AttentionLayer", "GatedActivation", "MoELayer",
]
