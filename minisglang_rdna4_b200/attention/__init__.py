"""Attention backends. ``--attention-backend`` is accepted for compatibility with the
reference's launch lines; every value maps to the one sm_100a paged backend."""
from .base import AttnMetadata, BaseAttnBackend
from .paged import PagedAttentionBackend


def create_attention_backend(name: str, num_q_heads: int, num_kv_heads: int, head_dim: int, device,
                             max_batch: int = 0, max_seq_len: int = 0, single_split: bool = False
                             ) -> BaseAttnBackend:
    return PagedAttentionBackend(num_q_heads, num_kv_heads, head_dim, device, max_batch, max_seq_len,
                                 single_split)


__all__ = ["AttnMetadata", "BaseAttnBackend", "PagedAttentionBackend", "create_attention_backend"]
