"""Multi-GPU runtime: process launch lives in ``bergson_b200.distributed``; this package
holds the peer-memory heap and the collectives that are fused into our kernels."""

from .peer import PeerHeap, gathered_scores, reduce_scatter_gram, symmetric_memory_available

__all__ = ["PeerHeap", "gathered_scores", "reduce_scatter_gram", "symmetric_memory_available"]
