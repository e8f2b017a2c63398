"""Sharded ``FusedEmbeddingCollection`` (``torchrec/distributed/fused_embedding.py:31``)."""
from torchrec_b200.distributed.fused_embeddingbag import FusedEmbeddingCollectionSharder, ShardedFusedEmbeddingCollection  # noqa: F401
