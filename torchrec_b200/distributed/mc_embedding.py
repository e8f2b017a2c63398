"""Sharded ``ManagedCollisionEmbeddingCollection`` (``torchrec/distributed/mc_embedding.py:67``)."""
from torchrec_b200.distributed.mc_embedding_modules import (  # noqa: F401
    ManagedCollisionEmbeddingCollectionContext,
    ManagedCollisionEmbeddingCollectionSharder,
    ShardedManagedCollisionEmbeddingCollection,
)
