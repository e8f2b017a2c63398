"""Sharded ``ManagedCollisionEmbeddingBagCollection`` (``torchrec/distributed/mc_embeddingbag.py:52``)."""
from torchrec_b200.distributed.mc_embedding_modules import (  # noqa: F401
    ManagedCollisionEmbeddingBagCollectionContext,
    ManagedCollisionEmbeddingBagCollectionSharder,
    ShardedManagedCollisionEmbeddingBagCollection,
)
