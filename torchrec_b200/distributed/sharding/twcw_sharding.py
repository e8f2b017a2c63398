"""Table-column-wise sharding: column-wise with all column shards of a table kept on one node
(the planner's partitioner enforces the co-location); the runtime is the column-wise one.
Counterpart of ``torchrec/distributed/sharding/twcw_sharding.py``.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from torchrec_b200.distributed.embedding_sharding import EmbeddingShardingInfo
from torchrec_b200.distributed.sharding.cw_sharding import CwPooledEmbeddingSharding
from torchrec_b200.distributed.types import QuantizedCommCodecs, ShardingEnv, ShardingType


class TwCwPooledEmbeddingSharding(CwPooledEmbeddingSharding):
    sharding_type = ShardingType.TABLE_COLUMN_WISE

    def __init__(self, sharding_infos: List[EmbeddingShardingInfo], env: ShardingEnv, device: Optional[torch.device] = None,
                 permute_embeddings: bool = False, qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None) -> None:
        super().__init__(sharding_infos, env, device, permute_embeddings=permute_embeddings, qcomm_codecs_registry=qcomm_codecs_registry)
