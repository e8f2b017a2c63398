"""Table-column-wise sharding: column-wise, with all column blocks of a table kept on one node.  The co-location is a property of
the plan (the planner's partitioner enforces it); at run time the blocks are routed exactly like column-wise ones
(cf. ``torchrec/distributed/sharding/twcw_sharding.py``)."""
from __future__ import annotations

from torchrec_b200.distributed.sharding.cw_sharding import CwPooledEmbeddingSharding
from torchrec_b200.distributed.types import ShardingType


class TwCwPooledEmbeddingSharding(CwPooledEmbeddingSharding):
    sharding_type = ShardingType.TABLE_COLUMN_WISE
