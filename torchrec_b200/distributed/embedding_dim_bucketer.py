"""Group a rank's table shards by row width before they are batched into kernels.

One batched lookup handles mixed widths, but a kernel sized for the widest row wastes lanes on narrow ones and a row cache is
allocated in units of the widest row, so shards are split into buckets of similar *byte* width: one bucket, one per distinct
width, or one per 128-byte line count.  Counterpart of ``torchrec/distributed/embedding_dim_bucketer.py:18-160``."""
from __future__ import annotations

from enum import Enum
from typing import Callable, Dict, List

from torchrec_b200.distributed.embedding_types import ShardedEmbeddingTable
from torchrec_b200.modules.embedding_configs import DATA_TYPE_NUM_BITS, DataType


class EmbDimBucketerPolicy(Enum):
    SINGLE_BUCKET = "single_bucket"
    ALL_BUCKETS = "all_buckets"
    CACHELINE_BUCKETS = "cacheline_buckets"


class EmbDimBucketer:
    """``get_bucket(dim, dtype)`` -> bucket id in ``range(bucket_count())`` for the shards given at construction."""

    def __init__(self, embedding_tables: List[ShardedEmbeddingTable], cfg: EmbDimBucketerPolicy) -> None:
        self.cacheline = 128
        group_of: Dict[EmbDimBucketerPolicy, Callable[[int], int]] = {
            EmbDimBucketerPolicy.SINGLE_BUCKET: lambda nbytes: 0,
            EmbDimBucketerPolicy.ALL_BUCKETS: lambda nbytes: nbytes,
            EmbDimBucketerPolicy.CACHELINE_BUCKETS: lambda nbytes: nbytes // self.cacheline,
        }
        if cfg not in group_of:
            raise ValueError(f"Invalid bucketization config {cfg}")
        group_ids: Dict[int, int] = {}
        self.emb_dim_buckets: Dict[int, int] = {}
        for table in embedding_tables:
            nbytes = self.dim_in_bytes(table.local_cols, table.data_type)
            group = group_of[cfg](nbytes)
            # bucket ids follow first appearance, so the grouping is deterministic for a given table order
            self.emb_dim_buckets.setdefault(nbytes, group_ids.setdefault(group, len(group_ids)))
        self.num_buckets = max(len(group_ids), 1)

    def bucket_count(self) -> int:
        return self.num_buckets

    def get_bucket(self, embedding_dim: int, dtype: DataType) -> int:
        return 0 if self.num_buckets == 1 else self.bucket(embedding_dim, dtype)

    def bucket(self, dim: int, dtype: DataType) -> int:
        return self.emb_dim_buckets[self.dim_in_bytes(dim, dtype)]

    def dim_in_bytes(self, dim: int, dtype: DataType) -> int:
        return dim * DATA_TYPE_NUM_BITS[dtype] // 8
