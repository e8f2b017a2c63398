"""Sharded ``KeyedJaggedTensorPool`` (``torchrec/distributed/keyed_jagged_tensor_pool.py``)."""
from torchrec_b200.distributed.object_pool import KeyedJaggedTensorPoolSharder, ShardedKeyedJaggedTensorPool  # noqa: F401
