"""Sharded ``TensorPool`` (``torchrec/distributed/tensor_pool.py``)."""
from torchrec_b200.distributed.object_pool import ShardedTensorPool, TensorPoolSharder  # noqa: F401
