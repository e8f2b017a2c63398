"""``LocalShardsWrapper``: several local shards (with global offsets) behind one tensor object.

A ``DTensor`` can only hold one local tensor; column-wise and grid sharding put several shards of
one table on a rank.  The wrapper carries those shards plus their offsets and implements the
distributed-checkpoint hooks (``__create_write_items__`` / ``__create_chunk_list__`` /
``__get_tensor_shard__``).  PyTorch ships the class (it was upstreamed from the reference's
``torchrec/distributed/shards_wrapper.py:30``); it is re-exported here so that state dicts are
type-compatible with the reference's.
"""
from torch.distributed.tensor._shards_wrapper import LocalShardsWrapper  # noqa: F401

__all__ = ["LocalShardsWrapper"]
