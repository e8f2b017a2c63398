"""Base class of the per-group embedding kernels and the sharded state-dict builder
(``torchrec/distributed/embedding_kernel.py:42-300``)."""
from torchrec_b200.distributed.batched_embedding_kernel import BaseEmbedding, get_state_dict  # noqa: F401
