"""``TableBatchedEmbeddingSlice``: a parameter that is a ``[rows, dim]`` view into the flat weight buffer of a table-batched kernel
and reports the matching slice of that buffer's gradient (``torchrec/distributed/composable/table_batched_embedding_slice.py:17``)."""
from torchrec_b200.distributed.batched_embedding_kernel import TableBatchedEmbeddingSlice  # noqa: F401
