"""torchrec_b200: a Blackwell-native sharded-embedding recommender framework.

Top-level exports mirror ``torchrec/__init__.py:10-30``.
"""
from torchrec_b200.modules.embedding_configs import (  # noqa: F401
    DataType,
    EmbeddingBagConfig,
    EmbeddingConfig,
    EmbeddingTableConfig,
    PoolingType,
)
from torchrec_b200.modules.embedding_modules import (  # noqa: F401
    EmbeddingBagCollection,
    EmbeddingBagCollectionInterface,
    EmbeddingCollection,
    EmbeddingCollectionInterface,
)
from torchrec_b200.sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor, KeyedTensor  # noqa: F401
from torchrec_b200.streamable import Multistreamable, Pipelineable  # noqa: F401

__version__ = "0.1.0"
