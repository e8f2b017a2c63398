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

from torchrec_b200.version import __version__  # noqa: E402,F401


def __getattr__(name: str):
    """``torchrec_b200.distributed``, ``.quant`` and ``.tracer`` resolve on first use (importing them eagerly would load the whole runtime)."""
    import importlib

    if name in ("distributed", "quant", "inference", "metrics", "optim", "datasets", "models", "fx"):
        return importlib.import_module(f"torchrec_b200.{name}")
    if name == "tracer":
        return importlib.import_module("torchrec_b200.fx.tracer")
    raise AttributeError(f"module 'torchrec_b200' has no attribute {name!r}")
