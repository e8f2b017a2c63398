"""Dynamic embedding: unbounded global ids mapped onto bounded HBM-resident tables that act as a cache of a
host/remote parameter store (C++ core in ``csrc/cpu/tde_*``).

Cf. ``contrib/dynamic_embedding/src/torchrec_dynamic_embedding`` of the reference."""
from torchrec_b200.contrib.dynamic_embedding.id_transformer import IDTransformer, TransformResult  # noqa: F401
from torchrec_b200.contrib.dynamic_embedding.id_transformer_collection import IDTransformerCollection  # noqa: F401
from torchrec_b200.contrib.dynamic_embedding.id_transformer_group import IDTransformerGroup  # noqa: F401
from torchrec_b200.contrib.dynamic_embedding.ps import PS, PSCollection  # noqa: F401
from torchrec_b200.contrib.dynamic_embedding.utils import register_io  # noqa: F401
from torchrec_b200.contrib.dynamic_embedding.dataloader import DataLoader, save, wrap  # noqa: F401
from torchrec_b200.contrib.dynamic_embedding.tensor_list import TensorList  # noqa: F401
