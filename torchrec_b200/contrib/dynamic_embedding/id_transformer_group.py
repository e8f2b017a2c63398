"""All id-transformer collections of a model, keyed by the path of the embedding module they serve."""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
from torch import nn

from torchrec_b200.contrib.dynamic_embedding.id_transformer_collection import IDTransformerCollection
from torchrec_b200.contrib.dynamic_embedding.ps import PSCollection
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


class IDTransformerGroup:
    def __init__(self, url: str, module: nn.Module, configs_dict: Dict[str, list], *, eviction_config: Optional[dict] = None,
                 transform_config: Optional[dict] = None, ps_config: Optional[dict] = None) -> None:
        """``configs_dict``: ``{path of an embedding module inside `module`: its table configs}``."""
        self._collections: Dict[str, IDTransformerCollection] = {}
        sd = module.state_dict()
        for path, configs in configs_dict.items():
            prefix = f"{path}." if path else ""
            table_sd = {}
            plan = {}
            for cfg in configs:
                for container in ("embedding_bags", "embeddings"):
                    k = f"{prefix}{container}.{cfg.name}.weight"
                    if k in sd:
                        table_sd[f"{cfg.name}.weight"] = sd[k]
                plan[cfg.name] = (cfg.num_embeddings, cfg.embedding_dim)
            ps = PSCollection(path, plan, table_sd, url, ps_config)
            self._collections[path] = IDTransformerCollection(configs, eviction_config, transform_config, ps)

    def transform(self, kjt_dict: Dict[str, KeyedJaggedTensor]) -> Tuple[Dict[str, KeyedJaggedTensor], List]:
        out: Dict[str, KeyedJaggedTensor] = {}
        handles: List = []
        for path, kjt in kjt_dict.items():
            out[path], hs = self._collections[path].transform(kjt)
            handles.extend(hs)
        return out, handles

    def save(self) -> None:
        for c in self._collections.values():
            c.save()
