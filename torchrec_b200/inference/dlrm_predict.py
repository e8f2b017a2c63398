"""Serving wrapper of DLRM (``torchrec/inference/dlrm_predict.py``): a ``PredictModule`` that takes the request dictionary
(``float_features`` and the ``id_list_features`` KJT) and a ``PredictFactory`` that builds, quantizes and places the model."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch
from torch import nn

from torchrec_b200.datasets.criteo import DEFAULT_CAT_NAMES, DEFAULT_INT_NAMES
from torchrec_b200.inference.modules import BatchingMetadata, PredictFactory, PredictModule, quantize_embeddings
from torchrec_b200.models.dlrm import DLRM
from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig
from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


def create_training_batch(args: Any) -> Any:
    """A random Criteo-shaped batch sized by ``args.batch_size`` / ``args.num_embedding_features`` (sample input for packaging)."""
    from torchrec_b200.inference.client import create_training_batch as _create

    return _create(args)


@dataclass
class DLRMModelConfig:
    dense_arch_layer_sizes: List[int]
    dense_in_features: int
    embedding_dim: int
    id_list_features_keys: List[str]
    num_embeddings_per_feature: List[int]
    over_arch_layer_sizes: List[int]
    sample_input: Optional[Any] = None
    num_embeddings: int = 0


def default_dlrm_config(num_embeddings: int = 100_000) -> DLRMModelConfig:
    return DLRMModelConfig(dense_arch_layer_sizes=[512, 256, 64], dense_in_features=len(DEFAULT_INT_NAMES), embedding_dim=64, id_list_features_keys=list(DEFAULT_CAT_NAMES),
                           num_embeddings_per_feature=[num_embeddings] * len(DEFAULT_CAT_NAMES), over_arch_layer_sizes=[512, 512, 256, 1])


class DLRMPredictModule(PredictModule):
    """``forward({"float_features": [B, n], "id_list_features": KJT}) -> {"default": [B]}`` (sigmoid scores)."""

    def __init__(self, embedding_bag_collection: nn.Module, dense_in_features: int, dense_arch_layer_sizes: List[int], over_arch_layer_sizes: List[int],
                 id_list_features_keys: List[str], dense_device: Optional[torch.device] = None) -> None:
        module = DLRM(embedding_bag_collection=embedding_bag_collection, dense_in_features=dense_in_features, dense_arch_layer_sizes=dense_arch_layer_sizes,
                      over_arch_layer_sizes=over_arch_layer_sizes, dense_device=dense_device)
        super().__init__(module, str(dense_device) if dense_device is not None else None)
        self.id_list_features_keys: List[str] = id_list_features_keys

    def predict_forward(self, batch: Dict[str, Any]) -> Any:
        try:
            logits = self.predict_module(batch["float_features"], batch["id_list_features"])
            return {"default": torch.sigmoid(logits.float()).squeeze(-1)}
        except Exception as e:
            raise RuntimeError(f"DLRM predict failed: {type(e).__name__}: {e}") from e


class DLRMPredictFactory(PredictFactory):
    def __init__(self, model_config: Optional[DLRMModelConfig] = None, quantize: bool = True, device: Optional[str] = None) -> None:
        self.model_config = model_config or default_dlrm_config()
        self.quantize = quantize
        self.device = device or ("cuda" if torch.cuda.is_available() else "cpu")

    def create_predict_module(self, world_size: int = 1, device: Optional[str] = None) -> nn.Module:
        cfg = self.model_config
        dev = torch.device(device or self.device)
        tables = [EmbeddingBagConfig(name=f"t_{k}", embedding_dim=cfg.embedding_dim, num_embeddings=n, feature_names=[k])
                  for k, n in zip(cfg.id_list_features_keys, cfg.num_embeddings_per_feature)]
        ebc = EmbeddingBagCollection(tables=tables, device=torch.device("cpu"))
        module = DLRMPredictModule(ebc, cfg.dense_in_features, cfg.dense_arch_layer_sizes, cfg.over_arch_layer_sizes, cfg.id_list_features_keys, dense_device=torch.device("cpu"))
        module = self.run_weights_independent_tranformations(module)
        module = self.run_weights_dependent_transformations(module)
        return module.to(dev) if dev.type != "meta" else module

    def batching_metadata(self) -> Dict[str, BatchingMetadata]:
        return {"float_features": BatchingMetadata(type="dense", device=self.device, pinned=[]),
                "id_list_features": BatchingMetadata(type="sparse", device=self.device, pinned=[])}

    def result_metadata(self) -> str:
        return "dict_of_tensor"

    def run_weights_independent_tranformations(self, predict_module: nn.Module) -> nn.Module:
        return predict_module

    def run_weights_dependent_transformations(self, predict_module: nn.Module) -> nn.Module:
        if self.quantize:
            predict_module = quantize_embeddings(predict_module, dtype=torch.qint8, inplace=True)
        return predict_module.eval()

    def model_inputs_data(self) -> Dict[str, Any]:
        return {"id_list_features": list(self.model_config.id_list_features_keys), "float_features": self.model_config.dense_in_features}
