"""``FeatureProcessedEmbeddingBagCollection``: feature processors applied to the KJT, then a weighted EBC lookup
(``torchrec/modules/fp_embedding_modules.py:48``)."""
from __future__ import annotations

from typing import Dict, List, Set, Tuple, Union

import torch
from torch import nn

from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
from torchrec_b200.modules.feature_processor_ import FeatureProcessor, FeatureProcessorsCollection
from torchrec_b200.sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor, KeyedTensor


def apply_feature_processors_to_kjt(features: KeyedJaggedTensor, feature_processors: Dict[str, nn.Module]) -> KeyedJaggedTensor:
    """Per-feature processors: rebuild the KJT from the processed ``JaggedTensor``s (unprocessed features get weight 1)."""
    jt_dict = features.to_dict()
    processed_weights = []
    for key in features.keys():
        jt = jt_dict[key]
        if key in feature_processors:
            w = feature_processors[key](jt).weights()
        else:
            w = torch.ones(jt.values().shape[0], device=jt.values().device)
        processed_weights.append(w)
    return KeyedJaggedTensor(keys=features.keys(), values=features.values(), weights=torch.cat(processed_weights) if processed_weights else features.weights_or_none(),
                             lengths=features.lengths(), offsets=features._offsets, stride=features._stride, length_per_key=features._length_per_key,
                             offset_per_key=features._offset_per_key, index_per_key=features._index_per_key)


class FeatureProcessorDictWrapper(FeatureProcessorsCollection):
    def __init__(self, feature_processors: nn.ModuleDict) -> None:
        super().__init__()
        self._feature_processors = feature_processors

    def forward(self, features: KeyedJaggedTensor) -> KeyedJaggedTensor:
        return apply_feature_processors_to_kjt(features, self._feature_processors)


class FeatureProcessedEmbeddingBagCollection(nn.Module):
    def __init__(self, embedding_bag_collection: EmbeddingBagCollection, feature_processors: Union[Dict[str, FeatureProcessor], FeatureProcessorsCollection]) -> None:
        super().__init__()
        self._embedding_bag_collection = embedding_bag_collection
        self._feature_processors: Union[nn.ModuleDict, FeatureProcessorsCollection]
        if isinstance(feature_processors, FeatureProcessorsCollection):
            self._feature_processors = feature_processors
        else:
            self._feature_processors = nn.ModuleDict(feature_processors)
        assert embedding_bag_collection.is_weighted(), "EmbeddingBagCollection must accept weighted inputs for feature processor"
        feature_names: Set[str] = set()
        for cfg in embedding_bag_collection.embedding_bag_configs():
            feature_names.update(cfg.feature_names)
        if isinstance(self._feature_processors, nn.ModuleDict):
            for k in self._feature_processors.keys():
                assert k in feature_names, f"feature processor key {k} is not a feature of the EmbeddingBagCollection"

    def split(self) -> Tuple[FeatureProcessorsCollection, EmbeddingBagCollection]:
        if isinstance(self._feature_processors, nn.ModuleDict):
            return FeatureProcessorDictWrapper(self._feature_processors), self._embedding_bag_collection
        return self._feature_processors, self._embedding_bag_collection

    def forward(self, features: KeyedJaggedTensor) -> KeyedTensor:
        if isinstance(self._feature_processors, FeatureProcessorsCollection):
            fp_features = self._feature_processors(features)
        else:
            fp_features = apply_feature_processors_to_kjt(features, self._feature_processors)
        return self._embedding_bag_collection(fp_features)
