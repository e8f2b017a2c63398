"""``FeatureProcessedEmbeddingBagCollection``: per-id weights computed by feature processors, then a weighted pooled lookup
(``torchrec/modules/fp_embedding_modules.py:48``).

Processors come either as a dict ``feature -> FeatureProcessor`` (each sees the ``JaggedTensor`` of its feature) or as one
``FeatureProcessorsCollection`` that rewrites the whole KJT.  Internally both are driven through one callable, ``_reweigh``; the
attribute ``_feature_processors`` keeps the form the caller gave, so checkpoints keep their key names.
"""
from __future__ import annotations

from typing import Dict, Tuple, Union

import torch
from torch import nn

from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
from torchrec_b200.modules.feature_processor_ import FeatureProcessor, FeatureProcessorsCollection
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor, KeyedTensor


def apply_feature_processors_to_kjt(features: KeyedJaggedTensor, feature_processors: Dict[str, nn.Module]) -> KeyedJaggedTensor:
    """The same ids with the weights the per-feature processors assign; a feature without a processor weighs 1 per id."""
    per_feature = features.to_dict()
    weights = []
    for key in features.keys():
        jt = per_feature[key]
        processor = feature_processors[key] if key in feature_processors else None
        weights.append(processor(jt).weights() if processor is not None else jt.values().new_ones(jt.values().shape[0], dtype=torch.float32))
    return KeyedJaggedTensor(
        keys=features.keys(), values=features.values(), weights=torch.cat(weights) if weights else features.weights_or_none(), lengths=features.lengths(),
        offsets=features._offsets, stride=features._stride, length_per_key=features._length_per_key, offset_per_key=features._offset_per_key,
        index_per_key=features._index_per_key)


class FeatureProcessorDictWrapper(FeatureProcessorsCollection):
    """A dict of per-feature processors behind the collection interface."""

    def __init__(self, feature_processors: nn.ModuleDict) -> None:
        super().__init__()
        self._feature_processors = feature_processors

    def forward(self, features: KeyedJaggedTensor) -> KeyedJaggedTensor:
        return apply_feature_processors_to_kjt(features, self._feature_processors)


class FeatureProcessedEmbeddingBagCollection(nn.Module):
    def __init__(self, embedding_bag_collection: EmbeddingBagCollection, feature_processors: Union[Dict[str, FeatureProcessor], FeatureProcessorsCollection]) -> None:
        super().__init__()
        if not embedding_bag_collection.is_weighted():
            raise AssertionError("EmbeddingBagCollection must accept weighted inputs for feature processor")
        self._embedding_bag_collection = embedding_bag_collection
        whole_kjt = isinstance(feature_processors, FeatureProcessorsCollection)
        self._feature_processors: Union[nn.ModuleDict, FeatureProcessorsCollection] = feature_processors if whole_kjt else nn.ModuleDict(feature_processors)
        if not whole_kjt:
            known = {f for cfg in embedding_bag_collection.embedding_bag_configs() for f in cfg.feature_names}
            strangers = [k for k in self._feature_processors.keys() if k not in known]
            assert not strangers, f"feature processor key {strangers[0]} is not a feature of the EmbeddingBagCollection"

    def _reweigh(self, features: KeyedJaggedTensor) -> KeyedJaggedTensor:
        fp = self._feature_processors
        return fp(features) if isinstance(fp, FeatureProcessorsCollection) else apply_feature_processors_to_kjt(features, fp)

    def split(self) -> Tuple[FeatureProcessorsCollection, EmbeddingBagCollection]:
        """``(processors as one collection, the embedding module)``: what a sharder needs to place the two halves."""
        fp = self._feature_processors
        return (fp if isinstance(fp, FeatureProcessorsCollection) else FeatureProcessorDictWrapper(fp)), self._embedding_bag_collection

    def forward(self, features: KeyedJaggedTensor) -> KeyedTensor:
        return self._embedding_bag_collection(self._reweigh(features))
