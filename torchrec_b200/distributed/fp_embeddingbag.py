"""Sharded ``FeatureProcessedEmbeddingBagCollection``: the embedding bags are sharded like any ``EmbeddingBagCollection``, the
feature processors (position weights) are replicated and run on every rank *after* the input distribution, on the ids that
rank looks up; their gradient flows back through the lookup's per-sample weights and is averaged by the model's data-parallel wrapper.
Counterpart of ``torchrec/distributed/fp_embeddingbag.py:48``."""
from __future__ import annotations

from typing import Any, Dict, Iterator, List, Optional, Tuple, Type, Union

import torch
from torch import nn

from torchrec_b200.distributed.embedding_types import BaseEmbeddingSharder, KJTList, ShardedEmbeddingModule
from torchrec_b200.distributed.embeddingbag import EmbeddingBagCollectionContext, EmbeddingBagCollectionSharder, ShardedEmbeddingBagCollection
from torchrec_b200.distributed.types import Awaitable, LazyAwaitable, ParameterSharding, QuantizedCommCodecs, ShardingEnv, ShardingType
from torchrec_b200.modules.feature_processor_ import FeatureProcessorsCollection
from torchrec_b200.modules.fp_embedding_modules import FeatureProcessedEmbeddingBagCollection, apply_feature_processors_to_kjt
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor, KeyedTensor


def param_dp_sync(kt: KeyedTensor, no_op_tensor: torch.Tensor) -> KeyedTensor:
    """Ties the output to every processor parameter so that DDP sees all of them used on every rank."""
    kt._values = kt._values + no_op_tensor
    return kt


class ShardedFeatureProcessedEmbeddingBagCollection(ShardedEmbeddingModule[KJTList, List[torch.Tensor], KeyedTensor, EmbeddingBagCollectionContext]):
    def __init__(self, module: FeatureProcessedEmbeddingBagCollection, table_name_to_parameter_sharding: Dict[str, ParameterSharding],
                 ebc_sharder: EmbeddingBagCollectionSharder, env: ShardingEnv, device: torch.device, module_fqn: Optional[str] = None) -> None:
        super().__init__()
        self._device = device
        self._env = env
        self._embedding_bag_collection: ShardedEmbeddingBagCollection = ebc_sharder.shard(
            module._embedding_bag_collection, table_name_to_parameter_sharding, env=env, device=device,
            module_fqn=(module_fqn + "._embedding_bag_collection") if module_fqn else None)
        self._embedding_bag_collection.disable_fused_engine()  # the processors run between input dist and lookup
        # row-wise input distributions must ship the position of every id in its bag
        for sharding in self._embedding_bag_collection._embedding_shardings:
            if hasattr(sharding, "_has_feature_processor"):
                sharding._has_feature_processor = True
        self._lookups = self._embedding_bag_collection._lookups
        self._is_collection = False
        self._feature_processors: Union[nn.ModuleDict, FeatureProcessorsCollection]
        if isinstance(module._feature_processors, FeatureProcessorsCollection):
            self._feature_processors = module._feature_processors.copy(device) if hasattr(module._feature_processors, "copy") else module._feature_processors.to(device)
            self._is_collection = True
        else:
            self._feature_processors = nn.ModuleDict({k: (fp.copy(device) if hasattr(fp, "copy") else fp.to(device)) for k, fp in module._feature_processors.items()})
            self._is_collection = False
        # the processors stay ordinary replicated parameters: the data-parallel wrapper of the whole model averages their gradient
        self._no_op_zero = torch.zeros((1, 1), device=device)

    # ---- pipeline stages ---------------------------------------------------------------------------------
    def input_dist(self, ctx: EmbeddingBagCollectionContext, features: KeyedJaggedTensor) -> Awaitable[Awaitable[KJTList]]:
        if not self._is_collection and features.weights_or_none() is None:
            features = KeyedJaggedTensor(keys=features.keys(), values=features.values(), lengths=features.lengths(), offsets=features._offsets, stride=features._stride,
                                         weights=torch.ones(features.values().numel(), dtype=torch.float32, device=features.device()))
        return self._embedding_bag_collection.input_dist(ctx, features)

    def apply_feature_processors_to_kjt_list(self, dist_input: KJTList) -> KJTList:
        out = []
        for features in dist_input:
            if self._is_collection:
                out.append(self._feature_processors(features))
            else:
                out.append(apply_feature_processors_to_kjt(features, self._feature_processors))
        return KJTList(out)

    def compute(self, ctx: EmbeddingBagCollectionContext, dist_input: KJTList) -> List[torch.Tensor]:
        return self._embedding_bag_collection.compute(ctx, self.apply_feature_processors_to_kjt_list(dist_input))

    def output_dist(self, ctx: EmbeddingBagCollectionContext, output: List[torch.Tensor]) -> LazyAwaitable[KeyedTensor]:
        lazy = self._embedding_bag_collection.output_dist(ctx, output)
        return self.add_fp_params_grad_sync_callback(lazy)

    def compute_and_output_dist(self, ctx: EmbeddingBagCollectionContext, input: KJTList) -> LazyAwaitable[KeyedTensor]:
        lazy = self._embedding_bag_collection.compute_and_output_dist(ctx, self.apply_feature_processors_to_kjt_list(input))
        return self.add_fp_params_grad_sync_callback(lazy)

    def add_fp_params_grad_sync_callback(self, pooled: LazyAwaitable[KeyedTensor]) -> LazyAwaitable[KeyedTensor]:
        params = [p for p in self._feature_processors.parameters() if p.requires_grad]
        if params:
            no_op = self._no_op_zero * torch.cat([p.view(-1)[:1] for p in params]).sum().view(1, 1)
            pooled.callbacks.append(lambda kt: param_dp_sync(kt, no_op.to(kt.values().dtype)))
        return pooled

    def create_context(self) -> EmbeddingBagCollectionContext:
        return self._embedding_bag_collection.create_context()

    # ---- module surface ------------------------------------------------------------------------------------
    def sharded_parameter_names(self, prefix: str = "") -> Iterator[str]:
        yield from self._embedding_bag_collection.sharded_parameter_names((prefix + "." if prefix else "") + "_embedding_bag_collection")

    @property
    def unsharded_module_type(self) -> Type[FeatureProcessedEmbeddingBagCollection]:
        return FeatureProcessedEmbeddingBagCollection


class FeatureProcessedEmbeddingBagCollectionSharder(BaseEmbeddingSharder[FeatureProcessedEmbeddingBagCollection]):
    def __init__(self, ebc_sharder: Optional[EmbeddingBagCollectionSharder] = None, qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None) -> None:
        super().__init__(qcomm_codecs_registry=qcomm_codecs_registry)
        self._ebc_sharder = ebc_sharder or EmbeddingBagCollectionSharder(qcomm_codecs_registry=self.qcomm_codecs_registry)

    def shard(self, module: FeatureProcessedEmbeddingBagCollection, params: Dict[str, ParameterSharding], env: ShardingEnv,
              device: Optional[torch.device] = None, module_fqn: Optional[str] = None) -> ShardedFeatureProcessedEmbeddingBagCollection:
        if device is None:
            device = torch.device("cuda") if torch.cuda.is_available() else torch.device("cpu")
        return ShardedFeatureProcessedEmbeddingBagCollection(module, params, ebc_sharder=self._ebc_sharder, env=env, device=device, module_fqn=module_fqn)

    @property
    def fused_params(self) -> Optional[Dict[str, Any]]:
        return self._ebc_sharder.fused_params

    def shardable_parameters(self, module: FeatureProcessedEmbeddingBagCollection) -> Dict[str, nn.Parameter]:
        return self._ebc_sharder.shardable_parameters(module._embedding_bag_collection)

    @property
    def module_type(self) -> Type[FeatureProcessedEmbeddingBagCollection]:
        return FeatureProcessedEmbeddingBagCollection

    def sharding_types(self, compute_device_type: str) -> List[str]:
        # data-parallel tables would hide the processors' gradient path behind a second DDP: left out, like the reference
        return [t for t in self._ebc_sharder.sharding_types(compute_device_type) if t != ShardingType.DATA_PARALLEL.value]
