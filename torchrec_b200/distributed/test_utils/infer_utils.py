"""Fixtures for inference tests: build and quantize the small test model, place its quantized collections over local devices,
wrappers that take plain tensors instead of a KJT or a ``ModelInput``, and comparison helpers.
Counterpart of ``torchrec/distributed/test_utils/infer_utils.py:98-1118``."""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple, Union

import torch
from torch import nn

from torchrec_b200.distributed.quant_embedding import QuantEmbeddingCollectionSharder
from torchrec_b200.distributed.quant_embeddingbag import QuantEmbeddingBagCollectionSharder
from torchrec_b200.distributed.quant_state import WeightSpec
from torchrec_b200.distributed.test_utils.test_model import ModelInput, TestSparseNN
from torchrec_b200.distributed.types import ModuleSharder, ParameterSharding, ShardingEnv
from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig, EmbeddingConfig
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor, KeyedTensor


@dataclass
class TestModelInfo:
    __test__ = False
    sparse_device: torch.device
    dense_device: torch.device
    num_features: int
    num_float_features: int
    num_weighted_features: int
    tables: Union[List[EmbeddingBagConfig], List[EmbeddingConfig]] = field(default_factory=list)
    weighted_tables: List[EmbeddingBagConfig] = field(default_factory=list)
    model: nn.Module = field(default_factory=nn.Module)
    quant_model: nn.Module = field(default_factory=nn.Module)
    sharders: List[ModuleSharder] = field(default_factory=list)


class TestQuantEBCSharder(QuantEmbeddingBagCollectionSharder):
    """Offers one sharding type / kernel and only the named tables."""

    __test__ = False

    def __init__(self, sharding_type: str, kernel_type: str, fused_params: Optional[Dict[str, Any]] = None, shardable_params: Optional[List[str]] = None) -> None:
        super().__init__(fused_params=fused_params, shardable_params=shardable_params)
        self._sharding_type, self._kernel_type = sharding_type, kernel_type

    def sharding_types(self, compute_device_type: str) -> List[str]:
        return [self._sharding_type]

    def compute_kernels(self, sharding_type: str, compute_device_type: str) -> List[str]:
        return [self._kernel_type]


class TestQuantECSharder(QuantEmbeddingCollectionSharder):
    __test__ = False

    def __init__(self, sharding_type: str, kernel_type: str, fused_params: Optional[Dict[str, Any]] = None, shardable_params: Optional[List[str]] = None) -> None:
        super().__init__(fused_params=fused_params, shardable_params=shardable_params)
        self._sharding_type, self._kernel_type = sharding_type, kernel_type

    def sharding_types(self, compute_device_type: str) -> List[str]:
        return [self._sharding_type]

    def compute_kernels(self, sharding_type: str, compute_device_type: str) -> List[str]:
        return [self._kernel_type]


class KJTInputWrapper(nn.Module):
    """Calls a KJT-taking module from the KJT's plain components."""

    def __init__(self, module_kjt_input: nn.Module) -> None:
        super().__init__()
        self._module_kjt_input = module_kjt_input

    def forward(self, keys: List[str], values: torch.Tensor, weights: Optional[torch.Tensor] = None, lengths: Optional[torch.Tensor] = None,
                offsets: Optional[torch.Tensor] = None):
        return self._module_kjt_input(KeyedJaggedTensor(keys=keys, values=values, weights=weights, lengths=lengths, offsets=offsets))


class TorchTypesModelInputWrapper(nn.Module):
    """Calls a ``ModelInput``-taking module from plain tensors (see ``model_input_to_forward_args``)."""

    def __init__(self, module: nn.Module) -> None:
        super().__init__()
        self._module = module

    def forward(self, float_features: torch.Tensor, idlist_features_keys: List[str], idlist_features_values: torch.Tensor,
                idscore_features_keys: List[str], idscore_features_values: torch.Tensor, idscore_features_weights: Optional[torch.Tensor],
                label: torch.Tensor, idlist_features_lengths: Optional[torch.Tensor] = None, idlist_features_offsets: Optional[torch.Tensor] = None,
                idscore_features_lengths: Optional[torch.Tensor] = None, idscore_features_offsets: Optional[torch.Tensor] = None):
        idlist = KeyedJaggedTensor(keys=idlist_features_keys, values=idlist_features_values, lengths=idlist_features_lengths, offsets=idlist_features_offsets)
        idscore = (KeyedJaggedTensor(keys=idscore_features_keys, values=idscore_features_values, weights=idscore_features_weights,
                                     lengths=idscore_features_lengths, offsets=idscore_features_offsets) if idscore_features_keys else None)
        return self._module(ModelInput(float_features=float_features, idlist_features=idlist, idscore_features=idscore, label=label))


def model_input_to_forward_args_kjt(mi: ModelInput):
    kjt = mi.idlist_features
    assert isinstance(kjt, KeyedJaggedTensor)
    return kjt.keys(), kjt.values(), kjt.weights_or_none(), kjt.lengths_or_none(), kjt.offsets_or_none()


def model_input_to_forward_args(mi: ModelInput):
    a, b = mi.idlist_features, mi.idscore_features
    assert isinstance(a, KeyedJaggedTensor)
    return (mi.float_features, a.keys(), a.values(), b.keys() if b is not None else [], b.values() if b is not None else torch.empty(0, dtype=torch.int64),
            b.weights_or_none() if b is not None else None, mi.label, a.lengths_or_none(), a.offsets_or_none(),
            b.lengths_or_none() if b is not None else None, b.offsets_or_none() if b is not None else None)


def prep_inputs(model_info: TestModelInfo, world_size: int, batch_size: int = 1, count: int = 5, seed: int = 0) -> List[ModelInput]:
    return [ModelInput.generate(batch_size=batch_size, world_size=world_size, num_float_features=model_info.num_float_features, tables=model_info.tables,
                                weighted_tables=model_info.weighted_tables, pooling_avg=3, random_seed=seed + i)[1][0].to(model_info.sparse_device) for i in range(count)]


def quantize(module: nn.Module, inplace: bool = False, output_type: torch.dtype = torch.float, register_tbes: bool = False,
             quant_state_dict_split_scale_bias: bool = False, weight_dtype: torch.dtype = torch.qint8,
             per_table_weight_dtypes: Optional[Dict[str, torch.dtype]] = None) -> nn.Module:
    """Row-wise quantize every embedding collection under ``module``."""
    from torchrec_b200.inference.modules import quantize_embeddings
    from torchrec_b200.quant.embedding_modules import MODULE_ATTR_QUANT_STATE_DICT_SPLIT_SCALE_BIAS, MODULE_ATTR_REGISTER_TBES_BOOL
    from torchrec_b200.quant.embedding_modules import EmbeddingBagCollection as QEBC
    from torchrec_b200.quant.embedding_modules import EmbeddingCollection as QEC

    out = quantize_embeddings(module if inplace else copy.deepcopy(module), dtype=weight_dtype, inplace=True, output_dtype=output_type,
                              per_table_weight_dtype=per_table_weight_dtypes)
    for m in out.modules():
        if isinstance(m, (QEBC, QEC)):
            setattr(m, MODULE_ATTR_REGISTER_TBES_BOOL, register_tbes)
            setattr(m, MODULE_ATTR_QUANT_STATE_DICT_SPLIT_SCALE_BIAS, quant_state_dict_split_scale_bias)
    return out


def create_test_model(num_embeddings: int, emb_dim: int, world_size: int, batch_size: int, dense_device: torch.device, sparse_device: torch.device,
                      num_features: int = 1, num_float_features: int = 8, num_weighted_features: int = 1, quant_state_dict_split_scale_bias: bool = False) -> TestModelInfo:
    """Small model, its quantized copy, and everything a test needs to generate inputs for it."""
    tables = [EmbeddingBagConfig(num_embeddings=num_embeddings, embedding_dim=emb_dim, name=f"table_{i}", feature_names=[f"feature_{i}"]) for i in range(num_features)]
    weighted = [EmbeddingBagConfig(num_embeddings=num_embeddings, embedding_dim=emb_dim, name=f"weighted_table_{i}", feature_names=[f"weighted_feature_{i}"])
                for i in range(num_weighted_features)]
    info = TestModelInfo(sparse_device=sparse_device, dense_device=dense_device, num_features=num_features, num_float_features=num_float_features,
                         num_weighted_features=num_weighted_features, tables=tables, weighted_tables=weighted)
    info.model = TestSparseNN(tables=tables, weighted_tables=weighted, num_float_features=num_float_features, dense_device=dense_device, sparse_device=sparse_device).eval()
    info.quant_model = quantize(info.model, inplace=False, quant_state_dict_split_scale_bias=quant_state_dict_split_scale_bias)
    return info


def shard_qebc(mi: TestModelInfo, sharding_type: str, device: torch.device, expected_shards: Optional[List[List[Tuple[Tuple[int, int, int, int], str]]]] = None,
               world_size: int = 2) -> nn.Module:
    """Copy of ``mi.quant_model`` whose quantized bag collections are placed over ``world_size`` local devices, tables dealt round robin."""
    from torchrec_b200.distributed.quant_embeddingbag import ShardedQuantEmbeddingBagCollection
    from torchrec_b200.quant.embedding_modules import EmbeddingBagCollection as QEBC

    model = copy.deepcopy(mi.quant_model)
    env = ShardingEnv.from_local(world_size=world_size, rank=0)
    for parent in list(model.modules()):
        for name, child in list(parent.named_children()):
            if isinstance(child, QEBC):
                placement = {cfg.name: ParameterSharding(sharding_type=sharding_type, compute_kernel="quant", ranks=[i % world_size])
                             for i, cfg in enumerate(child.embedding_bag_configs())}
                setattr(parent, name, ShardedQuantEmbeddingBagCollection(child, placement, env, device=device))
    return model


def assert_close(expected: Any, actual: Any) -> None:
    """Compare KeyedTensors, dictionaries of (jagged) tensors, or tensors, moving ``actual`` to ``expected``'s device."""
    if isinstance(expected, KeyedTensor):
        assert isinstance(actual, KeyedTensor) and expected.keys() == actual.keys() and expected.length_per_key() == actual.length_per_key()
        assert_close(expected.values(), actual.values())
    elif isinstance(expected, dict):
        assert sorted(expected.keys()) == sorted(actual.keys())
        for k, e in expected.items():
            if isinstance(e, torch.Tensor):
                assert_close(e, actual[k])
            else:
                assert_close(e.lengths(), actual[k].lengths())
                assert_close(e.values(), actual[k].values())
    else:
        if isinstance(actual, torch.Tensor) and isinstance(expected, torch.Tensor) and actual.device != expected.device:
            actual = actual.to(expected.device)
        torch.testing.assert_close(expected, actual)


def assert_weight_spec(weights_spec: Dict[str, WeightSpec], all_expected_shards: List[List[Tuple[Tuple[int, int, int, int], str]]], ebc_fqn: str,
                       weights_prefix: str, all_table_names: List[str], sharding_type: str) -> None:
    """Check ``sharded_tbes_weights_spec`` output against ``((row offset, col offset, rows, cols), "rank:<r>/...")`` per table shard;
    one kernel per rank is assumed."""
    slot: Dict[int, int] = {}
    for table, shards in zip(all_table_names, all_expected_shards):
        unsharded = f"{ebc_fqn}.{weights_prefix}.{table}.weight"
        for (off_r, off_c, rows, cols), placement in shards:
            kernel = int(placement.split("rank:")[1].split("/")[0]) if "rank:" in placement else 0
            key = f"{ebc_fqn}.tbes.{kernel}.{slot.get(kernel, 0)}.{table}.weight"
            slot[kernel] = slot.get(kernel, 0) + 1
            spec = weights_spec[key]
            assert (spec.fqn, spec.shard_offsets, spec.shard_sizes, spec.sharding_type) == (unsharded, [off_r, off_c], [rows, cols], sharding_type), (key, spec)
            for part in ("qscale", "qbias"):
                q = weights_spec[f"{key}_{part}"]
                assert (q.fqn, q.shard_offsets, q.shard_sizes, q.sharding_type) == (f"{unsharded}_{part}", [off_r, 0], [rows, 2], sharding_type), (key, q)
