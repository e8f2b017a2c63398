"""Builders shared by the benchmarks: model configs (small test model, DeepFM, DLRM), synthetic inputs, a planner restricted to one
sharding type and kernel, the sharded model with its combined optimizer, and the train pipeline by name.
Counterpart of ``torchrec/distributed/benchmark/benchmark_utils.py:59-535``."""
from __future__ import annotations

import abc
from dataclasses import dataclass, field, fields
from typing import Any, Dict, List, Optional, Tuple, Type, Union

import torch
import torch.distributed as dist
from torch import nn

from torchrec_b200.distributed.embedding_types import EmbeddingComputeKernel
from torchrec_b200.distributed.model_parallel import DistributedModelParallel
from torchrec_b200.distributed.planner import EmbeddingShardingPlanner, HeteroEmbeddingShardingPlanner, ParameterConstraints, Topology
from torchrec_b200.distributed.planner.constants import NUM_POOLINGS, POOLING_FACTOR
from torchrec_b200.distributed.test_utils.test_model import ModelInput, TestEBCSharder, TestOverArch, TestSparseNN
from torchrec_b200.distributed.train_pipeline import (
    PrefetchTrainPipelineSparseDist,
    TrainPipelineBase,
    TrainPipelineFusedSparseDist,
    TrainPipelineSemiSync,
    TrainPipelineSparseDist,
)
from torchrec_b200.distributed.types import ShardingEnv, ShardingType
from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig
from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
from torchrec_b200.optim.keyed import CombinedOptimizer, KeyedOptimizerWrapper
from torchrec_b200.optim.optimizers import in_backward_optimizer_filter


@dataclass
class BaseModelConfig(abc.ABC):
    """What every benchmark model needs to build itself and its inputs."""

    batch_size: int = 8192
    batch_sizes: Optional[List[int]] = None
    num_float_features: int = 10
    feature_pooling_avg: int = 10
    use_offsets: bool = False
    dev_str: str = ""
    long_kjt_indices: bool = True
    long_kjt_offsets: bool = True
    long_kjt_lengths: bool = True
    pin_memory: bool = True

    @abc.abstractmethod
    def generate_model(self, tables: List[EmbeddingBagConfig], weighted_tables: List[EmbeddingBagConfig], dense_device: torch.device) -> nn.Module: ...


@dataclass
class TestSparseNNConfig(BaseModelConfig):
    __test__ = False
    embedding_groups: Optional[Dict[str, List[str]]] = None
    over_arch_clazz: Type[nn.Module] = TestOverArch
    postproc_module: Optional[nn.Module] = None

    def generate_model(self, tables, weighted_tables, dense_device) -> nn.Module:
        return TestSparseNN(tables=tables, num_float_features=self.num_float_features, weighted_tables=weighted_tables, dense_device=dense_device,
                            sparse_device=torch.device("meta"), over_arch_clazz=self.over_arch_clazz, postproc_module=self.postproc_module,
                            embedding_groups=self.embedding_groups)


class _BatchAdapter(nn.Module):
    """Feeds a ``(dense, KJT)`` model from a ``ModelInput`` and adds the training loss."""

    def __init__(self, model: nn.Module, probabilities: bool) -> None:
        super().__init__()
        self.model = model
        self._probabilities = probabilities

    def forward(self, batch: ModelInput):
        out = self.model(batch.float_features, batch.idlist_features).squeeze(-1)
        if not self.training:
            return out
        loss_fn = torch.nn.functional.binary_cross_entropy if self._probabilities else torch.nn.functional.binary_cross_entropy_with_logits
        return loss_fn(out.float(), batch.label.float()), out


@dataclass
class DeepFMConfig(BaseModelConfig):
    hidden_layer_size: int = 20
    deep_fm_dimension: int = 5

    def generate_model(self, tables, weighted_tables, dense_device) -> nn.Module:
        from torchrec_b200.models.deepfm import SimpleDeepFMNN

        ebc = EmbeddingBagCollection(tables=tables, device=torch.device("meta"))
        net = SimpleDeepFMNN(num_dense_features=self.num_float_features, embedding_bag_collection=ebc, hidden_layer_size=self.hidden_layer_size,
                             deep_fm_dimension=self.deep_fm_dimension)
        for name in ("dense_arch", "inter_arch", "over_arch"):
            getattr(net, name).to(dense_device)
        return _BatchAdapter(net, probabilities=True)


@dataclass
class DLRMConfig(BaseModelConfig):
    dense_arch_layer_sizes: List[int] = field(default_factory=lambda: [20, 128])
    over_arch_layer_sizes: List[int] = field(default_factory=lambda: [5, 1])

    def generate_model(self, tables, weighted_tables, dense_device) -> nn.Module:
        from torchrec_b200.models.dlrm import DLRM

        ebc = EmbeddingBagCollection(tables=tables, device=torch.device("meta"))
        return _BatchAdapter(DLRM(ebc, self.num_float_features, self.dense_arch_layer_sizes, self.over_arch_layer_sizes, dense_device=dense_device), probabilities=False)


_MODEL_CONFIGS: Dict[str, Type[BaseModelConfig]] = {"test_sparse_nn": TestSparseNNConfig, "deepfm": DeepFMConfig, "dlrm": DLRMConfig}


def create_model_config(model_name: str, **kwargs: Any) -> BaseModelConfig:
    """Config by name; keyword arguments the chosen config does not know are dropped."""
    if model_name not in _MODEL_CONFIGS:
        raise ValueError(f"Unknown model name: {model_name}")
    cls = _MODEL_CONFIGS[model_name]
    known = {f.name for f in fields(cls)}
    return cls(**{k: v for k, v in kwargs.items() if k in known})


def generate_pipeline(pipeline_type: str, emb_lookup_stream: str, model: nn.Module, opt: torch.optim.Optimizer, device: torch.device, apply_jit: bool = False):
    """``base`` | ``sparse`` | ``fused`` | ``semi`` | ``prefetch``."""
    if pipeline_type == "base":
        assert not apply_jit, "JIT is not supported for base pipeline"
        return TrainPipelineBase(model=model, optimizer=opt, device=device)
    if pipeline_type == "semi":
        return TrainPipelineSemiSync(model=model, optimizer=opt, device=device, start_batch=0, apply_jit=apply_jit)
    if pipeline_type == "fused":
        return TrainPipelineFusedSparseDist(model=model, optimizer=opt, device=device, emb_lookup_stream=emb_lookup_stream, apply_jit=apply_jit)
    table = {"sparse": TrainPipelineSparseDist, "prefetch": PrefetchTrainPipelineSparseDist}
    if pipeline_type not in table:
        raise RuntimeError(f"Unknown pipeline type: {pipeline_type}")
    return table[pipeline_type](model=model, optimizer=opt, device=device, apply_jit=apply_jit)


def generate_data(tables: List[EmbeddingBagConfig], weighted_tables: List[EmbeddingBagConfig], model_config: BaseModelConfig, batch_sizes: List[int]) -> List[ModelInput]:
    """One local batch per entry of ``batch_sizes`` (pinned when asked and possible)."""
    device = torch.device(model_config.dev_str) if model_config.dev_str else None
    out = []
    for i, bs in enumerate(batch_sizes):
        _, (local,) = ModelInput.generate(batch_size=bs, world_size=1, num_float_features=model_config.num_float_features, tables=tables,
                                          weighted_tables=weighted_tables, pooling_avg=model_config.feature_pooling_avg, device=device,
                                          indices_dtype=torch.int64 if model_config.long_kjt_indices else torch.int32,
                                          lengths_dtype=torch.int64 if model_config.long_kjt_lengths else torch.int32, random_seed=1000 + i)
        if model_config.pin_memory and device is None and torch.cuda.is_available():
            local = ModelInput(local.float_features.pin_memory(), local.idlist_features.pin_memory() if local.idlist_features is not None else None,
                               local.idscore_features.pin_memory() if local.idscore_features is not None else None, local.label.pin_memory())
        out.append(local)
    return out


def generate_planner(planner_type: str, topology: Topology, tables: Optional[List[EmbeddingBagConfig]], weighted_tables: Optional[List[EmbeddingBagConfig]],
                     sharding_type: ShardingType, compute_kernel: EmbeddingComputeKernel, batch_sizes: List[int],
                     pooling_factors: Optional[List[float]] = None, num_poolings: Optional[List[float]] = None):
    """Planner (``embedding`` or ``hetero``) whose every table is held to one sharding type and one kernel."""
    n = len(batch_sizes)
    pooling_factors = pooling_factors if pooling_factors is not None else [POOLING_FACTOR] * n
    num_poolings = num_poolings if num_poolings is not None else [NUM_POOLINGS] * n
    assert len(pooling_factors) == n and len(num_poolings) == n, "The length of pooling_factors and num_poolings must match the number of batches."
    constraints: Dict[str, ParameterConstraints] = {}
    for group, weighted in ((tables or [], False), (weighted_tables or [], True)):
        for t in group:
            constraints[t.name] = ParameterConstraints(sharding_types=[sharding_type.value], compute_kernels=[compute_kernel.value], device_group=topology.compute_device,
                                                       pooling_factors=pooling_factors, num_poolings=num_poolings, batch_sizes=batch_sizes, is_weighted=weighted)
    if planner_type == "embedding":
        return EmbeddingShardingPlanner(topology=topology, constraints=constraints or None)
    if planner_type == "hetero":
        return HeteroEmbeddingShardingPlanner(topology_groups={topology.compute_device: topology}, constraints=constraints or None)
    raise RuntimeError(f"Unknown planner type: {planner_type}")


def generate_sharded_model_and_optimizer(model: nn.Module, sharding_type: str, kernel_type: str, pg: dist.ProcessGroup, device: torch.device,
                                         fused_params: Dict[str, Any], dense_optimizer: str = "SGD", dense_lr: float = 0.1,
                                         dense_momentum: Optional[float] = None, dense_weight_decay: Optional[float] = None,
                                         planner: Optional[Union[EmbeddingShardingPlanner, HeteroEmbeddingShardingPlanner]] = None) -> Tuple[nn.Module, torch.optim.Optimizer]:
    """Shard ``model`` (collective plan when a planner is given, else the default plan of the restricted sharder) and pair the fused
    embedding optimizer with a dense optimizer by name."""
    sharders = [TestEBCSharder(sharding_type=sharding_type, kernel_type=kernel_type, fused_params=fused_params)]
    plan = planner.collective_plan(model, sharders, pg) if planner is not None else None
    dmp = DistributedModelParallel(module=model, env=ShardingEnv.from_process_group(pg), init_data_parallel=True, device=device, sharders=sharders, plan=plan).to(device)
    kwargs: Dict[str, Any] = {"lr": dense_lr}
    if dense_momentum is not None:
        kwargs["momentum"] = dense_momentum
    if dense_weight_decay is not None:
        kwargs["weight_decay"] = dense_weight_decay
    opt_cls = getattr(torch.optim, dense_optimizer)
    dense = KeyedOptimizerWrapper(dict(in_backward_optimizer_filter(dmp.named_parameters())), lambda params: opt_cls(params, **kwargs))
    return dmp, CombinedOptimizer([dmp.fused_optimizer, dense])
