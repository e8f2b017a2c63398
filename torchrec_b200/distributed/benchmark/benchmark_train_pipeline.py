"""Train-pipeline benchmark: a DLRM(-DCN) over synthetic data, sharded by the planner, stepped through a chosen pipeline.

    python -m torchrec_b200.distributed.benchmark.benchmark_train_pipeline --pipeline sparse --num_batches 20 --batch_size 8192
    torchrun --nproc-per-node 8 -m torchrec_b200.distributed.benchmark.benchmark_train_pipeline --yaml_config cfg.yml

Flags come from the dataclasses below through ``cmd_conf``.  Counterpart of
``torchrec/distributed/benchmark/benchmark_train_pipeline.py:61-408``."""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import List, Optional

import torch
import torch.distributed as dist

from torchrec_b200.distributed.benchmark.benchmark_base import BenchmarkResult, benchmark_func, cmd_conf


@dataclass
class RunOptions:
    world_size: int = 1
    num_batches: int = 10
    warmup_batches: int = 3
    pipeline: str = "sparse"  # base | sparse | fused | semisync | prefetch
    dense_optimizer: str = "SGD"
    dense_lr: float = 0.1
    sparse_lr: float = 0.1
    profile: str = ""
    backend: str = ""  # default: nccl with GPUs, gloo otherwise


@dataclass
class EmbeddingTablesConfig:
    num_tables: int = 8
    num_embeddings: int = 100_000
    embedding_dim: int = 128
    pooling_factor: int = 10


@dataclass
class ModelConfig:
    model: str = "dlrm"  # dlrm | dlrm_dcn
    batch_size: int = 8192
    num_float_features: int = 13
    dense_arch_layer_sizes: List[int] = field(default_factory=lambda: [512, 256, 128])
    over_arch_layer_sizes: List[int] = field(default_factory=lambda: [1024, 512, 1])
    dcn_num_layers: int = 3
    dcn_low_rank_dim: int = 512


def _build_pipeline(name: str, model, optimizer, device):
    from torchrec_b200.distributed import train_pipeline as tp

    cls = {"base": tp.TrainPipelineBase, "sparse": tp.TrainPipelineSparseDist, "fused": tp.TrainPipelineFusedSparseDist, "semisync": tp.TrainPipelineSemiSync,
           "prefetch": tp.PrefetchTrainPipelineSparseDist}[name]
    return cls(model, optimizer, device)


def run(run_option: RunOptions, table_config: EmbeddingTablesConfig, model_config: ModelConfig) -> BenchmarkResult:
    from torchrec_b200.datasets.random import RandomRecDataset
    from torchrec_b200.distributed.embeddingbag import EmbeddingBagCollectionSharder
    from torchrec_b200.distributed.model_parallel import DistributedModelParallel
    from torchrec_b200.distributed.planner import EmbeddingShardingPlanner, ParameterConstraints, Topology
    from torchrec_b200.distributed.types import ShardingEnv
    from torchrec_b200.models.dlrm import DLRM, DLRM_DCN, DLRMTrain
    from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig
    from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
    from torchrec_b200.optim.apply_optimizer_in_backward import apply_optimizer_in_backward
    from torchrec_b200.optim.keyed import CombinedOptimizer, KeyedOptimizerWrapper
    from torchrec_b200.optim.optimizers import in_backward_optimizer_filter
    from torchrec_b200.optim.rowwise_adagrad import RowWiseAdagrad

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    use_cuda = torch.cuda.is_available()
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group(run_option.backend or ("nccl" if use_cuda else "gloo"), rank=rank, world_size=world)
    keys = [f"f{i}" for i in range(table_config.num_tables)]
    tables = [EmbeddingBagConfig(name=f"t{i}", embedding_dim=table_config.embedding_dim, num_embeddings=table_config.num_embeddings, feature_names=[k]) for i, k in enumerate(keys)]
    ebc = EmbeddingBagCollection(tables=tables, device=torch.device("meta"))
    if model_config.model == "dlrm_dcn":
        net = DLRM_DCN(ebc, model_config.num_float_features, model_config.dense_arch_layer_sizes[:-1] + [table_config.embedding_dim], model_config.over_arch_layer_sizes,
                       dcn_num_layers=model_config.dcn_num_layers, dcn_low_rank_dim=model_config.dcn_low_rank_dim, dense_device=device)
    else:
        net = DLRM(ebc, model_config.num_float_features, model_config.dense_arch_layer_sizes[:-1] + [table_config.embedding_dim], model_config.over_arch_layer_sizes, dense_device=device)
    model = DLRMTrain(net)
    apply_optimizer_in_backward(RowWiseAdagrad, model.model.sparse_arch.parameters(), {"lr": run_option.sparse_lr})
    sharders = [EmbeddingBagCollectionSharder()]
    constraints = {t.name: ParameterConstraints(pooling_factors=[float(table_config.pooling_factor)]) for t in tables}
    planner = EmbeddingShardingPlanner(topology=Topology(world_size=world, local_world_size=world, compute_device=device.type), batch_size=model_config.batch_size, constraints=constraints)
    plan = planner.collective_plan(model, sharders, dist.group.WORLD)
    dmp = DistributedModelParallel(model, env=ShardingEnv.from_process_group(dist.group.WORLD), device=device, plan=plan, sharders=sharders)
    dense_cls = getattr(torch.optim, run_option.dense_optimizer)
    dense_opt = KeyedOptimizerWrapper(dict(in_backward_optimizer_filter(dmp.named_parameters())), lambda p: dense_cls(p, lr=run_option.dense_lr))
    optimizer = CombinedOptimizer([dmp.fused_optimizer, dense_opt])
    ds = RandomRecDataset(keys=keys, batch_size=model_config.batch_size, hash_size=table_config.num_embeddings, ids_per_feature=table_config.pooling_factor,
                          num_dense=model_config.num_float_features, manual_seed=1234 + rank, num_generated_batches=4)
    batches = [b.pin_memory() if use_cuda else b for b in ds.batch_generator._generated_batches]
    pipe = _build_pipeline(run_option.pipeline, dmp, optimizer, device)

    def endless():
        i = 0
        while True:
            yield batches[i % len(batches)]
            i += 1

    it = endless()
    res = benchmark_func(f"{run_option.pipeline}-{model_config.model}", lambda: pipe.progress(it), num_iters=run_option.num_batches,
                         warmup_iters=run_option.warmup_batches, device=device, rank=rank, profile_dir=run_option.profile)
    if rank == 0:
        print(res)
        ms = float(res.runtime_percentile(50))
        print(f"p50 {ms:.3f} ms/step -> {model_config.batch_size * world / ms * 1e3:.0f} samples/s over {world} rank(s)")
    return res


@cmd_conf
def main(run_option: RunOptions, table_config: EmbeddingTablesConfig, model_config: ModelConfig) -> None:
    run(run_option, table_config, model_config)


if __name__ == "__main__":
    main()
