"""Canonical training script: DLRM on synthetic click data, embeddings sharded by the planner, optimizer fused into the
embedding backward, dense part data-parallel, stepped by ``TrainPipelineSparseDist``.

    python examples/golden_training/train_dlrm.py --num_iterations 20
    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 8 examples/golden_training/train_dlrm.py

(cf. ``examples/golden_training/train_dlrm.py`` of the reference.)"""
from __future__ import annotations

import argparse
import os
import sys
from typing import List, Optional

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from torchrec_b200.datasets.random import RandomRecDataset  # noqa: E402
from torchrec_b200.distributed.embeddingbag import EmbeddingBagCollectionSharder  # noqa: E402
from torchrec_b200.distributed.model_parallel import DistributedModelParallel  # noqa: E402
from torchrec_b200.distributed.planner import EmbeddingShardingPlanner, Topology  # noqa: E402
from torchrec_b200.distributed.train_pipeline import TrainPipelineSparseDist  # noqa: E402
from torchrec_b200.distributed.types import ShardingEnv  # noqa: E402
from torchrec_b200.metrics.metric_module import RecMetricModule, generate_metric_module  # noqa: E402
from torchrec_b200.metrics.metrics_config import DefaultTaskInfo, MetricsConfig, RecMetricDef, RecMetricEnum, ThroughputDef  # noqa: E402
from torchrec_b200.models.dlrm import DLRM, DLRMTrain  # noqa: E402
from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig  # noqa: E402
from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection  # noqa: E402
from torchrec_b200.optim.apply_optimizer_in_backward import apply_optimizer_in_backward  # noqa: E402
from torchrec_b200.optim.keyed import CombinedOptimizer, KeyedOptimizerWrapper  # noqa: E402
from torchrec_b200.optim.optimizers import in_backward_optimizer_filter  # noqa: E402
from torchrec_b200.optim.rowwise_adagrad import RowWiseAdagrad  # noqa: E402


def train(num_embeddings: int = 100_000, embedding_dim: int = 64, num_tables: int = 8, dense_arch_layer_sizes: Optional[List[int]] = None,
          over_arch_layer_sizes: Optional[List[int]] = None, learning_rate: float = 0.1, batch_size: int = 2048, num_iterations: int = 50) -> float:
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if torch.cuda.is_available():
        device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
        torch.cuda.set_device(device)
        backend = "nccl"
    else:
        device, backend = torch.device("cpu"), "gloo"
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29541")
        dist.init_process_group(backend, rank=rank, world_size=world)
    keys = [f"cat_{i}" for i in range(num_tables)]
    tables = [EmbeddingBagConfig(name=f"t_{k}", embedding_dim=embedding_dim, num_embeddings=num_embeddings, feature_names=[k]) for k in keys]
    # build on the meta device: tables are materialised shard by shard on their ranks
    model = DLRMTrain(DLRM(EmbeddingBagCollection(tables=tables, device=torch.device("meta")), dense_in_features=13,
                           dense_arch_layer_sizes=dense_arch_layer_sizes or [128, embedding_dim], over_arch_layer_sizes=over_arch_layer_sizes or [256, 128, 1],
                           dense_device=device))
    apply_optimizer_in_backward(RowWiseAdagrad, model.model.sparse_arch.parameters(), {"lr": learning_rate})
    sharders = [EmbeddingBagCollectionSharder()]
    planner = EmbeddingShardingPlanner(topology=Topology(world_size=world, local_world_size=world, compute_device=device.type), batch_size=batch_size)
    plan = planner.collective_plan(model, sharders, dist.group.WORLD)
    dmp = DistributedModelParallel(model, env=ShardingEnv.from_process_group(dist.group.WORLD), device=device, plan=plan, sharders=sharders)
    dense_opt = KeyedOptimizerWrapper(dict(in_backward_optimizer_filter(dmp.named_parameters())), lambda p: torch.optim.Adagrad(p, lr=learning_rate))
    optimizer = CombinedOptimizer([dmp.fused_optimizer, dense_opt])
    pipeline = TrainPipelineSparseDist(dmp, optimizer, device)
    data = iter(RandomRecDataset(keys=keys, batch_size=batch_size, hash_size=num_embeddings, ids_per_feature=3, num_dense=13, manual_seed=rank))
    metrics = generate_metric_module(
        RecMetricModule, MetricsConfig(rec_tasks=[DefaultTaskInfo], rec_metrics={RecMetricEnum.NE: RecMetricDef(rec_tasks=[DefaultTaskInfo], window_size=batch_size * world * 10)},
                                      throughput_metric=ThroughputDef(warmup_steps=5), compute_interval_steps=10),
        batch_size=batch_size, world_size=world, my_rank=rank, state_metrics_mapping={}, device=device)
    last = float("nan")
    for it in range(num_iterations):
        loss, logits, labels = pipeline.progress(data)  # the model's second output: (detached loss, logits, labels)
        metrics.update({"prediction": torch.sigmoid(logits.detach().float()), "label": labels.detach().float(), "weight": torch.ones_like(labels, dtype=torch.float)})
        if metrics.should_compute():
            res = metrics.compute()
            last = float(loss)
            if rank == 0:
                print(f"iter {it + 1}: loss {last:.4f} " + " ".join(f"{k.split('|')[1]}={float(v):.4g}" for k, v in res.items() if "window" in k or "total" in k), flush=True)
    return last


def main(argv: List[str]) -> None:
    p = argparse.ArgumentParser()
    p.add_argument("--num_embeddings", type=int, default=100_000)
    p.add_argument("--embedding_dim", type=int, default=64)
    p.add_argument("--num_tables", type=int, default=8)
    p.add_argument("--batch_size", type=int, default=2048)
    p.add_argument("--num_iterations", type=int, default=50)
    p.add_argument("--learning_rate", type=float, default=0.1)
    a = p.parse_args(argv)
    train(a.num_embeddings, a.embedding_dim, a.num_tables, None, None, a.learning_rate, a.batch_size, a.num_iterations)


if __name__ == "__main__":
    main(sys.argv[1:])
