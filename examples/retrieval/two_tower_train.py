"""Train the two-tower model on synthetic (user, item, label) triples with a sharded embedding collection, then build the
retrieval module and query it.

    python examples/retrieval/two_tower_train.py --num_iterations 30
    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 2 examples/retrieval/two_tower_train.py

(cf. ``examples/retrieval/two_tower_train.py`` and ``two_tower_retrieval.py`` of the reference.)"""
from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from two_tower import TwoTower, TwoTowerRetrieval, TwoTowerTrainTask  # noqa: E402

from torchrec_b200.datasets.utils import Batch  # noqa: E402
from torchrec_b200.distributed.model_parallel import DistributedModelParallel  # noqa: E402
from torchrec_b200.distributed.planner import EmbeddingShardingPlanner, Topology  # noqa: E402
from torchrec_b200.distributed.train_pipeline import TrainPipelineSparseDist  # noqa: E402
from torchrec_b200.distributed.types import ShardingEnv  # noqa: E402
from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig  # noqa: E402
from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection  # noqa: E402
from torchrec_b200.optim.apply_optimizer_in_backward import apply_optimizer_in_backward  # noqa: E402
from torchrec_b200.optim.keyed import CombinedOptimizer, KeyedOptimizerWrapper  # noqa: E402
from torchrec_b200.optim.optimizers import in_backward_optimizer_filter  # noqa: E402
from torchrec_b200.optim.rowwise_adagrad import RowWiseAdagrad  # noqa: E402
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor  # noqa: E402


def batches(n: int, batch_size: int, num_users: int, num_items: int, gen: torch.Generator):
    """A user likes the items congruent to its id modulo 7: learnable from ids alone."""
    for _ in range(n):
        users = torch.randint(0, num_users, (batch_size,), generator=gen)
        items = torch.randint(0, num_items, (batch_size,), generator=gen)
        labels = ((users % 7) == (items % 7)).float()
        kjt = KeyedJaggedTensor(keys=["userId", "movieId"], values=torch.cat([users, items]), lengths=torch.ones(2 * batch_size, dtype=torch.int64))
        yield Batch(dense_features=torch.zeros(batch_size, 1), sparse_features=kjt, labels=labels)


def main() -> None:
    p = argparse.ArgumentParser()
    p.add_argument("--num_users", type=int, default=70)
    p.add_argument("--num_items", type=int, default=140)
    p.add_argument("--embedding_dim", type=int, default=32)
    p.add_argument("--layer_sizes", type=str, default="64,32")
    p.add_argument("--batch_size", type=int, default=256)
    p.add_argument("--num_iterations", type=int, default=300)
    p.add_argument("--learning_rate", type=float, default=0.05)
    a = p.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    if torch.cuda.is_available():
        device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
        torch.cuda.set_device(device)
        backend = "nccl"
    else:
        device, backend = torch.device("cpu"), "gloo"
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29552")
        dist.init_process_group(backend, rank=rank, world_size=world)
    torch.manual_seed(0)
    tables = [EmbeddingBagConfig(name="t_userId", embedding_dim=a.embedding_dim, num_embeddings=a.num_users, feature_names=["userId"], weight_init_min=-0.5, weight_init_max=0.5),
              EmbeddingBagConfig(name="t_movieId", embedding_dim=a.embedding_dim, num_embeddings=a.num_items, feature_names=["movieId"], weight_init_min=-0.5, weight_init_max=0.5)]  # away from the saddle at zero
    ebc = EmbeddingBagCollection(tables=tables, device=torch.device("meta"))
    task = TwoTowerTrainTask(TwoTower(ebc, [int(x) for x in a.layer_sizes.split(",")], device=device))
    apply_optimizer_in_backward(RowWiseAdagrad, task.two_tower.ebc.parameters(), {"lr": a.learning_rate})
    planner = EmbeddingShardingPlanner(topology=Topology(world_size=world, compute_device=device.type, local_world_size=world), batch_size=a.batch_size, debug=False)
    plan = planner.collective_plan(task, pg=dist.group.WORLD)
    dmp = DistributedModelParallel(task, env=ShardingEnv.from_process_group(dist.group.WORLD), device=device, plan=plan)
    dense = KeyedOptimizerWrapper(dict(in_backward_optimizer_filter(dmp.named_parameters())), lambda ps: torch.optim.Adagrad(ps, lr=a.learning_rate))
    pipe = TrainPipelineSparseDist(dmp, CombinedOptimizer([dmp.fused_optimizer, dense]), device)
    it = iter(batches(a.num_iterations, a.batch_size, a.num_users, a.num_items, torch.Generator().manual_seed(10 + rank)))
    losses = []
    while True:
        try:
            losses.append(float(pipe.progress(it)[0]))
        except StopIteration:
            break
    if rank == 0:
        print(f"loss: first 10 steps {sum(losses[:10]) / 10:.4f} -> last 10 steps {sum(losses[-10:]) / 10:.4f}", flush=True)
    if world == 1:
        # retrieval needs the whole candidate table on one device: rebuild an unsharded copy from the state dict
        full_ebc = EmbeddingBagCollection(tables=tables, device=device)
        full = TwoTower(full_ebc, [int(x) for x in a.layer_sizes.split(",")], device=device)
        sd = {k[len("two_tower."):]: (v.local_shards()[0].tensor if hasattr(v, "local_shards") else v) for k, v in dmp.state_dict().items() if k.startswith("two_tower.")}
        sd.pop("bias", None)
        full.load_state_dict(sd)
        retrieval = TwoTowerRetrieval(full.eval(), a.num_items, k=5)
        users = torch.arange(4)
        top = retrieval(KeyedJaggedTensor(keys=["userId"], values=users.to(device), lengths=torch.ones(4, dtype=torch.int64, device=device)))
        print("top-5 items per user:", top.tolist(), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
