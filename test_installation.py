"""Smoke test of an installation: trains a tiny sharded model for a few steps on whatever this machine has (one process, CPU/gloo
or the first GPU/NCCL) and prints the losses (cf. ``test_installation.py`` of the reference).

    python test_installation.py
"""
from __future__ import annotations

import os
import sys

import torch
import torch.distributed as dist


def main() -> int:
    from torchrec_b200.datasets.random import RandomRecDataset
    from torchrec_b200.distributed.model_parallel import DistributedModelParallel
    from torchrec_b200.distributed.train_pipeline import TrainPipelineSparseDist
    from torchrec_b200.models.dlrm import DLRM, DLRMTrain
    from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig
    from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
    from torchrec_b200.optim.apply_optimizer_in_backward import apply_optimizer_in_backward
    from torchrec_b200.optim.keyed import CombinedOptimizer, KeyedOptimizerWrapper
    from torchrec_b200.optim.optimizers import in_backward_optimizer_filter
    from torchrec_b200.optim.rowwise_adagrad import RowWiseAdagrad

    use_cuda = torch.cuda.is_available()
    device = torch.device("cuda:0") if use_cuda else torch.device("cpu")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29561")
    dist.init_process_group("nccl" if use_cuda else "gloo", rank=0, world_size=1)
    keys = [f"f{i}" for i in range(4)]
    tables = [EmbeddingBagConfig(name=f"t{i}", embedding_dim=16, num_embeddings=1000, feature_names=[k]) for i, k in enumerate(keys)]
    model = DLRMTrain(DLRM(EmbeddingBagCollection(tables=tables, device=torch.device("meta")), dense_in_features=8, dense_arch_layer_sizes=[16, 16],
                           over_arch_layer_sizes=[16, 1], dense_device=device))
    apply_optimizer_in_backward(RowWiseAdagrad, model.model.sparse_arch.parameters(), {"lr": 0.01})
    dmp = DistributedModelParallel(model, device=device)
    dense = KeyedOptimizerWrapper(dict(in_backward_optimizer_filter(dmp.named_parameters())), lambda ps: torch.optim.SGD(ps, lr=0.1))
    pipe = TrainPipelineSparseDist(dmp, CombinedOptimizer([dmp.fused_optimizer, dense]), device)
    ds = RandomRecDataset(keys=keys, batch_size=32, hash_sizes=[1000] * 4, ids_per_features=[3] * 4, num_dense=8, manual_seed=0, num_batches=12)
    it = iter(ds)
    losses = []
    while True:
        try:
            losses.append(float(pipe.progress(it)[0]))
        except StopIteration:
            break
    print(f"device {device}, {len(losses)} steps, loss {losses[0]:.4f} -> {losses[-1]:.4f}")
    dist.destroy_process_group()
    ok = len(losses) == 12 and all(l == l for l in losses)
    print("installation OK" if ok else "installation BROKEN")
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
